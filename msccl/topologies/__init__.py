"""Topology constructors (``from msccl.topologies import *`` mirrors the reference package)."""
from .topology import Topology
from .generic import fully_connected, hub_and_spoke, ring, line, star
from .nvidia import dgx1, dgx_a100, b200_nvswitch, nvlink_only
from .amd import amd4, amd8
from .distributed import distributed_fully_connected, distributed_hub_and_spoke
from .transformers import reverse_topology, binarize_topology
