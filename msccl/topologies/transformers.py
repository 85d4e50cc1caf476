"""Topology-to-topology transformations.  Parity: reference ``msccl/topologies/transformers.py:6-24``."""
from .topology import Topology


def reverse_topology(topology):
    """Flip the direction of every link and of every switch."""
    n = topology.num_nodes()
    flipped = [[topology.links[s][d] for s in range(n)] for d in range(n)]
    switches = [(dsts, srcs, bw, f'{name}_reversed') for srcs, dsts, bw, name in topology.switches]
    return Topology(f'Reverse{topology.name}', flipped, switches)


def binarize_topology(topology):
    """Keep only connectivity: every existing link gets bandwidth 1 and switches are dropped.
    (Like the reference, the result is indexed transposed; callers use it on symmetric
    connectivity or together with its own link() accessor.)"""
    n = topology.num_nodes()
    links = [[1 if topology.links[s][d] > 0 else 0 for s in range(n)] for d in range(n)]
    return Topology(f'Binarized{topology.name}', links, [])
