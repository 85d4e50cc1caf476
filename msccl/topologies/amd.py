"""AMD xGMI machine topologies.  Parity: reference ``msccl/topologies/amd.py:6-26``."""
from .topology import Topology


def amd4():
    """Four GPUs in a square: 0-1, 0-2, 1-3, 2-3."""
    edges = {(0, 1), (0, 2), (1, 3), (2, 3)}
    links = [[1 if (min(s, d), max(s, d)) in edges else 0 for s in range(4)] for d in range(4)]
    return Topology('AMD4', links)


def amd8():
    """Eight GPUs; link weights 5/6 are relative xGMI bandwidths.  Ranks fall in two
    classes A={0,2,3,5}, B={1,4,6,7}: same-class pairs get 6, cross-class pairs 5."""
    cls_a = {0, 2, 3, 5}
    links = [[0 if s == d else (6 if (s in cls_a) == (d in cls_a) else 5) for s in range(8)]
             for d in range(8)]
    return Topology('AMD8', links)
