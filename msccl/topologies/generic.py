"""Generic topology constructors.  Parity: reference ``msccl/topologies/generic.py:6-52``."""
from .topology import Topology


def _matrix(n, connected):
    return [[1 if connected(src, dst) else 0 for src in range(n)] for dst in range(n)]


def fully_connected(num_nodes):
    return Topology(f'FullyConnected(n={num_nodes})', _matrix(num_nodes, lambda s, d: s != d))


def hub_and_spoke(num_nodes):
    """All-to-all unit links plus one ingress and one egress switch of bandwidth 1 per node
    (the NVSwitch model: a GPU's port is the bottleneck, not the fabric)."""
    switches = []
    for node in range(num_nodes):
        rest = [o for o in range(num_nodes) if o != node]
        switches.append(([node], rest, 1, f'node_{node}_out'))
        switches.append((rest, [node], 1, f'node_{node}_in'))
    return Topology(f'HubAndSpoke(n={num_nodes})', _matrix(num_nodes, lambda s, d: s != d), switches)


def ring(num_nodes):
    n = num_nodes
    return Topology(f'Ring(n={n})', _matrix(n, lambda s, d: s != d and ((s - d) % n in (1, n - 1))))


def line(num_nodes):
    return Topology(f'Line(n={num_nodes})', _matrix(num_nodes, lambda s, d: abs(s - d) == 1))


def star(num_nodes, non_blocking=True):
    """Node 0 is the centre.  With ``non_blocking=False`` the centre's port is a shared switch."""
    links = _matrix(num_nodes, lambda s, d: (s == 0) != (d == 0))
    switches = []
    if not non_blocking:
        points = list(range(1, num_nodes))
        switches = [([0], points, 1, 'to_points'), (points, [0], 1, 'from_points')]
    return Topology(f'Star(n={num_nodes})', links, switches)
