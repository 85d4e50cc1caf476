"""Multi-machine topologies made of copies of a local topology.

Parity: reference ``msccl/topologies/distributed.py:6-41``.
"""
from .topology import Topology


def _tile(local, copies, remote_bw):
    """Link matrix of ``copies`` replicas; cross-replica pairs get ``remote_bw``."""
    n = local.num_nodes()
    total = n * copies
    links = [[local.links[d % n][s % n] if s // n == d // n else remote_bw
              for s in range(total)] for d in range(total)]
    switches = []
    for srcs, dsts, bw, name in local.switches:
        for i in range(copies):
            shift = i * n
            switches.append(([s + shift for s in srcs], [d + shift for d in dsts], bw,
                             f'copy_{i}_{name}_local'))
    return links, switches


def distributed_fully_connected(local_topology, num_copies, remote_bw):
    links, switches = _tile(local_topology, num_copies, remote_bw)
    name = f'DistributedFullyConnected(local={local_topology.name},copies={num_copies},bw={remote_bw})'
    return Topology(name, links, switches)


def distributed_hub_and_spoke(local_topology, num_copies, remote_bw):
    """Like :func:`distributed_fully_connected` but each machine's NIC is a shared switch."""
    n = local_topology.num_nodes()
    links, switches = _tile(local_topology, num_copies, remote_bw)
    total = n * num_copies
    for i in range(num_copies):
        inside = list(range(i * n, (i + 1) * n))
        outside = [k for k in range(total) if k // n != i]
        switches.append((inside, outside, remote_bw, f'copy_{i}_out_remote'))
        switches.append((outside, inside, remote_bw, f'copy_{i}_in_remote'))
    name = f'DistributedHubAndSpoke(local={local_topology.name},copies={num_copies},bw={remote_bw})'
    return Topology(name, links, switches)
