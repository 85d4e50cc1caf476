"""All-to-all programs.

``alltoall_hierarchical`` and ``alltoall_three_step`` express the algorithms of the reference's
``msccl/programs/alltoall_a100_yifan.py:6-39`` and ``msccl/programs/alltoall_a100_8kp1.py:6-79``
(identical DSL call sequences).  ``alltoall_direct`` is the single-box NVSwitch algorithm.
"""
from msccl.language import Buffer, chunk


def alltoall_direct(size, lanes=1):
    """Every rank writes chunk (dst, lane) straight into the destination's output (chunk_factor
    = ``lanes``).  One step; the right algorithm when every pair has full port bandwidth."""
    for src in range(size):
        for dst in range(size):
            for lane in range(lanes):
                c = chunk(src, Buffer.input, dst * lanes + lane)
                c.copy(dst, Buffer.output, src * lanes + lane, ch=lane)


def alltoall_hierarchical(num_nodes, gpus_per_node):
    """Two-step all-to-all over ``num_nodes`` machines: data for machine n2 is first regrouped
    inside the machine so that local GPU g holds everything bound for GPU g of n2 (scratch
    ``copy_<n2>``), then one cross-machine transfer per GPU pair delivers ``gpus_per_node``
    chunks at once."""
    for n1 in range(num_nodes):
        peers = [(n1 + k) % num_nodes for k in range(1, num_nodes)]
        for n2 in peers:
            for g1 in range(gpus_per_node):
                for g2 in range(gpus_per_node):
                    c = chunk(n1 * gpus_per_node + g1, Buffer.input, n2 * gpus_per_node + g2)
                    c.copy(n1 * gpus_per_node + g2, f'copy_{n2}')
        for n2 in peers:
            for g in range(gpus_per_node):
                rank = n1 * gpus_per_node + g
                c = chunk(rank, f'copy_{n2}', 0, 8)
                c.copy(n2 * gpus_per_node + g, Buffer.output, c.get_dst_index(),
                       ch=((n1 + n2) % 8) * 2 + (rank % 2) + 2)
    for rank in range(num_nodes * gpus_per_node):
        first = (rank // gpus_per_node) * gpus_per_node
        for g in range(gpus_per_node):
            c = chunk(rank, Buffer.input, first + g)
            c.copy(c.get_dst_rank(), Buffer.output, c.get_dst_index())


def alltoall_three_step(num_nodes, gpus_per_node, instances=1, ib_connections=1):
    """Three-step all-to-all: for every ordered machine pair one designated GPU gathers all
    traffic (scratch named by the pair), a single large cross-machine transfer (optionally split
    over ``ib_connections`` channels) moves it, and the receiving GPU scatters it locally."""
    def rank_of(node, gpu):
        return node * gpus_per_node + gpu

    def gateways(n1, n2):
        def local(a, b):
            return (b if a > b else b - 1) % gpus_per_node
        return rank_of(n1, local(n1, n2)), rank_of(n2, local(n2, n1))

    staged = {}          # (n1, n2) -> reference covering everything gathered for that pair
    for n1 in range(num_nodes):
        for g1 in range(gpus_per_node):
            r1 = rank_of(n1, g1)
            for inst in range(instances):
                for n2 in range(num_nodes):
                    if n1 != n2:
                        c = chunk(r1, Buffer.input, n2 * gpus_per_node * instances + inst * gpus_per_node,
                                  gpus_per_node)
                        out_gpu, _ = gateways(n1, n2)
                        c = c.copy(out_gpu, buffer=(n1, n2), ch=inst * 2)
                        staged[(n1, n2)] = staged[(n1, n2)].group(c) if (n1, n2) in staged else c
                    else:
                        for g2 in range(gpus_per_node):
                            r2 = rank_of(n2, g2)
                            c = chunk(r1, Buffer.input, r2 * instances + inst)
                            c.copy(r2, buffer=Buffer.output, index=c.get_dst_index(), ch=inst * 2)

    for (n1, n2), everything in staged.items():
        _, in_gpu = gateways(n1, n2)
        for lane, part in enumerate(everything.split(ib_connections)):
            # with one connection per pair, alternate channels 0/1 to use both NICs
            wire = part.rank % 2 if ib_connections == 1 else lane
            landed = part.copy(in_gpu, buffer=(n1, n2), ch=wire)
            for piece in landed.split(gpus_per_node * gpus_per_node):
                piece.copy(piece.get_dst_rank(), buffer=Buffer.output, index=piece.get_dst_index(),
                           ch=lane * 2 + 1)
