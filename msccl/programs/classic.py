"""Classic collective algorithms written in MSCCLang: recursive doubling / halving, hierarchical
(two-level) all-reduce, tree-reduced all-pairs, and the point-to-point "all to next" pipeline
collective.  They cover the algorithm families of the reference's ``examples/mscclang`` directory
(allgather_recursive_doubling.py, allreduce_recursive_doubling_halving.py, hierarchical_allreduce.py,
allreduce_a100_allpairs_v2.py, alltonext_forward.py / alltonext_backward.py) as importable functions.
"""
from msccl.language import Buffer, chunk
from msccl.language.collectives import Collective
from msccl.language.symbolic import Chunk


# ------------------------------------------------------------------ recursive doubling / halving
def allgather_recursive_doubling(size):
    """In-place all-gather in log2(size) exchanges: at distance d every rank swaps the d chunks it
    has gathered so far with rank ^ d."""
    d = 1
    while d < size:
        for rank in range(size):
            peer, first = rank ^ d, (rank // d) * d
            chunk(rank, Buffer.output, first, size=d).copy(peer, Buffer.output, first, sendtb=peer, recvtb=rank)
        d *= 2


def allreduce_recursive_halving_doubling(size):
    """In-place all-reduce on ``size`` chunks: recursive vector halving (reduce-scatter) followed by
    recursive vector doubling (all-gather)."""
    d = size // 2
    while d >= 1:
        for rank in range(size):
            peer = rank ^ d
            first = (peer // d) * d
            mine = chunk(rank, Buffer.input, first, size=d)
            chunk(peer, Buffer.output, first, size=d).reduce(mine, sendtb=peer, recvtb=rank, ch=0)
        d //= 2
    d = 1
    while d < size:
        for rank in range(size):
            peer, first = rank ^ d, (rank // d) * d
            chunk(rank, Buffer.output, first, size=d).copy(peer, Buffer.output, first, sendtb=peer, recvtb=rank, ch=0)
        d *= 2


# ------------------------------------------------------------------------- hierarchical all-reduce
def _ring_reduce_scatter(n, first_rank=0, rank_step=1, width=1, chunk_offset=0, chunk_stride=1, ch=-1):
    for k in range(n):
        index = k * chunk_stride * width + chunk_offset
        for hop in range(n - 1):
            src = ((hop + 1 + k) % n) * rank_step + first_rank
            dst = ((hop + 2 + k) % n) * rank_step + first_rank
            chunk(dst, Buffer.input, index, width).reduce(chunk(src, Buffer.input, index, width), ch=ch)


def _ring_all_gather(n, first_rank=0, rank_step=1, width=1, chunk_offset=0, chunk_stride=1, ch=-1):
    for k in range(n):
        index = k * chunk_stride * width + chunk_offset
        for hop in range(n - 1):
            src = ((hop + k) % n) * rank_step + first_rank
            dst = ((hop + 1 + k) % n) * rank_step + first_rank
            chunk(src, Buffer.input, index, width).copy(dst, Buffer.input, index, ch=ch)


def hierarchical_allreduce(gpus_per_node, num_nodes, manual_channels=False):
    """Two-level in-place all-reduce on ``gpus_per_node*num_nodes`` chunks: ring reduce-scatter inside
    every node, ring reduce-scatter then ring all-gather across nodes between GPUs of equal local
    index, ring all-gather inside every node.  ``manual_channels`` pins the phases to separate
    channels (intra-node phases per chunk offset, the cross-node phases on two more)."""
    def pick(value):
        return value if manual_channels else -1

    for node in range(num_nodes):
        for off in range(num_nodes):
            _ring_reduce_scatter(gpus_per_node, first_rank=node * gpus_per_node, chunk_offset=off,
                                 chunk_stride=num_nodes, ch=pick(off))
    for g in range(gpus_per_node):
        _ring_reduce_scatter(num_nodes, first_rank=g, rank_step=gpus_per_node, chunk_offset=g * num_nodes,
                             ch=pick(g % 2 + num_nodes * 2))
    for g in range(gpus_per_node):
        _ring_all_gather(num_nodes, first_rank=g, rank_step=gpus_per_node, chunk_offset=g * num_nodes,
                         ch=pick(g % 2 + num_nodes * 2))
    for node in range(num_nodes):
        for off in range(num_nodes):
            _ring_all_gather(gpus_per_node, first_rank=node * gpus_per_node, chunk_offset=off,
                             chunk_stride=num_nodes, ch=pick(off + num_nodes))


# ------------------------------------------------------------------ all-pairs with a reduction tree
def allreduce_allpairs_tree(size):
    """All-pairs all-reduce on ``size`` chunks where the owner sums the received copies with a binary
    tree spread over its threadblocks instead of one long chain (``size`` a power of two)."""
    for src in range(size):
        for owner in range(size):
            if src != owner:
                chunk(src, Buffer.input, owner).copy(owner, 'scratch', sendtb=owner, recvtb=src)
    for r in range(size):
        level = 2
        while level <= size:
            for i in range(size // level):
                acc = chunk(r, Buffer.input, r) if i == 0 else chunk(r, 'scratch', i - 1)
                acc.reduce(chunk(r, 'scratch', i + size // level - 1), sendtb=i)
            level *= 2
    for owner in range(size):
        for dst in range(size):
            if owner != dst:
                chunk(owner, Buffer.input, owner).copy(dst, Buffer.input, owner, sendtb=dst, recvtb=owner)


# ------------------------------------------------------------------------------ all-to-next
class AllToNext(Collective):
    """Pipeline hand-over: the chunks of rank r must end up in the output of rank r+1 (``forward``)
    or r-1 (backward).  A custom collective: ``name`` stays 'custom'."""

    def __init__(self, num_ranks, chunk_factor, inplace=False, forward=True):
        super().__init__(num_ranks, chunk_factor, inplace)
        self.forward = forward

    def _target(self, r):
        t = r + 1 if self.forward else r - 1
        return t if 0 <= t < self.num_ranks else None

    def init_buffers(self):
        per_rank = []
        for r in range(self.num_ranks):
            t = self._target(r)
            data = [Chunk(r, c, t, c) if t is not None else None for c in range(self.chunk_factor)]
            per_rank.append({Buffer.input: data, Buffer.output: [None] * self.chunk_factor})
        return per_rank

    def check(self, prog):
        ok = True
        for r in range(self.num_ranks):
            t = self._target(r)
            if t is None:
                continue
            out = prog.buffers[t][Buffer.output]
            for c in range(self.chunk_factor):
                got = out[c]
                if got is None or got.origin_rank != r or got.origin_index != c:
                    print(f'Rank {t} chunk {c} is incorrect should be ({r}, {c}) given {got}')
                    ok = False
        return ok


def alltonext(num_nodes, gpus_per_node=8, forward=True):
    """Every GPU passes its ``gpus_per_node`` chunks to the next (previous) GPU of the pipeline.
    Inside a node that is one direct copy; the hop between nodes is spread over all GPUs of both nodes
    so that every NIC carries one chunk: scatter inside the sending node, one cross-node copy per
    GPU pair, gather on the receiving GPU."""
    size = num_nodes * gpus_per_node
    step = 1 if forward else -1

    def rank(node, g):
        return node * gpus_per_node + g

    edge_g = gpus_per_node - 1 if forward else 0          # the GPU whose neighbour lives on the other node
    for node in range(num_nodes):
        for g in range(gpus_per_node):
            r = rank(node, g)
            nxt = r + step
            if not 0 <= nxt < size:
                continue
            if g != edge_g:
                chunk(r, Buffer.input, 0, gpus_per_node).copy(nxt, Buffer.output, 0, ch=g % 2)
                continue
            other = node + step
            tag = f's{node}->{other}'
            for c in range(gpus_per_node):
                piece = chunk(r, Buffer.input, c)
                if c != edge_g:                               # scatter inside my node first
                    piece = piece.copy(rank(node, c), tag, 0, ch=c % 2)
                if rank(other, c) != nxt:                     # cross-node copy to the matching GPU, gathered below
                    piece = piece.copy(rank(other, c), tag, 0, ch=c % 2)
                piece.copy(nxt, Buffer.output, piece.get_dst_index(), ch=c % 2)


# ------------------------------------------------------------------------------ binomial tree
def allreduce_binomial_tree(size, chunks=1):
    """In-place all-reduce along a binomial tree rooted at rank 0: in round d every rank whose index has bit d
    set (and no lower bit) is folded into the rank ``2^d`` below it, then the sum travels back down the same
    edges.  ``2 ceil(log2 size)`` steps for any ``size``; ``chunks`` = chunk factor of the collective.
    (The reference's ``examples/mscclang/allreduce_binomial_tree.py`` no longer runs against its own API.)"""
    dist = 1
    edges = []
    while dist < size:
        for child in range(dist, size, 2 * dist):
            edges.append((child, child - dist))
        dist *= 2
    for child, parent in edges:                           # up: reduce into the parent
        chunk(parent, Buffer.input, 0, chunks).reduce(chunk(child, Buffer.input, 0, chunks))
    for child, parent in reversed(edges):                 # down: the parent's value replaces the child's
        chunk(parent, Buffer.input, 0, chunks).copy(child, Buffer.input, 0)
