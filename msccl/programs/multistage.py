"""All-reduce programs that span more than one group of GPUs: two machines joined by one link per GPU, a
four-GPU box made of two NVLink pairs, and a pipeline in which one stage reduces and the next stage
receives the result.

Parity (behaviour, not text): reference ``examples/mscclang/allreduce_a100_multinode_allpairs.py``,
``allreduce_a100_ncv4.py``, ``pipeline_a100_ring.py`` and ``pipeline_a100_allpairs.py``.  The two pipeline
examples of the reference declare themselves as an ``AllReduce`` over both stages and switch ``Check()``
off because that is not what they compute; here they get a collective of their own (``StageAllReduce``)
whose check holds.
"""
from msccl.language import Buffer, chunk
from msccl.language.collectives import Collective
from msccl.language.symbolic import Chunk, ReduceChunk


# ------------------------------------------------------------------ two (or more) machines, all pairs
def allreduce_multinode_allpairs(gpus_per_node, num_nodes=2):
    """In-place all-reduce with ``chunk_factor = gpus_per_node``.  GPU l of every machine owns chunk l:
    all-pairs scatter and local reduction inside each machine, exchange and reduction of the owned chunk
    between the GPUs with equal local index of all machines (one cross-machine link per GPU), all-pairs
    broadcast inside each machine."""
    g = gpus_per_node

    def rank(node, local):
        return node * g + local

    for node in range(num_nodes):                       # scatter: chunk l of everyone goes to local GPU l
        for src in range(g):
            for owner in range(g):
                if src != owner:
                    chunk(rank(node, src), Buffer.input, owner).copy(rank(node, owner), f'in{node}', src)
    for node in range(num_nodes):                       # local reduction into the owned chunk
        for owner in range(g):
            acc = chunk(rank(node, owner), Buffer.input, owner)
            for src in range(g):
                if src != owner:
                    acc.reduce(chunk(rank(node, owner), f'in{node}', src))
    for owner in range(g):                              # partial sums cross machines between equal local indices
        for a in range(num_nodes):
            for b in range(num_nodes):
                if a != b:
                    chunk(rank(a, owner), Buffer.input, owner).copy(rank(b, owner), 'across', a)
    for owner in range(g):
        for b in range(num_nodes):
            acc = chunk(rank(b, owner), Buffer.input, owner)
            for a in range(num_nodes):
                if a != b:
                    acc.reduce(chunk(rank(b, owner), 'across', a))
    for node in range(num_nodes):                       # broadcast inside each machine
        for owner in range(g):
            for dst in range(g):
                if dst != owner:
                    chunk(rank(node, owner), Buffer.input, owner).copy(rank(node, dst), Buffer.input, owner)


# ------------------------------------------------------------------ four GPUs in two NVLink pairs
def allreduce_two_pairs():
    """In-place all-reduce on 4 GPUs with ``chunk_factor = 2``, for boxes where GPUs (0,1) and (2,3) share a
    fast link: chunk c is reduced inside each pair onto the GPU of parity c, the two partial sums are
    exchanged and added across the pairs, and the result is copied back inside the pairs."""
    size = 4
    for c in range(2):
        owners = [r for r in range(size) if r % 2 == c]
        for r in owners:                                 # inside the pair
            chunk(r, Buffer.input, c).reduce(chunk(r ^ 1, Buffer.input, c))
        for r in owners:                                 # across the pairs, through scratch
            chunk(r, Buffer.input, c).copy((r + 2) % size, 'other-pair', c)
        for r in owners:
            chunk(r, Buffer.input, c).reduce(chunk(r, 'other-pair', c))
        for r in owners:                                 # back to the partner
            chunk(r, Buffer.input, c).copy(r ^ 1, Buffer.input, c)


# ------------------------------------------------------------------ reduce in one stage, deliver to the next
class StageAllReduce(Collective):
    """2 * ``size`` ranks.  The inputs of stage 0 (ranks 0 .. size-1) are summed; every rank of stage 1
    (ranks size .. 2 size - 1) must end up with the sum in its input buffer.  What stage 0 is left with is
    not constrained.  A custom collective: ``name`` stays 'custom'."""

    def __init__(self, size, chunk_factor):
        super().__init__(2 * size, chunk_factor, True)
        self.size = size

    def init_buffers(self):
        per_rank = []
        for r in range(self.num_ranks):
            data = [Chunk(r, c) for c in range(self.chunk_factor)]
            per_rank.append({Buffer.input: data, Buffer.output: data})
        return per_rank

    def check(self, prog):
        ok = True
        for c in range(self.chunk_factor):
            want = ReduceChunk(-1, [Chunk(r, c) for r in range(self.size)])
            for t in range(self.size, 2 * self.size):
                got = prog.buffers[t][Buffer.input][c]
                if got != want:
                    print(f'Rank {t} chunk {c} is incorrect: should be the sum over stage 0, given {got}')
                    ok = False
        return ok


def pipeline_allreduce_ring(size, channels=1):
    """``StageAllReduce(size, size)``: ring reduction inside stage 0 (chunk i ends on rank i - 1), hand-over
    of every finished chunk to the rank of stage 1 with the same local index, ring propagation inside
    stage 1.  ``channels`` spreads the chunks of a ring over that many channels."""
    for step in range(size - 1):
        for index in range(size):
            src, dst = (index + step) % size, (index + step + 1) % size
            chunk(dst, Buffer.input, index).reduce(chunk(src, Buffer.input, index), ch=index % channels)
    for index in range(size):
        done_on = (index - 1) % size
        chunk(done_on, Buffer.input, index).copy(done_on + size, Buffer.input, index, ch=done_on % 2)
    for step in range(size - 1):
        for index in range(size):
            src, dst = (index - 1 + step) % size, (index + step) % size
            chunk(src + size, Buffer.input, index).copy(dst + size, Buffer.input, index, ch=index % channels)


def pipeline_allreduce_allpairs(size):
    """``StageAllReduce(size, size)``: all-pairs scatter and local reduction inside stage 0 (rank r owns
    chunk r), hand-over of the owned chunk to rank r of stage 1, all-pairs broadcast inside stage 1."""
    for src in range(size):
        for owner in range(size):
            if src != owner:
                chunk(src, Buffer.input, owner).copy(owner, 'gathered', src)
    for owner in range(size):
        acc = chunk(owner, Buffer.input, owner)
        for src in range(size):
            if src != owner:
                acc.reduce(chunk(owner, 'gathered', src))
        acc.copy(owner + size, Buffer.input, owner, ch=owner % 2)
    for owner in range(size):
        for dst in range(size):
            if dst != owner:
                chunk(owner + size, Buffer.input, owner).copy(dst + size, Buffer.input, owner)


# ------------------------------------------------------------------ rows x columns
def allreduce_2d(rows, cols):
    """In-place all-reduce with ``chunk_factor = rows * cols`` on GPUs arranged in ``cols`` columns of ``rows``
    GPUs (GPU id = column * rows + row), columns being the fast direction (NVLink) and rows the slow one (PCIe
    or network): reduce-scatter inside the columns, reduce-scatter of the column results along the rows (only
    1 / rows of the data crosses the slow links), all-gather along the rows, all-gather inside the columns.
    Chunk ``i * cols + j`` is owned by row i after the first phase and by GPU (row i, column j) after the second.
    (The reference's ``examples/mscclang/allreduce_a100_pcie_hierarchical.py`` fails its own ``Check()``.)"""
    def gpu(row, col):
        return col * rows + row

    for col in range(cols):                               # 1. reduce-scatter inside every column
        for owner_row in range(rows):
            for src_row in range(rows):
                if src_row != owner_row:
                    for j in range(cols):
                        idx = owner_row * cols + j
                        chunk(gpu(owner_row, col), Buffer.input, idx).reduce(chunk(gpu(src_row, col), Buffer.input, idx))
    for row in range(rows):                               # 2. reduce-scatter along every row
        for j in range(cols):
            idx = row * cols + j
            for src_col in range(cols):
                if src_col != j:
                    chunk(gpu(row, j), Buffer.input, idx).reduce(chunk(gpu(row, src_col), Buffer.input, idx))
    for row in range(rows):                               # 3. all-gather along every row
        for j in range(cols):
            idx = row * cols + j
            for dst_col in range(cols):
                if dst_col != j:
                    chunk(gpu(row, j), Buffer.input, idx).copy(gpu(row, dst_col), Buffer.input, idx)
    for col in range(cols):                               # 4. all-gather inside every column
        for row in range(rows):
            for dst_row in range(rows):
                if dst_row != row:
                    chunk(gpu(row, col), Buffer.input, row * cols, cols).copy(gpu(dst_row, col), Buffer.input, row * cols)


def allgather_two_pairs():
    """All-gather (``chunk_factor = 1``, not in place) on 4 GPUs made of two NVLink pairs: every GPU gives its
    chunk to its partner and to one GPU of the other pair, which passes it on to its own partner, so each
    chunk crosses the slow link between the pairs once."""
    size = 4
    for r in range(size):
        mine = chunk(r, Buffer.input, 0)
        mine.copy(r, Buffer.output, r)
        mine.copy(r ^ 1, Buffer.output, r)
        across = mine.copy((r + 2) % size, Buffer.output, r)
        across.copy(((r + 2) % size) ^ 1, Buffer.output, r)


# ------------------------------------------------------------------ reduce inside groups, gather everywhere
class ReduceGather(Collective):
    """``groups`` groups of ``gpus_per_group`` GPUs; every GPU has ``gpus_per_group`` input chunks.  Output chunk
    ``q * gpus_per_group + j`` of every GPU = sum over the GPUs of group q of their input chunk j.
    A custom collective (``name`` stays 'custom').  (The reference's ``examples/mscclang/reducegather.py``
    defines the same idea but no longer runs against its own API.)"""

    def __init__(self, groups, gpus_per_group):
        super().__init__(groups * gpus_per_group, 1, False)
        self.groups, self.gpus_per_group = groups, gpus_per_group

    def init_buffers(self):
        return [{Buffer.input: [Chunk(r, j) for j in range(self.gpus_per_group)], Buffer.output: [None] * self.num_ranks}
                for r in range(self.num_ranks)]

    def expected(self, index):
        q, j = divmod(index, self.gpus_per_group)
        return ReduceChunk(-1, [Chunk(q * self.gpus_per_group + m, j) for m in range(self.gpus_per_group)])

    def check(self, prog):
        ok = True
        for r in range(self.num_ranks):
            for index in range(self.num_ranks):
                got = prog.buffers[r][Buffer.output][index]
                if got != self.expected(index):
                    print(f'Rank {r} output chunk {index} is incorrect: given {got}')
                    ok = False
        return ok


def reduce_gather(groups, gpus_per_group):
    """``ReduceGather(groups, gpus_per_group)``: all-pairs reduce-scatter inside every group (member j sums
    input chunk j of its group into its output slot), then every result is copied to every other GPU."""
    g = gpus_per_group
    for q in range(groups):
        for j in range(g):
            owner = q * g + j
            slot = q * g + j
            acc = chunk(owner, Buffer.input, j).copy(owner, Buffer.output, slot)
            for m in range(g):
                if m != j:
                    acc.reduce(chunk(q * g + m, Buffer.input, j))
    for owner in range(groups * g):
        for dst in range(groups * g):
            if dst != owner:
                chunk(owner, Buffer.output, owner).copy(dst, Buffer.output, owner)


# ------------------------------------------------------------------ DGX-1 machines, one chunk
DGX1_PATH = (1, 3, 2, 6, 7, 5, 4, 0)      # a path through all 8 GPUs of a DGX-1 that only uses NVLink


def allreduce_dgx1_chain(num_nodes=2):
    """Latency-oriented in-place all-reduce of one chunk over ``num_nodes`` DGX-1 machines (topology
    ``distributed_fully_connected(dgx1(), num_nodes, 1)``): the chunk is summed along an NVLink path through
    each machine, the machines' sums are exchanged between the GPUs at the end of the paths and added, and the
    result travels back along the paths.  (Same idea as the reference's ``examples/mscclang/allreduce_dgx1.py``,
    which is written against an API the reference no longer has.)"""
    def rank(node, step):
        return DGX1_PATH[step] + 8 * node

    last = len(DGX1_PATH) - 1
    for node in range(num_nodes):                         # sum along the path
        for step in range(1, last + 1):
            chunk(rank(node, step), Buffer.input, 0).reduce(chunk(rank(node, step - 1), Buffer.input, 0))
    for a in range(num_nodes):                            # path ends exchange their sums
        for b in range(num_nodes):
            if a != b:
                chunk(rank(a, last), Buffer.input, 0).copy(rank(b, last), 'machines', a)
    for b in range(num_nodes):
        for a in range(num_nodes):
            if a != b:
                chunk(rank(b, last), Buffer.input, 0).reduce(chunk(rank(b, last), 'machines', a))
    for node in range(num_nodes):                         # and back
        for step in range(last - 1, -1, -1):
            chunk(rank(node, step + 1), Buffer.input, 0).copy(rank(node, step), Buffer.input, 0)
