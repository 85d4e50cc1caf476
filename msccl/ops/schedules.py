"""The communication schedules of the fused kernels, written as MSCCLang programs, and their lowering into the
order tables the kernels take as arguments.

What the fused kernels (``csrc/fused_tp.cu``, ``csrc/moe_a2a.cu``) move, and in which order, is an ordinary MSCCL
program: one chunk per 128-row block, copied (all-gather, dispatch) or reduced (reduce-scatter, combine) between
ranks.  The functions here state those programs in the DSL, so that a schedule can be checked (``Check()``),
validated and executed by the CPU interpreter, and then lower the compiled MSCCL-IR into the row-block order of the
GEMM tiles (``lower_all_gather``, ``lower_reduce_scatter``): the kernels read that table, so another program gives
another tile order without touching the CUDA code.

* all-gather -> GEMM: rank r pushes its blocks to every peer, block by block; a GEMM tile of row block b
  waits for chunk b only (``all_gather_blocks``);
* GEMM -> reduce-scatter: block-major - every rank produces block 0 for each owner, then block 1, ... - so that
  an owner can add up block b while the later blocks are still being computed (``reduce_scatter_blocks``);
* MoE: dispatch and combine are all-to-alls with one chunk per (source, destination) pair (``dispatch_blocks``;
  the kernels send a variable number of rows inside each chunk).

Lowering rule: the threadblocks of a GPU run side by side, each its steps in order, so the transfers of a GPU are
listed in rounds - round k takes the k-th transfer of every threadblock, threadblocks in id order.
"""
import functools

from msccl.language import Buffer, MSCCLProgram, chunk
from msccl.language.collectives import AllGather, AllToAll, ReduceScatter
from msccl.topologies import fully_connected


def all_gather_blocks(ranks, blocks_per_rank, channels=2):
    """MSCCL-IR of the all-gather inside all-gather -> GEMM: chunk = one 128-row block, block b on channel
    ``b % channels``."""
    prog = MSCCLProgram(f'ag_gemm_schedule_{ranks}x{blocks_per_rank}', fully_connected(ranks),
                        AllGather(ranks, blocks_per_rank, False), 1)
    with prog:
        for block in range(blocks_per_rank):                 # block-major: early blocks unblock GEMM tiles first
            for src in range(ranks):
                mine = chunk(src, Buffer.input, block)
                mine.copy(src, Buffer.output, src * blocks_per_rank + block)
                for step in range(1, ranks):
                    mine.copy((src + step) % ranks, Buffer.output, src * blocks_per_rank + block, ch=block % channels)
        assert prog.check()
    return prog


def reduce_scatter_blocks(ranks, blocks_per_rank, channels=1):
    """MSCCL-IR of the reduce-scatter inside GEMM -> reduce-scatter: every rank's partial block goes to the
    block's owner; the owner adds the n partials.  Block b travels on channel ``b % channels``: with one channel
    there is one connection per owner and the rounds of the lowering are the blocks (block 0 of every owner, then
    block 1, ...); with more channels a round holds ``channels`` blocks of every owner."""
    prog = MSCCLProgram(f'gemm_rs_schedule_{ranks}x{blocks_per_rank}c{channels}', fully_connected(ranks),
                        ReduceScatter(ranks, blocks_per_rank, False), 1)
    with prog:
        for block in range(blocks_per_rank):
            for src in range(ranks):
                for step in range(1, ranks):
                    owner = (src + step) % ranks
                    chunk(src, Buffer.input, owner * blocks_per_rank + block).copy(owner, ('partial', src), block,
                                                                                  ch=block % channels)
        for owner in range(ranks):
            for block in range(blocks_per_rank):
                acc = chunk(owner, Buffer.input, owner * blocks_per_rank + block).copy(owner, Buffer.output, block)
                for src in range(ranks):
                    if src != owner:
                        acc.reduce(chunk(owner, ('partial', src), block))
        assert prog.check()
    return prog


def dispatch_blocks(ranks):
    """MSCCL-IR of the MoE token exchange (dispatch; combine is the same program run in the other direction):
    chunk (src, dst) holds the rows source ``src`` routes to the experts of rank ``dst``."""
    prog = MSCCLProgram(f'moe_dispatch_schedule_{ranks}', fully_connected(ranks), AllToAll(ranks, 1, False), 1)
    with prog:
        for src in range(ranks):
            for step in range(ranks):
                dst = (src + step) % ranks
                chunk(src, Buffer.input, dst).copy(dst, Buffer.output, src)
        assert prog.check()
    return prog


# ---------------------------------------------------------------------------------- lowering into order tables
def _rounds(gpu, pick):
    """Transfers of one GPU in rounds: ``pick(step)`` returns the items a step contributes (or nothing)."""
    lanes = []
    for tb in gpu.tbs:
        lane = []
        for st in tb.steps:
            lane.extend(pick(st) or ())
        if lane:
            lanes.append(lane)
    out = []
    for k in range(max((len(lane) for lane in lanes), default=0)):
        for lane in lanes:
            if k < len(lane):
                out.append(lane[k])
    return out


def _produce_order(algo, rank):
    """The (owner, block) row blocks in the order ``rank`` produces them: its sends out of the input buffer, in
    rounds; the rank's own block b (a local copy in the program: nothing to send) follows the last remote
    transfer of block index b."""
    gpu = algo.gpus[rank]
    per_rank = gpu.o_chunks

    def sends(st):
        if st.type == 's' and st.srcbuf == 'i':
            return [((st.srcoff + j) // per_rank, (st.srcoff + j) % per_rank) for j in range(st.cnt)]

    order = [item for item in _rounds(gpu, sends) if item[0] != rank]
    for block in range(per_rank):
        last = max((i for i, (_, b) in enumerate(order) if b == block), default=len(order) - 1)
        order.insert(last + 1, (rank, block))
    assert sorted(order) == [(o, b) for o in range(algo.ngpus) for b in range(per_rank)], 'not a reduce-scatter schedule'
    return order


def lower_reduce_scatter(algo, rank):
    """``(order, reduce_order)`` for ``rank`` from the MSCCL-IR of a ``reduce_scatter_blocks``-shaped program.

    ``order``: the (owner, block) row blocks in the order this rank's GEMM tiles produce them.  ``reduce_order``:
    this rank's own blocks in the order they become complete, i.e. sorted by the latest position at which any
    rank produces its contribution to the block."""
    order = _produce_order(algo, rank)
    per_rank = algo.gpus[rank].o_chunks
    complete = {b: 0 for b in range(per_rank)}
    for src in range(algo.ngpus):
        theirs = order if src == rank else _produce_order(algo, src)
        for position, (owner, block) in enumerate(theirs):
            if owner == rank:
                complete[block] = max(complete[block], position)
    reduce_order = sorted(range(per_rank), key=lambda b: (complete[b], b))
    return order, reduce_order


def lower_all_gather(algo, rank):
    """The (source, block) row blocks in the order the GEMM tiles of ``rank`` consume them, from the MSCCL-IR of an
    ``all_gather_blocks``-shaped program: the rank's own blocks first (they need no transfer), then the received
    blocks in rounds."""
    gpu = algo.gpus[rank]
    per_rank = gpu.i_chunks

    def receives(st):
        if st.type in ('r', 'rcs') and st.dstbuf == 'o':
            return [((st.dstoff + j) // per_rank, (st.dstoff + j) % per_rank) for j in range(st.cnt)]

    order = [(rank, b) for b in range(per_rank)] + [item for item in _rounds(gpu, receives) if item[0] != rank]
    assert sorted(order) == [(s, b) for s in range(algo.ngpus) for b in range(per_rank)], 'not an all-gather schedule'
    return order


@functools.lru_cache(maxsize=None)
def fused_tp_tables(ranks, blocks_per_rank, rank, ag_channels=1, rs_channels=1):
    """Order tables of the two fused tensor-parallel kernels for ``rank``: ``(all-gather order, reduce-scatter
    order, reduce order)``, each a flat list of ints ready to upload."""
    from msccl.xml import load_xml
    if ranks == 1:                       # nothing moves: the blocks in sequence
        own = [v for b in range(blocks_per_rank) for v in (0, b)]
        return own, list(own), list(range(blocks_per_rank))
    ag = lower_all_gather(load_xml(all_gather_blocks(ranks, blocks_per_rank, ag_channels).generate_xml()), rank)
    rs, red = lower_reduce_scatter(load_xml(reduce_scatter_blocks(ranks, blocks_per_rank, rs_channels).generate_xml()), rank)
    flat = lambda pairs: [v for pair in pairs for v in pair]      # noqa: E731
    return flat(ag), flat(rs), list(red)
