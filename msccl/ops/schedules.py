"""The communication schedules of the fused kernels, written as MSCCLang programs.

The fused kernels (``csrc/fused_tp.cu``, ``csrc/moe_a2a.cu``) are hand-written, but what they move and in
which order is an ordinary MSCCL program: one chunk per 128-row block, copied (all-gather, dispatch) or
reduced (reduce-scatter, combine) between ranks.  The functions here state those programs in the DSL so that
the schedule can be checked (``Check()``), validated and executed by the CPU interpreter, and compared with
alternatives through the executor; the kernels implement the same chunk order with the GEMM tiles in
between:

* all-gather -> GEMM: rank r pushes its blocks to every peer, block by block; a GEMM tile of row block b
  waits for chunk b only (``all_gather_blocks``);
* GEMM -> reduce-scatter: partial tiles go to their owner in owner-major order starting at rank + 1, so that at
  any moment every rank sends to a different owner (``reduce_scatter_blocks``);
* MoE: dispatch and combine are all-to-alls with one chunk per (source, destination) pair (``dispatch_blocks``;
  the kernels send a variable number of rows inside each chunk).
"""
from msccl.language import Buffer, MSCCLProgram, chunk
from msccl.language.collectives import AllGather, AllToAll, ReduceScatter
from msccl.topologies import fully_connected


def all_gather_blocks(ranks, blocks_per_rank):
    """MSCCL-IR of the all-gather inside all-gather -> GEMM: chunk = one 128-row block."""
    prog = MSCCLProgram(f'ag_gemm_schedule_{ranks}x{blocks_per_rank}', fully_connected(ranks),
                        AllGather(ranks, blocks_per_rank, False), 1)
    with prog:
        for block in range(blocks_per_rank):                 # block-major: early blocks unblock GEMM tiles first
            for src in range(ranks):
                mine = chunk(src, Buffer.input, block)
                mine.copy(src, Buffer.output, src * blocks_per_rank + block)
                for step in range(1, ranks):
                    mine.copy((src + step) % ranks, Buffer.output, src * blocks_per_rank + block, ch=block % 2)
        assert prog.check()
    return prog


def reduce_scatter_blocks(ranks, blocks_per_rank):
    """MSCCL-IR of the reduce-scatter inside GEMM -> reduce-scatter: every rank's partial block goes to the
    block's owner, owners visited in the order rank + 1, rank + 2, ...; the owner adds the n partials."""
    prog = MSCCLProgram(f'gemm_rs_schedule_{ranks}x{blocks_per_rank}', fully_connected(ranks),
                        ReduceScatter(ranks, blocks_per_rank, False), 1)
    with prog:
        for src in range(ranks):
            for step in range(1, ranks):
                owner = (src + step) % ranks
                for block in range(blocks_per_rank):
                    chunk(src, Buffer.input, owner * blocks_per_rank + block).copy(owner, ('partial', src), block, ch=block % 2)
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
