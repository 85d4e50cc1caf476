"""Run one MSCCLang all-reduce program with all ranks emulated on one GPU (a small, self-contained
target for timing and for profilers).

    python -m msccl.runtime.bench_emulated --ranks 8 --mbytes 64 --iters 3 --algo ring
    python -m msccl.runtime.bench_emulated --direct twoshot --mbytes 256 --iters 3

``--direct`` runs one of the direct (non-interpreted) kernels in its one-rank form on a one-process communicator:
the cross-rank barrier has a single participant and every "peer" is the GPU itself, so the loop that moves the data
runs alone - the form a profiler can replay.
"""
import argparse
import json

import torch

from msccl.language import MSCCLProgram, ThreadblockPolicy
from msccl.language.collectives import AllReduce
from msccl.programs.allreduce import allreduce_ring, allreduce_two_shot
from msccl.runtime import Communicator, Executor
from msccl.topologies import fully_connected
from msccl.xml import load_xml


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--ranks', type=int, default=8)
    ap.add_argument('--mbytes', type=int, default=64, help='message size per rank (MiB)')
    ap.add_argument('--iters', type=int, default=5)
    ap.add_argument('--algo', default='ring', choices=['ring', 'two_shot'])
    ap.add_argument('--instances', type=int, default=4)
    ap.add_argument('--protocol', default='Simple', choices=['Simple', 'LL', 'LL128'])
    ap.add_argument('--direct', default=None, choices=['twoshot', 'oneshot', 'push'],
                    help='time a direct kernel in its one-rank form instead of an interpreted program')
    args = ap.parse_args()
    if args.direct:
        return direct(args)
    n = args.ranks
    prog = MSCCLProgram(args.algo, fully_connected(n), AllReduce(n, n, True), args.instances, protocol=args.protocol,
                        threadblock_policy=ThreadblockPolicy.manual)
    with prog:
        if args.algo == 'ring':
            allreduce_ring(n, 4)
        else:
            allreduce_two_shot(n)
    comm = Communicator.emulated(n, fifo_bytes=128 << 20)
    ex = Executor(comm)
    plan = ex.compile(load_xml(prog.generate_xml()))
    numel = (args.mbytes << 20) // 2
    bufs = {r: torch.randn(numel, device='cuda').bfloat16() for r in range(n)}
    ex.run(plan, bufs)
    ex.check()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.iters):
        ex.run(plan, bufs)
    stop.record()
    ex.check()
    ms = start.elapsed_time(stop) / args.iters
    nbytes = numel * 2
    print(json.dumps({'algo': args.algo, 'ranks': n, 'bytes_per_rank': nbytes, 'threadblocks': plan.grid, 'us': round(ms * 1e3, 1),
                      'emulated_busbw_gbs': round(nbytes * 2 * (n - 1) / n / ms / 1e6, 1)}))
    comm.close()


def direct(args):
    import os
    import torch.distributed as dist
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29579')
    torch.cuda.set_device(0)
    dist.init_process_group('nccl', rank=0, world_size=1, device_id=torch.device('cuda', 0))
    nbytes = args.mbytes << 20
    comm = Communicator.from_process_group(arena_bytes=2 * nbytes + (8 << 20), fifo_bytes=16 << 20)
    nat = comm.native
    sym, offset = comm.symmetric_empty(nbytes // 2, torch.bfloat16)
    out, out_offset = comm.symmetric_empty(nbytes // 2, torch.bfloat16)
    src = torch.randn(nbytes // 2, device='cuda').bfloat16()
    sym.copy_(src)
    stream = torch.cuda.current_stream().cuda_stream
    if args.direct == 'twoshot':
        fn = lambda: nat.twoshot_allreduce(comm.dev_heap_bases, 0, offset, nbytes, 1, 0, 1, comm.dev_syncs,       # noqa: E731
                                           comm.timeout_ns, 64, stream)
    elif args.direct == 'push':
        fn = lambda: nat.push_blocks(src.data_ptr(), True, comm.dev_heap_bases, 0, out_offset, nbytes, 0, 1,      # noqa: E731
                                     comm.dev_syncs, comm.timeout_ns, 64, stream)
    else:
        small = min(nbytes, comm.ll_max_bytes)
        nbytes = small
        fn = lambda: nat.oneshot(src.data_ptr(), out.data_ptr(), comm.dev_staging, small, comm.ll_slot_bytes, 1, 0, 1,   # noqa: E731
                                 comm.sync_ptr(0), comm.timeout_ns, 32, 0, stream)
    fn()
    comm.check()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.iters):
        fn()
    stop.record()
    comm.check()
    ms = start.elapsed_time(stop) / args.iters
    print(json.dumps({'kernel': args.direct, 'ranks': 1, 'bytes': nbytes, 'us': round(ms * 1e3, 1),
                      'gbs_read_plus_written': round(2 * nbytes / ms / 1e6, 1)}))
    comm.close()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
