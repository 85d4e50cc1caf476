"""Run one MSCCLang all-reduce program with all ranks emulated on one GPU (a small, self-contained
target for timing and for profilers).

    python -m msccl.runtime.bench_emulated --ranks 8 --mbytes 64 --iters 3 --algo ring
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
    ap.add_argument('--protocol', default='Simple', choices=['Simple', 'LL'])
    args = ap.parse_args()
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


if __name__ == '__main__':
    main()
