#!/usr/bin/env python
"""NCCL baseline on the same box: busBW of all_reduce / all_gather / reduce_scatter / all_to_all
through torch.distributed, device-timed (CUDA events), max over ranks, nccl-tests conventions
(busBW = algBW * 2(n-1)/n for all-reduce, * (n-1)/n for the others).

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 baseline/nccl_bench.py --out nccl.json
"""
import argparse
import json
import os

import torch
import torch.distributed as dist


def timed(fn, iters, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device='cuda', dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--min-log2', type=int, default=10)
    ap.add_argument('--max-log2', type=int, default=30)
    ap.add_argument('--step-log2', type=int, default=1)
    ap.add_argument('--collectives', default='allreduce,allgather,reduce_scatter,alltoall')
    ap.add_argument('--dtype', default='bf16')
    ap.add_argument('--out', default=None)
    args = ap.parse_args()
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    rank, n = dist.get_rank(), dist.get_world_size()
    dtype = {'bf16': torch.bfloat16, 'fp16': torch.float16, 'fp32': torch.float32}[args.dtype]
    esize = torch.empty((), dtype=dtype).element_size()
    rows = []
    for coll in args.collectives.split(','):
        for lg in range(args.min_log2, args.max_log2 + 1, args.step_log2):
            nbytes = 1 << lg          # all-reduce: buffer size; others: total (gathered / scattered) size per rank
            numel = nbytes // esize
            if numel % n:
                continue
            iters = 100 if nbytes <= (1 << 20) else (20 if nbytes <= (1 << 26) else 8)
            if coll == 'allreduce':
                x = torch.zeros(numel, device='cuda', dtype=dtype)
                fn, factor = (lambda: dist.all_reduce(x)), 2 * (n - 1) / n
            elif coll == 'allgather':
                x = torch.zeros(numel // n, device='cuda', dtype=dtype)
                y = torch.zeros(numel, device='cuda', dtype=dtype)
                fn, factor = (lambda: dist.all_gather_into_tensor(y, x)), (n - 1) / n
            elif coll == 'reduce_scatter':
                x = torch.zeros(numel, device='cuda', dtype=dtype)
                y = torch.zeros(numel // n, device='cuda', dtype=dtype)
                fn, factor = (lambda: dist.reduce_scatter_tensor(y, x)), (n - 1) / n
            else:
                x = torch.zeros(numel, device='cuda', dtype=dtype)
                y = torch.zeros(numel, device='cuda', dtype=dtype)
                fn, factor = (lambda: dist.all_to_all_single(y, x)), (n - 1) / n
            ms = timed(fn, iters)
            rows.append({'collective': coll, 'algo': 'nccl', 'nranks': n, 'bytes': nbytes, 'time_us': round(ms * 1e3, 2),
                         'algbw_gbs': round(nbytes / ms / 1e6, 3), 'busbw_gbs': round(nbytes * factor / ms / 1e6, 3)})
            if rank == 0:
                print(rows[-1], flush=True)
    if rank == 0 and args.out:
        with open(args.out, 'w') as f:
            json.dump({'nccl': '.'.join(map(str, torch.cuda.nccl.version())), 'dtype': args.dtype, 'rows': rows}, f, indent=1)
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
