"""Time the fused compute + collective kernels one by one (and give profilers a small target).

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 -m msccl.ops.bench_fused --tokens 8192
    python -m msccl.ops.bench_fused --tokens 4096 --only ag_gemm --iters 1     # one rank: every block is local

Prints one JSON line: per kernel the CUDA-event time (max over ranks), the tensor throughput and the fraction of the
roofline - the slower of the FLOPs at the measured cuBLAS bf16 peak and the bytes that must cross NVLink at the
measured 770 GB/s per direction (both overridable).  With one rank nothing crosses NVLink: the kernels then run their
degenerate single-GPU form (all blocks local, the reducers add one slab), which is what a profiler can replay.
"""
import argparse
import json
import os

import torch

KERNELS = ('ag_gemm', 'gemm_rs', 'ag_gemm_mxfp8', 'gemm_rs_mxfp8', 'moe')


def main(argv=None):
    import torch.distributed as dist
    from msccl.ops import check_gemm_errors
    from msccl.ops.fused_tp import FusedTensorParallel
    from msccl.ops.gemm import interleave_gate_up, pack_mx_scales, quantize_mxfp8
    from msccl.runtime import Communicator
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument('--tokens', type=int, default=8192)
    ap.add_argument('--hidden', type=int, default=4096)
    ap.add_argument('--ffn', type=int, default=14336, help='full FFN width (sharded over the ranks)')
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--only', default='', help='comma-separated subset of ' + ', '.join(KERNELS))
    ap.add_argument('--peak-tflops', type=float, default=1695.0, help='bf16 GEMM peak the roofline uses (fp8: twice that)')
    ap.add_argument('--link-gbs', type=float, default=770.0, help='NVLink bandwidth per direction per GPU')
    args = ap.parse_args(argv)
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    if 'RANK' not in os.environ:
        os.environ.update(RANK='0', WORLD_SIZE='1', MASTER_ADDR='127.0.0.1', MASTER_PORT=os.environ.get('MASTER_PORT', '29577'))
    dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    rank, n = dist.get_rank(), dist.get_world_size()
    only = set(filter(None, args.only.split(','))) or set(KERNELS)
    comm = Communicator.from_process_group(fifo_bytes=16 << 20, arena_bytes=2 << 30)
    rows, shard = args.tokens // n, args.ffn // n
    hidden = args.hidden
    tp = FusedTensorParallel(comm, rows, hidden)
    gen = torch.Generator(device='cuda').manual_seed(5 + rank)
    x = torch.randn(rows, hidden, device='cuda', generator=gen).bfloat16()
    wg = (torch.randn(shard, hidden, device='cuda', generator=gen) * 0.02).bfloat16()
    wu = (torch.randn(shard, hidden, device='cuda', generator=gen) * 0.02).bfloat16()
    wd = (torch.randn(hidden, shard, device='cuda', generator=gen) * 0.02).bfloat16()
    h = torch.empty(args.tokens, shard, device='cuda', dtype=torch.bfloat16)
    y = torch.empty(rows, hidden, device='cuda', dtype=torch.bfloat16)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / args.iters], device='cuda', dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def entry(ms, flops, link_bytes, peak):
        ideal_ms = max(flops / (peak * 1e12), link_bytes / (args.link_gbs * 1e9)) * 1e3
        return {'us': round(ms * 1e3, 1), 'tflops': round(flops / ms / 1e9, 1), 'roofline_us': round(ideal_ms * 1e3, 1),
                'fraction_of_roofline': round(ideal_ms / ms, 3), 'bound': 'compute' if flops / (peak * 1e12) >= link_bytes / (args.link_gbs * 1e9) else 'nvlink'}

    out = {'n_gpus': n, 'tokens': args.tokens, 'hidden': hidden, 'ffn': args.ffn, 'multicast': bool(comm.mc_base)}
    flops_up = 2.0 * args.tokens * hidden * 2 * shard
    flops_down = 2.0 * args.tokens * shard * hidden
    gathered_in = (n - 1) * rows * hidden             # elements every rank receives in the all-gather
    scattered_out = (n - 1) * rows * hidden           # elements every rank sends in the reduce-scatter
    if 'ag_gemm' in only:
        wgu = interleave_gate_up(wg, wu)
        out['ag_gemm_swiglu'] = entry(timed(lambda: tp.all_gather_gemm(x, wgu, epilogue='swiglu', out=h)), flops_up, gathered_in * 2,
                                      args.peak_tflops)
    if 'gemm_rs' in only:
        out['gemm_rs'] = entry(timed(lambda: tp.gemm_reduce_scatter(h, wd, out=y)), flops_down, scattered_out * 2, args.peak_tflops)
    if 'ag_gemm_mxfp8' in only or 'gemm_rs_mxfp8' in only:
        pack = lambda s: pack_mx_scales(s, row_multiple=128)                                     # noqa: E731
        guq, gus = quantize_mxfp8(interleave_gate_up(wg, wu, tile=tp.mx_gate_up_tile).float())
        wdq, wds = quantize_mxfp8(wd.float())
        xq, xs = quantize_mxfp8(x.float())
        gus_p, wds_p, xs_p = pack(gus), pack(wds), pack(xs)
        if 'ag_gemm_mxfp8' in only:
            ms = timed(lambda: tp.all_gather_gemm_mxfp8(xq, xs_p, guq, gus_p, epilogue='swiglu', out=h))
            out['ag_gemm_swiglu_mxfp8'] = entry(ms, flops_up, gathered_in * (1 + 1 / 32), 2 * args.peak_tflops)
        if 'gemm_rs_mxfp8' in only:
            hq, hs = quantize_mxfp8(torch.randn(args.tokens, shard, device='cuda', generator=gen))
            hs_p = pack(hs)
            ms = timed(lambda: tp.gemm_reduce_scatter_mxfp8(hq, hs_p, wdq, wds_p, out=y))
            out['gemm_rs_mxfp8'] = entry(ms, flops_down, scattered_out * 2, 2 * args.peak_tflops)
    check_gemm_errors()
    if 'moe' in only:
        from msccl.parallel.expert_parallel import ExpertParallelMoE
        tokens, ffn_moe, per_gpu, topk = min(args.tokens, 4096), args.ffn, 8, 2
        layer = ExpertParallelMoE(comm, tokens, hidden, ffn_moe, per_gpu * n, topk)
        xm = torch.randn(tokens, hidden, device='cuda', generator=gen).bfloat16()
        logits = torch.randn(tokens, per_gpu * n, device='cuda', generator=gen)
        ym = torch.empty_like(xm)
        ms = timed(lambda: layer(xm, gate_logits=logits, out=ym))
        check_gemm_errors()
        flops = 2.0 * tokens * topk * 3 * hidden * ffn_moe
        crossing = 2.0 * tokens * topk * hidden * 2 * (n - 1) / n          # dispatch and combine, bf16
        out['moe_layer'] = dict(entry(ms, flops, crossing, args.peak_tflops), tokens_per_gpu=tokens, experts=per_gpu * n, topk=topk)
    if rank == 0:
        print('FUSED_BENCH ' + json.dumps(out), flush=True)
    comm.close()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
