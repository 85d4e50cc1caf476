"""Multi-process worker for the fused tensor-parallel kernels (run under torchrun).

Numerics: compared with a plain PyTorch fp32 reference of the same operation (all-gather, matmul,
SwiGLU; matmul, reduce-scatter).  With ``--bench`` also times the Llama-3-8B MLP shapes against the
NCCL + cuBLAS pipeline on the same GPUs.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from msccl.ops import check_gemm_errors  # noqa: E402
from msccl.ops.fused_tp import FusedTensorParallel  # noqa: E402
from msccl.ops.gemm import interleave_gate_up  # noqa: E402
from msccl.runtime import Communicator  # noqa: E402


def timed(fn, iters, warmup=3):
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


def check(comm, rank, n, rows, hidden, ffn_shard, calls=3):
    tp = FusedTensorParallel(comm, rows, hidden, comm_ctas=4)
    gen = torch.Generator(device='cuda').manual_seed(100 + rank)
    wg = (torch.randn(ffn_shard, hidden, device='cuda', generator=gen) * 0.05).bfloat16()
    wu = (torch.randn(ffn_shard, hidden, device='cuda', generator=gen) * 0.05).bfloat16()
    wd = (torch.randn(hidden, ffn_shard, device='cuda', generator=gen) * 0.05).bfloat16()
    wgu = interleave_gate_up(wg, wu)
    for call in range(calls):
        x = torch.randn(rows, hidden, device='cuda', generator=gen).bfloat16()
        full = torch.empty(n * rows, hidden, device='cuda', dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, x)
        # all-gather -> GEMM, plain and SwiGLU
        plain = tp.all_gather_gemm(x, wg)
        h = tp.all_gather_gemm(x, wgu, epilogue='swiglu')
        check_gemm_errors()
        want_plain = full.float() @ wg.float().t()
        want_h = torch.nn.functional.silu(want_plain) * (full.float() @ wu.float().t())
        for got, want, name in ((plain, want_plain, 'ag_gemm'), (h, want_h, 'ag_gemm_swiglu')):
            err = (got.float() - want).abs().max().item()
            assert err <= 2e-2 * want.abs().max().item() + 1e-3, (name, call, err)
        # GEMM -> reduce-scatter
        y = tp.gemm_reduce_scatter(h, wd)
        check_gemm_errors()
        partial = (h.float() @ wd.float().t())
        dist.all_reduce(partial)
        want_y = partial[rank * rows:(rank + 1) * rows]
        err = (y.float() - want_y).abs().max().item()
        assert err <= 3e-2 * want_y.abs().max().item() + 1e-3, ('gemm_rs', call, err)
    dist.barrier()
    assert tp.pair and tp.mx_gate_up_tile == 256, 'CTA pairs are the default when the row blocks pair up'
    check_mxfp8(tp, comm, rank, n, rows, hidden, ffn_shard, gen)
    tp.pair = False                                         # the single-CTA block-scaled kernels
    check_mxfp8(tp, comm, rank, n, rows, hidden, ffn_shard, gen)
    tp.pair = True


def check_mxfp8(tp, comm, rank, n, rows, hidden, ffn_shard, gen):
    """The block-scaled fp8 variants against the fp32 product of the dequantised operands."""
    from msccl.ops.gemm import dequantize_mxfp8, pack_mx_scales, quantize_mxfp8
    wg = torch.randn(ffn_shard, hidden, device='cuda', generator=gen) * 0.05
    wu = torch.randn(ffn_shard, hidden, device='cuda', generator=gen) * 0.05
    wd = torch.randn(hidden, ffn_shard, device='cuda', generator=gen) * 0.05
    wgq, wgs = quantize_mxfp8(wg)
    wuq, wus = quantize_mxfp8(wu)
    wdq, wds = quantize_mxfp8(wd)
    # gate and up rows interleaved in groups of 64 (single CTAs) or 128 (CTA pairs): the scales are per row, so they
    # interleave the same way
    tile = tp.mx_gate_up_tile
    guq = interleave_gate_up(wgq.view(torch.uint8), wuq.view(torch.uint8), tile=tile).view(torch.float8_e4m3fn)
    gus = interleave_gate_up(wgs, wus, tile=tile)
    pack = lambda t: pack_mx_scales(t, row_multiple=128)                                  # noqa: E731
    for call in range(3):
        x = torch.randn(rows, hidden, device='cuda', generator=gen)
        xq, xs = quantize_mxfp8(x)
        x_deq = dequantize_mxfp8(xq, xs)
        full = torch.empty(n * rows, hidden, device='cuda')
        dist.all_gather_into_tensor(full, x_deq)
        plain = tp.all_gather_gemm_mxfp8(xq, pack(xs), wgq, pack(wgs))
        h = tp.all_gather_gemm_mxfp8(xq, pack(xs), guq, pack(gus), epilogue='swiglu')
        check_gemm_errors()
        want_plain = full @ dequantize_mxfp8(wgq, wgs).t()
        want_h = torch.nn.functional.silu(want_plain) * (full @ dequantize_mxfp8(wuq, wus).t())
        for got, want, name in ((plain, want_plain, 'ag_gemm_mxfp8'), (h, want_h, 'ag_gemm_mxfp8_swiglu')):
            err = (got.float() - want).abs().max().item()
            assert err <= 2e-2 * want.abs().max().item() + 1e-3, (name, call, err)
        hq, hs = quantize_mxfp8(h.float())
        y = tp.gemm_reduce_scatter_mxfp8(hq, pack(hs), wdq, pack(wds))
        check_gemm_errors()
        partial = dequantize_mxfp8(hq, hs) @ dequantize_mxfp8(wdq, wds).t()
        partial = partial.bfloat16().float()                    # the partial sums travel as bf16
        dist.all_reduce(partial)
        want_y = partial[rank * rows:(rank + 1) * rows]
        err = (y.float() - want_y).abs().max().item()
        assert err <= 3e-2 * want_y.abs().max().item() + 1e-3, ('gemm_rs_mxfp8', call, err)
    dist.barrier()


def bench(comm, rank, n, tokens, hidden, ffn, iters):
    rows, shard = tokens // n, ffn // n
    tp = FusedTensorParallel(comm, rows, hidden, comm_ctas=int(os.environ.get('MSCCL_COMM_CTAS', '16')))
    x = torch.randn(rows, hidden, device='cuda').bfloat16()
    wg = (torch.randn(shard, hidden, device='cuda') * 0.02).bfloat16()
    wu = (torch.randn(shard, hidden, device='cuda') * 0.02).bfloat16()
    wd = (torch.randn(hidden, shard, device='cuda') * 0.02).bfloat16()
    wgu = interleave_gate_up(wg, wu)
    wgu_plain = torch.cat([wg, wu]).contiguous()
    h = torch.empty(tokens, shard, device='cuda', dtype=torch.bfloat16)
    y = torch.empty(rows, hidden, device='cuda', dtype=torch.bfloat16)

    def fused():
        tp.all_gather_gemm(x, wgu, epilogue='swiglu', out=h)
        tp.gemm_reduce_scatter(h, wd, out=y)

    full = torch.empty(tokens, hidden, device='cuda', dtype=torch.bfloat16)
    part = torch.empty(tokens, hidden, device='cuda', dtype=torch.bfloat16)

    def pipeline():
        dist.all_gather_into_tensor(full, x)
        gu = full @ wgu_plain.t()
        hh = torch.nn.functional.silu(gu[:, :shard]) * gu[:, shard:]
        torch.matmul(hh, wd.t(), out=part)
        dist.reduce_scatter_tensor(y, part)

    t_ag = timed(lambda: tp.all_gather_gemm(x, wgu, epilogue='swiglu', out=h), iters)
    t_rs = timed(lambda: tp.gemm_reduce_scatter(h, wd, out=y), iters)
    t_fused = timed(fused, iters)
    check_gemm_errors()
    t_pipe = timed(pipeline, iters)
    t_gemm_only = timed(lambda: torch.matmul(full, wgu_plain.t()), iters)
    flops_ag = 2.0 * tokens * hidden * 2 * shard
    flops_rs = 2.0 * tokens * shard * hidden
    if rank == 0:
        print('FUSED_TP_BENCH ' + json.dumps({
            'n_gpus': n, 'tokens': tokens, 'hidden': hidden, 'ffn': ffn,
            'ag_gemm_swiglu_us': round(t_ag * 1e3, 1), 'gemm_rs_us': round(t_rs * 1e3, 1),
            'fused_mlp_us': round(t_fused * 1e3, 1), 'nccl_cublas_mlp_us': round(t_pipe * 1e3, 1),
            'cublas_up_gemm_only_us': round(t_gemm_only * 1e3, 1),
            'ag_gemm_tflops': round(flops_ag / t_ag / 1e9, 1), 'gemm_rs_tflops': round(flops_rs / t_rs / 1e9, 1),
            'fused_tokens_per_s': round(tokens / (t_fused * 1e-3)), 'pipeline_tokens_per_s': round(tokens / (t_pipe * 1e-3)),
            'multicast': bool(comm.mc_base)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--bench', action='store_true')
    ap.add_argument('--tokens', type=int, default=8192)
    ap.add_argument('--iters', type=int, default=20)
    args = ap.parse_args()
    local = int(os.environ['LOCAL_RANK'])
    torch.cuda.set_device(local)
    dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    rank, n = dist.get_rank(), dist.get_world_size()
    comm = Communicator.from_process_group(fifo_bytes=16 << 20, arena_bytes=640 << 20)
    check(comm, rank, n, rows=256, hidden=512, ffn_shard=512)
    if rank == 0:
        print('FUSED_TP_OK', flush=True)
    if args.bench:
        bench(comm, rank, n, args.tokens, 4096, 14336 // 8 * n if n < 8 else 14336, args.iters)
    comm.close()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
