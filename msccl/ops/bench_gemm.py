"""Time (and give profilers a small target for) the tcgen05 GEMM on one GPU.

    python -m msccl.ops.bench_gemm --m 8192 --n 3584 --k 4096 --iters 20 [--swiglu] [--fp8] [--cublas]
"""
import argparse
import json

import torch

from msccl.ops.gemm import check_gemm_errors, gemm_bf16


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--m', type=int, default=8192)
    ap.add_argument('--n', type=int, default=3584)
    ap.add_argument('--k', type=int, default=4096)
    ap.add_argument('--bn', type=int, default=256)
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--swiglu', action='store_true')
    ap.add_argument('--pair', type=int, default=-1, help='1: CTA-pair kernel (cta_group::2), 0: single-CTA kernel, -1: default')
    ap.add_argument('--fp8', action='store_true', help='block-scaled e4m3 kernel (MX scales per 32 K elements)')
    ap.add_argument('--cublas', action='store_true', help='also time torch.matmul (cuBLAS) on the same operands')
    args = ap.parse_args()
    a = torch.randn(args.m, args.k, device='cuda').bfloat16()
    b = (torch.randn(args.n, args.k, device='cuda') * 0.02).bfloat16()
    out = torch.empty(args.m, args.n // 2 if args.swiglu else args.n, device='cuda', dtype=torch.bfloat16)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.iters):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / args.iters

    if args.fp8:
        from msccl.ops.gemm import gemm_mxfp8, pack_mx_scales, quantize_mxfp8
        aq, sa = quantize_mxfp8(a.float())
        bq, sb = quantize_mxfp8(b.float())
        sa, sb = pack_mx_scales(sa), pack_mx_scales(sb)
        ms = timed(lambda: gemm_mxfp8(aq, sa, bq, sb, out=out, pair=None if args.pair < 0 else bool(args.pair)))
    else:
        ms = timed(lambda: gemm_bf16(a, b, out=out, bn=args.bn, epilogue='swiglu' if args.swiglu else 'none',
                                     pair=None if args.pair < 0 else bool(args.pair)))
    check_gemm_errors()
    flops = 2.0 * args.m * args.n * args.k
    row = {'m': args.m, 'n': args.n, 'k': args.k, 'bn': 128 if args.fp8 else args.bn, 'swiglu': args.swiglu, 'fp8': args.fp8, 'pair': args.pair, 'us': round(ms * 1e3, 1),
           'tflops': round(flops / ms / 1e9, 1)}
    if args.cublas and args.fp8:
        # library reference for fp8: cuBLASLt through torch._scaled_mm with one scale per tensor
        one = torch.ones((), device='cuda', dtype=torch.float32)
        bt = bq.t()
        ms_c = timed(lambda: torch._scaled_mm(aq, bt, scale_a=one, scale_b=one, out_dtype=torch.bfloat16))
        row.update({'cublaslt_fp8_us': round(ms_c * 1e3, 1), 'cublaslt_fp8_tflops': round(flops / ms_c / 1e9, 1)})
    elif args.cublas:
        full = torch.empty(args.m, args.n, device='cuda', dtype=torch.bfloat16)
        ms_c = timed(lambda: torch.matmul(a, b.t(), out=full))
        row.update({'cublas_us': round(ms_c * 1e3, 1), 'cublas_tflops': round(flops / ms_c / 1e9, 1)})
    print(json.dumps(row))


if __name__ == '__main__':
    main()
