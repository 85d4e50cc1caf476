"""The tcgen05 GEMMs on one B200: bf16 (CTA pairs) with a fused SwiGLU epilogue, and block-scaled fp8.

    python examples/runtime/gemm.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from msccl.ops import check_gemm_errors, gemm_bf16  # noqa: E402
from msccl.ops.gemm import (dequantize_mxfp8, gemm_mxfp8, interleave_gate_up, pack_mx_scales,  # noqa: E402
                            quantize_mxfp8)


def main():
    tokens, hidden, ffn = 2048, 4096, 3584
    x = torch.randn(tokens, hidden, device='cuda').bfloat16()
    w_gate = (torch.randn(ffn, hidden, device='cuda') * 0.02).bfloat16()
    w_up = (torch.randn(ffn, hidden, device='cuda') * 0.02).bfloat16()
    # one kernel: (gate | up) projection and silu(gate) * up; weights interleaved per 256-row tile
    h = gemm_bf16(x, interleave_gate_up(w_gate, w_up), epilogue='swiglu')
    check_gemm_errors()
    want = torch.nn.functional.silu(x.float() @ w_gate.float().t()) * (x.float() @ w_up.float().t())
    print('SwiGLU MLP up-projection: max abs error', (h.float() - want).abs().max().item())

    # MX fp8: e4m3 values with one power-of-two scale per 32 K elements; the tensor core applies the scales
    xq, xs = quantize_mxfp8(x.float())
    wq, ws = quantize_mxfp8(w_up.float())
    y = gemm_mxfp8(xq, pack_mx_scales(xs), wq, pack_mx_scales(ws))
    check_gemm_errors()
    exact = dequantize_mxfp8(xq, xs) @ dequantize_mxfp8(wq, ws).t()
    full = x.float() @ w_up.float().t()
    print('fp8 GEMM against its dequantised operands: max abs error', (y.float() - exact).abs().max().item())
    print('fp8 GEMM against the bf16 product: relative error',
          ((y.float() - full).norm() / full.norm()).item())


if __name__ == '__main__':
    main()
