"""Tensor + sequence parallel SwiGLU MLP: activations sharded by tokens, weights by the FFN dimension.

``forward`` = all-gather -> (gate|up) GEMM -> SwiGLU  (one fused kernel)  then
            down GEMM -> reduce-scatter               (one fused kernel).

``precision='mxfp8'`` runs both kernels on block-scaled fp8 operands (OCP MX: e4m3 values, one power-of-two scale per
32 K elements): the weights are quantised once, the activations per call (the token shard before the all-gather, the
SwiGLU output before the down projection); accumulation is fp32 and the result bf16 either way.
"""
import torch

from msccl.ops.fused_tp import FusedTensorParallel
from msccl.ops.gemm import interleave_gate_up, pack_mx_scales, quantize_mxfp8, quantize_mxfp8_packed


class TensorParallelMLP:
    def __init__(self, comm, tokens_per_rank, hidden, ffn, w_gate=None, w_up=None, w_down=None, std=0.02, seed=0,
                 precision='bf16'):
        """``ffn`` is the full FFN width; this rank holds ``ffn / world`` of it.  Weights default to N(0, std)."""
        assert precision in ('bf16', 'mxfp8')
        self.precision = precision
        self.comm = comm
        self.shard = ffn // comm.world
        assert self.shard * comm.world == ffn and self.shard % 128 == 0
        dev = f'cuda:{comm.device}'
        gen = torch.Generator(device=dev).manual_seed(seed + comm.rank)
        mk = lambda *s: (torch.randn(*s, device=dev, generator=gen) * std).bfloat16()   # noqa: E731
        w_gate = mk(self.shard, hidden) if w_gate is None else w_gate
        w_up = mk(self.shard, hidden) if w_up is None else w_up
        self.w_gate_up = interleave_gate_up(w_gate, w_up)
        self.w_down = mk(hidden, self.shard) if w_down is None else w_down.contiguous()
        self.fused = FusedTensorParallel(comm, tokens_per_rank, hidden)
        self.h = torch.empty(comm.world * tokens_per_rank, self.shard, dtype=torch.bfloat16, device=dev)
        if precision == 'mxfp8':
            gu = interleave_gate_up(w_gate, w_up, tile=self.fused.mx_gate_up_tile)   # 256 on CTA pairs, 128 on single CTAs
            self.wq_gate_up, s = quantize_mxfp8(gu.float())
            self.sf_gate_up = pack_mx_scales(s, row_multiple=128)
            self.wq_down, s = quantize_mxfp8(self.w_down.float())
            self.sf_down = pack_mx_scales(s, row_multiple=128)

    def forward(self, x_local, out=None):
        """x_local: [tokens_per_rank, hidden] -> this rank's [tokens_per_rank, hidden] of the MLP output."""
        if self.precision == 'mxfp8':
            xq, sx = quantize_mxfp8_packed(x_local)                  # one kernel each: values + packed scales
            self.fused.all_gather_gemm_mxfp8(xq, sx, self.wq_gate_up, self.sf_gate_up, epilogue='swiglu', out=self.h)
            hq, sh = quantize_mxfp8_packed(self.h)
            return self.fused.gemm_reduce_scatter_mxfp8(hq, sh, self.wq_down, self.sf_down, out=out)
        self.fused.all_gather_gemm(x_local, self.w_gate_up, epilogue='swiglu', out=self.h)
        return self.fused.gemm_reduce_scatter(self.h, self.w_down, out=out)

    __call__ = forward
