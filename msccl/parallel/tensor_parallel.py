"""Tensor + sequence parallel SwiGLU MLP: activations sharded by tokens, weights by the FFN dimension.

``forward`` = all-gather -> (gate|up) GEMM -> SwiGLU  (one fused kernel)  then
            down GEMM -> reduce-scatter               (one fused kernel).
"""
import torch

from msccl.ops.fused_tp import FusedTensorParallel
from msccl.ops.gemm import interleave_gate_up


class TensorParallelMLP:
    def __init__(self, comm, tokens_per_rank, hidden, ffn, w_gate=None, w_up=None, w_down=None, std=0.02, seed=0):
        """``ffn`` is the full FFN width; this rank holds ``ffn / world`` of it.  Weights default to N(0, std)."""
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

    def forward(self, x_local, out=None):
        """x_local: [tokens_per_rank, hidden] -> this rank's [tokens_per_rank, hidden] of the MLP output."""
        self.fused.all_gather_gemm(x_local, self.w_gate_up, epilogue='swiglu', out=self.h)
        return self.fused.gemm_reduce_scatter(self.h, self.w_down, out=out)

    __call__ = forward
