"""Fused MoE expert parallelism on sm_100a: top-k dispatch all-to-all fused with the grouped gate/up
GEMM (+SwiGLU), and the grouped down GEMM fused with the combine all-to-all (``csrc/moe_a2a.cu``).

Experts are sharded contiguously over the ranks (expert e lives on rank ``e // local_experts``).
"""
import os

import torch

from msccl.ops.gemm import _errors, interleave_gate_up
from msccl.runtime.comm import Communicator


def _align(v, a):
    return (v + a - 1) // a * a


def route_top_k(gate_logits, topk=2):
    """Softmax over experts, keep the ``topk`` largest, renormalise.  Returns (expert ids [T, k] int64,
    weights [T, k] fp32)."""
    probs = torch.softmax(gate_logits.float(), dim=-1)
    weights, experts = torch.topk(probs, topk, dim=-1)
    return experts, weights / weights.sum(dim=-1, keepdim=True)


class FusedMoE:
    def __init__(self, comm: Communicator, tokens: int, hidden: int, ffn: int, num_experts: int, topk: int = 2,
                 capacity_factor: float = 2.0, comm_ctas: int = 16):
        if comm.emulated_mode:
            raise ValueError('the fused MoE kernels need one process per GPU')
        n = comm.world
        assert num_experts % n == 0 and hidden % 256 == 0 and ffn % 128 == 0
        self.comm, self.n = comm, n
        self.tokens, self.hidden, self.ffn, self.num_experts, self.topk = tokens, hidden, ffn, num_experts, topk
        self.local_experts = num_experts // n
        expected = n * tokens * topk / num_experts
        self.cap = _align(int(expected * capacity_factor) + 128, 128)
        self.comm_ctas = int(os.environ.get('MSCCL_COMM_CTAS', comm_ctas))
        # CTA pairs (cta_group::2) by default; MSCCL_MOE_PAIR=0 selects the single-CTA kernels
        self.pair = os.environ.get('MSCCL_MOE_PAIR', '1') != '0' and self.comm_ctas % 2 == 0 and hidden % 256 == 0
        le, cap = self.local_experts, self.cap
        counts_p = _align(n * num_experts * 4, 256)
        meta_p = _align(le * cap * 16, 256)
        disp_p = le * cap * hidden * 2
        comb_p = tokens * topk * hidden * 2
        total = 2 * (counts_p + meta_p + disp_p + comb_p)
        _, self.moe_off = comm.symmetric_empty(total // 2, torch.bfloat16)
        offs = [0, 2 * counts_p, 2 * counts_p + 2 * meta_p, 2 * counts_p + 2 * meta_p + 2 * disp_p]
        self.layout = offs + [counts_p, meta_p, disp_p, comb_p]
        self.h = torch.empty(le * cap, ffn, dtype=torch.bfloat16, device=f'cuda:{comm.device}')
        self.sms = comm.native.sm_count()
        self.launches = 0
        dev = f'cuda:{comm.device}'
        self._sorted = torch.empty(tokens * topk, dtype=torch.int32, device=dev)
        self._start = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
        self._route_e = torch.empty(tokens, topk, dtype=torch.int32, device=dev)
        self._route_w = torch.empty(tokens, topk, dtype=torch.float32, device=dev)

    def route(self, gate_logits, stream=None):
        """``route_top_k`` in one kernel of this package: gate logits [tokens, num_experts] -> (expert ids [tokens, k]
        int32, weights [tokens, k] fp32).  The tensors returned are reused by the next call."""
        assert gate_logits.shape == (self.tokens, self.num_experts)
        logits = gate_logits.float().contiguous()
        stream_h = (stream or torch.cuda.current_stream()).cuda_stream
        self.comm.native.moe_topk(logits.data_ptr(), self.tokens, self.num_experts, self.topk, self._route_e.data_ptr(),
                                  self._route_w.data_ptr(), stream_h)
        self.launches += 1
        return self._route_e, self._route_w

    def pack_weights(self, w_gate, w_up, w_down):
        """w_gate / w_up: [local_experts, ffn, hidden]; w_down: [local_experts, hidden, ffn] -> the stacked
        layouts the kernels read."""
        gu = torch.cat([interleave_gate_up(w_gate[e], w_up[e]) for e in range(self.local_experts)]).contiguous()
        return gu, w_down.reshape(self.local_experts * self.hidden, self.ffn).contiguous()

    def forward(self, x, experts, weights, w_gate_up, w_down, out=None, stream=None):
        """x [tokens, hidden] bf16; experts/weights [tokens, topk] from ``route_top_k``.  Returns y [tokens, hidden]."""
        c = self.comm
        assert x.shape == (self.tokens, self.hidden) and x.is_contiguous() and x.dtype == torch.bfloat16
        assert experts.shape == (self.tokens, self.topk) and weights.shape == (self.tokens, self.topk)
        flat = experts.reshape(-1).to(torch.int32).contiguous()
        copy_weight = weights.reshape(-1).float().contiguous()
        if out is None:
            out = torch.empty_like(x)
        stream_h = (stream or torch.cuda.current_stream()).cuda_stream
        # stable counting sort of the copies by expert: the order and the per-expert prefix the dispatch kernel reads
        sorted_copy, expert_start = self._sorted, self._start
        c.native.moe_sort(flat.data_ptr(), flat.numel(), self.num_experts, sorted_copy.data_ptr(), expert_start.data_ptr(), stream_h)
        geom = [c.rank, self.n, self.tokens, self.topk, self.hidden, self.ffn, self.num_experts, self.local_experts,
                self.cap, self.comm_ctas]
        args = (geom, self.layout, c.dev_heap_bases, list(c.heap_ptrs), c.off_fused, self.moe_off, x.data_ptr(),
                sorted_copy.data_ptr(), expert_start.data_ptr(), copy_weight.data_ptr(), w_gate_up.data_ptr(),
                self.h.data_ptr(), w_down.data_ptr(), out.data_ptr(), _errors(x.device).data_ptr(), self.sms, stream_h)
        c.native.moe_phase(0, *args, self.pair)
        c.native.moe_phase(1, *args, self.pair)
        self.launches += 3
        self._keep = (flat, copy_weight)                           # alive until the kernels have run
        return out
