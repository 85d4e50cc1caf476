"""Expert-parallel MoE layer: top-k routing, fused dispatch + expert FFN + combine."""
import torch

from msccl.ops.moe import FusedMoE


class ExpertParallelMoE:
    def __init__(self, comm, tokens, hidden, ffn, num_experts, topk=2, std=0.02, seed=0, capacity_factor=2.0):
        self.comm = comm
        self.topk = topk
        dev = f'cuda:{comm.device}'
        gen = torch.Generator(device=dev).manual_seed(seed + comm.rank)
        self.moe = FusedMoE(comm, tokens, hidden, ffn, num_experts, topk, capacity_factor)
        le = self.moe.local_experts
        mk = lambda *s: (torch.randn(*s, device=dev, generator=gen) * std).bfloat16()   # noqa: E731
        self.w_gate_up, self.w_down = self.moe.pack_weights(mk(le, ffn, hidden), mk(le, ffn, hidden), mk(le, hidden, ffn))
        gate_gen = torch.Generator(device=dev).manual_seed(seed)       # the router is replicated
        self.w_router = (torch.randn(num_experts, hidden, device=dev, generator=gate_gen) * std).bfloat16()

    def forward(self, x, gate_logits=None, out=None):
        if gate_logits is None:
            gate_logits = x @ self.w_router.t()
        experts, weights = self.moe.route(gate_logits)       # top-k of the softmax, renormalised (route_top_k in one kernel)
        return self.moe.forward(x, experts, weights, self.w_gate_up, self.w_down, out=out)

    __call__ = forward
