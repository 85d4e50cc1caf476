"""The fused compute + collective layers on the GPUs of one box: a tensor-parallel SwiGLU MLP (all-gather -> GEMM and
GEMM -> reduce-scatter in one kernel each, bf16 and block-scaled fp8) and an expert-parallel MoE layer (routing,
dispatch, expert FFN and combine in four kernels), each checked against a PyTorch fp32 computation.

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/runtime/fused_layers.py
    python examples/runtime/fused_layers.py                 # one GPU: every block is local

The collectives these kernels fuse are the reference's AllGather, ReduceScatter and AllToAll (msccl/language/collectives.py).
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from msccl.ops import check_gemm_errors  # noqa: E402
from msccl.ops.moe import route_top_k  # noqa: E402
from msccl.parallel import ExpertParallelMoE, TensorParallelMLP  # noqa: E402
from msccl.runtime import Communicator  # noqa: E402


def main():
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    if 'RANK' not in os.environ:
        os.environ.update(RANK='0', WORLD_SIZE='1', MASTER_ADDR='127.0.0.1', MASTER_PORT='29590')
    dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    rank, n = dist.get_rank(), dist.get_world_size()
    comm = Communicator.from_process_group(fifo_bytes=16 << 20, arena_bytes=1 << 30)
    tokens_per_rank, hidden, ffn = 1024, 2048, 1024 * n
    gen = torch.Generator(device='cuda').manual_seed(11 + rank)
    x = torch.randn(tokens_per_rank, hidden, device='cuda', generator=gen).bfloat16()

    # ---- tensor + sequence parallel MLP: tokens sharded over the ranks, the FFN dimension too
    for precision in ('bf16', 'mxfp8'):
        mlp = TensorParallelMLP(comm, tokens_per_rank, hidden, ffn, precision=precision, seed=3)
        y = mlp(x)
        check_gemm_errors()
        # the same layer from its bf16 weights in fp32: all tokens, this rank's FFN shard, summed over the ranks
        full = torch.empty(n * tokens_per_rank, hidden, device='cuda', dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, x)
        shard = ffn // n
        gate_up = mlp.w_gate_up.float().view(-1, 2, 128, hidden)          # interleaved per 256 rows: 128 gate, 128 up
        w_gate, w_up = gate_up[:, 0].reshape(shard, hidden), gate_up[:, 1].reshape(shard, hidden)
        h = torch.nn.functional.silu(full.float() @ w_gate.t()) * (full.float() @ w_up.t())
        partial = h.bfloat16().float() @ mlp.w_down.float().t()
        dist.all_reduce(partial)
        want = partial[rank * tokens_per_rank:(rank + 1) * tokens_per_rank]
        err = (y.float() - want).abs().max().item() / want.abs().max().item()
        if rank == 0:
            print(f'tensor-parallel MLP ({precision}): {mlp.fused.launches} fused launches, relative error {err:.4f}')

    # ---- expert-parallel MoE: 4 experts per GPU, top-2 routing
    experts = 4 * n
    moe = ExpertParallelMoE(comm, tokens_per_rank, hidden, 1024, experts, topk=2, seed=5)
    logits = torch.randn(tokens_per_rank, experts, device='cuda', generator=gen)
    y = moe(x, gate_logits=logits)
    check_gemm_errors()
    ids, weights = route_top_k(logits, 2)                                   # the routing the layer computes on the device
    dev_ids, dev_weights = moe.moe.route(logits)
    same = torch.equal(dev_ids.long(), ids) and (dev_weights - weights).abs().max().item() < 1e-5
    if rank == 0:
        print(f'expert-parallel MoE: output {tuple(y.shape)}, finite {bool(torch.isfinite(y.float()).all())}, '
              f'device routing equals softmax + top-k: {same}')
    comm.close()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
