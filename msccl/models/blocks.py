"""The two model blocks named by the benchmark configurations, with random-initialised weights."""
from msccl.parallel.expert_parallel import ExpertParallelMoE
from msccl.parallel.tensor_parallel import TensorParallelMLP


def llama3_8b_mlp(comm, tokens=8192):
    """Llama-3-8B MLP (hidden 4096, FFN 14336, SwiGLU) tensor-parallel over ``comm.world`` GPUs, ``tokens`` in total."""
    assert tokens % comm.world == 0
    return TensorParallelMLP(comm, tokens // comm.world, 4096, 14336)


def moe_block_64x2(comm, tokens_per_gpu=4096, experts_per_gpu=8):
    """MoE block: hidden 4096, expert FFN 4096->14336->4096 SwiGLU, 8 experts per GPU, top-2 routing."""
    return ExpertParallelMoE(comm, tokens_per_gpu, 4096, 14336, experts_per_gpu * comm.world, topk=2,
                             capacity_factor=1.5)
