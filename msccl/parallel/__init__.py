"""Parallelism building blocks on top of the executor and the fused kernels: data-parallel gradient buckets,
tensor/sequence-parallel MLP, expert-parallel MoE, and pipeline hand-over on NCCL point-to-point."""
from msccl.parallel.tensor_parallel import TensorParallelMLP  # noqa: F401
from msccl.parallel.expert_parallel import ExpertParallelMoE  # noqa: F401
from msccl.parallel.pipeline import PipelineP2P  # noqa: F401
from msccl.parallel.data_parallel import FlatGradients  # noqa: F401
