"""Hand-written sm_100a compute kernels (tcgen05 GEMM and its fused variants) as PyTorch callables."""
from msccl.ops.gemm import gemm_bf16, GemmKernelError, check_gemm_errors  # noqa: F401
