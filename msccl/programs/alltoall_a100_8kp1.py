"""Import path kept for programs written against msccl-tools; the code lives in ``msccl.programs.alltoall``."""
from msccl.programs.alltoall import alltoall_three_step  # noqa: F401
