"""Import path kept for programs written against msccl-tools; the code lives in ``msccl.programs.alltoall``."""
from msccl.programs.alltoall import alltoall_hierarchical  # noqa: F401
