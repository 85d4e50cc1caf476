"""Import path kept for programs written against msccl-tools; the code lives in ``msccl.programs.allreduce``."""
from msccl.programs.allreduce import allreduce_ring  # noqa: F401
