"""Import path kept for programs written against msccl-tools (``msccl.language.passes``); the code lives in ``msccl.language.compiler.verify``."""
from msccl.language.compiler.verify import check_dependency_cycles, check_threadblock_ordering  # noqa: F401,F403
