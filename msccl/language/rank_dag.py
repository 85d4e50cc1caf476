"""Import path kept for programs written against msccl-tools (``msccl.language.rank_dag``); the code lives in ``msccl.language.dag``."""
from msccl.language.dag import InstructionDAG  # noqa: F401,F403
