"""Import path kept for programs written against msccl-tools (``msccl.language.chunk``); the code lives in ``msccl.language.symbolic``."""
from msccl.language.symbolic import Chunk, ReduceChunk  # noqa: F401,F403
