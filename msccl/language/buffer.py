"""Import path kept for programs written against msccl-tools (``msccl.language.buffer``); the code lives in ``msccl.language.symbolic``."""
from msccl.language.symbolic import BufferSlice  # noqa: F401,F403
