"""Import path kept for programs written against msccl-tools (``msccl.steps_bound``); the code lives in ``msccl.synth.bounds``."""
from msccl.synth.bounds import lower_bound_steps  # noqa: F401
