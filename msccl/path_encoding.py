"""Import path kept for programs written against msccl-tools (``msccl.path_encoding``); the code lives in ``msccl.synth.smt_paths``."""
from msccl.synth.smt_paths import PathEncoding, PathEncodingBase  # noqa: F401
