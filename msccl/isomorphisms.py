"""Import path kept for programs written against msccl-tools (``msccl.isomorphisms``); the code lives in ``msccl.synth.symmetry``."""
from msccl.synth.symmetry import Permutation, find_isomorphisms  # noqa: F401
