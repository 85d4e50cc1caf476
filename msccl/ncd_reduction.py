"""Import path kept for programs written against msccl-tools (``msccl.ncd_reduction``); the code lives in ``msccl.synth.duality``."""
from msccl.synth.duality import ReductionNotApplicableError, non_combining_dual, recover_primal_algorithm, wrap_try_ncd_reduction  # noqa: F401
