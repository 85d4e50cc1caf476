"""Import path kept for programs written against msccl-tools (``msccl.strategies``); the code lives in ``msccl.synth.search``."""
from msccl.synth.search import solve_instance, solve_least_steps, solve_all_latency_bandwidth_tradeoffs, prune_pareto_optimal  # noqa: F401
