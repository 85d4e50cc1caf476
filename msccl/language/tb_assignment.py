"""Import path kept for programs written against msccl-tools (``msccl.language.tb_assignment``); the code lives in ``msccl.language.compiler.schedule``."""
from msccl.language.compiler.schedule import auto_assign_tbs, manual_assign_tbs, topo_sort_instrs, channel_assignment  # noqa: F401,F403
