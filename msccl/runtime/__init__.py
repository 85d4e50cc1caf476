"""Native executor for MSCCL-IR on B200: symmetric memory, interpreter kernel, direct kernels."""
from msccl.runtime.comm import Communicator, CommError, ExecutorError  # noqa: F401
from msccl.runtime.executor import DevicePlan, Executor  # noqa: F401
from msccl.runtime.plan import PlanError, compile_plan  # noqa: F401
from msccl.runtime.liveness import Liveness, PeerLostError  # noqa: F401
