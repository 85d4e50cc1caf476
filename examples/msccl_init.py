"""Using the plan registry: register own algorithms, let ``msccl.init`` pick per size range, then run
collectives through the native executor (one process per GPU under torchrun) or plain
``torch.distributed``."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import msccl  # noqa: E402
from msccl.autosynth.registry import register_msccl_program, register_synthesis_plan  # noqa: E402
from msccl.collectives import allgather  # noqa: E402
from msccl.language.mscclir import ThreadblockPolicy  # noqa: E402
from msccl.ncclize import ncclize  # noqa: E402
from msccl.programs.allreduce import allreduce_ring  # noqa: E402
from msccl.strategies import solve_least_steps  # noqa: E402
from msccl.topologies import fully_connected, hub_and_spoke  # noqa: E402


# A synthesized plan: least-steps all-gather on the NVSwitch model, valid from 64 KB to 256 MB.
@register_synthesis_plan('allgather', 'mybox', sizes=('64KB', '256MB'))
def synthesized_allgather(machines):
    return ncclize(solve_least_steps(hub_and_spoke(8), allgather(8)), instances=2)


# An MSCCLang plan with a higher priority on an overlapping range.
@register_msccl_program(fully_connected(8), 'allreduce', 'mybox', chunk_factor=8, inplace=True, instances=4,
                        sizes=('1MB', None), priority=1, threadblock_policy=ThreadblockPolicy.manual)
def my_ring(prog, machines):
    allreduce_ring(8, 4)


if __name__ == '__main__':
    msccl.init('mybox', 1, ('allgather', ('64KB', '1MB')), (msccl.Collective.allreduce, '16MB'))
    print('plan table written to', os.environ['MSCCL_CONFIG'])
    print(open(os.environ['MSCCL_CONFIG']).read())
    # With GPUs: executor = msccl.runtime.Executor(msccl.runtime.Communicator.from_process_group()).load_plan_table()
