"""MSCCL-IR programs that use the in-switch (NVLS) extension steps: build, validate, run on the CPU interpreter.

    python examples/runtime/in_switch_programs.py 8 4 > allreduce_nvls.xml

With GPUs, ``Executor.run(executor.compile(xml), tensor_from_symmetric_empty)`` hands the same program to the native
``multimem`` kernel.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from msccl.interp import run_reference_check  # noqa: E402
from msccl.language.ext_nvls import allgather_nvls, allreduce_nvls, reduce_scatter_nvls  # noqa: E402
from msccl.xml import load_xml  # noqa: E402
from msccl.xml.validator import validate  # noqa: E402


def main():
    ranks = int(sys.argv[1]) if len(sys.argv) > 1 else 8
    instances = int(sys.argv[2]) if len(sys.argv) > 2 else 4
    for build in (allreduce_nvls, allgather_nvls, reduce_scatter_nvls):
        algo = load_xml(build(ranks, instances))
        problems = validate(algo)
        verdict = run_reference_check(algo, race_check=True) if not problems else problems
        print(f'{algo.name}: {sum(len(g.tbs) for g in algo.gpus)} threadblocks, {verdict}', file=sys.stderr)
    print(allreduce_nvls(ranks, instances))


if __name__ == '__main__':
    main()
