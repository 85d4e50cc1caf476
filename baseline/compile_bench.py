"""Time the MSCCLang compiler (program body -> MSCCL-IR XML) on a few large programs with whichever ``msccl`` package
is first on ``sys.path``: this repository's, or the unmodified reference installed under ``baseline/_ref``.

    PYTHONPATH=. python baseline/compile_bench.py                              # this repository
    PYTHONPATH=baseline/shims:baseline/_ref python baseline/compile_bench.py    # the reference

The program bodies are loaded by file path from ``msccl/programs`` of this repository; they use only
``msccl.language.chunk`` / ``Buffer``, which both packages provide (reference msccl/language/__init__.py:175-190).
The all-pairs program is replicated in batches, not interleaved: this repository refuses the interleaved form for
programs that address a chunk with two different extents.
"""
import contextlib
import importlib.util
import io
import os
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bodies(name):
    spec = importlib.util.spec_from_file_location(f'_bodies_{name}', os.path.join(ROOT, 'msccl', 'programs', name + '.py'))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def main():
    from msccl.language import XML, MSCCLProgram
    from msccl.language.collectives import AllReduce, AllToAll
    from msccl.topologies import fully_connected
    ar, a2a = _bodies('allreduce'), _bodies('alltoall')
    cases = [('allreduce_allpairs, 8 ranks, 4 instances', 8, lambda: AllReduce(8, 64, True), lambda: ar.allreduce_allpairs(8), 4, False),
             ('allreduce_ring, 8 ranks, 4 channels, 8 instances', 8, lambda: AllReduce(8, 8, True), lambda: ar.allreduce_ring(8, 4), 8, True),
             ('alltoall three-step, 2 x 8 ranks, 2 instances', 16, lambda: AllToAll(16, 1, False),
              lambda: a2a.alltoall_three_step(2, 8, 1), 2, True),
             ('alltoall hierarchical, 4 x 8 ranks', 32, lambda: AllToAll(32, 1, False), lambda: a2a.alltoall_hierarchical(4, 8), 1, True)]
    for name, ranks, collective, body, instances, interleaved in cases:
        start = time.perf_counter()
        text = io.StringIO()
        with MSCCLProgram(name, fully_connected(ranks), collective(), instances, interleaved_replication=interleaved):
            body()
            with contextlib.redirect_stdout(text):
                XML()
        print(f'{name}: {time.perf_counter() - start:.2f} s, {len(text.getvalue())} bytes of XML', flush=True)


if __name__ == '__main__':
    main()
