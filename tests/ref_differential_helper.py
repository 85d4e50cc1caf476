"""Compile a fixed list of MSCCLang programs with whichever ``msccl`` package is first on ``sys.path`` and write
one XML file per program into the directory given as the only argument.

tests/test_reference_differential.py runs this twice, once against this repository's package and once against
the installed reference, and compares the outputs.  The program bodies come from
``msccl/programs/{allreduce,allgather,alltoall}.py`` of this repository, loaded by file path: they use nothing but
``msccl.language.Buffer`` and ``msccl.language.chunk``, which both packages provide.
"""
import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PROGRAMS = os.path.join(os.path.dirname(HERE), 'msccl', 'programs')


def _load(name):
    spec = importlib.util.spec_from_file_location(f'_bodies_{name}', os.path.join(PROGRAMS, name + '.py'))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def cases():
    from msccl.language.collectives import AllGather, AllReduce, AllToAll, ReduceScatter
    ar, ag, a2a = _load('allreduce'), _load('allgather'), _load('alltoall')
    M = 'manual'
    return [
        ('ring_8_4_x4_ll128', lambda: AllReduce(8, 8, True), lambda: ar.allreduce_ring(8, 4), 4, dict(protocol='LL128', policy=M)),
        ('ring_8_1_x1', lambda: AllReduce(8, 8, True), lambda: ar.allreduce_ring(8, 1), 1, dict(policy=M)),
        ('ring_4_2_x2_ll', lambda: AllReduce(4, 4, True), lambda: ar.allreduce_ring(4, 2), 2, dict(protocol='LL', policy=M)),
        ('ring_2_1_x8', lambda: AllReduce(2, 2, True), lambda: ar.allreduce_ring(2, 1), 8, dict(policy=M)),
        ('allpairs_8_x2_nop', lambda: AllReduce(8, 64, True), lambda: ar.allreduce_allpairs(8), 2,
         dict(protocol='LL', policy=M, interleaved_replication=False, dependence_nop=True)),
        ('allpairs_4_x1', lambda: AllReduce(4, 16, True), lambda: ar.allreduce_allpairs(4), 1, dict(policy=M)),
        ('allpairs_4_x4_ll', lambda: AllReduce(4, 16, True), lambda: ar.allreduce_allpairs(4), 4,
         dict(protocol='LL', policy=M, interleaved_replication=False)),
        ('one_shot_8', lambda: AllReduce(8, 1, True), lambda: ar.allreduce_one_shot(8), 1, dict(protocol='LL', policy=M)),
        ('one_shot_4_x2', lambda: AllReduce(4, 1, True), lambda: ar.allreduce_one_shot(4), 2, dict(protocol='LL', policy=M)),
        ('two_shot_8_x2', lambda: AllReduce(8, 8, True), lambda: ar.allreduce_two_shot(8), 2, dict(policy=M)),
        ('two_shot_2_x8', lambda: AllReduce(2, 2, True), lambda: ar.allreduce_two_shot(2), 8, dict(policy=M)),
        ('a2a_direct_8', lambda: AllToAll(8, 1, False), lambda: a2a.alltoall_direct(8), 1, {}),
        ('a2a_direct_4_x4', lambda: AllToAll(4, 1, False), lambda: a2a.alltoall_direct(4), 4, dict(protocol='LL')),
        ('a2a_two_step_2x8', lambda: AllToAll(16, 1, False), lambda: a2a.alltoall_hierarchical(2, 8), 1, {}),
        ('a2a_two_step_3x8_ll128', lambda: AllToAll(24, 1, False), lambda: a2a.alltoall_hierarchical(3, 8), 1,
         dict(protocol='LL128')),
        ('a2a_three_step_2x8', lambda: AllToAll(16, 1, False), lambda: a2a.alltoall_three_step(2, 8, 1), 1, {}),
        ('a2a_three_step_2x4_x2', lambda: AllToAll(8, 1, False), lambda: a2a.alltoall_three_step(2, 4, 1), 2, {}),
        ('ag_direct_8', lambda: AllGather(8, 1, False), lambda: ag.allgather_direct(8), 1, {}),
        ('ag_direct_4_x2', lambda: AllGather(4, 1, False), lambda: ag.allgather_direct(4), 2, {}),
        ('ag_ring_8_2', lambda: AllGather(8, 1, False), lambda: ag.allgather_ring(8, 2), 1, {}),
        ('ag_ring_4_1_x2', lambda: AllGather(4, 1, False), lambda: ag.allgather_ring(4, 1), 2, dict(protocol='LL')),
        ('rs_direct_4_x2', lambda: ReduceScatter(4, 1, False), lambda: ag.reduce_scatter_direct(4), 2, {}),
    ]


def main(out_dir):
    from msccl.language import MSCCLProgram
    try:
        from msccl.language import ThreadblockPolicy
    except ImportError:                      # the reference keeps the enum in its IR module
        from msccl.language.ir import ThreadblockPolicy
    from msccl.topologies import fully_connected
    os.makedirs(out_dir, exist_ok=True)
    for name, coll, body, instances, opts in cases():
        opts = dict(opts)
        policy = opts.pop('policy', None)
        if policy == 'manual':
            opts['threadblock_policy'] = ThreadblockPolicy.manual
        collective = coll()
        prog = MSCCLProgram(name, fully_connected(collective.num_ranks), collective, instances, **opts)
        with prog:
            body()
            import contextlib
            import io
            from msccl.language import XML
            text = io.StringIO()
            with contextlib.redirect_stdout(text):
                XML()
        with open(os.path.join(out_dir, name + '.xml'), 'w') as f:
            f.write(text.getvalue())
    print('DONE', flush=True)


if __name__ == '__main__':
    main(sys.argv[1])
