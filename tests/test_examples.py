"""Regression targets for the example algorithms: threadblock / step / channel totals of the XML
the reference tool emits for the same programs and arguments, and execution on the CPU interpreter."""
import os
import subprocess
import sys

import pytest

from msccl.interp import run_reference_check
from msccl.language import MSCCLProgram, ThreadblockPolicy
from msccl.language.collectives import AllGather, AllReduce, AllToAll
from msccl.programs import classic
from msccl.programs.allreduce import allreduce_allpairs, allreduce_ring
from msccl.programs.alltoall import alltoall_direct, alltoall_hierarchical, alltoall_three_step
from msccl.topologies import fully_connected
from msccl.xml import load_xml, validate

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
M = ThreadblockPolicy.manual

#        name, collective, body, instances, options, (ngpus, proto, nchannels, nchunksperloop, tbs, steps)
CASES = [
    ('ring_8_4_4', lambda: AllReduce(8, 8, True), lambda: allreduce_ring(8, 4), 4,
     dict(protocol='LL128', threadblock_policy=M), (8, 'LL128', 16, 32, 128, 480)),
    ('allpairs_8_2', lambda: AllReduce(8, 64, True), lambda: allreduce_allpairs(8), 2,
     dict(protocol='LL', threadblock_policy=M, interleaved_replication=False, dependence_nop=True),
     (8, 'LL', 2, 128, 128, 2672)),
    ('allpairs_tree_8', lambda: AllReduce(8, 8, True), lambda: classic.allreduce_allpairs_tree(8), 1,
     dict(protocol='LL', threadblock_policy=M, interleaved_replication=False), (8, 'LL', 1, 8, 60, 298)),
    ('halving_doubling_8', lambda: AllReduce(8, 8, True), lambda: classic.allreduce_recursive_halving_doubling(8), 1,
     dict(protocol='LL', threadblock_policy=M, interleaved_replication=False), (8, 'LL', 1, 8, 24, 104)),
    ('hierarchical_auto', lambda: AllReduce(8, 8, True), lambda: classic.hierarchical_allreduce(4, 2), 1,
     dict(interleaved_replication=False), (8, 'Simple', 12, 8, 112, 144)),
    ('hierarchical_manual', lambda: AllReduce(8, 8, True), lambda: classic.hierarchical_allreduce(4, 2, True), 1,
     dict(interleaved_replication=False), (8, 'Simple', 6, 8, 48, 160)),
    ('ag_recursive_doubling', lambda: AllGather(8, 1, True), lambda: classic.allgather_recursive_doubling(8), 1,
     dict(threadblock_policy=M), (8, 'Simple', 1, 8, 24, 56)),
    ('a2a_allpairs', lambda: AllToAll(8, 1, False), lambda: alltoall_direct(8), 1, {}, (8, 'Simple', 1, 8, 112, 120)),
    ('a2a_two_step', lambda: AllToAll(16, 1, False), lambda: alltoall_hierarchical(2, 8), 1, {},
     (16, 'Simple', 6, 16, 256, 624)),
    ('a2a_three_step', lambda: AllToAll(16, 1, False), lambda: alltoall_three_step(2, 8, 1), 1, {},
     (16, 'Simple', 2, 16, 258, 528)),
    ('alltonext_forward', lambda: classic.AllToNext(16, 8, False, True), lambda: classic.alltonext(2, 8, True), 1, {},
     (16, 'Simple', 2, 8, 66, 66)),
    ('alltonext_backward', lambda: classic.AllToNext(16, 8, False, False), lambda: classic.alltonext(2, 8, False), 1, {},
     (16, 'Simple', 2, 8, 66, 66)),
]


@pytest.mark.parametrize('name,make_coll,body,instances,options,want', CASES, ids=[c[0] for c in CASES])
def test_example_totals_and_execution(name, make_coll, body, instances, options, want):
    coll = make_coll()
    prog = MSCCLProgram(name, fully_connected(coll.num_ranks), coll, instances, **options)
    with prog:
        body()
        assert prog.check()
    algo = load_xml(prog.generate_xml())
    got = (algo.ngpus, algo.proto, algo.nchannels, algo.nchunksperloop, algo.num_threadblocks(), algo.num_steps())
    assert got == want
    assert validate(algo) == []
    assert run_reference_check(algo, 2, race_check=True).startswith('pass')


@pytest.mark.parametrize('script,args', [('allreduce_ring.py', '4 2 1'), ('custom_collective.py', ''),
                                         ('alltonext.py', '2 1 --backward'), ('allgather_direct.py', '4 2')])
def test_example_scripts_run(script, args):
    run = subprocess.run([sys.executable, os.path.join(ROOT, 'examples', 'mscclang', script)] + args.split() + ['--execute'],
                         capture_output=True, text=True)
    assert run.returncode == 0, run.stderr
    assert run.stdout.startswith('<algo ') and 'interpreter: pass' in run.stderr


def test_init_and_synthesis_examples_run(clean_env):
    run = subprocess.run([sys.executable, os.path.join(ROOT, 'examples', 'msccl_init.py')], capture_output=True, text=True)
    assert run.returncode == 0 and 'synthesized_allgather' in run.stdout and 'run my_ring' in run.stdout, run.stdout + run.stderr
    run = subprocess.run([sys.executable, os.path.join(ROOT, 'examples', 'synthesis', 'allgather_pareto.py')],
                         capture_output=True, text=True)
    assert run.returncode == 0 and 'interpreter: pass' in run.stdout, run.stdout + run.stderr


def test_in_switch_and_b200_synthesis_examples_run(tmp_path):
    run = subprocess.run([sys.executable, os.path.join(ROOT, 'examples', 'runtime', 'in_switch_programs.py'), '4', '2'],
                         capture_output=True, text=True)
    assert run.returncode == 0, run.stderr
    assert run.stdout.startswith('<algo') and run.stderr.count('pass (race-free)') == 3
    out = tmp_path / 'ag4.xml'
    run = subprocess.run([sys.executable, os.path.join(ROOT, 'examples', 'synthesis', 'allgather_b200.py'), '--gpus', '4',
                          '--instances', '2', '-o', str(out)], capture_output=True, text=True)
    assert run.returncode == 0, run.stderr
    from msccl.interp import run_reference_check
    from msccl.xml import load_xml_file
    assert run_reference_check(load_xml_file(str(out))) == 'pass'
