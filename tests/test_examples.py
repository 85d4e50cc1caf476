"""Regression targets for the example algorithms: threadblock / step / channel totals of the XML
the reference tool emits for the same programs and arguments, and execution on the CPU interpreter."""
import os
import subprocess
import sys

import pytest

from msccl.interp import run_reference_check
from msccl.language import MSCCLProgram, ThreadblockPolicy
from msccl.language.collectives import AllGather, AllReduce, AllToAll
from msccl.programs import classic, multistage
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
    # programs spanning several groups of GPUs: totals recorded from this compiler (the reference's scripts use
    # other chunk factors and manual threadblocks, so its totals are not comparable)
    ('multinode_allpairs_4x2', lambda: AllReduce(8, 4, True), lambda: multistage.allreduce_multinode_allpairs(4, 2), 1, {},
     (8, 'Simple', 1, 4, 64, 168)),
    ('two_pairs', lambda: AllReduce(4, 2, True), multistage.allreduce_two_pairs, 1, {}, (4, 'Simple', 1, 2, 16, 32)),
    ('pipeline_ring_4', lambda: multistage.StageAllReduce(4, 4), lambda: multistage.pipeline_allreduce_ring(4, 2), 1, {},
     (8, 'Simple', 2, 4, 24, 40)),
    ('pipeline_allpairs_4', lambda: multistage.StageAllReduce(4, 4), lambda: multistage.pipeline_allreduce_allpairs(4), 1, {},
     (8, 'Simple', 2, 4, 56, 76)),
    ('allreduce_2d_3x3_batched', lambda: AllReduce(9, 9, True), lambda: multistage.allreduce_2d(3, 3), 2,
     dict(interleaved_replication=False), None),
    ('allgather_two_pairs', lambda: AllGather(4, 1, False), multistage.allgather_two_pairs, 2, {}, None),
    ('binomial_tree_6', lambda: AllReduce(6, 1, True), lambda: classic.allreduce_binomial_tree(6), 2, {}, None),
    ('reduce_gather_2x3', lambda: multistage.ReduceGather(2, 3), lambda: multistage.reduce_gather(2, 3), 2, {}, None),
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
    assert want is None or got == want
    assert validate(algo) == []
    assert run_reference_check(algo, 2, race_check=True).startswith('pass')


@pytest.mark.parametrize('script,args', [('allreduce_ring.py', '4 2 1'), ('custom_collective.py', ''),
                                         ('alltonext.py', '2 1 --backward'), ('allgather_direct.py', '4 2'),
                                         ('allreduce_multinode_allpairs.py', '2 3 2'), ('allreduce_two_pairs.py', '2'),
                                         ('pipeline_allreduce.py', '4 2 --channels 2'),
                                         ('pipeline_allreduce.py', '3 1 --allpairs'),
                                         ('allreduce_binomial_tree.py', '6 2'), ('allreduce_2d.py', '3 3 2'),
                                         ('allgather_two_pairs.py', '3'), ('allreduce_dgx1_chain.py', '2 2'),
                                         ('reduce_gather.py', '2 2 1')])
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


@pytest.mark.parametrize('body', ['ring', 'allpairs'])
def test_pipeline_stage_allreduce_numbers(body):
    # the custom collective is checked numerically here: every rank of stage 1 holds the sum of stage 0's inputs
    import torch
    from msccl.interp import Interpreter
    size = 4
    prog = MSCCLProgram('stage', fully_connected(2 * size), multistage.StageAllReduce(size, size), 2)
    with prog:
        if body == 'ring':
            multistage.pipeline_allreduce_ring(size, 2)
        else:
            multistage.pipeline_allreduce_allpairs(size)
        assert prog.check()
    algo = load_xml(prog.generate_xml())
    elems = 3
    gen = torch.Generator().manual_seed(5)
    inputs = [torch.randint(-9, 9, (size * 2 * elems,), generator=gen).float() for _ in range(2 * size)]
    machine = Interpreter(algo, elems, race_check=True)
    for r, data in enumerate(inputs):
        machine.set_input(r, data)
    machine.run()
    want = sum(inputs[:size])
    for t in range(size, 2 * size):
        assert torch.equal(machine.buffers[t]['i'][:want.numel()], want)     # in place: the result is in the input buffer


def test_collective_file_and_device_order_examples(tmp_path):
    target = tmp_path / 'send.json'
    run = subprocess.run([sys.executable, os.path.join(ROOT, 'examples', 'custom_collective_file.py'), str(target)],
                         capture_output=True, text=True)
    assert run.returncode == 0 and target.exists(), run.stderr
    run = subprocess.run([sys.executable, '-m', 'msccl', 'solve', 'least-steps', 'DGX1', 'custom', '--collective-file',
                          str(target), '--no-save'], capture_output=True, text=True, cwd=ROOT)
    assert run.returncode == 0 and '2→' in run.stdout, run.stdout + run.stderr
    run = subprocess.run([sys.executable, os.path.join(ROOT, 'examples', 'device_order.py'), '--demo'],
                         capture_output=True, text=True)
    assert run.returncode == 0 and run.stdout.count('Permutation(') == 4, run.stdout + run.stderr


def test_mixed_extents_are_refused_under_interleaved_replication():
    # one step moves three chunks that other steps handle one by one: copy i of the two kinds of step would get
    # different sub-chunks, and the dependency between them would not cover the shared data
    prog = MSCCLProgram('2d', fully_connected(9), AllReduce(9, 9, True), 2)
    with prog:
        multistage.allreduce_2d(3, 3)
    with pytest.raises(RuntimeError, match='interleaved_replication=False'):
        prog.generate_xml()
    single = MSCCLProgram('2d', fully_connected(9), AllReduce(9, 9, True), 1)      # one instance: nothing to interleave
    with single:
        multistage.allreduce_2d(3, 3)
    assert run_reference_check(load_xml(single.generate_xml()), 2, race_check=True) == 'pass (race-free)'


def test_reduce_gather_numbers():
    import torch
    from msccl.interp import Interpreter
    groups, g, elems = 2, 3, 2
    prog = MSCCLProgram('rg', fully_connected(groups * g), multistage.ReduceGather(groups, g), 2)
    with prog:
        multistage.reduce_gather(groups, g)
        assert prog.check()
    algo = load_xml(prog.generate_xml())
    gen = torch.Generator().manual_seed(1)
    inputs = [torch.randint(-5, 5, (g * 2 * elems,), generator=gen).float() for _ in range(groups * g)]
    machine = Interpreter(algo, elems, race_check=True)
    for r, data in enumerate(inputs):
        machine.set_input(r, data)
    machine.run()
    want = torch.cat([sum(inputs[q * g + m] for m in range(g)) for q in range(groups)])
    for r in range(groups * g):
        assert torch.equal(machine.buffers[r]['o'][:want.numel()], want)
