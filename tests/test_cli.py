"""End-to-end command line tests (``python -m msccl ...``), after the reference's tests/test_cli.py."""
import os
import subprocess
import sys

from msccl.collectives import build_collective
from msccl.serialization import save_msccl_object
from msccl.topologies import Topology

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def msccl_cli(args, expect=0):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get('PYTHONPATH', ''))
    run = subprocess.run([sys.executable, '-m', 'msccl'] + args.split(), env=env, capture_output=True, text=True)
    if expect is not None:
        assert (run.returncode == 0) == (expect == 0), run.stdout + run.stderr
    return run


def ncclizes(path):
    msccl_cli(f'ncclize {path} -o ncclized.msccl.xml -f')
    assert os.path.exists('ncclized.msccl.xml')
    assert 'ok (' in msccl_cli('check ncclized.msccl.xml --elems 2 --race-check').stdout


def test_help():
    assert 'solve' in msccl_cli('--help').stdout


def test_solve_instance(in_tempdir):
    msccl_cli('solve instance Ring Allgather --nodes 4 --steps 1 -o algo.json')
    assert not os.path.exists('algo.json')
    msccl_cli('solve instance Ring Allgather --nodes 2 --steps 1 -o algo.json')
    assert os.path.exists('algo.json')
    assert 'use -f/--force' in msccl_cli('solve instance Ring Allgather --nodes 2 --steps 1 -o algo.json').stderr
    msccl_cli('solve instance Ring Allgather --nodes 2 --steps 1 -o algo.json --force')
    ncclizes('algo.json')
    out = msccl_cli('solve instance Ring Allgather --nodes 2 --steps 1 --no-save').stdout
    assert 'Allgather(n=2)-Ring(n=2)-steps=1 algorithm:' in out and '0:0→1' in out
    msccl_cli('solve instance Ring Allgather --steps 1', expect=1)            # sized topology needs -n
    msccl_cli('solve instance DGX1 Allgather -n 4 --steps 1', expect=1)       # fixed topology size clash
    msccl_cli('solve instance Ring Allgather -n 2 -s 2 -r 1', expect=1)       # rounds < steps


def test_extra_memory(in_tempdir):
    msccl_cli('solve instance Ring -n 4 Alltoall -s 2 --extra-memory 0 -o algo.json')
    ncclizes('algo.json')


def test_least_steps_and_pareto(in_tempdir):
    msccl_cli('solve least-steps Ring Allgather --nodes 2')
    assert 'Checking for fewer steps' in msccl_cli('solve least-steps Ring Allgather --nodes 2 --initial-steps 2').stdout
    os.mkdir('a'), os.mkdir('b')
    assert 'Found 1 Pareto optimal algorithms. Pruned 1' in msccl_cli('solve pareto-optimal Ring Allgather --nodes 4 -d a').stdout
    assert os.listdir('a') == ['Allgather.n4-Ring.n4-steps2.rounds3.chunks2.msccl.json']
    msccl_cli('solve pareto-optimal Ring Allgather --nodes 4 -d b --save-eagerly')
    assert len(os.listdir('b')) == 2
    msccl_cli('solve pareto-optimal Ring Alltoall --nodes 2 --assume-rpc-bound 1/1 --no-save')
    msccl_cli('solve pareto-optimal Ring Alltoall --nodes 2 --no-monotonic-feasibility --no-save')


def test_ncclize_options(in_tempdir):
    msccl_cli('solve instance Ring Allgather --nodes 2 --steps 1 -o algo.json')
    msccl_cli('ncclize algo.json -o ncclized1.msccl.xml')
    assert os.path.exists('ncclized1.msccl.xml')
    for flags in ('--channel-policy One', '--channel-policy MatchTopology', '--no-merge-contiguous',
                  '--no-pretty-print', '--instances 2', '--no-scratch'):
        msccl_cli(f'ncclize algo.json -f {flags}')
    assert os.path.exists('Allgather.n2-Ring.n2-steps1.msccl.xml')
    msccl_cli('solve instance Star Alltoall --nodes 4 --steps 2 --rounds 4 -o algo_scratch.json')
    msccl_cli('ncclize algo_scratch.json -f --remap-scratch')
    msccl_cli('ncclize algo_scratch.json -f --greedy-scratch-sorting')
    msccl_cli('ncclize algo_scratch.json --remap-scratch --no-remap-scratch', expect=1)


def test_custom_topology_and_collective(in_tempdir):
    save_msccl_object(Topology('CT', [[0, 1], [1, 0]]), 'topo.json')
    save_msccl_object(build_collective('CC', 2, 1, lambda r, c: r == 0, lambda r, c: r == 1), 'coll.json')
    msccl_cli('solve instance custom custom --topology-file topo.json --collective-file coll.json -s 1 --no-save')
    msccl_cli('solve instance custom Allgather -s 1', expect=1)


def test_analyses():
    assert '7/6' in msccl_cli('analyze rounds DGX1 Allgather').stdout
    assert '4 isomorphisms found.' in msccl_cli('analyze isomorphisms DGX1 DGX1').stdout
    assert '7 rounds' in msccl_cli('analyze rounds HubAndSpoke -n 8 Allgather').stdout
    assert 'ReverseRing' in msccl_cli('analyze rounds Ring -n 3 -t reverse Broadcast --root 1').stdout


def test_distribute_greedy(in_tempdir):
    msccl_cli('solve instance Ring Alltoall --nodes 4 --steps 2 -o local.json')
    msccl_cli('distribute alltoall-greedy local.json DistributedFullyConnected --copies 3 -o dist.json')
    ncclizes('dist.json')
    msccl_cli('distribute alltoall-greedy local.json DistributedHubAndSpoke --nodes 8 --no-save')
    msccl_cli('distribute alltoall-greedy local.json DistributedHubAndSpoke --nodes 5', expect=1)


def test_distribute_gather_scatter(in_tempdir):
    msccl_cli('solve instance DGX1 Gather --root 5 --steps 2 -o gather.json')
    msccl_cli('solve instance DGX1 Scatter --root 5 --steps 2 -o scatter.json')
    msccl_cli('distribute alltoall-gather-scatter gather.json scatter.json --copies 2 -o alltoall.json')
    ncclizes('alltoall.json')


def test_distribute_gather_scatter_multiroot(in_tempdir):
    msccl_cli('solve instance Ring -n 3 MultirootGather --roots 0 1 --steps 1 -o gather.json')
    msccl_cli('solve instance Ring -n 3 MultirootScatter --roots 1 2 --steps 1 -o scatter.json')
    msccl_cli('distribute alltoall-gather-scatter gather.json scatter.json --copies 2 -o alltoall.json')
    ncclizes('alltoall.json')


def test_distribute_subproblem(in_tempdir):
    msccl_cli('distribute alltoall-create-subproblem Line -n 2 --copies 2')
    coll, topo = 'AlltoallSubproblem.n2.copies2.msccl.json', 'Subtopo.localLine.n2.relays.0.msccl.json'
    assert os.path.exists(coll) and os.path.exists(topo)
    msccl_cli(f'solve instance custom custom --topology-file {topo} --collective-file {coll} -s 3 -r 4 -o subalgo.json')
    msccl_cli('distribute alltoall-stitch-subproblem subalgo.json --copies 2 -o stitched.json')
    ncclizes('stitched.json')


def test_compose_allreduce(in_tempdir):
    msccl_cli('solve instance DGX1 ReduceScatter -s 2 -r 3 -c 2 -o reducescatter.json')
    msccl_cli('solve instance DGX1 Allgather -s 2 -r 3 -c 2 -o allgather.json')
    msccl_cli('compose allreduce reducescatter.json allgather.json -o allreduce.json')
    ncclizes('allreduce.json')


def test_plans_list():
    out = msccl_cli('plans list').stdout
    assert 'ndv4_ring_allreduce_config2' in out and 'b200_allreduce_two_shot_8' in out


def test_check_reports_problems(in_tempdir):
    with open('bad.xml', 'w') as f:
        f.write('<algo name="bad" proto="Simple" nchannels="1" nchunksperloop="1" ngpus="2" coll="custom" inplace="0">'
                '<gpu id="0" i_chunks="1" o_chunks="1" s_chunks="0"><tb id="0" send="1" recv="-1" chan="0">'
                '<step s="0" type="s" srcbuf="i" srcoff="0" dstbuf="o" dstoff="0" cnt="1" depid="-1" deps="-1" hasdep="0"/>'
                '</tb></gpu><gpu id="1" i_chunks="1" o_chunks="1" s_chunks="0"></gpu></algo>')
    run = msccl_cli('check bad.xml', expect=1)
    assert 'sends but 0 receives' in run.stdout
