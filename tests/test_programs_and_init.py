"""Shipped programs, plan registry and msccl.init (reference tests/test_programs.py, test_autosynth.py)."""
import os
import xml.etree.ElementTree as ET

import pytest

import msccl
from msccl.autosynth.registry import register_ef_file, register_synthesis_plan, synthesis_plans
from msccl.interp import run_reference_check
from msccl.language import MSCCLProgram, ThreadblockPolicy, Check
from msccl.language.collectives import AllGather, AllReduce, AllToAll, ReduceScatter
from msccl.topologies import fully_connected
from msccl.xml import load_plan_table, load_xml, validate


def _compile(name, coll, body, instances=1, **kw):
    prog = MSCCLProgram(name, fully_connected(coll.num_ranks), coll, instances, **kw)
    with prog:
        body()
        assert Check()
    return load_xml(prog.generate_xml())


def _tb_steps(algo):
    return algo.num_threadblocks(), algo.num_steps()


def test_alltoall_hierarchical():
    from msccl.programs.alltoall_a100_yifan import alltoall_hierarchical
    algo = _compile('hierarchical_all_to_all', AllToAll(32, 1, False), lambda: alltoall_hierarchical(4, 8))
    assert validate(algo) == [] and run_reference_check(algo, 1).startswith('pass')


def test_alltoall_three_step():
    from msccl.programs.alltoall_a100_8kp1 import alltoall_three_step
    algo = _compile('three_step', AllToAll(72, 1, False), lambda: alltoall_three_step(9, 8))
    assert validate(algo) == []
    small = _compile('three_step', AllToAll(16, 1, False), lambda: alltoall_three_step(2, 8))
    assert _tb_steps(small) == (258, 528) and small.nchannels == 2
    assert run_reference_check(small, 1, race_check=True).startswith('pass')


def test_allreduce_ring_registered_shape():
    from msccl.programs.allreduce_a100_ring import allreduce_ring
    algo = _compile('allreduce_ring', AllReduce(8, 8, True), lambda: allreduce_ring(8, 8), 4,
                    protocol='LL128', threadblock_policy=ThreadblockPolicy.manual)
    assert validate(algo) == [] and algo.proto == 'LL128'
    four = _compile('allreduce_ring', AllReduce(8, 8, True), lambda: allreduce_ring(8, 4), 4,
                    protocol='LL128', threadblock_policy=ThreadblockPolicy.manual)
    assert _tb_steps(four) == (128, 480) and four.nchannels == 16 and four.nchunksperloop == 32
    assert run_reference_check(four, 2, race_check=True).startswith('pass')


def test_allreduce_allpairs_registered_shape():
    from msccl.programs.allreduce_allpairs import allreduce_allpairs
    algo = _compile('allreduce_allpairs', AllReduce(8, 64, True), lambda: allreduce_allpairs(8), 2,
                    protocol='LL', threadblock_policy=ThreadblockPolicy.manual,
                    interleaved_replication=False, dependence_nop=True)
    assert _tb_steps(algo) == (128, 2672) and algo.nchannels == 2 and algo.nchunksperloop == 128
    assert validate(algo) == [] and run_reference_check(algo, 1, race_check=True).startswith('pass')


@pytest.mark.parametrize('n', [2, 4, 8])
def test_b200_programs(n):
    from msccl.programs.allgather import allgather_direct, allgather_ring, reduce_scatter_direct
    from msccl.programs.allreduce import allreduce_one_shot, allreduce_two_shot
    from msccl.programs.alltoall import alltoall_direct
    manual = dict(threadblock_policy=ThreadblockPolicy.manual)
    cases = [
        _compile('one_shot', AllReduce(n, 1, True), lambda: allreduce_one_shot(n), 1, **manual),
        _compile('one_shot_l2', AllReduce(n, 2, True), lambda: allreduce_one_shot(n, 2), 1, **manual),
        _compile('two_shot', AllReduce(n, n, True), lambda: allreduce_two_shot(n), 4, **manual),
        _compile('two_shot_l2', AllReduce(n, 2 * n, True), lambda: allreduce_two_shot(n, 2), 1, **manual),
        _compile('a2a', AllToAll(n, 1, False), lambda: alltoall_direct(n), 2),
        _compile('ag', AllGather(n, 1, False), lambda: allgather_direct(n), 2),
        _compile('ag_ring', AllGather(n, 1, False), lambda: allgather_ring(n)),
        _compile('rs', ReduceScatter(n, 1, False), lambda: reduce_scatter_direct(n), 2),
    ]
    for algo in cases:
        assert validate(algo) == [], algo.name
        assert run_reference_check(algo, 3, race_check=True).startswith('pass'), algo.name
    assert cases[0].max_tbs_per_gpu() == n - 1


def test_init_selects_ndv4_allreduce_plans(capsys, clean_env):
    for sizes, plan in [((512, 1024), 'ndv4_allpairs_allreduce_config1 with LL protocol'),
                        ((82944, 458752), 'ndv4_allpairs_allreduce_config2 with LL protocol'),
                        ((458752, 2129920), 'ndv4_ring_allreduce_config1 with LL protocol'),
                        ((2129920, 22806528), 'ndv4_ring_allreduce_config2 with LL128 protocol')]:
        msccl.init('ndv4', 1, (msccl.Collective.allreduce, sizes))
        assert plan in capsys.readouterr().out


def test_init_selects_ndv4_alltoall_plans(capsys, clean_env):
    msccl.init('ndv4', 8, (msccl.Collective.alltoall, ('1MB', '32MB')))
    assert 'ndv4_alltoall_hierarchical_config1 with LL128 protocol' in capsys.readouterr().out
    msccl.init('ndv4', 8, (msccl.Collective.alltoall, ('32MB', '64MB')))
    assert 'ndv4_alltoall_hierarchical_config2 with Simple protocol' in capsys.readouterr().out


def test_init_environment(capsys, clean_env):
    msccl.init('not_a_machine_type', 4, ('alltoall', 0))
    assert 'No plan found' in capsys.readouterr().out
    assert 'MSCCL_CONFIG' not in os.environ and 'NCCL_ALGO' not in os.environ

    msccl.init('ndv2', 2, ('alltoall', '1MB'))
    assert 'synthesize_ndv2_relay_alltoall' in capsys.readouterr().out
    assert 'NCCL_IB_AR_THRESHOLD' not in os.environ and os.environ['NCCL_ALGO'] == 'MSCCL,RING,TREE'
    table = load_plan_table(os.environ['MSCCL_CONFIG'])
    assert len(table) == 1 and table[0].min_bytes == 1000000 and table[0].proto == 'Simple'
    assert table[0].algo.ngpus == 16 and table[0].algo.coll == 'alltoall'
    assert table[0].algo.gpus[0].i_chunks == 128 and table[0].algo.gpus[0].s_chunks > 0
    assert validate(table[0].algo) == []

    os.environ['NCCL_ALGO'] = 'RING,FAKE_MSCCL'
    msccl.init('ndv4', 8, (msccl.Collective.alltoall, '2MB'))
    assert 'ndv4_alltoall' in capsys.readouterr().out
    assert 'NCCL_IB_AR_THRESHOLD' in os.environ and os.environ['NCCL_ALGO'] == 'MSCCL,RING,FAKE_MSCCL'

    os.environ['NCCL_ALGO'] = 'HELLO,MSCCL,WORLD'
    msccl.init('ndv4', 16, (msccl.Collective.alltoall, '35MB'))
    assert 'ndv4_alltoall' in capsys.readouterr().out and os.environ['NCCL_ALGO'] == 'HELLO,MSCCL,WORLD'


def test_init_b200_plan_table(capsys, clean_env):
    msccl.init('b200', 1, ('allreduce', (0, None)), ('alltoall', '1MB'), ('allgather', '64KB'))
    out = capsys.readouterr().out
    assert 'b200_allreduce_one_shot_8 with LL protocol' in out
    assert 'b200_allreduce_in_switch_8' in out                                     # from 64 KB: reduced inside the switch
    assert 'b200_allreduce_two_shot' not in out                                    # the peer-store programs lose to it there
    assert 'b200_alltoall_direct_ll128_8 with LL128 protocol' in out              # 128-byte lines between LL and Simple
    root = ET.parse(os.environ['MSCCL_CONFIG']).getroot()
    assert root.tag == 'msccl_algos' and [e.get('proto') for e in root.findall('load')].count('LL128') == 1
    for entry in load_plan_table(os.environ['MSCCL_CONFIG']):
        assert validate(entry.algo) == [] and entry.algo.ngpus == 8


def test_registration_variants(tmp_path, capsys, clean_env):
    @register_synthesis_plan('allgather', 'fancy_machine', sizes=(0, '4MB'))
    def dummy_plan(machines):
        return '<algo/>'

    @register_synthesis_plan('allgather', ['m1', 'm2'], sizes=('1GiB', None))
    def dummy_plan2(machines):
        return '<algo/>'

    assert synthesis_plans[('allgather', 'm1')][-1][3] == (2 ** 30, float('inf'))
    assert synthesis_plans[('allgather', 'fancy_machine')][-1][3] == (0, 4000000)
    path = tmp_path / 'custom.xml'
    path.write_text('<algo/>')
    register_ef_file(str(path), 'broadcast', 'testbox', 3, sizes=('1KB', '2KB'), priority=2)
    register_ef_file('/nonexistent', 'broadcast', 'testbox', 3, sizes=('1KB', '4KB'), priority=1)
    msccl.init('testbox', 3, ('broadcast', (0, '8KB')))
    out = capsys.readouterr().out
    assert f'from 1 KB to 2 KB is load {path}' in out and 'from 2 KB to 4 KB is load /nonexistent' in out
    assert 'from 0 bytes to 1 KB. Falling back to NCCL baseline' in out
    assert 'testbox' in msccl.tabulate_plans()


def test_plan_listing_matches_reference_rows():
    rows = [[cell.strip() for cell in line.strip('|').split('|')] for line in msccl.tabulate_plans().splitlines()[2:]]
    for want in [['ndv2', 'alltoall', '>=2', '1 MB', 'infinity', 'Simple', '0', 'call synthesize_ndv2_relay_alltoall'],
                 ['ndv4', 'allreduce', '1', '512 bytes', '82.94 KB', 'LL', '0', 'run ndv4_allpairs_allreduce_config1'],
                 ['ndv4', 'allreduce', '1', '2.13 MB', '22.81 MB', 'LL128', '0', 'run ndv4_ring_allreduce_config2'],
                 ['ndv4', 'alltoall', '8,16,32,64', '1 MB', '32 MB', 'LL128', '0', 'run ndv4_alltoall_hierarchical_config1'],
                 ['ndv4', 'alltoall', '2,4', '1 KB', 'infinity', 'Simple', '0', 'run ndv4_alltoall_hierarchical_config2'],
                 ['ndv4', 'alltoall', '64', '32 MB', 'infinity', 'Simple', '0', 'run ndv4_alltoall_three_step']]:
        assert want in rows, want


@pytest.mark.parametrize('machine', ['b200x2', 'b200x4', 'b200x8'])
def test_every_registered_b200_plan_fits_the_executor(machine):
    # each registered plan compiles to tables within the executor's limits (threadblocks per rank, channels, steps)
    from msccl.autosynth.registry import synthesis_plans
    from msccl.language.ext_nvls import classify
    from msccl.runtime.plan import K_MAX_CHANNELS, K_MAX_TBS, compile_plan
    from msccl.xml import load_xml_file
    import msccl.autosynth.plans_b200  # noqa: F401  (registers on import)
    seen = 0
    for (coll, mtype), entries in list(synthesis_plans.items()):
        if mtype != machine:
            continue
        for entry in entries:
            algo = load_xml_file(entry[1](1))
            assert validate(algo) == [], algo.name
            if classify(algo) is not None:           # a program of in-switch steps runs on the native kernel of its shape
                seen += 1
                continue
            plan = compile_plan(algo, [0], 64 << 10)
            assert algo.nchannels <= K_MAX_CHANNELS and len(algo.gpus[0].tbs) <= K_MAX_TBS, algo.name
            assert plan.total_tbs() == len(algo.gpus[0].tbs)
            seen += 1
    assert seen >= 10


def test_b200_allreduce_ranges_follow_the_measurements(capsys, clean_env):
    # two GPUs: one-shot LL, then the two-channel ring in LL, LL128 and Simple; four GPUs: one-shot LL, then the in-switch program
    msccl.init('b200x2', 1, ('allreduce', (0, None)))
    out = capsys.readouterr().out
    assert 'from 0 bytes to 32 KB is run b200_allreduce_one_shot_2 with LL protocol' in out
    assert 'from 32 KB to 2 MB is run b200_allreduce_ring_2_ll with LL protocol' in out
    assert 'from 2 MB to 8 MB is run b200_allreduce_ring_2_ll128 with LL128 protocol' in out
    assert 'from 8 MB to infinity is run b200_allreduce_ring_2 with Simple protocol' in out
    entries = load_plan_table(os.environ['MSCCL_CONFIG'])
    ring = [e.algo for e in entries if e.algo.name.startswith('b200_allreduce_ring_2')]
    assert len(ring) == 3 and all(len(a.gpus[0].tbs) == 128 and a.nchannels == 128 for a in ring)
    msccl.init('b200x4', 1, ('allreduce', (0, None)))
    out = capsys.readouterr().out
    assert 'from 0 bytes to 64 KB is run b200_allreduce_one_shot_4 with LL protocol' in out
    assert 'b200_allreduce_in_switch_4' in out and 'two_shot' not in out
    from msccl.language.ext_nvls import classify
    kinds = [classify(e.algo) for e in load_plan_table(os.environ['MSCCL_CONFIG'])]
    assert kinds.count('allreduce') >= 1 and kinds[0] is None
