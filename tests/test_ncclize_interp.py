"""ncclize lowering, XML loader/validator and the CPU interpreter (incl. the 8x1 MiB ring config)."""
import pytest
import torch

from msccl.collectives import allgather, alltoall, reduce_scatter
from msccl.instance import Instance
from msccl.interp import (DeadlockError, Interpreter, RaceError, run_algorithm, run_reference_check)
from msccl.language import Buffer, MSCCLProgram, ThreadblockPolicy, chunk
from msccl.language.collectives import AllGather, AllReduce
from msccl.ncclize import ChannelPolicy, ncclize
from msccl.path_encoding import PathEncoding
from msccl.programs.allreduce import allreduce_ring
from msccl.strategies import solve_least_steps
from msccl.topologies import dgx1, fully_connected, hub_and_spoke, ring, star
from msccl.xml import load_xml, validate
from msccl.xml.validator import find_deadlock


def test_ncclize_ring_allgather_structure():
    algo = PathEncoding(ring(4), allgather(4)).solve(Instance(2))
    text = ncclize(algo)
    assert text.splitlines()[0] == ('<algo name="Allgather(n=4)-Ring(n=4)-steps=2" proto="Simple" nchannels="1" '
                                    'ngpus="4" inplace="0" coll="allgather" nchunksperloop="4">')
    ir = load_xml(text)
    assert validate(ir) == []
    for gpu in ir.gpus:
        assert (gpu.i_chunks, gpu.o_chunks, gpu.s_chunks) == (1, 4, 0)
        last = gpu.tbs[-1]
        assert (last.send, last.recv) == (-1, -1) and [st.type for st in last.steps] == ['cpy']
    assert run_reference_check(ir, 3, race_check=True).startswith('pass')


@pytest.mark.parametrize('options', [
    {}, {'channel_policy': ChannelPolicy.One}, {'merge_contiguous': False}, {'instances': 3},
    {'greedy_scratch_sorting': True}, {'use_scratch': False}, {'pretty_print': False}])
def test_ncclize_option_matrix_executes(options):
    algo = PathEncoding(star(4), alltoall(4)).solve(Instance(2, extra_rounds=2))
    ir = load_xml(ncclize(algo, **options))
    if options.get('use_scratch', True):
        assert validate(ir) == []
        assert run_reference_check(ir, 2, race_check=True).startswith('pass')
    else:
        assert ir.gpus[0].s_chunks > 0      # scratch is addressed behind the output buffer


def test_ncclize_scratch_remap_and_errors():
    algo = PathEncoding(star(4), alltoall(4)).solve(Instance(2, extra_rounds=2))
    plain = load_xml(ncclize(algo))
    remapped = load_xml(ncclize(algo, remap_scratch=True))
    assert max(g.s_chunks for g in remapped.gpus) <= max(g.s_chunks for g in plain.gpus)
    assert run_reference_check(remapped, 2).startswith('pass')
    with pytest.raises(ValueError):
        ncclize(PathEncoding(ring(4), allgather(4)).solve(Instance(2)).__class__(
            'p', allgather(4), ring(4), Instance(2, pipeline=1), []))


@pytest.mark.parametrize('make,topo', [(allgather, dgx1()), (reduce_scatter, dgx1()),
                                       (allgather, hub_and_spoke(8)), (alltoall, fully_connected(4))])
def test_synthesized_algorithms_execute(make, topo):
    algo = solve_least_steps(topo, make(topo.num_nodes()))
    ir = load_xml(ncclize(algo, instances=2))
    assert validate(ir) == []
    assert run_reference_check(ir, 2, race_check=True).startswith('pass')


def test_composed_allreduce_executes():
    from msccl.composers import compose_allreduce
    rs = solve_least_steps(dgx1(), reduce_scatter(8))
    ag = solve_least_steps(dgx1(), allgather(8))
    ir = load_xml(ncclize(compose_allreduce(rs, ag)))
    assert validate(ir) == [] and ir.coll == 'allreduce'
    assert run_reference_check(ir, 2, race_check=True).startswith('pass')


def test_ring_allreduce_8x1MiB_bit_exact():
    """8 ranks, 8 chunks, 4 channels, manual schedule, fp32 N(0,1), 1 MiB per rank; compared bit
    for bit with sums done in ring order: chunk i is accumulated starting at rank i."""
    n, elems = 8, 262144
    prog = MSCCLProgram('allreduce_ring', fully_connected(n), AllReduce(n, n, True), 1,
                        threadblock_policy=ThreadblockPolicy.manual)
    with prog:
        allreduce_ring(n, 4)
    ir = load_xml(prog.generate_xml())
    assert validate(ir) == [] and ir.nchannels == 4 and ir.nchunksperloop == 8
    assert all(len(g.tbs) == 4 for g in ir.gpus)
    assert {st.type for g in ir.gpus for tb in g.tbs for st in tb.steps} == {'s', 'rrs', 'rrcs', 'rcs', 'r'}
    gen = torch.Generator().manual_seed(1234)
    inputs = [torch.randn(elems, generator=gen) for _ in range(n)]
    outputs = run_algorithm(ir, inputs, elems // n)
    per = elems // n
    want = torch.empty(elems)
    for i in range(n):
        acc = inputs[i][i * per:(i + 1) * per].clone()
        for hop in range(1, n):
            acc = inputs[(i + hop) % n][i * per:(i + 1) * per] + acc
        want[i * per:(i + 1) * per] = acc
    for r in range(n):
        assert torch.equal(outputs[r], want)
    assert torch.allclose(want.double(), sum(t.double() for t in inputs), atol=1e-5)


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
def test_low_precision_sums_round_per_addition(dtype):
    prog = MSCCLProgram('ring', fully_connected(4), AllReduce(4, 4, True), 1)
    with prog:
        allreduce_ring(4, 1)
    ir = load_xml(prog.generate_xml())
    gen = torch.Generator().manual_seed(7)
    inputs = [torch.randn(64, generator=gen).to(dtype) for _ in range(4)]
    out = run_algorithm(ir, inputs, 16, dtype=dtype)
    acc = inputs[0][:16]
    for hop in range(1, 4):
        acc = (inputs[hop][:16].float() + acc.float()).to(dtype)
    assert torch.equal(out[0][:16], acc) and all(torch.equal(out[0], o) for o in out)


def _xml(tbs):
    body = ''.join(f'<gpu id="{r}" i_chunks="1" o_chunks="1" s_chunks="0">{t}</gpu>' for r, t in enumerate(tbs))
    return f'<algo name="t" proto="Simple" nchannels="1" nchunksperloop="1" ngpus="{len(tbs)}" coll="custom" inplace="0">{body}</algo>'


def _step(s, kind, depid=-1, deps=-1, hasdep=0, src='i', dst='o'):
    return (f'<step s="{s}" type="{kind}" srcbuf="{src}" srcoff="0" dstbuf="{dst}" dstoff="0" cnt="1" '
            f'depid="{depid}" deps="{deps}" hasdep="{hasdep}"/>')


def test_validator_and_deadlock_detection():
    # each GPU receives before it sends: a cross-rank cycle
    cyc = _xml([f'<tb id="0" send="{1 - r}" recv="{1 - r}" chan="0">{_step(0, "r")}{_step(1, "s")}</tb>'
                for r in range(2)])
    ir = load_xml(cyc)
    assert any('deadlock' in p for p in validate(ir))
    with pytest.raises(DeadlockError):
        Interpreter(ir, 1).run()
    # unmatched send
    lone = load_xml(_xml(['<tb id="0" send="1" recv="-1" chan="0">' + _step(0, 's') + '</tb>', '']))
    assert any('sends but 0 receives' in p for p in validate(lone))
    # out of bounds and bad dependency
    bad = _xml(['<tb id="0" send="-1" recv="-1" chan="0">'
                '<step s="0" type="cpy" srcbuf="i" srcoff="3" dstbuf="o" dstoff="0" cnt="1" depid="5" deps="0" hasdep="0"/>'
                '</tb>'])
    problems = validate(load_xml(bad))
    assert any('exceeds' in p for p in problems) and any('depid 5' in p for p in problems)
    assert any('unknown protocol' in p for p in validate(load_xml(_xml(['']).replace('Simple', 'Turbo'))))
    # a bounded FIFO turns "send twice, then the peer receives" into a deadlock only at depth 1
    two = _xml(['<tb id="0" send="1" recv="1" chan="0">' + _step(0, 's') + _step(1, 's') + _step(2, 'r') + '</tb>',
                '<tb id="0" send="0" recv="0" chan="0">' + _step(0, 's') + _step(1, 's') + _step(2, 'r') + _step(3, 'r') + '</tb>'])
    ir2 = load_xml(two.replace('</tb></gpu><gpu id="1"', _step(3, 'r') + '</tb></gpu><gpu id="1"'))
    assert find_deadlock(ir2) == [] and find_deadlock(ir2, fifo_depth=1) != []


def test_race_detection_catches_missing_dependency():
    prog = MSCCLProgram('racy', fully_connected(2), AllGather(2, 1, False), 1,
                        threadblock_policy=ThreadblockPolicy.manual)
    with prog:
        c = chunk(0, Buffer.input, 0).copy(1, 'tmp', 0, sendtb=0, recvtb=0, ch=0)
        c.copy(1, Buffer.output, 0, sendtb=1, ch=0)
        chunk(0, Buffer.input, 0).copy(0, Buffer.output, 0, sendtb=1)
        chunk(1, Buffer.input, 0).copy(1, Buffer.output, 1, sendtb=1)
        chunk(1, Buffer.input, 0).copy(0, Buffer.output, 1, sendtb=2, recvtb=2, ch=1)
    ir = load_xml(prog.generate_xml())
    assert run_reference_check(ir, 2, race_check=True).startswith('pass')
    for tb in ir.gpus[1].tbs:                  # drop the wait of the local copy on the receive
        for st in tb.steps:
            if st.type == 'cpy' and st.srcbuf == 's':
                st.depid, st.deps = -1, -1
    with pytest.raises((RaceError, AssertionError)):
        it = Interpreter(ir, 2, race_check=True)
        it.set_input(0, torch.ones(2))
        it.set_input(1, torch.ones(2))
        it.run()
        raise AssertionError('schedule happened to be ordered')


def test_copy_threadblocks_split_local_copies():
    # the local copies of a rank spread over several threadblocks: same result, one copy step per block
    from msccl.collectives import allgather
    from msccl.instance import Instance
    from msccl.interp import run_reference_check
    from msccl.ncclize import ncclize
    from msccl.path_encoding import PathEncoding
    from msccl.topologies import fully_connected
    from msccl.xml import load_xml
    topo = fully_connected(4)
    algo = PathEncoding(topo, allgather(4)).solve(Instance(1))
    assert algo is not None
    one = load_xml(ncclize(algo, instances=4))
    many = load_xml(ncclize(algo, instances=4, copy_threadblocks=4))
    assert run_reference_check(one) == 'pass' and run_reference_check(many) == 'pass'

    def copy_blocks(ir):
        return [sum(1 for tb in g.tbs if any(st.type == 'cpy' for st in tb.steps)) for g in ir.gpus]
    assert copy_blocks(one) == [1] * 4
    assert copy_blocks(many) == [4] * 4
    for g in many.gpus:
        cnts = sorted(st.cnt for tb in g.tbs for st in tb.steps if st.type == 'cpy')
        assert cnts == [1, 1, 1, 1]


@pytest.mark.parametrize('ranks,instances', [(2, 1), (4, 2), (8, 4)])
def test_in_switch_extension_programs(ranks, instances):
    # bar / mmar / mmb / mmr: validated, executed race-free by the CPU interpreter, recognised by the executor
    from msccl.language.ext_nvls import allgather_nvls, allreduce_nvls, classify, reduce_scatter_nvls
    from msccl.xml import load_xml
    from msccl.xml.validator import validate
    for build, coll in ((allreduce_nvls, 'allreduce'), (allgather_nvls, 'allgather'), (reduce_scatter_nvls, 'reduce_scatter')):
        algo = load_xml(build(ranks, instances))
        assert validate(algo) == []
        assert classify(algo) == coll
        assert run_reference_check(algo, race_check=True).startswith('pass')
        assert sum(st.type == 'bar' for g in algo.gpus for tb in g.tbs for st in tb.steps) == 2 * ranks * instances


def test_in_switch_sum_is_rounded_once_and_barriers_are_checked():
    from msccl.language.ext_nvls import allreduce_nvls, classify
    from msccl.xml import load_xml
    from msccl.xml.validator import find_deadlock, validate
    text = allreduce_nvls(4)
    algo = load_xml(text)
    # bf16: 256 + 1 + 1 + 1 is 259 -> 260 when summed in fp32 and rounded once; rounding after every addition gives 256
    inputs = [torch.full((4 * 8,), v, dtype=torch.bfloat16) for v in (256.0, 1.0, 1.0, 1.0)]
    out = run_algorithm(algo, inputs, 8, dtype=torch.bfloat16)
    assert all(torch.all(o == 260.0) for o in out)
    # a GPU that skips its first barrier: counts differ, and the others can never pass
    broken = text.replace('<step s="0" type="bar"', '<step s="0" type="nop"', 1)
    bad = load_xml(broken)
    assert any('barrier counts differ' in p for p in validate(bad))
    assert find_deadlock(bad)
    assert classify(bad) is None
    # a classic program is not mistaken for an in-switch one
    ring = MSCCLProgram('ring', fully_connected(4), AllReduce(4, 4, True), 1)
    with ring:
        allreduce_ring(4, 1)
    assert classify(load_xml(ring.generate_xml())) is None


def test_program_summary_and_cost_estimate():
    from msccl.xml.analysis import estimate_us, summarize
    n = 8
    prog = MSCCLProgram('ring', fully_connected(n), AllReduce(n, n, True), 1, threadblock_policy=ThreadblockPolicy.manual)
    with prog:
        allreduce_ring(n, 1)
    algo = load_xml(prog.generate_xml())
    s = summarize(algo)
    # a ring all-reduce passes every chunk through 2 (n - 1) hops, one more step for the first local read
    assert s.complete and 2 * (n - 1) <= s.depth <= 2 * (n - 1) + 1
    assert set(s.sent_chunks.values()) == {2 * (n - 1)} and set(s.sending_tbs.values()) == {1}
    small, large = estimate_us(algo, 8 << 10, summary=s), estimate_us(algo, 1 << 30, summary=s)
    assert abs(small - (11.0 + s.depth * 5.0)) < 1.0               # launch and per-step latency dominate
    bytes_out = 2 * (n - 1) / n * (1 << 30)
    assert abs(large - (11.0 + s.depth * 5.0 + bytes_out / 50e3)) < 1.0   # one sending threadblock at 50 GB/s
    # LL128 carries 120 bytes of payload per 128-byte line, LL 8 per 16
    ll128 = load_xml(prog.generate_xml().replace('proto="Simple"', 'proto="LL128"'))
    assert abs(estimate_us(ll128, 1 << 30) - (11.0 + s.depth * 3.0 + bytes_out * (128 / 120) / 50e3)) < 1.0
    # more instances: same depth, proportionally more sending threadblocks
    prog4 = MSCCLProgram('ring4', fully_connected(n), AllReduce(n, n, True), 4, threadblock_policy=ThreadblockPolicy.manual)
    with prog4:
        allreduce_ring(n, 1)
    s4 = summarize(load_xml(prog4.generate_xml()))
    assert s4.depth == s.depth and set(s4.sending_tbs.values()) == {4}
    # a program that cannot finish is reported as incomplete
    from msccl.language.ext_nvls import allreduce_nvls
    stuck = load_xml(allreduce_nvls(4).replace('<step s="0" type="bar"', '<step s="0" type="nop"', 1))
    assert not summarize(stuck).complete
