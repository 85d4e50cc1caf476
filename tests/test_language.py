"""MSCCLang DSL and compiler behaviour (same expectations as the reference's tests/test_language.py)."""
import re

import pytest

from msccl.language import *  # noqa: F401,F403
from msccl.language.collectives import AllGather, AllReduce, AllToAll, Collective, ReduceScatter
from msccl.language.routines import allgather_ring_inplace, allreduce_ring_inplace
from msccl.topologies import fully_connected, line
from msccl.xml import load_xml, validate
from msccl.interp import run_reference_check


class Send(Collective):
    """chunk c of rank 0 must reach output[c] of rank 2."""
    def init_buffers(self):
        return [{Buffer.input: [Chunk(r, c, 2, c) if r == 0 else None for c in range(self.chunk_factor)],
                 Buffer.output: [None] * self.chunk_factor} for r in range(self.num_ranks)]

    def check(self, prog):
        out = prog.buffers[2][Buffer.output]
        return all(ch is not None and ch.origin_rank == 0 and ch.origin_index == 0 for ch in out)


class Reduce(Collective):
    """input[0] of rank 2 must hold the sum over all ranks."""
    def init_buffers(self):
        return [{Buffer.input: [Chunk(r, c, -1, c) for c in range(self.chunk_factor)],
                 Buffer.output: [None] * self.chunk_factor} for r in range(self.num_ranks)]

    def check(self, prog):
        want = ReduceChunk(-1, [Chunk(r, 0) for r in range(self.num_ranks)])
        got = prog.buffers[2][Buffer.input][0]
        return got is not None and got == want


def test_send_via_scratch():
    with MSCCLProgram('send', line(3), Send(3, 1, False), 1):
        chunk(0, Buffer.input, 0).copy(1, 'scratch').copy(2, Buffer.output, 0)
        assert Check()


def test_reduce_chain():
    with MSCCLProgram('reduce', line(3), Reduce(3, 1, True), 1):
        c10 = chunk(1, Buffer.input, 0).reduce(chunk(0, Buffer.input, 0))
        chunk(2, Buffer.input, 0).reduce(c10)
        assert Check()


def test_local_copy_and_reduce(capsys):
    with MSCCLProgram('cpy', fully_connected(3), Send(3, 1, False), 1):
        chunk(0, Buffer.input, 0).copy(2, 'scratch').copy(2, Buffer.output, 0)
        assert Check()
    with MSCCLProgram('local-reduce', line(3), Reduce(3, 1, True), 1):
        c = chunk(1, Buffer.input, 0).reduce(chunk(0, Buffer.input, 0))
        c = c.copy(2, 'scratch', 0)
        chunk(2, Buffer.input, 0).reduce(c)
        XML()
        assert Check()
    text = capsys.readouterr().out
    assert 'type="re"' in text and 'type="rrc"' in text


def test_no_link_is_rejected():
    with MSCCLProgram('nolink', line(3), Send(3, 1, False), 1):
        with pytest.raises(AssertionError):
            chunk(0, Buffer.input, 0).copy(2, Buffer.output, 0)


def test_scratch_index_defaults():
    with MSCCLProgram('test', fully_connected(3), AllReduce(3, 3, False), 1) as prog:
        chunk(0, Buffer.input, 0).copy(2, 'scratch', 2)
        assert chunk(2, 'scratch', 2).index == 2
        assert chunk(1, Buffer.input, 0).copy(2, 'scratch').index == 3
        assert chunk(2, 'scratch', 0) is None
        prog.generate_xml()


def test_program_order_dependency():
    prog = MSCCLProgram('test', fully_connected(2), AllReduce(2, 2, False), 1)
    with prog:
        chunk(1, Buffer.input, 0).copy(0, 'sc', 1)
        chunk(0, Buffer.input, 0).copy(1, Buffer.input, 0)     # must wait for the send above
    prog.lower()
    op = prog.instr_dag.operations[(1, Buffer.input, 0)]
    assert op.inst == Instruction.start
    assert op.next[0].inst == Instruction.send and op.next[0].next[0].inst == Instruction.recv


def test_builtin_collectives_two_ranks():
    fc = fully_connected(2)
    with MSCCLProgram('allgather', fc, AllGather(2, 1, True), 1):
        chunk(0, Buffer.input, 0).copy(1, Buffer.output, 0)
        chunk(1, Buffer.input, 0).copy(0, Buffer.output, 1)
        assert Check()
    with MSCCLProgram('reducescatter', fc, ReduceScatter(2, 1, True), 1):
        chunk(1, Buffer.input, 1).reduce(chunk(0, Buffer.input, 1))
        chunk(0, Buffer.input, 0).reduce(chunk(1, Buffer.input, 0))
        assert Check()
    with MSCCLProgram('alltoall', fc, AllToAll(2, 1, False), 1):
        for r in range(2):
            for d in range(2):
                chunk(r, Buffer.input, d).copy(d, Buffer.output, r)
        assert Check()
    with MSCCLProgram('allreduce', fc, AllReduce(2, 2, True), 1):
        chunk(1, Buffer.output, 0).reduce(chunk(0, Buffer.input, 0)).copy(0, Buffer.input, 0)
        chunk(0, Buffer.input, 1).reduce(chunk(1, Buffer.input, 1)).copy(1, Buffer.input, 1)
        assert Check()
    with MSCCLProgram('incomplete', fc, AllGather(2, 1, False), 1):
        chunk(0, Buffer.input, 0).copy(1, Buffer.output, 0)
        assert not Check()


def test_instruction_fusion():
    prog = MSCCLProgram('allreduce', fully_connected(3), AllReduce(3, 3, True), 1,
                        threadblock_policy=ThreadblockPolicy.manual)
    with prog:
        lane = dict(sendtb=0, recvtb=0, ch=0)
        c01 = chunk(1, Buffer.input, 0, 3).reduce(chunk(0, Buffer.input, 0, 3), **lane)
        c012 = chunk(2, Buffer.input, 0, 3).reduce(c01, **lane)
        c012.copy(0, Buffer.input, 0, **lane).copy(1, Buffer.input, 0, **lane)
        assert Check()
    gpus = prog.lower().gpus
    kinds = [[op.inst for op in g.threadblocks[0].ops] for g in gpus]
    assert kinds[0] == [Instruction.send, Instruction.recv_copy_send]
    assert kinds[1] == [Instruction.recv_reduce_send, Instruction.recv]
    assert kinds[2] == [Instruction.recv_reduce_copy_send]


def test_fusion_can_be_disabled():
    prog = MSCCLProgram('nofuse', fully_connected(3), AllGather(3, 1, True), 1, instr_fusion=False)
    with prog:
        allgather_ring_inplace(3)
    kinds = {op.inst for g in prog.lower().gpus for tb in g.threadblocks for op in tb.ops}
    assert kinds == {Instruction.send, Instruction.recv}


def _alltoall2(instances, interleaved=True):
    prog = MSCCLProgram('alltoall', fully_connected(2), AllToAll(2, 1, False), instances,
                        interleaved_replication=interleaved)
    with prog:
        for r in range(2):
            for d in range(2):
                chunk(r, Buffer.input, d).copy(d, Buffer.output, r)
    return prog


def test_replication():
    base, double = _alltoall2(1).lower(), _alltoall2(2).lower()
    for g1, g2 in zip(base.gpus, double.gpus):
        assert 2 * len(g1.threadblocks) == len(g2.threadblocks)
    inter = load_xml(_alltoall2(2, True).generate_xml())
    batch = load_xml(_alltoall2(2, False).generate_xml())
    recv = lambda a: sorted((st.srcoff, st.dstoff) for tb in a.gpus[0].tbs for st in tb.steps if st.type == 'r')
    assert recv(inter) == [(0, 2), (1, 3)]      # chunk k -> 2k+i
    assert recv(batch) == [(0, 1), (2, 3)]      # chunk k -> k + i*len(buffer)
    assert inter.nchannels == 2 and validate(inter) == [] and validate(batch) == []


def test_illegal_manual_threadblock():
    prog = MSCCLProgram('alltoall', fully_connected(3), AllToAll(3, 1, False), 1,
                        threadblock_policy=ThreadblockPolicy.manual)
    with prog:
        chunk(0, Buffer.input, 0).copy(1, Buffer.output, 0, sendtb=0, recvtb=1)
        chunk(0, Buffer.input, 1).copy(2, Buffer.output, 0, sendtb=0, recvtb=1)
        with pytest.raises(Exception, match='Illegal threadblock assignment'):
            prog.generate_xml()


def test_context_rules():
    prog = MSCCLProgram('a', fully_connected(2), AllGather(2, 1, True), 1)
    with pytest.raises(RuntimeError):
        chunk(0, Buffer.input, 0)
    with prog:
        with pytest.raises(RuntimeError):
            MSCCLProgram('b', fully_connected(2), AllGather(2, 1, True), 1).__enter__()
    with pytest.raises(AssertionError):
        MSCCLProgram('c', fully_connected(2), AllGather(2, 1, True), 1, protocol='Fast')


def test_split_and_group():
    with MSCCLProgram('sg', fully_connected(2), AllReduce(2, 4, True), 1):
        whole = chunk(0, Buffer.input, 0, 4)
        parts = whole.split(2)
        assert [(p.index, p.size) for p in parts] == [(0, 2), (2, 2)]
        again = parts[1].group(parts[0])
        assert (again.index, again.size) == (0, 4)
        with pytest.raises(AssertionError):
            whole.split(3)
        assert whole.get_origin_rank() == 0 and whole.get_origin_index(2) == 2


def test_routines_and_hierarchies():
    with MSCCLProgram('ag', fully_connected(4), AllGather(4, 1, True), 1):
        allgather_ring_inplace(4)
        assert Check()
    with MSCCLProgram('ag2', fully_connected(8), AllGather(8, 1, True), 1):
        allgather_ring_inplace(4, 0, 0)
        allgather_ring_inplace(4, 4, 4)
        for r in range(8):
            at = 0 if r < 4 else 4
            chunk(r, Buffer.output, at, 4).copy((r + 4) % 8, Buffer.output, at)
        assert Check()
    with MSCCLProgram('ar', fully_connected(4), AllReduce(4, 4, True), 1):
        allreduce_ring_inplace(4)
        assert Check()
    prog = MSCCLProgram('ar2', fully_connected(8), AllReduce(8, 8, True), 1)
    with prog:
        allreduce_ring_inplace(4, 0, 0)
        allreduce_ring_inplace(4, 0, 4, ch=1)
        allreduce_ring_inplace(4, 4, 4)
        allreduce_ring_inplace(4, 4, 0, ch=1)
        for r in range(8):
            peer, at = (r + 4) % 8, (0 if r < 4 else 4)
            c = chunk(peer, Buffer.output, at, 4)
            c.reduce(chunk(r, Buffer.output, at, 4))
            c.copy(r, Buffer.output, at)
        assert Check()
    algo = load_xml(prog.generate_xml())
    assert validate(algo) == [] and run_reference_check(algo, 2, race_check=True).startswith('pass')


def test_ring_xml_golden_shape():
    """4-rank in-place ring all-reduce, auto policy: one threadblock per GPU running
    s, rrs, rrs, rrcs, rcs, rcs, r with offsets rotated by rank."""
    prog = MSCCLProgram('allreduce_ring', fully_connected(4), AllReduce(4, 4, True), 1)
    with prog:
        allreduce_ring_inplace(4)
    text = prog.generate_xml()
    assert text.splitlines()[0] == ('<algo name="allreduce_ring" proto="Simple" nchannels="1" nchunksperloop="4" '
                                    'ngpus="4" coll="allreduce" inplace="1">')
    algo = load_xml(text)
    for r, gpu in enumerate(algo.gpus):
        assert (gpu.i_chunks, gpu.o_chunks, gpu.s_chunks) == (4, 0, 0) and len(gpu.tbs) == 1
        tb = gpu.tbs[0]
        assert (tb.send, tb.recv, tb.chan) == ((r + 1) % 4, (r - 1) % 4, 0)
        assert [st.type for st in tb.steps] == ['s', 'rrs', 'rrs', 'rrcs', 'rcs', 'rcs', 'r']
        assert [st.dstoff for st in tb.steps] == [r, (r - 1) % 4, (r - 2) % 4, (r + 1) % 4, r, (r - 1) % 4, (r - 2) % 4]
    assert re.search(r'<step s="0" type="s" srcbuf="i" srcoff="0" dstbuf="i" dstoff="0" cnt="1" depid="-1" '
                     r'deps="-1" hasdep="0" />', text)


def test_dependence_nop_hoists_reduce_waits():
    from msccl.programs.allreduce import allreduce_allpairs
    prog = MSCCLProgram('ap', fully_connected(4), AllReduce(4, 16, True), 1, protocol='LL',
                        threadblock_policy=ThreadblockPolicy.manual, dependence_nop=True)
    with prog:
        allreduce_allpairs(4)
        assert Check()
    algo = load_xml(prog.generate_xml())
    assert validate(algo) == []
    for gpu in algo.gpus:
        for tb in gpu.tbs:
            kinds = [st.type for st in tb.steps]
            if 're' in kinds:
                first = kinds.index('re')
                later = [st for st in tb.steps[first + 1:] if st.type == 're']
                assert all(st.depid == -1 for st in later)
    assert run_reference_check(algo, 2, race_check=True).startswith('pass')


def test_dot_export():
    prog = MSCCLProgram('dot', fully_connected(2), AllGather(2, 1, True), 1)
    with prog:
        allgather_ring_inplace(2)
    text = prog.to_dot()
    assert text.startswith('digraph mscclang {') and '->' in text


def test_compile_pass_times_are_recorded(monkeypatch, capsys):
    from msccl.language import MSCCLProgram
    from msccl.language.collectives import AllReduce
    from msccl.programs.allreduce import allreduce_ring
    from msccl.topologies import fully_connected
    monkeypatch.setenv('MSCCL_PROFILE', '1')
    prog = MSCCLProgram('timed_ring', fully_connected(4), AllReduce(4, 4, True), 2)
    with prog:
        allreduce_ring(4, 2)
    xml = prog.generate_xml()
    assert xml.startswith('<algo')
    assert list(prog.pass_times)[:3] == ['order edges', 'fuse instructions', 'chunk steps and priorities']
    assert 'write XML' in prog.pass_times and all(t >= 0 for t in prog.pass_times.values())
    err = capsys.readouterr().err
    assert 'MSCCL: compile passes of timed_ring' in err and 'assign threadblocks and channels' in err
    prog.generate_xml()                                     # cached text: no second report
    assert capsys.readouterr().err == ''


def test_in_switch_steps_in_the_dsl():
    # bar / mmar / mmb / mmr written through the DSL: Check(), XML, validator, interpreter, executor classification
    from msccl.interp import run_reference_check
    from msccl.language import Buffer, MSCCLProgram, chunk
    from msccl.language.collectives import AllGather, AllReduce, ReduceScatter
    from msccl.language.ext_nvls import (allreduce_nvls, classify, in_switch_allreduce, in_switch_broadcast,
                                         in_switch_reduce)
    from msccl.topologies import fully_connected
    from msccl.xml import load_xml
    from msccl.xml.validator import validate
    n = 4
    cases = ((AllReduce(n, n, True), lambda r: in_switch_allreduce(r, Buffer.input, r), 'allreduce'),
             (AllGather(n, 1, True), lambda r: in_switch_broadcast(r, Buffer.output, r), 'allgather'),
             (ReduceScatter(n, 1, False), lambda r: in_switch_reduce(r, Buffer.input, r, Buffer.output, 0), 'reduce_scatter'))
    for instances in (1, 3):
        for coll, step, kind in cases:
            prog = MSCCLProgram(f'{kind}_in_switch', fully_connected(n), coll, instances)
            with prog:
                assert not prog.check()                       # nothing has moved yet
                for r in range(n):
                    step(r)
                assert prog.check()
            algo = load_xml(prog.generate_xml())
            assert validate(algo) == [] and classify(algo) == kind
            assert run_reference_check(algo, race_check=True) == 'pass (race-free)'
            assert [len(g.tbs) for g in algo.gpus] == [instances] * n
    # the DSL program and the ready-made builder describe the same steps
    prog = MSCCLProgram('x', fully_connected(n), AllReduce(n, n, True), 2)
    with prog:
        for r in range(n):
            in_switch_allreduce(r, Buffer.input, r)
    mine, ready = load_xml(prog.generate_xml()), load_xml(allreduce_nvls(n, 2))
    shape = lambda a: [[(tb.chan, [(st.type, st.srcbuf, st.srcoff, st.dstbuf, st.dstoff) for st in tb.steps]) for tb in g.tbs]  # noqa: E731
                       for g in a.gpus]
    assert shape(mine) == shape(ready)
    # no mixing with classic steps, in either order
    prog = MSCCLProgram('mixed', fully_connected(n), AllReduce(n, n, True), 1)
    with prog:
        in_switch_allreduce(0, Buffer.input, 0)
        with pytest.raises(RuntimeError):
            chunk(0, Buffer.input, 1).copy(1, Buffer.input, 1)
    prog = MSCCLProgram('mixed2', fully_connected(n), AllReduce(n, n, True), 1)
    with prog:
        chunk(1, Buffer.input, 0).reduce(chunk(0, Buffer.input, 0))
        with pytest.raises(RuntimeError):
            in_switch_allreduce(0, Buffer.input, 1)
