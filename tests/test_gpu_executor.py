"""Interpreter kernel on one GPU: every rank of a program runs as threadblocks of one cooperative
launch (emulated communicator); results are compared bit for bit with the CPU interpreter."""
import pytest
import torch

from msccl.collectives import allgather, alltoall
from msccl.interp import input_chunks_of, run_algorithm
from msccl.language import MSCCLProgram, ThreadblockPolicy
from msccl.language.collectives import AllGather, AllReduce, AllToAll, ReduceScatter
from msccl.language.routines import allgather_ring_inplace
from msccl.ncclize import ncclize
from msccl.programs.allgather import allgather_direct, allgather_ring, reduce_scatter_direct
from msccl.programs.allreduce import allreduce_allpairs, allreduce_one_shot, allreduce_ring, allreduce_two_shot
from msccl.programs.alltoall import alltoall_direct
from msccl.strategies import solve_least_steps
from msccl.topologies import fully_connected, hub_and_spoke
from msccl.xml import load_xml

pytestmark = pytest.mark.gpu
MANUAL = ThreadblockPolicy.manual


def _program(name, coll, body, instances=1, **kw):
    prog = MSCCLProgram(name, fully_connected(coll.num_ranks), coll, instances, **kw)
    with prog:
        body()
    return load_xml(prog.generate_xml())


def _cases():
    return {
        'ring8_simple': lambda: _program('ring', AllReduce(8, 8, True), lambda: allreduce_ring(8, 4), 1,
                                         threadblock_policy=MANUAL),
        'ring8_ll_x2': lambda: _program('ring', AllReduce(8, 8, True), lambda: allreduce_ring(8, 4), 2,
                                        threadblock_policy=MANUAL, protocol='LL'),
        'ring4_ll128': lambda: _program('ring', AllReduce(4, 4, True), lambda: allreduce_ring(4, 2), 2,
                                        threadblock_policy=MANUAL, protocol='LL128'),
        'allpairs4_ll_nop': lambda: _program('allpairs', AllReduce(4, 16, True), lambda: allreduce_allpairs(4), 2,
                                             threadblock_policy=MANUAL, protocol='LL',
                                             interleaved_replication=False, dependence_nop=True),
        'one_shot8': lambda: _program('one_shot', AllReduce(8, 1, True), lambda: allreduce_one_shot(8), 1,
                                      threadblock_policy=MANUAL, protocol='LL'),
        'two_shot8_x2': lambda: _program('two_shot', AllReduce(8, 8, True), lambda: allreduce_two_shot(8), 2,
                                         threadblock_policy=MANUAL),
        'alltoall8': lambda: _program('a2a', AllToAll(8, 1, False), lambda: alltoall_direct(8), 1),
        'allgather8_direct': lambda: _program('ag', AllGather(8, 1, False), lambda: allgather_direct(8), 1),
        'allgather4_ring_inplace': lambda: _program('agr', AllGather(4, 1, True), lambda: allgather_ring_inplace(4)),
        'allgather8_ring': lambda: _program('agr', AllGather(8, 1, False), lambda: allgather_ring(8, 2)),
        'reduce_scatter4': lambda: _program('rs', ReduceScatter(4, 1, False), lambda: reduce_scatter_direct(4), 2),
        'synth_allgather_nvswitch': lambda: load_xml(ncclize(solve_least_steps(hub_and_spoke(8), allgather(8)))),
        'synth_alltoall_fc4': lambda: load_xml(ncclize(solve_least_steps(fully_connected(4), alltoall(4)))),
    }


def _run_both(algo, chunk_elems, dtype, fifo_bytes, direct='auto', misalign=0):
    from msccl.runtime import Communicator, Executor
    comm = Communicator.emulated(algo.ngpus, fifo_bytes=fifo_bytes)
    try:
        ex = Executor(comm)
        plan = ex.compile(algo)

        def place(t):
            """A device copy of ``t`` that starts ``misalign`` elements past a 16-byte boundary."""
            if not misalign:
                return t.cuda()
            holder = torch.zeros(t.numel() + misalign, dtype=t.dtype, device='cuda')
            holder[misalign:].copy_(t)
            return holder[misalign:]

        gen = torch.Generator().manual_seed(42)
        host_in = [torch.randn(input_chunks_of(algo, r) * chunk_elems, generator=gen).to(dtype)
                   for r in range(algo.ngpus)]
        want = run_algorithm(algo, host_in, chunk_elems, dtype=dtype)
        dev_in, dev_out = {}, {}
        for r in range(algo.ngpus):
            if algo.inplace and algo.coll == 'allgather':
                full = torch.zeros(algo.gpus[r].o_chunks * chunk_elems, dtype=dtype)
                per = input_chunks_of(algo, r) * chunk_elems
                full[r * per:(r + 1) * per] = host_in[r]
                dev_in[r] = place(full)
            else:
                dev_in[r] = place(host_in[r])
                if algo.gpus[r].o_chunks > 0 and not algo.inplace:
                    dev_out[r] = place(torch.zeros(algo.gpus[r].o_chunks * chunk_elems, dtype=dtype))
        got = ex.run(plan, dev_in, dev_out, direct=direct)
        ex.check()
        assert ex.launches == 1
        for r in range(algo.ngpus):
            g = got[r].cpu()
            w = want[r]
            n = min(g.numel(), w.numel())
            assert torch.equal(g[:n].view(torch.uint8), w[:n].view(torch.uint8)), f'rank {r} differs'
        plan.close()
    finally:
        comm.close()


@pytest.mark.parametrize('name', list(_cases()))
def test_programs_bit_exact_fp32(name):
    _run_both(_cases()[name](), 256, torch.float32, 8 << 20)


@pytest.mark.parametrize('name', ['ring8_simple', 'ring8_ll_x2', 'two_shot8_x2', 'allpairs4_ll_nop', 'alltoall8'])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
def test_low_precision_bit_exact(name, dtype):
    _run_both(_cases()[name](), 1024, dtype, 8 << 20)


@pytest.mark.parametrize('name', ['ring8_simple', 'ring8_ll_x2', 'two_shot8_x2', 'synth_allgather_nvswitch'])
def test_many_iterations_through_small_fifos(name):
    # 1 MiB of FIFO per rank forces tiles much smaller than a chunk: 40000-element chunks take
    # several iterations and the last tile is partial
    _run_both(_cases()[name](), 40000, torch.float32, 1 << 20)


@pytest.mark.parametrize('name', ['ring8_simple', 'two_shot8_x2', 'alltoall8', 'allgather8_ring', 'reduce_scatter4',
                                  'synth_allgather_nvswitch'])
def test_fifo_only_path_matches_too(name):
    # the same programs with stores into the receivers' buffers switched off: every tile takes the FIFO
    _run_both(_cases()[name](), 4096, torch.float32, 8 << 20, direct=False)


@pytest.mark.parametrize('name', ['ring4_ll128', 'ring8_ll128_x2', 'allgather8_ll128', 'allpairs4_ll128'])
@pytest.mark.parametrize('dtype,chunk', [(torch.float32, 256), (torch.bfloat16, 40000), (torch.float16, 1000)])
def test_ll128_lines(name, dtype, chunk):
    # 128-byte lines with 120 bytes of payload: chunks that do not fill their last line, several iterations
    cases = dict(_cases())
    cases['ring8_ll128_x2'] = lambda: _program('ring', AllReduce(8, 8, True), lambda: allreduce_ring(8, 4), 2,
                                               threadblock_policy=MANUAL, protocol='LL128')
    cases['allgather8_ll128'] = lambda: _program('ag', AllGather(8, 1, False), lambda: allgather_direct(8), 1,
                                                 protocol='LL128')
    cases['allpairs4_ll128'] = lambda: _program('allpairs', AllReduce(4, 16, True), lambda: allreduce_allpairs(4), 1,
                                                threadblock_policy=MANUAL, protocol='LL128')
    _run_both(cases[name](), chunk, dtype, 1 << 20)


@pytest.mark.parametrize('name', ['ring8_simple', 'ring8_ll_x2', 'ring4_ll128', 'two_shot8_x2', 'alltoall8',
                                  'synth_allgather_nvswitch', 'allpairs4_ll_nop'])
@pytest.mark.parametrize('dtype,chunk,misalign', [(torch.float16, 500, 0), (torch.bfloat16, 1001, 0), (torch.float32, 333, 0),
                                                  (torch.float32, 256, 1), (torch.bfloat16, 4099, 3)])
def test_chunks_that_are_not_multiples_of_16_bytes(name, dtype, chunk, misalign):
    # 500 fp16 elements = 1000 bytes per chunk (a synthesised all-gather cut into 3 chunks meets such sizes), odd
    # element counts, and buffers that do not start on a 16-byte boundary: element-wide accesses
    _run_both(_cases()[name](), chunk, dtype, 2 << 20, misalign=misalign)


def test_batched_reduces_match_separate_ones():
    # all-pairs all-reduce: each rank adds the n - 1 received copies into its chunk; the runs of `re` steps are
    # executed as one multi-input add and must round exactly like the separate passes of the CPU interpreter
    for dtype in (torch.float32, torch.bfloat16):
        for nop in (False, True):
            algo = _program('allpairs', AllReduce(8, 64, True), lambda: allreduce_allpairs(8), 1,
                            threadblock_policy=MANUAL, dependence_nop=nop)
            from msccl.runtime.plan import compile_plan
            assert compile_plan(algo, range(8), 64 << 10).batched_steps > 0
            _run_both(algo, 2048, dtype, 8 << 20)


def test_step_outside_the_declared_buffer_is_reported_not_executed():
    """The kernel checks every step against the buffer sizes the host declared.  Here the declared sizes are
    smaller than the tensors really are, so the "out-of-range" step still lies inside owned memory whatever the
    check does; the launch must stop with the bounds status and leave the output untouched."""
    from msccl.runtime import Communicator, Executor, ExecutorError
    algo = _program('ag', AllGather(4, 1, False), lambda: allgather_direct(4))
    comm = Communicator.emulated(4, fifo_bytes=1 << 20)
    try:
        comm.timeout_ns = int(1e9)        # the other ranks wait this long for the rank that stopped
        ex = Executor(comm)
        plan = ex.compile(algo)
        ins = {r: torch.full((256,), float(r + 1), device='cuda') for r in range(4)}
        outs = {r: torch.zeros(4 * 256, device='cuda') for r in range(4)}
        # rank 2 declares an output of three chunks; the program writes four
        declared = {r: (256, 4 * 256 if r != 2 else 3 * 256, 0) for r in range(4)}
        ex.run(plan, ins, outs, declared_elems=declared)
        with pytest.raises(ExecutorError):
            ex.check()
        status = comm.native.read_status(comm.sync_ptr(2))
        assert status[0] == 6 and status[1] == 2          # STATUS_BOUNDS, reported by rank 2
        assert torch.all(outs[2][3 * 256:] == 0)
        comm.reset_after_failure()
        comm.timeout_ns = int(20e9)
        out = ex.run(plan, ins, outs)
        ex.check()
        assert torch.equal(out[2].view(4, 256)[:, 0].cpu(), torch.tensor([1.0, 2.0, 3.0, 4.0]))
    finally:
        comm.close()


def test_step_trace_records_every_step():
    from msccl.runtime import Communicator, Executor
    algo = _cases()['ring8_simple']()
    comm = Communicator.emulated(8, fifo_bytes=4 << 20)
    try:
        ex = Executor(comm)
        plan = ex.compile(algo)
        ins = {r: torch.ones(8 * 65536, device='cuda') for r in range(8)}
        ex.run(plan, ins, trace=True)
        ex.check()
        rows = ex.last_trace()
        assert len(rows) == algo.num_steps()
        assert all(r['end_ns'] >= r['start_ns'] >= 0 and r['wait_ns'] >= 0 and r['move_ns'] >= 0 for r in rows)
        assert any(r['move_ns'] > 0 for r in rows) and max(r['end_ns'] for r in rows) < 5e9
        assert torch.all(ins[0] == 8.0)
    finally:
        comm.close()


def test_direct_stores_were_taken_and_counters_survive_mixed_launches():
    """Launches with and without direct stores alternate on one communicator: tile counters, opened-slot counters
    and the mode bits in the tail words must stay consistent."""
    from msccl.runtime import Communicator, Executor
    ag = _cases()['allgather8_ring']()
    ring = _cases()['ring8_simple']()
    comm = Communicator.emulated(8, fifo_bytes=4 << 20)
    try:
        ex = Executor(comm)
        p_ag, p_ring = ex.compile(ag), ex.compile(ring)
        assert p_ag.host.direct_steps > 0 and p_ring.host.direct_steps > 0
        for round_ in range(6):
            direct = round_ % 3 != 1
            ins = {r: torch.full((65536,), float(r + round_), device='cuda') for r in range(8)}
            out = ex.run(p_ag, ins, direct=direct)
            ex.check()
            assert ex.last_direct_mask == (7 if direct else 0)
            want = torch.arange(8, dtype=torch.float32) + round_
            assert all(torch.equal(out[r].view(8, -1)[:, 5].cpu(), want) for r in range(8))
            red = {r: torch.full((8 * 4096,), float(r + round_), device='cuda') for r in range(8)}
            ex.run(p_ring, red, direct=not direct)
            ex.check()
            assert all(torch.all(red[r] == float(sum(range(8)) + 8 * round_)) for r in range(8))
    finally:
        comm.close()


def test_repeated_launches_reuse_flags():
    from msccl.runtime import Communicator, Executor
    algo = _cases()['ring8_simple']()
    comm = Communicator.emulated(8, fifo_bytes=4 << 20)
    try:
        ex = Executor(comm)
        plan = ex.compile(algo)
        other = ex.compile(_cases()['two_shot8_x2']())
        for round_ in range(4):
            ins = {r: torch.full((8 * 512,), float(r + round_), device='cuda') for r in range(8)}
            out = ex.run(plan if round_ % 2 == 0 else other, ins)
            ex.check()
            expect = float(sum(r + round_ for r in range(8)))
            assert all(torch.all(out[r] == expect) for r in range(8))
    finally:
        comm.close()


def test_wait_runs_out_and_context_survives():
    """A receive that nothing feeds gives up after the (short) limit, reports where it waited, and
    the device stays usable."""
    from msccl.runtime import Communicator, Executor, ExecutorError
    from msccl.runtime.executor import DevicePlan
    import msccl.runtime.plan as plan_mod
    lonely = load_xml(
        '<algo name="lonely" proto="Simple" nchannels="1" nchunksperloop="1" ngpus="2" coll="custom" inplace="0">'
        '<gpu id="0" i_chunks="1" o_chunks="1" s_chunks="0"><tb id="0" send="-1" recv="1" chan="0">'
        '<step s="0" type="r" srcbuf="i" srcoff="0" dstbuf="o" dstoff="0" cnt="1" depid="-1" deps="-1" hasdep="0"/>'
        '</tb></gpu><gpu id="1" i_chunks="1" o_chunks="1" s_chunks="0"></gpu></algo>')
    comm = Communicator.emulated(2, fifo_bytes=1 << 20)
    try:
        comm.timeout_ns = int(0.2e9)
        ex = Executor(comm)
        real_compile = plan_mod.compile_plan
        import msccl.runtime.executor as exec_mod
        exec_mod.compile_plan = lambda algo, ranks, slot, check=True: real_compile(algo, ranks, slot, check=False)
        try:
            plan = DevicePlan(comm, lonely)
        finally:
            exec_mod.compile_plan = real_compile
        ins = {r: torch.ones(64, device='cuda') for r in range(2)}
        ex.run(plan, ins)
        with pytest.raises(ExecutorError) as err:
            ex.check()
        assert err.value.code == 2 and err.value.rank == 0 and err.value.aux0 == 1
        comm.reset_after_failure()
        comm.timeout_ns = int(20e9)
        good = ex.compile(_program('ag', AllGather(2, 1, False), lambda: allgather_direct(2)))
        out = ex.run(good, {0: torch.full((64,), 1.0, device='cuda'), 1: torch.full((64,), 2.0, device='cuda')})
        ex.check()
        assert torch.equal(out[0][:64], torch.full((64,), 1.0, device='cuda'))
        assert torch.equal(out[1][64:], torch.full((64,), 2.0, device='cuda'))
    finally:
        comm.close()
