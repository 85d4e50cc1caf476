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


def _run_both(algo, chunk_elems, dtype, fifo_bytes):
    from msccl.runtime import Communicator, Executor
    comm = Communicator.emulated(algo.ngpus, fifo_bytes=fifo_bytes)
    try:
        ex = Executor(comm)
        plan = ex.compile(algo)
        gen = torch.Generator().manual_seed(42)
        host_in = [torch.randn(input_chunks_of(algo, r) * chunk_elems, generator=gen).to(dtype)
                   for r in range(algo.ngpus)]
        want = run_algorithm(algo, host_in, chunk_elems, dtype=dtype)
        dev_in, dev_out = {}, {}
        for r in range(algo.ngpus):
            if algo.inplace and algo.coll == 'allgather':
                full = torch.zeros(algo.gpus[r].o_chunks * chunk_elems, dtype=dtype, device='cuda')
                per = input_chunks_of(algo, r) * chunk_elems
                full[r * per:(r + 1) * per] = host_in[r].cuda()
                dev_in[r] = full
            else:
                dev_in[r] = host_in[r].cuda()
                if algo.gpus[r].o_chunks > 0 and not algo.inplace:
                    dev_out[r] = torch.zeros(algo.gpus[r].o_chunks * chunk_elems, dtype=dtype, device='cuda')
        got = ex.run(plan, dev_in, dev_out)
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
