"""Host-side analyses of ``msccl.runtime.plan.compile_plan`` (direct stores, slot opening, batched reduces,
tile geometry and limits) and the table checks of the allocation-free entry point.  Nothing here needs a GPU:
the entry point rejects bad tables before it makes its first CUDA call."""
import ctypes
import struct

import pytest

from msccl.language import MSCCLProgram, ThreadblockPolicy
from msccl.language.collectives import AllGather, AllReduce, AllToAll
from msccl.programs.allgather import allgather_direct, allgather_ring
from msccl.programs.allreduce import allreduce_allpairs, allreduce_ring, allreduce_two_shot
from msccl.programs.alltoall import alltoall_direct
from msccl.runtime import plan as P
from msccl.topologies import fully_connected
from msccl.xml import load_xml

MANUAL = ThreadblockPolicy.manual


def _program(name, coll, body, instances=1, **kw):
    prog = MSCCLProgram(name, fully_connected(coll.num_ranks), coll, instances, **kw)
    with prog:
        body()
    return load_xml(prog.generate_xml())


def _steps(plan):
    return [P._STEP.unpack_from(plan.step_bytes, i * 32) for i in range(len(plan.step_bytes) // 32)]


def _tbs(plan):
    return [P._TB.unpack_from(plan.tb_bytes, i * 64) for i in range(len(plan.tb_bytes) // 64)]


def test_all_gather_receives_are_direct_and_open_from_the_start():
    algo = _program('ag', AllGather(4, 1, False), lambda: allgather_direct(4))
    plan = P.compile_plan(algo, range(4), 64 << 10)
    steps = _steps(plan)
    sends = [s for s in steps if s[0] == P.STEP_CODES['s']]
    recvs = [s for s in steps if s[0] == P.STEP_CODES['r']]
    assert sends and all(s[9] & P.SF_DIRECT_SEND for s in sends)
    assert recvs and all(s[9] & P.SF_DIRECT_RECV for s in recvs)
    # a send names the receiver's slot: output buffer, chunk = the sender's rank
    tbs = _tbs(plan)
    for tb in tbs:
        rank, nsteps, begin = tb[0], tb[5], tb[6]
        for s in steps[begin:begin + nsteps]:
            if s[0] == P.STEP_CODES['s']:
                assert s[10] == P.BUF_CODES['o'] and s[13] == rank
    # every receiving threadblock opens all of its slots when the kernel starts
    receiving = [tb for tb in tbs if tb[3] >= 0]
    assert receiving and all(tb[12] == tb[14] > 0 and tb[13] == 1 << P.BUF_CODES['o'] for tb in receiving)
    assert plan.eager_tbs == len(receiving) and plan.direct_bufs[0] == {'o'}
    # the FIFO-only compilation carries no flags at all
    plain = P.compile_plan(algo, range(4), 64 << 10, direct=False)
    assert all(s[9] == 0 for s in _steps(plain)) and all(tb[12] == 0 for tb in _tbs(plain))


def test_ring_all_reduce_opens_gather_slots_after_their_last_use():
    n = 4
    algo = _program('ring', AllReduce(n, n, True), lambda: allreduce_ring(n, 1), 1, threadblock_policy=MANUAL)
    plan = P.compile_plan(algo, range(n), 64 << 10)
    steps, tbs = _steps(plan), _tbs(plan)
    assert plan.eager_tbs == 0 and plan.direct_steps > 0
    for tb in tbs:
        nsteps, begin, at_start, nrecv = tb[5], tb[6], tb[12], tb[14]
        mine = steps[begin:begin + nsteps]
        # every receive is opened exactly once per iteration
        assert at_start + sum(s[14] + s[15] for s in mine) == nrecv
        # reducing receives (rrs / rrc / rrcs) never take their data in place
        for s in mine:
            if s[0] in (P.STEP_CODES['rrs'], P.STEP_CODES['rrc'], P.STEP_CODES['rrcs']):
                assert not s[9] & P.SF_DIRECT_RECV
    # the slots the gather phase receives into were read or written by the reduce phase of the same threadblock:
    # they open after a step, not at the start of the iteration
    assert any(s[14] > 0 for s in steps)


def test_all_pairs_reduces_are_batched_and_sources_keep_their_order():
    algo = _program('allpairs', AllReduce(4, 16, True), lambda: allreduce_allpairs(4), 1, threadblock_policy=MANUAL,
                    protocol='LL', dependence_nop=True)
    plan = P.compile_plan(algo, range(4), 64 << 10)
    assert plan.batched_steps > 0
    steps, tbs = _steps(plan), _tbs(plan)
    heads = 0
    for tb in tbs:
        nsteps, begin = tb[5], tb[6]
        mine = steps[begin:begin + nsteps]
        for i, s in enumerate(mine):
            if s[11] > 1:
                heads += 1
                run = mine[i:i + s[11]]
                res = [r for r in run if r[0] == P.STEP_CODES['re']]
                assert run[0][0] == P.STEP_CODES['re'] and run[-1][0] == P.STEP_CODES['re']
                assert 2 <= len(res) <= P.K_MAX_BATCH
                assert all(r[0] in (P.STEP_CODES['re'], P.STEP_CODES['nop']) for r in run)
                assert all((r[2], r[7], r[8]) == (s[2], s[7], s[8]) for r in res)       # one destination
    assert heads > 0
    assert P.compile_plan(algo, range(4), 64 << 10, batch=False).batched_steps == 0


def test_tile_geometry_by_protocol_and_width():
    algo = _program('a2a', AllToAll(4, 1, False), lambda: alltoall_direct(4))
    plan = P.compile_plan(algo, range(4), 64 << 10)
    slot = 64 << 10
    assert P.access_width(1024, 2) == 16 and P.access_width(500, 2) == 2 and P.access_width(1024, 4, [8]) == 4
    tile, its = P.tile_geometry(plan, 1 << 20, 2, slot, 16, proto=1)              # LL: half of the slot is payload
    assert tile == slot // 2 // 2 and its == -(-(1 << 20) // tile)
    tile, _ = P.tile_geometry(plan, 1 << 20, 2, slot, 16, proto=2)                # LL128: 120 of 128 bytes
    assert tile == (slot // 128 * 15 // 2) * 8
    tile, _ = P.tile_geometry(plan, 1 << 20, 2, slot, 2, proto=1)                 # one bf16 per 8-byte packet
    assert tile == slot // 8
    tile, _ = P.tile_geometry(plan, 999, 2, slot, 2, proto=0)                     # odd chunk: the whole chunk at once
    assert tile == 999
    with pytest.raises(P.PlanError):
        P.tile_geometry(plan, 1 << 20, 2, slot, 2, proto=2)                       # LL128 needs 16-byte chunks
    with pytest.raises(P.PlanError):
        P.tile_geometry(plan, 1 << 34, 2, 1024, 16, proto=1)                      # 2^20 iterations or more


def test_a_threadblock_with_too_many_steps_is_rejected():
    algo = _program('ag', AllGather(2, 1, False), lambda: allgather_direct(2))
    tb = algo.gpus[0].tbs[0]
    first = tb.steps[0]
    import copy
    tb.steps = [copy.copy(first) for _ in range(P.K_MAX_STEPS_PER_TB + 1)]
    with pytest.raises(P.PlanError, match='steps'):
        P.compile_plan(algo, range(2), 64 << 10, check=False)


# ---- table checks of the allocation-free entry point -------------------------------------------------------
def _library():
    from msccl.runtime.build import module_path
    lib = ctypes.CDLL(module_path())
    lib.msccl_exec_noalloc.restype = ctypes.c_int
    lib.msccl_exec_noalloc.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_int,
                                       ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
                                       ctypes.POINTER(ctypes.c_int), ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int,
                                       ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.msccl_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _call(lib, tb_bytes, step_bytes, n, scratch, chunk=64, slot=16 << 10, max_cnt=1, dtype=0, proto=0):
    # the buffer addresses are never dereferenced: every case below is turned away by the host-side checks
    ins = (ctypes.c_void_p * n)(*[0x10000 * (r + 1) for r in range(n)])
    outs = (ctypes.c_void_p * n)(*[0x900000 + 0x10000 * r for r in range(n)])
    sc = (ctypes.c_int * n)(*scratch)
    return lib.msccl_exec_noalloc(tb_bytes, len(tb_bytes) // 64, step_bytes, len(step_bytes) // 32, n, ins, outs, sc,
                                  chunk, slot, max_cnt, dtype, proto, None)


def _mutated(blob, fmt, index, field, value):
    rec = list(fmt.unpack_from(blob, index * fmt.size))
    rec[field] = value
    return blob[:index * fmt.size] + fmt.pack(*rec) + blob[(index + 1) * fmt.size:]


def test_noalloc_entry_point_rejects_inconsistent_tables():
    lib = _library()
    n = 4
    algo = _program('two_shot', AllReduce(n, n, True), lambda: allreduce_two_shot(n), 1, threadblock_policy=MANUAL)
    plan = P.compile_plan(algo, range(n), 16 << 10)
    scratch = [plan.extents[r]['s'] for r in range(n)]
    tbs, steps = plan.tb_bytes, plan.step_bytes
    ntb = len(tbs) // 64
    BAD, LARGE = 2, 1
    cases = {
        'step range past the table': (_mutated(tbs, P._TB, ntb - 1, 5, 10_000), steps, BAD),
        'connection id': (_mutated(tbs, P._TB, 0, 8 if P._TB.unpack_from(tbs, 0)[2] >= 0 else 9, 1023), steps, BAD),
        'rank': (_mutated(tbs, P._TB, 0, 0, 7), steps, BAD),
        'dependency outside the rank': (tbs, _mutated(steps, P._STEP, 0, 4, 127), BAD),
        'count above max_cnt': (tbs, _mutated(steps, P._STEP, 0, 8, 50), BAD),
        'buffer id': (tbs, _mutated(steps, P._STEP, 0, 2, 3), BAD),
        'fifo offset': (_mutated(tbs, P._TB, 0, 10, 1 << 30), _mutated(steps, P._STEP, 0, 0, 0), LARGE),
    }
    for name, (t, s, want) in cases.items():
        got = _call(lib, t, s, n, scratch)
        assert got in (want, BAD, LARGE) and got != 0, name
        assert lib.msccl_noalloc_last_error() != b'', name
    # scratch offsets beyond what the caller declared
    assert _call(lib, tbs, steps, n, [0] * n) == BAD and b'scratch' in lib.msccl_noalloc_last_error()
    # more threadblocks per rank than the progress array of a rank has entries
    one = P._TB.unpack_from(tbs, 0)
    flood = b''.join(P._TB.pack(0, i, -1, -1, 0, 0, 0, 140, -1, -1, 0, 0, 0, 0, 0, 0) for i in range(140))
    assert one is not None and _call(lib, flood, b'', 1, [0]) == LARGE
    # unknown protocol, slot size that is not a multiple of 1 KiB, LL128 with chunks that are not 16-byte multiples
    assert _call(lib, tbs, steps, n, scratch, proto=5) == BAD
    assert _call(lib, tbs, steps, n, scratch, slot=1000) == BAD
    assert _call(lib, tbs, steps, n, scratch, chunk=3, proto=2) == BAD
