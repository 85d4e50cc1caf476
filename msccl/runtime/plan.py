"""Compile a validated MSCCL-IR program into the flat device arrays the executor kernel reads.

Layout contract: ``csrc/msccl_device.h`` (``DevTb`` 48 bytes, ``DevStep`` 20 bytes).  Aliases of
the in-place collectives are resolved here, so the kernel sees plain (buffer, chunk) pairs.
"""
import struct
from dataclasses import dataclass, field
from typing import Dict, List

from msccl.xml.loader import AlgoIR
from msccl.xml.validator import validate

STEP_CODES = {'nop': 0, 's': 1, 'r': 2, 'rcs': 3, 'rrs': 4, 'rrc': 5, 'rrcs': 6, 'cpy': 7, 're': 8}
BUF_CODES = {'i': 0, 'o': 1, 's': 2}
PROTO_CODES = {'Simple': 0, 'LL': 1, 'LL128': 1}      # LL128 programs run on the LL packet path
K_MAX_RANKS = 16
K_MAX_CHANNELS = 64
K_MAX_TBS = 128
K_FIFO_SLOTS = 4
_TB = struct.Struct('<4h4i2i2q')
_STEP = struct.Struct('<4B2h3i')


class PlanError(ValueError):
    pass


@dataclass
class HostPlan:
    """Host-side description of a compiled program for a set of local ranks."""
    algo: AlgoIR
    local_ranks: List[int]
    tb_bytes: bytes = b''
    step_bytes: bytes = b''
    first_tb: Dict[int, int] = field(default_factory=dict)     # rank -> index of its first tb
    num_tbs: Dict[int, int] = field(default_factory=dict)
    in_conns: int = 0              # most incoming connections of any rank
    max_cnt: int = 1
    proto: int = 0
    extents: Dict[int, Dict[str, int]] = field(default_factory=dict)   # rank -> physical buffer -> chunks used

    def total_tbs(self):
        return sum(self.num_tbs[r] for r in self.local_ranks)


def fifo_index_tables(algo: AlgoIR):
    """For every rank, the incoming connections (src, chan) in a fixed order.  The position of a
    connection in this list selects its slots inside the receiver's FIFO area; sender and
    receiver derive the same table from the same XML."""
    incoming = {g.id: set() for g in algo.gpus}
    for g in algo.gpus:
        for tb in g.tbs:
            if tb.recv != -1 and any(st.is_recv() for st in tb.steps):
                incoming[g.id].add((tb.chan, tb.recv))
    return {r: {conn: i for i, conn in enumerate(sorted(conns))} for r, conns in incoming.items()}


def compile_plan(algo: AlgoIR, local_ranks, slot_bytes: int, check=True) -> HostPlan:
    if check:
        problems = validate(algo)
        if problems:
            raise PlanError('invalid MSCCL-IR: ' + '; '.join(problems[:5]))
    if algo.proto not in PROTO_CODES:
        raise PlanError(f'unknown protocol {algo.proto}')
    if algo.ngpus > K_MAX_RANKS:
        raise PlanError(f'{algo.ngpus} ranks exceed the executor limit of {K_MAX_RANKS}')
    if algo.nchannels > K_MAX_CHANNELS:
        raise PlanError(f'{algo.nchannels} channels exceed the executor limit of {K_MAX_CHANNELS}')
    if algo.max_tbs_per_gpu() > K_MAX_TBS:
        raise PlanError(f'{algo.max_tbs_per_gpu()} threadblocks per GPU exceed the executor limit of {K_MAX_TBS}')
    tables = fifo_index_tables(algo)
    plan = HostPlan(algo, list(local_ranks), proto=PROTO_CODES[algo.proto], max_cnt=max(algo.max_count(), 1),
                    in_conns=max((len(t) for t in tables.values()), default=0))
    stride = K_FIFO_SLOTS * slot_bytes
    tb_blob, step_blob = [], []
    nsteps_total = 0
    for rank in plan.local_ranks:
        gpu = algo.gpus[rank]
        plan.first_tb[rank] = len(tb_blob)
        plan.num_tbs[rank] = len(gpu.tbs)
        used = {'i': 0, 'o': 0, 's': 0}
        for tb in gpu.tbs:
            sends = any(st.is_send() for st in tb.steps)
            recvs = any(st.is_recv() for st in tb.steps)
            send_peer = tb.send if sends else -1
            recv_peer = tb.recv if recvs else -1
            send_conn = tb.chan * K_MAX_RANKS + send_peer if sends else -1
            recv_conn = tb.chan * K_MAX_RANKS + recv_peer if recvs else -1
            send_off = tables[send_peer][(tb.chan, rank)] * stride if sends else 0
            recv_off = tables[rank][(tb.chan, recv_peer)] * stride if recvs else 0
            tb_blob.append(_TB.pack(rank, tb.id, send_peer, recv_peer, tb.chan, len(tb.steps), nsteps_total,
                                    len(gpu.tbs), send_conn, recv_conn, send_off, recv_off))
            for st in tb.steps:
                if st.type not in STEP_CODES:
                    raise PlanError(f'step type {st.type!r} is not executable by the interpreter kernel')
                if st.type == 'nop':
                    sbuf, soff, dbuf, doff, cnt = 'i', 0, 'i', 0, 0
                else:
                    # local operand of receive-type steps is dst; src of s/cpy/re is local too
                    sbuf, soff = algo.resolve(rank, st.srcbuf, st.srcoff)
                    dbuf, doff = algo.resolve(rank, st.dstbuf, st.dstoff)
                    cnt = st.cnt
                    if st.type in ('s', 'cpy', 're'):
                        used[sbuf] = max(used[sbuf], soff + cnt)
                    if st.type != 's':
                        used[dbuf] = max(used[dbuf], doff + cnt)
                    if st.type in ('r', 'rcs', 'rrs', 'rrc', 'rrcs'):
                        sbuf, soff = 'i', 0       # the remote source slot is not addressed by the receiver
                    if st.type == 's':
                        dbuf, doff = 'i', 0       # nor the remote destination by the sender
                step_blob.append(_STEP.pack(STEP_CODES[st.type], BUF_CODES[sbuf], BUF_CODES[dbuf], int(st.hasdep),
                                            st.depid, st.deps, soff, doff, cnt))
            nsteps_total += len(tb.steps)
        plan.extents[rank] = used
    plan.tb_bytes = b''.join(tb_blob)
    plan.step_bytes = b''.join(step_blob)
    return plan


def chunk_geometry(algo: AlgoIR, rank: int, input_elems: int):
    """Elements per chunk for a call whose input on ``rank`` has ``input_elems`` elements."""
    g = algo.gpus[rank]
    if algo.inplace and algo.coll == 'allgather':
        chunks = g.o_chunks // algo.ngpus
    else:
        chunks = g.i_chunks
    if chunks <= 0 or input_elems % chunks != 0:
        raise PlanError(f'{input_elems} input elements are not divisible into {chunks} chunks')
    return input_elems // chunks


def tile_geometry(plan: HostPlan, chunk_elems: int, elem_size: int, slot_bytes: int):
    """(tile_elems, iterations): how many elements of each chunk one iteration moves so that the
    largest step (max_cnt chunks) fits into one FIFO slot."""
    if (chunk_elems * elem_size) % 16 != 0:
        raise PlanError(f'chunk of {chunk_elems} x {elem_size} bytes is not a multiple of 16 bytes')
    payload = slot_bytes if plan.proto == 0 else slot_bytes // 2
    per_vec = 16 // elem_size
    tile = (payload // (plan.max_cnt * elem_size)) // per_vec * per_vec
    if tile <= 0:
        raise PlanError('FIFO slot too small for this program')
    if plan.proto == 0:
        # Simple: a receiver starts on a tile only when the whole tile has landed, so a chunk is cut
        # into at least four tiles (of 256 KB or more) to overlap the two sides.
        quarter = -(-chunk_elems // 4)
        want = max((256 << 10) // (plan.max_cnt * elem_size), quarter)
        want = -(-want // per_vec) * per_vec
        tile = min(tile, want)
    tile = min(tile, chunk_elems)
    iterations = -(-chunk_elems // tile)
    return tile, iterations
