"""Compile a validated MSCCL-IR program into the flat device arrays the executor kernel reads.

Layout contract: ``csrc/msccl_device.h`` (``DevTb`` 64 bytes, ``DevStep`` 32 bytes).  Aliases of
the in-place collectives are resolved here, so the kernel sees plain (buffer, chunk) pairs.

Besides the translation, three analyses run here:

* **direct stores** - the k-th send of a connection is matched with the k-th receive on the peer.  When that
  receive is ``r`` or ``rcs`` the send is marked ``SF_DIRECT_SEND`` with the receiver's slot, and the receive
  ``SF_DIRECT_RECV``: on registered (symmetric) memory the sender then stores into the final slot and only the
  flag travels through the connection (the receive semantics of ``r`` / ``rcs``, reference
  ``msccl/language/rank_dag.py:128-154``).  ``rrc`` / ``rrs`` / ``rrcs`` keep the FIFO: the receiver has to add.
* **opening receive slots** - a sender may only store into a slot once nothing on the receiving GPU touches it
  any more before the receive.  For every receive the earliest such point is worked out from program order and
  the ``depid/deps`` edges: the start of the iteration (nothing touches the slot before the receive), the end of
  an earlier step of the same threadblock (the last one that touches it), or the receive step itself.  A tile
  whose slot is not yet open when the sender gets to it simply takes the FIFO, so this never adds a wait.
* **batched reduces** - a run of ``re`` steps into one destination (with the ``nop`` steps that carry their extra
  dependencies, reference ``msccl/language/ir.py:264-291``) becomes one multi-input add with one store.
"""
import struct
from dataclasses import dataclass, field
from typing import Dict, List

from msccl.xml.loader import AlgoIR
from msccl.xml.validator import validate

STEP_CODES = {'nop': 0, 's': 1, 'r': 2, 'rcs': 3, 'rrs': 4, 'rrc': 5, 'rrcs': 6, 'cpy': 7, 're': 8}
BUF_CODES = {'i': 0, 'o': 1, 's': 2}
PROTO_CODES = {'Simple': 0, 'LL': 1, 'LL128': 2}
K_MAX_RANKS = 16
K_MAX_CHANNELS = 128
K_MAX_TBS = 128
K_FIFO_SLOTS = 4
K_MAX_BATCH = 8                 # `re` steps fused into one pass (csrc/msccl_device.h kMaxBatch)
K_MAX_STEPS_PER_TB = 4094       # the progress word keeps 12 bits of step + 1 ...
K_MAX_ITERATIONS = 1 << 20      # ... and 20 bits of iteration
SF_DIRECT_SEND, SF_DIRECT_RECV = 1, 2
_TB = struct.Struct('<4h4i2i2q4i')
_STEP = struct.Struct('<4B2h3i4Bi2H')
assert _TB.size == 64 and _STEP.size == 32


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
    direct_bufs: Dict[int, set] = field(default_factory=dict)          # rank -> buffers ('i','o','s') that direct stores land in
    direct_steps: int = 0          # send steps that may store straight into the receiver's slot
    eager_tbs: int = 0             # threadblocks whose receives are all opened at kernel start
    batched_steps: int = 0         # `re` steps folded into a multi-input add

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


def _match_connections(algo: AlgoIR):
    """Pair the k-th send of every connection with the k-th receive on the peer.  Returns
    ``{(rank, tb index, step index): (peer rank, peer tb index, peer step index)}`` for both directions."""
    sends, recvs = {}, {}
    for g in algo.gpus:
        for ti, tb in enumerate(g.tbs):
            for si, st in enumerate(tb.steps):
                if st.is_send() and tb.send != -1:
                    sends.setdefault((g.id, tb.send, tb.chan), []).append((g.id, ti, si))
                if st.is_recv() and tb.recv != -1:
                    recvs.setdefault((tb.recv, g.id, tb.chan), []).append((g.id, ti, si))
    match = {}
    for conn, ss in sends.items():
        rr = recvs.get(conn, [])
        for a, b in zip(ss, rr):
            match[a] = b
            match[b] = a
    return match


def _slots(algo, rank, st):
    """Resolved (buffer, first chunk, count) ranges a step reads or writes on its own GPU."""
    out = []
    if st.type == 'nop':
        return out
    if st.type in ('s', 'cpy', 're'):
        b, o = algo.resolve(rank, st.srcbuf, st.srcoff)
        out.append((b, o, st.cnt))
    if st.type != 's':
        b, o = algo.resolve(rank, st.dstbuf, st.dstoff)
        out.append((b, o, st.cnt))
    return out


def _open_positions(algo: AlgoIR, match):
    """For every threadblock with receives: ``{(rank, tb index): (opens_at_start, {step: opens_after},
    {step: opens_before}, nrecv, bufmask)}``.

    Position of a receive R at step ``si``: 0 when no step of the GPU touches R's slots unless it is ordered after R;
    ``k + 1`` ("after step k") when all such steps are earlier steps of R's own threadblock, k the last of them;
    otherwise R opens the slots itself when it is reached (after its dependency wait: the other threadblocks'
    accesses must be ordered before it by ``depid/deps``, which the FIFO path relies on just the same).  Slots are
    opened in receive order, so a receive never opens before its predecessors on the connection."""
    result = {}
    for g in algo.gpus:
        rank = g.id
        index_of = {tb.id: ti for ti, tb in enumerate(g.tbs)}
        # successors in the happens-before graph of this GPU: program order plus dependency edges
        waiters = {}
        for ti, tb in enumerate(g.tbs):
            for si, st in enumerate(tb.steps):
                if st.depid >= 0 and st.depid in index_of:
                    waiters.setdefault((index_of[st.depid], st.deps), []).append((ti, si))
        touched = {}
        for ti, tb in enumerate(g.tbs):
            for si, st in enumerate(tb.steps):
                for b, o, c in _slots(algo, rank, st):
                    for k in range(o, o + c):
                        touched.setdefault((b, k), []).append((ti, si))

        def after(ti, si):
            """Earliest step index per threadblock that is ordered after (ti, si)."""
            first = {ti: si + 1}
            todo = [(ti, si)]
            while todo:
                t, s0 = todo.pop()
                for s in range(s0, len(g.tbs[t].steps)):
                    for (t2, s2) in waiters.get((t, s), []):
                        if s2 < first.get(t2, 1 << 30):
                            first[t2] = s2
                            todo.append((t2, s2))
            return first

        for ti, tb in enumerate(g.tbs):
            recv_steps = [(si, st) for si, st in enumerate(tb.steps) if st.is_recv()]
            if not recv_steps or tb.recv == -1:
                continue
            running, at_start, opens_after, opens_before, mask = 0, 0, {}, {}, 0
            for si, st in recv_steps:
                own = 0                               # encoded: 2k = after step k-1 (0: iteration start), 2si+1 = at step si
                capable = st.type in ('r', 'rcs') and (rank, ti, si) in match
                if capable:
                    b, o = algo.resolve(rank, st.dstbuf, st.dstoff)
                    mask |= 1 << BUF_CODES[b]
                    later = after(ti, si)
                    for k in range(o, o + st.cnt):
                        for (t2, s2) in touched.get((b, k), []):
                            if (t2, s2) == (ti, si) or s2 >= later.get(t2, 1 << 30):
                                continue
                            if t2 == ti:
                                own = max(own, 2 * (s2 + 1))
                            else:
                                own = max(own, 2 * si + 1)
                running = max(running, own)
                if running == 0:
                    at_start += 1
                elif running % 2 == 0:
                    opens_after[running // 2 - 1] = opens_after.get(running // 2 - 1, 0) + 1
                else:
                    opens_before[running // 2] = opens_before.get(running // 2, 0) + 1
            result[(rank, ti)] = (at_start, opens_after, opens_before, len(recv_steps), mask)
    return result


def _batches(tb):
    """``{first step index: number of steps}`` for runs of ``re`` steps into one destination (``nop`` steps may sit
    between them) that the kernel executes as one multi-input add."""
    out = {}
    steps = tb.steps
    i = 0
    while i < len(steps):
        st = steps[i]
        if st.type != 're':
            i += 1
            continue
        j, last_re, sources = i + 1, i, 1
        srcs = {(st.srcbuf, st.srcoff)}
        while j < len(steps) and sources < K_MAX_BATCH and j - i < 2 * K_MAX_BATCH:
            nx = steps[j]
            if nx.type == 'nop':
                j += 1
                continue
            same_dst = nx.type == 're' and (nx.dstbuf, nx.dstoff, nx.cnt) == (st.dstbuf, st.dstoff, st.cnt)
            # a source that overlaps the destination must see the partial sum of the steps before it: not batched
            overlaps = nx.type == 're' and nx.srcbuf == st.dstbuf and nx.srcoff < st.dstoff + st.cnt and st.dstoff < nx.srcoff + nx.cnt
            if not same_dst or overlaps:
                break
            srcs.add((nx.srcbuf, nx.srcoff))
            last_re, sources = j, sources + 1
            j += 1
        if sources > 1:
            out[i] = last_re - i + 1
            i = last_re + 1
        else:
            i += 1
    return out


def compile_plan(algo: AlgoIR, local_ranks, slot_bytes: int, check=True, direct=True, batch=True) -> HostPlan:
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
    longest = max((len(tb.steps) for g in algo.gpus for tb in g.tbs), default=0)
    if longest > K_MAX_STEPS_PER_TB:
        raise PlanError(f'a threadblock has {longest} steps, the executor handles at most {K_MAX_STEPS_PER_TB}')
    tables = fifo_index_tables(algo)
    plan = HostPlan(algo, list(local_ranks), proto=PROTO_CODES[algo.proto], max_cnt=max(algo.max_count(), 1),
                    in_conns=max((len(t) for t in tables.values()), default=0))
    simple = algo.proto == 'Simple'
    match = _match_connections(algo) if (direct and simple) else {}
    opens = _open_positions(algo, match) if match else {}
    for r in range(algo.ngpus):
        plan.direct_bufs[r] = set()
    stride = K_FIFO_SLOTS * slot_bytes
    tb_blob, step_blob = [], []
    nsteps_total = 0
    for rank in plan.local_ranks:
        gpu = algo.gpus[rank]
        plan.first_tb[rank] = len(tb_blob)
        plan.num_tbs[rank] = len(gpu.tbs)
        used = {'i': 0, 'o': 0, 's': 0}
        for ti, tb in enumerate(gpu.tbs):
            sends = any(st.is_send() for st in tb.steps)
            recvs = any(st.is_recv() for st in tb.steps)
            send_peer = tb.send if sends else -1
            recv_peer = tb.recv if recvs else -1
            send_conn = tb.chan * K_MAX_RANKS + send_peer if sends else -1
            recv_conn = tb.chan * K_MAX_RANKS + recv_peer if recvs else -1
            send_off = tables[send_peer][(tb.chan, rank)] * stride if sends else 0
            recv_off = tables[rank][(tb.chan, recv_peer)] * stride if recvs else 0
            batches = _batches(tb) if batch else {}
            at_start, opens_after, opens_before, _, recv_mask = opens.get((rank, ti), (0, {}, {}, 0, 0))
            nrecv = sum(1 for st in tb.steps if st.is_recv()) if recvs else 0
            packed = []
            for si, st in enumerate(tb.steps):
                if st.type not in STEP_CODES:
                    raise PlanError(f'step type {st.type!r} is not executable by the interpreter kernel')
                flags, rbuf, roff = 0, 0, 0
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
                    peer = match.get((rank, ti, si))
                    if peer is not None and st.is_send():
                        pr, pt, ps = peer
                        other = algo.gpus[pr].tbs[pt].steps[ps]
                        if other.type in ('r', 'rcs') and other.cnt == st.cnt:
                            pb, po = algo.resolve(pr, other.dstbuf, other.dstoff)
                            flags |= SF_DIRECT_SEND
                            rbuf, roff = BUF_CODES[pb], po
                            plan.direct_bufs[pr].add(pb)
                            plan.direct_steps += 1
                    if peer is not None and st.type in ('r', 'rcs'):
                        pr, pt, ps = peer
                        if algo.gpus[pr].tbs[pt].steps[ps].cnt == st.cnt:
                            flags |= SF_DIRECT_RECV
                            plan.direct_bufs[rank].add(dbuf)
                nb = batches.get(si, 0)
                if nb:
                    plan.batched_steps += sum(1 for k in range(si, si + nb) if tb.steps[k].type == 're')
                packed.append(_STEP.pack(STEP_CODES[st.type], BUF_CODES[sbuf], BUF_CODES[dbuf], int(st.hasdep),
                                         st.depid, st.deps, soff, doff, cnt, flags, rbuf, nb, 0, roff,
                                         opens_after.get(si, 0), opens_before.get(si, 0)))
            if nrecv > 0 and recv_mask and at_start == nrecv:
                plan.eager_tbs += 1
            tb_blob.append(_TB.pack(rank, tb.id, send_peer, recv_peer, tb.chan, len(tb.steps), nsteps_total,
                                    len(gpu.tbs), send_conn, recv_conn, send_off, recv_off, at_start, recv_mask, nrecv, 0))
            step_blob.extend(packed)
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


def access_width(chunk_elems: int, elem_size: int, pointers=()):
    """Bytes per access of the kernel: 16 when every chunk and buffer is a multiple of 16 bytes, else one element."""
    if (chunk_elems * elem_size) % 16 == 0 and all(p % 16 == 0 for p in pointers):
        return 16
    return elem_size


def tile_geometry(plan: HostPlan, chunk_elems: int, elem_size: int, slot_bytes: int, width: int = 16, proto=None):
    """(tile_elems, iterations): how many elements of each chunk one iteration moves so that the
    largest step (max_cnt chunks) fits into one FIFO slot.  ``width`` is the access size in bytes
    (``access_width``); ``proto`` overrides the plan's protocol (LL128 programs whose chunks are not
    multiples of 16 bytes run as LL)."""
    proto = plan.proto if proto is None else proto
    per_access = width // elem_size
    if (chunk_elems * elem_size) % width:
        raise PlanError(f'chunks of {chunk_elems * elem_size} bytes are not whole {width}-byte accesses')
    if proto == 2:
        if width != 16:
            raise PlanError('LL128 needs chunks that are multiples of 16 bytes')
        lines = slot_bytes // 128 // plan.max_cnt             # 15 units of 8 bytes per 128-byte line
        tile = (lines * 15 // 2) * per_access
    else:
        fifo_bytes = width if proto == 0 else (32 if width == 16 else 8)
        tile = slot_bytes // (plan.max_cnt * fifo_bytes) * per_access
    if tile <= 0:
        raise PlanError('FIFO slot too small for this program')
    if proto == 0:
        # Simple: a receiver starts on a tile only when the whole tile has landed, so a chunk is cut
        # into at least four tiles (of 256 KB or more) to overlap the two sides.
        quarter = -(-chunk_elems // 4)
        want = max((256 << 10) // (plan.max_cnt * elem_size), quarter)
        want = -(-want // per_access) * per_access
        tile = min(tile, want)
    tile = min(tile, chunk_elems)
    iterations = -(-chunk_elems // tile)
    if iterations >= K_MAX_ITERATIONS:
        raise PlanError(f'{iterations} iterations through FIFO slots of {slot_bytes} bytes exceed the executor limit '
                        f'of {K_MAX_ITERATIONS}: use a larger FIFO area')
    return tile, iterations
