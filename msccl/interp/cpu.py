"""CPU reference interpreter for MSCCL-IR XML.

Execution model (the contract the native executor implements as well):

* every GPU has an input, an output and a scratch buffer made of equally sized chunks; the
  in-place collectives alias them (``AlgoIR.resolve``);
* each ``<tb>`` runs its steps in order; a step with ``depid/deps`` first waits until
  threadblock ``depid`` of the same GPU has completed step ``deps``;
* every (source GPU, destination GPU, channel) is a FIFO of messages.  ``s`` pushes a copy of
  the local ``src`` chunks; ``r`` pops into the local ``dst``; ``rrc`` pops and adds into
  ``dst`` (``dst = dst + received``); ``rcs`` pops, stores to ``dst`` and pushes the same data
  on the send connection; ``rrs`` pops, adds the local ``dst`` and pushes the sum without
  storing it; ``rrcs`` pops, adds, stores and pushes; ``cpy`` / ``re`` are local copy / add;
  ``nop`` only waits;
* a FIFO holds at most ``fifo_depth`` messages - a sender blocks when it is full;
* extension steps of the B200 runtime (never written by the classic tool chain): ``bar`` - the k-th
  barrier of a channel on one GPU waits for the k-th barrier of that channel on every other GPU;
  ``mmr`` - local ``dst`` = sum over all GPUs of their ``src`` slot; ``mmb`` - the local ``src`` is
  stored into the ``dst`` slot of every GPU; ``mmar`` - the slot is replaced on every GPU by its sum over
  all GPUs.  They model the in-switch (NVLS) reduction and multicast store: the sum is formed in fp32
  and rounded once, whatever the number of GPUs.

Scheduling is cooperative and deterministic; if no threadblock can advance the interpreter
raises ``DeadlockError`` naming the blocked steps.  With ``race_check=True`` every access to a
chunk is checked against earlier conflicting accesses using vector clocks over program order,
dependency edges and message edges; an unordered pair raises ``RaceError``.

Arithmetic: element type is the tensor dtype; sums of bf16/fp16 are computed in fp32 and
rounded once per addition (torch CPU semantics), which is what the CUDA kernels do as well,
so results can be compared bit for bit.
"""
from collections import defaultdict, deque

import torch

from msccl.xml.loader import AlgoIR

DEFAULT_FIFO_DEPTH = 8


class DeadlockError(RuntimeError):
    pass


class RaceError(RuntimeError):
    pass


class _Clock:
    """Sparse vector clock."""
    __slots__ = ('v',)

    def __init__(self, v=None):
        self.v = dict(v) if v else {}

    def tick(self, who):
        self.v[who] = self.v.get(who, 0) + 1

    def join(self, other):
        for k, t in other.v.items():
            if t > self.v.get(k, 0):
                self.v[k] = t

    def snapshot(self):
        return _Clock(self.v)

    def covers(self, who, time):
        return self.v.get(who, 0) >= time


class Interpreter:
    def __init__(self, algo: AlgoIR, chunk_elems: int, dtype=torch.float32, fifo_depth=DEFAULT_FIFO_DEPTH,
                 race_check=False):
        self.algo = algo
        self.chunk = chunk_elems
        self.dtype = dtype
        self.fifo_depth = fifo_depth
        self.race_check = race_check
        self.buffers = []
        for g in algo.gpus:
            self.buffers.append({'i': torch.zeros(g.i_chunks * chunk_elems, dtype=dtype),
                                 'o': torch.zeros(g.o_chunks * chunk_elems, dtype=dtype),
                                 's': torch.zeros(g.s_chunks * chunk_elems, dtype=dtype)})
        self.fifos = defaultdict(deque)
        self.pc = {(g.id, tb.id): 0 for g in algo.gpus for tb in g.tbs}
        self.tbs = {(g.id, tb.id): tb for g in algo.gpus for tb in g.tbs}
        self.trace = []
        # race checking state
        self.clock = {key: _Clock() for key in self.pc}
        self.done_clock = {}                 # (rank, tb, step) -> clock snapshot after the step
        self.last_write = {}                 # (rank, buf, chunk) -> (tb key, time, description)
        self.reads_since = defaultdict(list)
        # cross-rank barriers
        self.bar_passed = defaultdict(int)   # tb key -> barriers passed
        self.bar_arrived = defaultdict(dict)  # (channel, index) -> {rank: clock snapshot}
        self.bar_progress = False            # set when a threadblock newly arrives at a barrier

    # ---------------------------------------------------------------- buffers
    def view(self, rank, buf, off, cnt):
        rbuf, roff = self.algo.resolve(rank, buf, off)
        c = self.chunk
        return self.buffers[rank][rbuf][roff * c:(roff + cnt) * c]

    def set_input(self, rank, data):
        """Fill the input buffer of ``rank`` (for an in-place all-gather: its slice of the output)."""
        flat = data.reshape(-1).to(self.dtype)
        if self.algo.inplace and self.algo.coll == 'allgather':
            per = self.algo.gpus[rank].o_chunks // self.algo.ngpus
            self.view(rank, 'i', 0, per)[:flat.numel()] = flat
        else:
            self.buffers[rank]['i'][:flat.numel()] = flat

    def get_output(self, rank):
        g = self.algo.gpus[rank]
        if self.algo.inplace:
            if self.algo.coll == 'allreduce' or self.algo.coll == 'alltoall':
                return self.buffers[rank]['i']
            if self.algo.coll == 'reduce_scatter':
                per = g.i_chunks // self.algo.ngpus
                return self.view(rank, 'o', 0, per)
        return self.buffers[rank]['o']

    # ------------------------------------------------------------ race checks
    def _touch(self, key, rank, buf, off, cnt, write, what):
        if not self.race_check:
            return
        clock = self.clock[key]
        rbuf, roff = self.algo.resolve(rank, buf, off)
        for i in range(roff, roff + cnt):
            slot = (rank, rbuf, i)
            prev = self.last_write.get(slot)
            if prev is not None and prev[0] != key and not clock.covers(prev[0], prev[1]):
                raise RaceError(f'{what} on gpu {rank} {rbuf}[{i}] is not ordered after the write by {prev[2]}')
            if write:
                for rd in self.reads_since[slot]:
                    if rd[0] != key and not clock.covers(rd[0], rd[1]):
                        raise RaceError(f'{what} overwrites gpu {rank} {rbuf}[{i}] without being ordered after '
                                        f'the read by {rd[2]}')
                self.last_write[slot] = (key, clock.v.get(key, 0), what)
                self.reads_since[slot] = []
            else:
                self.reads_since[slot].append((key, clock.v.get(key, 0), what))

    # ------------------------------------------------------------------ steps
    def _try_step(self, key):
        rank, tbid = key
        tb = self.tbs[key]
        st = tb.steps[self.pc[key]]
        if st.depid != -1 and self.pc[(rank, st.depid)] <= st.deps:
            return False
        if st.type == 'bar':
            return self._try_barrier(key, tb, st)
        inbox = self.fifos[(tb.recv, rank, tb.chan)] if st.is_recv() else None
        outbox = self.fifos[(rank, tb.send, tb.chan)] if st.is_send() else None
        if inbox is not None and not inbox:
            return False
        if outbox is not None and self.fifo_depth is not None and len(outbox) >= self.fifo_depth:
            return False

        what = f'gpu {rank} tb {tbid} step {st.s} ({st.type})'
        if self.race_check:
            self.clock[key].tick(key)
            if st.depid != -1:
                self.clock[key].join(self.done_clock[(rank, st.depid, st.deps)])

        t = st.type
        if t == 's':
            self._touch(key, rank, st.srcbuf, st.srcoff, st.cnt, False, what)
            payload = self.view(rank, st.srcbuf, st.srcoff, st.cnt).clone()
        elif t in ('cpy', 're'):
            src = self.view(rank, st.srcbuf, st.srcoff, st.cnt)
            dst = self.view(rank, st.dstbuf, st.dstoff, st.cnt)
            self._touch(key, rank, st.srcbuf, st.srcoff, st.cnt, False, what)
            self._touch(key, rank, st.dstbuf, st.dstoff, st.cnt, True, what)
            if t == 'cpy':
                dst.copy_(src)
            else:
                dst.copy_(dst + src)
            payload = None
        elif t == 'nop':
            payload = None
        elif t in ('mmr', 'mmb', 'mmar'):
            everyone = range(self.algo.ngpus)
            if t == 'mmb':
                self._touch(key, rank, st.srcbuf, st.srcoff, st.cnt, False, what)
                value = self.view(rank, st.srcbuf, st.srcoff, st.cnt).clone()
            else:
                for r in everyone:
                    self._touch(key, r, st.srcbuf, st.srcoff, st.cnt, False, what)
                total = sum(self.view(r, st.srcbuf, st.srcoff, st.cnt).float() for r in everyone)
                value = total.to(self.dtype)
            if t == 'mmr':
                self._touch(key, rank, st.dstbuf, st.dstoff, st.cnt, True, what)
                self.view(rank, st.dstbuf, st.dstoff, st.cnt).copy_(value)
            else:
                for r in everyone:
                    self._touch(key, r, st.dstbuf, st.dstoff, st.cnt, True, what)
                    self.view(r, st.dstbuf, st.dstoff, st.cnt).copy_(value)
            payload = None
        elif st.is_recv():
            received, msg_clock = inbox.popleft()
            if received.numel() != st.cnt * self.chunk:
                raise RuntimeError(f'{what}: message of {received.numel()} elements, expected {st.cnt * self.chunk}')
            if self.race_check:
                self.clock[key].join(msg_clock)
            # The local operand of every receive-type step is the dst slot: a fused step carries
            # the remote destination there, and fusion only happens when that equals (buffer
            # and index) the slot the data was received into.
            lbuf, loff = st.dstbuf, st.dstoff
            local = self.view(rank, lbuf, loff, st.cnt)
            if t == 'r':
                self._touch(key, rank, lbuf, loff, st.cnt, True, what)
                local.copy_(received)
                payload = None
            elif t == 'rrc':
                self._touch(key, rank, lbuf, loff, st.cnt, True, what)
                local.copy_(local + received)
                payload = None
            elif t == 'rcs':
                self._touch(key, rank, lbuf, loff, st.cnt, True, what)
                local.copy_(received)
                payload = received
            elif t == 'rrs':
                self._touch(key, rank, lbuf, loff, st.cnt, False, what)
                payload = local + received
            elif t == 'rrcs':
                self._touch(key, rank, lbuf, loff, st.cnt, True, what)
                local.copy_(local + received)
                payload = local.clone()
            else:
                raise RuntimeError(f'{what}: unsupported on the CPU interpreter')
        else:
            raise RuntimeError(f'{what}: unsupported on the CPU interpreter')
        if outbox is not None:
            outbox.append((payload, self.clock[key].snapshot() if self.race_check else None))
        if self.race_check and st.hasdep:
            self.done_clock[(rank, tbid, st.s)] = self.clock[key].snapshot()
        self.pc[key] += 1
        return True

    def _try_barrier(self, key, tb, st):
        rank, tbid = key
        meeting = (tb.chan, self.bar_passed[key])
        here = self.bar_arrived[meeting]
        if rank not in here:
            if self.race_check:
                self.clock[key].tick(key)
                if st.depid != -1:
                    self.clock[key].join(self.done_clock[(rank, st.depid, st.deps)])
            here[rank] = self.clock[key].snapshot() if self.race_check else None
            self.bar_progress = True
        if len(here) < self.algo.ngpus:
            return False
        if self.race_check:
            for other in here.values():          # everything before anyone's barrier is ordered before what follows
                self.clock[key].join(other)
            if st.hasdep:
                self.done_clock[(rank, tbid, st.s)] = self.clock[key].snapshot()
        self.bar_passed[key] += 1
        self.pc[key] += 1
        return True

    def run(self):
        pending = deque(k for k in self.pc if self.tbs[k].steps)
        stalled = 0
        while pending:
            key = pending.popleft()
            moved = False
            self.bar_progress = False
            while self.pc[key] < len(self.tbs[key].steps) and self._try_step(key):
                moved = True
            moved = moved or self.bar_progress   # arriving at a barrier lets the others through
            if self.pc[key] < len(self.tbs[key].steps):
                pending.append(key)
                stalled = 0 if moved else stalled + 1
                if stalled > len(pending):
                    blocked = [f'gpu {k[0]} tb {k[1]} step {self.tbs[k].steps[self.pc[k]].s} '
                               f'({self.tbs[k].steps[self.pc[k]].type})' for k in list(pending)[:8]]
                    raise DeadlockError('no threadblock can advance: ' + '; '.join(blocked))
            else:
                stalled = 0
        leftover = {c: len(q) for c, q in self.fifos.items() if q}
        if leftover:
            raise RuntimeError(f'messages left in FIFOs after the program ended: {leftover}')
        return self


def input_chunks_of(algo: AlgoIR, rank):
    """Number of chunks the caller supplies on ``rank``."""
    g = algo.gpus[rank]
    if algo.inplace and algo.coll == 'allgather':
        return g.o_chunks // algo.ngpus
    return g.i_chunks


def run_algorithm(algo: AlgoIR, inputs, chunk_elems, dtype=torch.float32, fifo_depth=DEFAULT_FIFO_DEPTH,
                  race_check=False):
    """Run ``algo`` with ``inputs[rank]`` as the input of each rank; returns the output tensors."""
    it = Interpreter(algo, chunk_elems, dtype, fifo_depth, race_check)
    for r in range(algo.ngpus):
        it.set_input(r, inputs[r])
    it.run()
    return [it.get_output(r).clone() for r in range(algo.ngpus)]


def expected_result(algo: AlgoIR, inputs, chunk_elems):
    """Mathematical result of the named collective in fp64 (None for custom collectives)."""
    n = algo.ngpus
    x = [t.reshape(-1).double() for t in inputs]
    if algo.coll == 'allreduce':
        total = sum(x)
        return [total.clone() for _ in range(n)]
    if algo.coll == 'allgather':
        cat = torch.cat(x)
        return [cat.clone() for _ in range(n)]
    if algo.coll == 'reduce_scatter':
        total = sum(x)
        per = total.numel() // n
        return [total[r * per:(r + 1) * per].clone() for r in range(n)]
    if algo.coll == 'alltoall':
        per = x[0].numel() // n
        return [torch.cat([x[src][r * per:(r + 1) * per] for src in range(n)]) for r in range(n)]
    return None


def run_reference_check(algo: AlgoIR, chunk_elems=4, race_check=False, seed=0):
    """Execute on seeded integer-valued data (sums are exact, so any summation order gives the
    same bits) and compare with the collective's definition.  Returns 'pass ...' or 'FAIL ...'."""
    gen = torch.Generator().manual_seed(seed)
    inputs = [torch.randint(-8, 9, (input_chunks_of(algo, r) * chunk_elems,), generator=gen).float()
              for r in range(algo.ngpus)]
    try:
        outputs = run_algorithm(algo, inputs, chunk_elems, race_check=race_check)
    except (DeadlockError, RaceError, RuntimeError, AssertionError) as e:
        return f'FAIL {type(e).__name__}: {e}'
    want = expected_result(algo, inputs, chunk_elems)
    if want is None:
        return 'pass (custom collective: executed, result not checked)'
    for r in range(algo.ngpus):
        got = outputs[r][:want[r].numel()].double()
        if got.numel() != want[r].numel() or not torch.equal(got, want[r]):
            return f'FAIL: gpu {r} output differs from the {algo.coll} definition'
    return 'pass' + (' (race-free)' if race_check else '')
