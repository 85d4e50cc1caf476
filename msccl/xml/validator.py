"""Static validation of MSCCL-IR: the checks an executor needs before it may trust a file.

The reference never inspects its own XML (only DAG-level checks exist, ``msccl/language/passes.py``);
a native executor cannot afford that.  ``validate`` returns a list of human-readable problems
(empty = valid):

* structure: gpu ids 0..ngpus-1, tb ids dense, step indices dense, known step types and buffers,
  protocol name, channel within ``nchannels``;
* bounds: every locally addressed slot lies inside ``i/o/s_chunks`` of its rank, and the remote
  side of sends/receives inside the peer's buffers;
* threadblock shape: sends only with a send peer, receives only with a receive peer;
* connections: each (src, dst, channel) has exactly one sending and one receiving threadblock,
  with equal numbers of sends and receives and equal ``cnt`` message by message;
* dependencies: ``depid/deps`` name an existing step of another threadblock, the target is
  marked ``hasdep``;
* deadlock freedom: the union of program order, dependency edges and send->receive matching
  must be acyclic (checked by abstract execution with unbounded FIFOs).
"""
from collections import defaultdict, deque

from msccl.xml.loader import PROTOCOLS, STEP_TYPES, AlgoIR

_BUFFERS = ('i', 'o', 's')


def _extent(gpu, buf):
    return {'i': gpu.i_chunks, 'o': gpu.o_chunks, 's': gpu.s_chunks}[buf]


def validate(algo: AlgoIR, max_problems=50):
    problems = []

    def report(msg):
        if len(problems) < max_problems:
            problems.append(msg)

    if algo.proto not in PROTOCOLS:
        report(f'unknown protocol {algo.proto!r}')
    if len(algo.gpus) != algo.ngpus or [g.id for g in algo.gpus] != list(range(algo.ngpus)):
        report(f'gpu ids {[g.id for g in algo.gpus]} are not 0..{algo.ngpus - 1}')
        return problems

    def check_slot(rank, buf, off, cnt, what):
        if buf not in _BUFFERS:
            report(f'{what}: unknown buffer {buf!r}')
            return
        rbuf, roff = algo.resolve(rank, buf, off)
        limit = _extent(algo.gpus[rank], rbuf)
        if off < 0 or roff + cnt > limit:
            report(f'{what}: {buf}[{off}:{off + cnt}] exceeds the {limit} chunks of buffer {rbuf!r} on gpu {rank}')

    senders = defaultdict(list)     # (src, dst, chan) -> [(tb id, [cnt...])]
    receivers = defaultdict(list)
    for gpu in algo.gpus:
        if [tb.id for tb in gpu.tbs] != list(range(len(gpu.tbs))):
            report(f'gpu {gpu.id}: threadblock ids are not dense')
        for tb in gpu.tbs:
            where = f'gpu {gpu.id} tb {tb.id}'
            if not 0 <= tb.chan < max(algo.nchannels, 1):
                report(f'{where}: channel {tb.chan} outside nchannels={algo.nchannels}')
            for peer, role in ((tb.send, 'send'), (tb.recv, 'recv')):
                if peer != -1 and not (0 <= peer < algo.ngpus and peer != gpu.id):
                    report(f'{where}: bad {role} peer {peer}')
            if [st.s for st in tb.steps] != list(range(len(tb.steps))):
                report(f'{where}: step indices are not dense')
            sent, received = [], []
            for st in tb.steps:
                at = f'{where} step {st.s}'
                if st.type not in STEP_TYPES:
                    report(f'{at}: unknown type {st.type!r}')
                    continue
                if st.type in ('nop', 'bar'):
                    pass
                else:
                    if st.cnt < 1:
                        report(f'{at}: cnt={st.cnt}')
                    if st.is_send():
                        if tb.send == -1:
                            report(f'{at}: {st.type} in a threadblock without send peer')
                        else:
                            sent.append(st.cnt)
                            if st.type == 's':
                                check_slot(gpu.id, st.srcbuf, st.srcoff, st.cnt, at + ' src')
                            check_slot(tb.send, st.dstbuf, st.dstoff, st.cnt, at + ' remote dst')
                    if st.is_recv():
                        if tb.recv == -1:
                            report(f'{at}: {st.type} in a threadblock without recv peer')
                        else:
                            received.append(st.cnt)
                            if st.type in ('r', 'rrc'):
                                check_slot(gpu.id, st.dstbuf, st.dstoff, st.cnt, at + ' dst')
                    if st.type in ('cpy', 're', 'mmr', 'mmb', 'mmar'):
                        check_slot(gpu.id, st.srcbuf, st.srcoff, st.cnt, at + ' src')
                        check_slot(gpu.id, st.dstbuf, st.dstoff, st.cnt, at + ' dst')
                if st.depid != -1:
                    if not 0 <= st.depid < len(gpu.tbs) or st.depid == tb.id:
                        report(f'{at}: depid {st.depid} is not another threadblock of gpu {gpu.id}')
                    elif not 0 <= st.deps < len(gpu.tbs[st.depid].steps):
                        report(f'{at}: deps {st.deps} is not a step of tb {st.depid}')
                    elif not gpu.tbs[st.depid].steps[st.deps].hasdep:
                        report(f'{at}: waits on tb {st.depid} step {st.deps}, which is not marked hasdep')
            if sent:
                senders[(gpu.id, tb.send, tb.chan)].append((tb.id, sent))
            if received:
                receivers[(tb.recv, gpu.id, tb.chan)].append((tb.id, received))

    # cross-rank barriers: the k-th `bar` of a channel on one GPU meets the k-th `bar` of that channel on
    # every other GPU, so each GPU needs the same number of them, issued by one threadblock per channel
    bars = defaultdict(dict)                      # channel -> gpu -> [tb ids issuing bars] / count
    for gpu in algo.gpus:
        for tb in gpu.tbs:
            n = sum(1 for st in tb.steps if st.type == 'bar')
            if n:
                bars[tb.chan].setdefault(gpu.id, []).append((tb.id, n))
    for chan, per_gpu in sorted(bars.items()):
        counts = {}
        for g in range(algo.ngpus):
            owners = per_gpu.get(g, [])
            if len(owners) > 1:
                report(f'gpu {g}: barriers of channel {chan} are issued by {len(owners)} threadblocks (must be one)')
            counts[g] = sum(n for _, n in owners)
        if len(set(counts.values())) > 1:
            report(f'channel {chan}: barrier counts differ between gpus: {counts}')

    for conn in sorted(set(senders) | set(receivers)):
        s, r = senders.get(conn, []), receivers.get(conn, [])
        src, dst, chan = conn
        if len(s) > 1 or len(r) > 1:
            report(f'connection {src}->{dst} channel {chan} is driven by {len(s)} sending and {len(r)} '
                   'receiving threadblocks (must be one each)')
        elif not s or not r:
            report(f'connection {src}->{dst} channel {chan}: {sum(len(x[1]) for x in s)} sends but '
                   f'{sum(len(x[1]) for x in r)} receives')
        elif s[0][1] != r[0][1]:
            report(f'connection {src}->{dst} channel {chan}: send counts {s[0][1][:8]} do not match receive '
                   f'counts {r[0][1][:8]}')
    if problems:
        return problems

    stuck = find_deadlock(algo)
    if stuck:
        report('deadlock: no threadblock can advance; waiting: ' + '; '.join(stuck[:6]))
    return problems


def find_deadlock(algo: AlgoIR, fifo_depth=None):
    """Abstractly execute the program (no data).  Returns [] if every threadblock finishes, else
    descriptions of the blocked threadblocks.  ``fifo_depth`` bounds in-flight messages per
    connection (None = unbounded)."""
    pc = {(g.id, tb.id): 0 for g in algo.gpus for tb in g.tbs}
    tbs = {(g.id, tb.id): tb for g in algo.gpus for tb in g.tbs}
    in_flight = defaultdict(int)
    arrived = defaultdict(set)                    # (channel, barrier index) -> gpus that reached it
    passed = defaultdict(int)                     # (gpu, tb) -> barriers already passed
    work = deque(pc)
    idle_rounds = 0
    while work and idle_rounds <= len(work):
        key = work.popleft()
        rank, _ = key
        tb = tbs[key]
        advanced = False
        while pc[key] < len(tb.steps):
            st = tb.steps[pc[key]]
            if st.depid != -1 and pc[(rank, st.depid)] <= st.deps:
                break
            if st.type == 'bar':
                meeting = (tb.chan, passed[key])
                if rank not in arrived[meeting]:
                    arrived[meeting].add(rank)
                    advanced = True               # arriving is progress: the others may now get through
                if len(arrived[meeting]) < algo.ngpus:
                    break
                passed[key] += 1
                pc[key] += 1
                advanced = True
                continue
            if st.is_recv() and in_flight[(tb.recv, rank, tb.chan)] == 0:
                break
            if st.is_send() and fifo_depth is not None and in_flight[(rank, tb.send, tb.chan)] >= fifo_depth:
                break
            if st.is_recv():
                in_flight[(tb.recv, rank, tb.chan)] -= 1
            if st.is_send():
                in_flight[(rank, tb.send, tb.chan)] += 1
            pc[key] += 1
            advanced = True
        if pc[key] < len(tb.steps):
            work.append(key)
        idle_rounds = 0 if advanced else idle_rounds + 1
    blocked = []
    for key in work:
        st = tbs[key].steps[pc[key]]
        blocked.append(f'gpu {key[0]} tb {key[1]} at step {st.s} ({st.type})')
    return blocked
