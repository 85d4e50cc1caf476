"""Static figures of an MSCCL-IR program and a latency/bandwidth estimate for one NVSwitch box.

``summarize(algo)`` executes the program abstractly (no data) and reports, per program: the depth of the
longest chain of steps that must run one after another (program order inside a threadblock, ``depid/deps``
edges, and the edge from every send to the receive that pops it), the chunks every GPU sends, and how many
of its threadblocks send.  ``estimate_us`` turns that into a time with the two-parameter model the
synthesis guide uses (reference ``examples/dgx1_allgather.ipynb`` cells 343-353: time = steps * alpha +
size * rounds / chunks * beta), with alpha and beta taken from measurements of this executor instead of 1:

    time = launch  +  depth * alpha  +  max over GPUs ( wire bytes sent / min(port bandwidth, sending threadblocks * per-CTA rate) )

Defaults, fitted to runs of the interpreter kernel on 2 B200: 11 us per launch (cooperative launch, the first flag
round trip, the drain at the end), then per dependent step 5 us for Simple (flag wait plus system-scope fence; a ring of
3 steps takes 29 us, a two-shot program of 5 steps 35 us at small sizes), 2.5 us for LL (3 steps: 19 us) and 3 us for
LL128; 50 GB/s per threadblock, 770 GB/s per NVLink port and direction; LL moves 16 bytes per 8 bytes of payload,
LL128 128 bytes per 120.  It is an estimate for choosing instance counts, not a measurement.
"""
from collections import defaultdict, deque
from dataclasses import dataclass, field

from msccl.xml.loader import AlgoIR

ALPHA_US = {'Simple': 5.0, 'LL': 2.5, 'LL128': 3.0}
LAUNCH_US = 11.0
WIRE_BYTES_PER_PAYLOAD_BYTE = {'Simple': 1.0, 'LL': 2.0, 'LL128': 128.0 / 120.0}
CTA_GBS = 50.0
PORT_GBS = 770.0


@dataclass
class ProgramSummary:
    depth: int = 0                                  # longest dependent chain, in steps
    sent_chunks: dict = field(default_factory=dict)   # gpu -> chunks it sends (all connections)
    sending_tbs: dict = field(default_factory=dict)   # gpu -> threadblocks with a send peer
    threadblocks: dict = field(default_factory=dict)  # gpu -> threadblocks
    steps: int = 0
    complete: bool = True                           # False if the abstract run got stuck (deadlock)


def summarize(algo: AlgoIR) -> ProgramSummary:
    out = ProgramSummary()
    pc = {(g.id, tb.id): 0 for g in algo.gpus for tb in g.tbs}
    tbs = {(g.id, tb.id): tb for g in algo.gpus for tb in g.tbs}
    level = {}                                      # (gpu, tb, step) -> depth of the chain ending there
    fifo = defaultdict(deque)                       # connection -> levels of the sends in flight
    arrived = defaultdict(dict)
    passed = defaultdict(int)
    for g in algo.gpus:
        out.threadblocks[g.id] = len(g.tbs)
        out.sending_tbs[g.id] = sum(1 for tb in g.tbs if tb.send != -1 and any(st.is_send() for st in tb.steps))
        out.sent_chunks[g.id] = sum(st.cnt for tb in g.tbs for st in tb.steps if st.is_send())
        out.steps += sum(len(tb.steps) for tb in g.tbs)
    work = deque(pc)
    idle = 0
    while work and idle <= len(work):
        key = work.popleft()
        rank, tbid = key
        tb = tbs[key]
        moved = False
        while pc[key] < len(tb.steps):
            st = tb.steps[pc[key]]
            if st.depid != -1 and pc[(rank, st.depid)] <= st.deps:
                break
            before = [level.get((rank, tbid, st.s - 1), 0)]
            if st.depid != -1:
                before.append(level[(rank, st.depid, st.deps)])
            if st.type == 'bar':
                meeting = (tb.chan, passed[key])
                if rank not in arrived[meeting]:
                    arrived[meeting][rank] = max(before)
                    moved = True
                if len(arrived[meeting]) < algo.ngpus:
                    break
                passed[key] += 1
                before.extend(arrived[meeting].values())
            else:
                if st.is_recv():
                    inbox = fifo[(tb.recv, rank, tb.chan)]
                    if not inbox:
                        break
                    before.append(inbox.popleft())
            mine = max(before) + (0 if st.type == 'nop' else 1)
            level[(rank, tbid, st.s)] = mine
            if st.is_send():
                fifo[(rank, tb.send, tb.chan)].append(mine)
            out.depth = max(out.depth, mine)
            pc[key] += 1
            moved = True
        if pc[key] < len(tb.steps):
            work.append(key)
        idle = 0 if moved else idle + 1
    out.complete = not work
    return out


def chunks_per_message(algo: AlgoIR) -> int:
    """How many chunks the caller's message is cut into (the buffer the size of a collective refers to)."""
    g = algo.gpus[0]
    if algo.coll == 'allgather':
        return max(g.o_chunks, 1)
    return max(g.i_chunks, 1)


def estimate_us(algo: AlgoIR, nbytes: int, alpha_us=None, cta_gbs=CTA_GBS, port_gbs=PORT_GBS, summary=None):
    """Estimated time in microseconds for a message of ``nbytes`` (the size the registry's ranges refer to:
    the input for all-reduce, reduce-scatter and all-to-all, the gathered output for all-gather)."""
    s = summary or summarize(algo)
    alpha = ALPHA_US.get(algo.proto, ALPHA_US['Simple']) if alpha_us is None else alpha_us
    chunk_bytes = nbytes / chunks_per_message(algo)
    wire = WIRE_BYTES_PER_PAYLOAD_BYTE.get(algo.proto, 1.0)     # flags travel with the data in LL and LL128
    slowest = 0.0
    for gpu, chunks in s.sent_chunks.items():
        if chunks == 0:
            continue
        rate = min(port_gbs, max(s.sending_tbs[gpu], 1) * cta_gbs)
        slowest = max(slowest, chunks * chunk_bytes * wire / (rate * 1e3))   # bytes / (GB/s) in us
    return LAUNCH_US + s.depth * alpha + slowest
