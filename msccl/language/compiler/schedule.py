"""Scheduling passes: depth annotation, global op order, channel and threadblock assignment.

Parity: reference ``msccl/language/rank_dag.py:181-200`` (chunk_step / priority) and
``msccl/language/tb_assignment.py:12-224`` (manual and automatic threadblock assignment,
topological instruction order, channel assignment with flow tracking and FIFO fix-up).
"""
import heapq
from collections import defaultdict

from msccl.language.mscclir import Instruction, Threadblock

MAX_CHANNELS = 32


# --------------------------------------------------------------------------- depths
def _successors(op):
    if op.is_send() and op.recv_match is not None:
        return op.next + [op.recv_match]
    return op.next


def annotate_depths(dag):
    """chunk_step = longest path from a start op (start = -1); priority = longest path to a
    sink.  A send's matching receive counts as a successor."""
    order = []            # reverse post-order over next + recv_match edges
    state = {}
    for root in dag.start_ops():
        if root in state:
            continue
        stack = [(root, iter(_successors(root)))]
        state[root] = 1
        while stack:
            node, it = stack[-1]
            child = next(it, None)
            if child is None:
                stack.pop()
                state[node] = 2
                order.append(node)
            elif child not in state:
                state[child] = 1
                stack.append((child, iter(_successors(child))))
    for op in order:                       # children are finished before their parents
        succ = _successors(op)
        op.priority = max((s.priority + 1 for s in succ), default=0)
    for op in reversed(order):             # parents first
        if op.inst == Instruction.start:
            op.chunk_step = -1
        for s in _successors(op):
            s.chunk_step = max(s.chunk_step, op.chunk_step + 1)


# ------------------------------------------------------------------- global ordering
def topo_sort_instrs(dag):
    """Order all ops so that a send precedes its receive and DAG predecessors come first;
    among ready ops prefer low chunk_step, then high priority, then low destination index."""
    counter = 0
    heap = []
    done = set()

    def push(op):
        nonlocal counter
        key = (op.chunk_step, -op.priority, op.dst.index, op.src.index, counter)
        counter += 1
        heapq.heappush(heap, (key, op))

    def ready(op):
        return all(p in done for p in op.prev)

    starts = list(dag.start_ops())
    done.update(starts)
    for st in starts:
        for o in st.next:
            if o.inst in (Instruction.send, Instruction.copy) or (o.inst == Instruction.reduce and ready(o)):
                push(o)
    ordered = []
    while heap:
        _, op = heapq.heappop(heap)
        if op in done:
            continue
        if not ready(op):
            continue         # a copy seeded from one start may still wait on another slot
        done.add(op)
        ordered.append(op)
        match = op.recv_match
        if match is not None and ready(match):
            push(match)
        for o in op.next:
            if o in done or not ready(o):
                continue
            if o.is_recv() and o.send_match is not None and o.send_match not in done:
                continue     # released by its send
            push(o)
    return ordered


# --------------------------------------------------------------- channel assignment
def channel_assignment(instrs, dag):
    """Give every send/receive pair a channel.

    Chains of fused ops (a "flow" Rw -> Rx -> Ry ...) must use one channel end to end, and two
    different flows through the same (sender, receiver) pair must not share a channel, because
    a threadblock owns exactly one (send peer, recv peer, channel).  Identical flows reuse their
    channel.  Finally, any pair whose FIFO order on a (src, dst, channel) connection differs
    between sender and receiver is moved to the next channel until the order is consistent."""
    everything = frozenset(range(MAX_CHANNELS))
    free_out = [defaultdict(lambda: set(everything)) for _ in range(dag.num_ranks)]
    free_in = [defaultdict(lambda: set(everything)) for _ in range(dag.num_ranks)]
    known_flows = []     # [(edge set, channel)]

    def reserve(sender, receiver, ch):
        free_out[sender][receiver].discard(ch)
        free_in[receiver][sender].discard(ch)

    def walk(op, allowed, path):
        if op.is_local():
            op.channel = 0
            return
        if not op.is_send():
            return
        match = op.recv_match
        sender, receiver = op.rank, match.rank
        allowed = free_out[sender][receiver] & free_in[receiver][sender] & allowed
        path.append(sender)
        if match.is_fused():
            walk(match, allowed, path)
            op.channel = match.channel
        else:
            path.append(receiver)
            edges = {(path[i - 1], path[i]) for i in range(1, len(path))}
            if op.channel != -1:
                ch = op.channel            # pinned by the user
            else:
                ch = next((c for f, c in known_flows if f == edges), -1)
                if ch == -1:
                    ch = min(allowed)
                    known_flows.append((edges, ch))
            op.channel = ch
            match.channel = ch
        reserve(sender, receiver, op.channel)

    for op in instrs:
        if op.inst == Instruction.send and op.recv_match.is_fused():
            walk(op, set(everything), [])

    again = True
    while again:
        again = False
        in_flight = defaultdict(list)      # (src, dst, ch) -> receives not yet matched
        for op in instrs:
            ch = max(op.channel, 0)
            if op.is_send():
                in_flight[(op.rank, op.dst.rank, ch)].append(op.recv_match)
            if op.is_recv():
                queue = in_flight[(op.src.rank, op.rank, ch)]
                if op in queue:
                    if queue[0] is op:
                        queue.pop(0)
                    else:
                        again = True
                        op.channel += 1
                        op.send_match.channel += 1
                        queue.remove(op)


# ----------------------------------------------------------- threadblock assignment
def _fits(tb, op):
    s, r = op.send_peer(), op.recv_peer()
    return ((tb.send == s or s == -1 or tb.send == -1)
            and (tb.recv == r or r == -1 or tb.recv == -1)
            and (tb.channel == op.channel or tb.channel == -1 or op.channel == -1))


def _place(tb, op):
    tb.ops.append(op)
    if op.is_send():
        tb.send = op.dst.rank
    if op.is_recv():
        tb.recv = op.src.rank
    op.step = len(tb.ops) - 1


def manual_assign_tbs(dag):
    """Honour the user's sendtb/recvtb/ch; reject a threadblock with two send peers, two
    receive peers or two channels."""
    for op in topo_sort_instrs(dag):
        tb = dag.tbs[op.rank].setdefault(op.tb, Threadblock())
        if not _fits(tb, op):
            raise Exception(
                f'Illegal threadblock assignment. Trying to add {op} to threadblock {op.tb}\n'
                f'Threadblock {op.tb} send:{tb.send} recv:{tb.recv} channel:{tb.channel}\n'
                f'Operation send:{op.send_peer()} recv:{op.recv_peer()} channel:{op.channel}')
        _place(tb, op)
        tb.channel = op.channel if op.channel != -1 else 0
        dag.num_channels[op.rank] = max(op.channel + 1, dag.num_channels[op.rank])


def _candidates(tbs, send, recv, channel):
    """Threadblocks able to host an op with these peers.  A connection (peer, channel) that
    some threadblock already owns must be reused, so that one is returned alone."""
    fitting = []
    for tbid, tb in tbs.items():
        channel_ok = channel == -1 or channel == tb.channel
        if channel_ok and ((send != -1 and tb.send == send) or (recv != -1 and tb.recv == recv)):
            return [tbid]
        if channel_ok and (send == -1 or tb.send == send) and (recv == -1 or tb.recv == recv):
            fitting.append(tbid)
    return fitting


def auto_assign_tbs(dag):
    instrs = topo_sort_instrs(dag)
    channel_assignment(instrs, dag)
    next_id = [0] * dag.num_ranks
    progress = [dict() for _ in range(dag.num_ranks)]     # tbid -> chunk_step of its last op
    for op in instrs:
        rank = op.rank
        s, r = op.send_peer(), op.recv_peer()
        ch = max(op.channel, 0)
        options = _candidates(dag.tbs[rank], s, r, ch)
        if options:
            tbid = options[0]
            for other in options:
                # prefer the candidate that is least far along
                if progress[rank][other] < progress[rank][tbid] and _fits(dag.tbs[rank][tbid], op):
                    tbid = other
        else:
            tbid = next_id[rank]
            next_id[rank] += 1
            dag.tbs[rank][tbid] = Threadblock(send=s, recv=r, channel=ch)
        tb = dag.tbs[rank][tbid]
        assert _fits(tb, op), (f'Failing: Operations uses channel {op.channel}, send:{s} recv:{r} {op}\n'
                               f'Threadblock uses send:{tb.send} recv:{tb.recv} channel:{tb.channel}')
        dag.num_channels[rank] = max(dag.num_channels[rank], ch + 1)
        _place(tb, op)
        op.tb = tbid
        progress[rank][tbid] = op.chunk_step
