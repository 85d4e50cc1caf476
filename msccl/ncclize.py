"""Lower a synthesized ``Algorithm`` (steps of address sends) to MSCCL-IR XML.

Pipeline:
  1. map abstract addresses to input / output / scratch indices per rank;
  2. optionally shrink scratch (SMT remap into dead input/output slots, or a greedy sort
     that makes merged transfers contiguous);
  3. turn each algorithm step into send/receive operation pairs - a receive into a slot
     that already holds data becomes ``rrc``; several senders into one slot in one step are
     serialised into sub-steps; contiguous transfers on an edge merge into one op with ``cnt``;
  4. spread the ops of an edge over channels, replicate instances;
  5. track read/write dependencies per buffer index;
  6. group ops into threadblocks (one direction+peer+channel each, never two groups that
     share an algorithm step), add a copy threadblock, expand extra waits into nops, emit.

Behavioural parity: reference ``msccl/ncclize.py:60-722``; attribute order of the ``<algo>``
element is that writer's (``name proto nchannels ngpus inplace coll nchunksperloop``).
"""
import bisect
import itertools
import math
import queue
import threading
import xml.etree.ElementTree as ET
from collections import defaultdict
from dataclasses import dataclass, field
from enum import Enum

import z3


class ChannelPolicy(Enum):
    One = 'One'
    MatchTopology = 'MatchTopology'

    def __str__(self):
        return self.value


@dataclass(eq=False)
class _Op:
    gpu: int
    peer: object
    step: int
    is_send: bool
    op_type: str
    src_buffer: object
    src_offset: object
    dst_buffer: object
    dst_offset: object
    cnt: int
    depends: list
    block_rbid: object = None
    idx: object = None          # position in the emitted threadblock (nops included)
    has_dependence: bool = False


@dataclass
class _Gpu:
    precopies: list
    postcopies: list
    inputs: dict
    outputs: dict
    input_chunks: int
    output_chunks: int
    scratch: dict = field(default_factory=dict)
    threadblocks: list = field(default_factory=list)

    def scratch_size(self):
        return max(self.scratch.values(), default=-1) + 1

    def locate(self, addr):
        if addr in self.inputs:
            return 'i', self.inputs[addr]
        if addr in self.outputs:
            return 'o', self.outputs[addr]
        if addr in self.scratch:
            return 's', self.scratch[addr]
        raise RuntimeError('Address is not mapped to a buffer')


@dataclass(eq=False)
class _Threadblock:
    channel: int
    rbid: object = None
    send: int = -1
    recv: int = -1
    steps: list = field(default_factory=list)   # algorithm-level ops
    ops: list = field(default_factory=list)     # emitted ops, nops included


def _local_copy(rank, src_buf, src_off, dst_buf, dst_off):
    return _Op(rank, None, -1, False, 'cpy', src_buf, src_off, dst_buf, dst_off, 1, [])


# ------------------------------------------------------------------ scratch policies
def _liveness(gpus, algorithm):
    """Per rank and buffer index: list of (first step, last step) intervals of use.  Inputs are
    live from before the start, outputs until after the end."""
    live = {rank: {'i': [[(-1, -1)] for _ in range(g.input_chunks)],
                   'o': [[(math.inf, math.inf)] for _ in range(g.output_chunks)],
                   's': [[(math.inf, -1)] for _ in g.scratch]} for rank, g in gpus.items()}
    for rank, g in gpus.items():
        # An address that is both input and output stays in its input slot and is copied to the
        # output after the last step, so that slot is occupied for the whole algorithm.  (The
        # reference omits this and can remap scratch on top of data the final copy still needs.)
        for addr, idx in g.inputs.items():
            if addr in g.outputs:
                live[rank]['i'][idx][0] = (-1, math.inf)
    for t, step in enumerate(algorithm.steps):
        for addr, src, dst in step.sends:
            for rank in (src, dst):
                try:
                    buf, idx = gpus[rank].locate(addr)
                except RuntimeError:
                    raise RuntimeError(f'Address {addr} not found in any buffer of rank {rank}.')
                lo, hi = live[rank][buf][idx][0]
                live[rank][buf][idx][0] = (min(lo, t), max(hi, t))
    return live


def _overlaps(a, b):
    return any(s1 <= e2 and s2 <= e1 for s1, e1 in a for s2, e2 in b)


def _remap_scratch_into_input_output(live, gpus, logging):
    """Per GPU, find with Z3 an assignment of scratch indices to the unified index space
    [inputs | outputs | scratch] such that no two live ranges collide and the scratch tail is
    as short as a one-second search gets it."""
    if logging:
        print('Remapping scratch into input/output...')
    print('Optimizing scratch mapping on all GPUs: ', end='', flush=True)
    for rank, gpu in gpus.items():
        ctx = z3.Context()
        solver = z3.Solver(ctx=ctx)
        where = [z3.Int(f'{i}_remap', ctx=ctx) for i in range(len(live[rank]['s']))]
        limit = z3.Int('idx_end', ctx=ctx)
        for i, mine in enumerate(live[rank]['s']):
            for j, other in enumerate(live[rank]['i']):
                if _overlaps(mine, other):
                    solver.add(where[i] != j)
            for j, other in enumerate(live[rank]['o']):
                if _overlaps(mine, other):
                    solver.add(where[i] != j + gpu.input_chunks)
            for j, other in enumerate(live[rank]['s']):
                if j != i and _overlaps(mine, other):
                    solver.add(where[i] != where[j])
            solver.add(where[i] >= 0, where[i] < limit)
        fixed = gpu.input_chunks + gpu.output_chunks
        found = queue.Queue()

        def shrink():
            for budget in range(fixed + gpu.scratch_size(), fixed - 1, -1):
                if solver.check(limit == budget) != z3.sat:
                    return
                try:
                    model = solver.model()
                    found.put({addr: model.eval(where[old], model_completion=True).as_long()
                               for addr, old in gpu.scratch.items()})
                except z3.Z3Exception:      # interrupted
                    return

        worker = threading.Thread(target=shrink)
        worker.start()
        worker.join(1)
        ctx.interrupt()
        worker.join()
        best = None
        while not found.empty():
            best = found.get()
        if best is None:
            print('x', end='', flush=True)
            continue
        print('.', end='', flush=True)
        new_scratch = {}
        new_live = [[] for _ in gpu.scratch]
        for addr, old in gpu.scratch.items():
            pos = best[addr]
            if pos < gpu.input_chunks:
                table, idx, ranges = gpu.inputs, pos, live[rank]['i'][pos]
            elif pos < fixed:
                idx = pos - gpu.input_chunks
                table, ranges = gpu.outputs, live[rank]['o'][idx]
            else:
                idx = pos - fixed
                table, ranges = new_scratch, new_live[idx]
            assert not _overlaps(ranges, live[rank]['s'][old])
            ranges.extend(live[rank]['s'][old])
            table[addr] = idx
        gpu.scratch = new_scratch
    print()
    if logging:
        worst = max(g.scratch_size() / (g.input_chunks + g.output_chunks) for g in gpus.values())
        print(f'Maximum scratch overhead is {worst * 100:.0f}%')


def _greedy_scratch_sort(algorithm, gpus):
    """Heuristic: allocate the address sets that travel together over one edge in one step
    contiguously (largest sets first), so that their transfers merge into single ops."""
    unplaced = {rank: set(g.scratch) | set(g.inputs) | set(g.outputs) for rank, g in gpus.items()}
    bundles = defaultdict(set)
    for t, step in enumerate(algorithm.steps):
        for addr, src, dst in step.sends:
            if addr in unplaced[src] and addr in unplaced[dst]:
                bundles[(t, src, dst)].add(addr)
    for g in gpus.values():
        g.scratch = {}
    for key in sorted(bundles, key=lambda k: len(bundles[k]), reverse=True):
        _t, src, dst = key
        bundle = bundles[key]
        addrs = sorted(bundle)

        def contiguous(table):
            return bundle <= table.keys() and all(table[b] == table[a] + 1 for a, b in zip(addrs, addrs[1:]))

        src_in = contiguous(gpus[src].inputs)
        src_done = src_in or contiguous(gpus[src].outputs) or contiguous(gpus[src].scratch)
        dst_in = contiguous(gpus[dst].inputs)
        dst_done = dst_in or contiguous(gpus[dst].outputs) or contiguous(gpus[dst].scratch)
        if not ((bundle <= unplaced[src] or src_done) and (bundle <= unplaced[dst] or dst_done)):
            continue
        unplaced[src] -= bundle
        unplaced[dst] -= bundle
        for addr in addrs:
            for rank, done, keep_input in ((src, src_done, src_in), (dst, dst_done, dst_in)):
                g = gpus[rank]
                if done:
                    if addr in g.inputs and addr in g.outputs:
                        cp = _local_copy(rank, 'i', g.inputs[addr], 'o', g.outputs[addr])
                        if keep_input:
                            g.postcopies.append(cp)
                            del g.outputs[addr]
                        else:
                            g.precopies.append(cp)
                            del g.inputs[addr]
                else:
                    g.scratch[addr] = len(g.scratch)
                    if addr in g.inputs:
                        g.precopies.append(_local_copy(src, 'i', g.inputs[addr], 's', g.scratch[addr]))
                        del g.inputs[addr]
                    if addr in g.outputs:
                        g.postcopies.append(_local_copy(src, 's', g.scratch[addr], 'o', g.outputs[addr]))
                        del g.outputs[addr]
    for rank, rest in unplaced.items():
        g = gpus[rank]
        for addr in sorted(rest):
            if addr not in g.inputs and addr not in g.outputs:
                g.scratch[addr] = len(g.scratch)


# --------------------------------------------------------------------- step lowering
def _merge_copies(copies):
    copies.sort(key=lambda c: (c.src_buffer, c.dst_buffer, c.src_offset, c.dst_offset))
    merged = []
    for c in copies:
        last = merged[-1] if merged else None
        if (last is not None and last.src_buffer == c.src_buffer and last.dst_buffer == c.dst_buffer
                and last.src_offset + last.cnt == c.src_offset and last.dst_offset + last.cnt == c.dst_offset):
            last.cnt += c.cnt
        else:
            merged.append(c)
    copies[:] = merged


def _intervals(gpus, src, dst, items, merge):
    """(srcbuf, srcoff, dstbuf, dstoff, recv_type, cnt) for the addresses sent src -> dst."""
    located = [gpus[src].locate(addr) + gpus[dst].locate(addr) + (kind,) for addr, kind in items]
    if not merge:
        return [entry + (1,) for entry in located]
    located.sort()
    out = []
    run_start = run_end = located[0]
    for entry in located[1:]:
        follows = (entry[0] == run_end[0] and entry[1] == run_end[1] + 1 and entry[2] == run_end[2]
                   and entry[3] == run_end[3] + 1 and entry[4] == run_end[4])
        if not follows:
            out.append(run_start + (run_end[1] - run_start[1] + 1,))
            run_start = entry
        run_end = entry
    out.append(run_start + (run_end[1] - run_start[1] + 1,))
    return out


def _spread_over_channels(intervals, num_chans):
    """Distribute intervals over ``num_chans`` channels with near-equal chunk totals, splitting
    an interval when nothing of the right size is left.  Returns interval + (channel,)."""
    pending = sorted(intervals, key=lambda x: x[-1])
    sizes = [x[-1] for x in pending]
    total = sum(sizes)
    quota = [total // num_chans + (1 if c < total % num_chans else 0) for c in range(num_chans)]
    placed = []
    chan = 0
    while pending:
        pick = -1
        if quota[chan] < sizes[-1]:
            at = bisect.bisect_left(sizes, quota[chan])
            if at < len(sizes) and sizes[at] == quota[chan]:
                pick = at
        sb, so, db, do, kind, cnt = pending.pop(pick)
        sizes.pop(pick)
        if cnt > quota[chan]:
            rest = cnt - quota[chan]
            cnt = quota[chan]
            at = bisect.bisect_left(sizes, rest)
            pending.insert(at, (sb, so + cnt, db, do + cnt, kind, rest))
            sizes.insert(at, rest)
        placed.append((sb, so, db, do, kind, cnt, chan))
        quota[chan] -= cnt
        assert quota[chan] >= 0
        if quota[chan] == 0:
            chan += 1
    return placed


def ncclize(algorithm, remap_scratch=None, channel_policy=ChannelPolicy.MatchTopology, pretty_print=True,
            use_scratch=True, merge_contiguous=True, greedy_scratch_sorting=False, instances=1,
            logging=False, copy_threadblocks=1):
    """Return the MSCCL-IR XML text (proto ``Simple``, ``inplace="0"``) for ``algorithm``.

    ``copy_threadblocks``: the local copies of a rank (input to scratch before, input or scratch to output
    after) run on this many threadblocks, each taking an equal share of every copy's chunks.  1 is the
    reference layout (one copy threadblock per rank, reference ncclize.py:622-630); on an executor that
    gives every threadblock its own SM a single block copying a large buffer becomes the critical path,
    and ``copy_threadblocks=instances`` removes it."""
    if algorithm.is_pipelined():
        raise ValueError('Pipelining is not supported.')
    if remap_scratch is None:
        remap_scratch = algorithm.instance.extra_memory is not None
        if remap_scratch and logging:
            print('Turning scratch remapping on to honor the memory limit set in the instance.')

    # 1. buffers
    gpus = {}
    for rank in algorithm.ranks():
        ins = {a: i for i, a in enumerate(sorted(algorithm.input_map.get(rank, ())))}
        outs = {a: i for i, a in enumerate(sorted(algorithm.output_map.get(rank, ())))}
        gpus[rank] = _Gpu([], [], ins, outs, len(ins), len(outs))
    for step in algorithm.steps:
        for addr, src, dst in step.sends:
            for g in (gpus[src], gpus[dst]):
                if addr not in g.inputs and addr not in g.outputs and addr not in g.scratch:
                    g.scratch[addr] = len(g.scratch)

    # 2. scratch policy
    if remap_scratch:
        _remap_scratch_into_input_output(_liveness(gpus, algorithm), gpus, logging)
        if algorithm.collective.is_combining:
            raise RuntimeError('Combining collectives are not supported yet with scratch remapping.')
    elif greedy_scratch_sorting:
        _greedy_scratch_sort(algorithm, gpus)
    else:
        for g in gpus.values():
            g.scratch = {a: i for i, a in enumerate(sorted(g.scratch))}

    # addresses that are both input and output stay in the input buffer and are copied at the end
    for rank, g in gpus.items():
        for addr in list(g.inputs):
            if addr in g.outputs:
                g.postcopies.append(_local_copy(rank, 'i', g.inputs[addr], 'o', g.outputs[addr]))
                del g.outputs[addr]
    for g in gpus.values():
        _merge_copies(g.precopies)
        _merge_copies(g.postcopies)
        if instances > 1:
            for cp in itertools.chain(g.precopies, g.postcopies):
                cp.src_offset *= instances
                cp.dst_offset *= instances
                cp.cnt *= instances
        if copy_threadblocks > 1:
            for copies in (g.precopies, g.postcopies):
                pieces = []
                for cp in copies:
                    share = -(-cp.cnt // copy_threadblocks)
                    for slot, first in enumerate(range(0, cp.cnt, share)):
                        piece = _Op(cp.gpu, None, cp.step, False, 'cpy', cp.src_buffer, cp.src_offset + first,
                                    cp.dst_buffer, cp.dst_offset + first, min(share, cp.cnt - first), [])
                        piece.copy_slot = slot
                        pieces.append(piece)
                copies[:] = pieces

    # 3-5. ops with dependencies
    by_channel = defaultdict(list)
    last_writers = defaultdict(list)
    readers_since = defaultdict(list)
    holds_data = [set(itertools.chain((('i', off) for off in g.inputs.values()),
                                      ((c.dst_buffer, c.dst_offset) for c in g.precopies)))
                  for g in gpus.values()]
    for rank, g in gpus.items():
        for cp in g.precopies:
            for i in range(cp.cnt):
                readers_since[(rank, cp.src_buffer, cp.src_offset + i)].append(cp)
                last_writers[(rank, cp.dst_buffer, cp.dst_offset + i)].append(cp)

    combining = algorithm.collective.is_combining
    chunked = algorithm.collective.chunk_up(algorithm.instance.chunks)
    content = {rank: defaultdict(frozenset) for rank in gpus}
    for c in chunked.chunks():
        for rank in chunked.ranks():
            if chunked.precondition(rank, c):
                content[rank][chunked.address(c)] = content[rank][chunked.address(c)] | {c}
    xml_step = 0
    for algo_step in algorithm.steps:
        # Serialise multiple arrivals at one destination slot into sub-steps and decide whether
        # an arrival overwrites ('r') or is added ('rrc').  ``content`` tracks which chunks of the
        # collective each (rank, address) currently holds: an arrival that already contains what
        # the slot holds replaces it (the all-gather half of an all-reduce), an arrival with
        # disjoint content is reduced into it.  (The reference reduces whenever the slot was
        # written before, which double counts in composed all-reduces.)
        sent_content = {(addr, src): content[src].get(addr, frozenset()) for addr, src, _dst in algo_step.sends}
        arrivals = defaultdict(list)
        for addr, src, dst in algo_step.sends:
            arrivals[(dst,) + gpus[dst].locate(addr)].append((src, addr))
        substeps = []
        for (dst, dbuf, doff), senders in arrivals.items():
            for k, (src, addr) in enumerate(senders):
                incoming = sent_content[(addr, src)]
                present = content[dst].get(addr, frozenset())
                fresh = k == 0 and (dbuf, doff) not in holds_data[dst]
                if fresh or not combining or present <= incoming:
                    kind, merged = 'r', incoming
                elif not (present & incoming):
                    kind, merged = 'rrc', present | incoming
                else:
                    raise RuntimeError(f'step {xml_step + 1}: address {addr} arriving at rank {dst} from rank {src} '
                                       'partly overlaps what the rank already reduced (would double count)')
                content[dst][addr] = merged
                while len(substeps) <= k:
                    substeps.append([])
                substeps[k].append((addr, src, dst, kind))

        for transfers in substeps:
            per_edge = defaultdict(list)
            for addr, src, dst, kind in transfers:
                per_edge[(src, dst)].append((addr, kind))
            wire = []
            for (src, dst), items in per_edge.items():
                spans = _intervals(gpus, src, dst, items, merge_contiguous)
                if channel_policy == ChannelPolicy.One:
                    spans = [s + (0,) for s in spans]
                elif channel_policy == ChannelPolicy.MatchTopology:
                    spans = _spread_over_channels(spans, algorithm.topology.link(src, dst))
                else:
                    raise AssertionError('Unhandled channel policy')
                for sb, so, db, do, kind, cnt, chan in spans:
                    for i in range(instances):
                        wire.append((src, dst, sb, so * instances + i * cnt, db, do * instances + i * cnt,
                                     kind, cnt, chan * instances + i))
            fresh_writers = defaultdict(list)
            fresh_readers = defaultdict(list)
            for src, dst, sb, so, db, do, kind, cnt, chan in wire:
                reads = [(src, sb, so + i) for i in range(cnt)]
                writes = [(dst, db, do + i) for i in range(cnt)]
                send_waits = list(dict.fromkeys(d for k in reads for d in last_writers[k]))
                recv_waits = list(dict.fromkeys(d for table in (readers_since, last_writers)
                                                for k in writes for d in table[k]))
                send_op = _Op(src, dst, xml_step, True, 's', sb, so, db, do, cnt, send_waits)
                recv_op = _Op(dst, src, xml_step, False, kind, sb, so, db, do, cnt, recv_waits)
                by_channel[chan] += [send_op, recv_op]
                for k in writes:
                    fresh_writers[k].append(recv_op)
                for k in reads:
                    fresh_readers[k].append(send_op)
            for key, ops in fresh_writers.items():
                if key in fresh_readers:
                    g, buf, off = key
                    raise RuntimeError(f'Encountered receive and send on the same buffer index on step '
                                       f'{xml_step + 1} (gpu={g}, buf={buf}, off={off})')
                last_writers[key] = ops
                readers_since[key] = []
            for key, ops in fresh_readers.items():
                readers_since[key].extend(ops)
            for src, dst, sb, so, db, do, kind, cnt, chan in wire:
                holds_data[dst].add((db, do))
            xml_step += 1

    for rank, g in gpus.items():
        for cp in g.postcopies:
            for i in range(cp.cnt):
                cp.depends.extend(last_writers[(rank, cp.src_buffer, cp.src_offset + i)])
                cp.depends.extend(readers_since[(rank, cp.dst_buffer, cp.dst_offset + i)])
                cp.depends.extend(last_writers[(rank, cp.dst_buffer, cp.dst_offset + i)])

    if instances > 1:
        def widen(table):
            return {a * instances + i: idx * instances + i for a, idx in table.items() for i in range(instances)}
        for g in gpus.values():
            g.inputs, g.outputs, g.scratch = widen(g.inputs), widen(g.outputs), widen(g.scratch)
            g.input_chunks *= instances
            g.output_chunks *= instances

    # 6. threadblocks
    groups = defaultdict(list)
    for chan, ops in by_channel.items():
        for op in ops:
            groups[(op.gpu, op.is_send, op.peer, chan)].append(op)
    pools = defaultdict(lambda: defaultdict(list))
    for (rank, is_send, peer, chan), ops in groups.items():
        steps_used = {op.step for op in ops}
        home = None
        for tb in pools[rank][chan]:
            current = tb.send if is_send else tb.recv
            if current in (-1, peer) and not any(o.step in steps_used for o in tb.steps):
                home = tb
                break
        if home is None:
            home = _Threadblock(chan)
            pools[rank][chan].append(home)
        if is_send:
            assert home.send in (-1, peer)
            home.send = peer
        else:
            assert home.recv in (-1, peer)
            home.recv = peer
        home.steps.extend(ops)

    for rank, g in gpus.items():
        g.threadblocks = sorted((tb for tbs in pools[rank].values() for tb in tbs),
                                key=lambda tb: (tb.send, tb.recv, tb.channel))
        slots = sorted({getattr(cp, 'copy_slot', 0) for cp in g.precopies + g.postcopies} | {0})
        for slot in slots:
            copies = _Threadblock(0)
            copies.steps = [cp for cp in g.precopies + g.postcopies if getattr(cp, 'copy_slot', 0) == slot]
            g.threadblocks.append(copies)
        for i, tb in enumerate(g.threadblocks):
            tb.rbid = i
            for op in tb.steps:
                op.block_rbid = i
    for g in gpus.values():
        for tb in g.threadblocks:
            for op in tb.steps:
                op.depends = [d for d in dict.fromkeys(op.depends) if d.block_rbid != op.block_rbid]
                for d in op.depends:
                    d.has_dependence = True
    for g in gpus.values():
        for tb in g.threadblocks:
            tb.steps.sort(key=lambda op: op.step)
            for op in tb.steps:
                for extra in op.depends[1:]:
                    tb.ops.append(_Op(op.gpu, None, op.step, False, 'nop', None, None, None, None, 0, [extra]))
                op.depends = op.depends[:1]
                tb.ops.append(op)
            for i, op in enumerate(tb.ops):
                op.idx = i

    # emit
    nchannels = 1 + max(tb.channel for g in gpus.values() for tb in g.threadblocks)
    algorithm.nchannels = nchannels
    algo = ET.Element('algo')
    algo.set('name', algorithm.name)
    algo.set('proto', 'Simple')
    algo.set('nchannels', str(nchannels))
    algo.set('ngpus', str(len(gpus)))
    algo.set('inplace', '0')
    algo.set('coll', algorithm.collective.runtime_name)
    algo.set('nchunksperloop', str(max(max(g.input_chunks, g.output_chunks) for g in gpus.values())))
    for rank, g in gpus.items():
        ge = ET.SubElement(algo, 'gpu')
        ge.set('id', str(rank))
        ge.set('i_chunks', str(g.input_chunks))
        ge.set('o_chunks', str(g.output_chunks))
        ge.set('s_chunks', str(g.scratch_size()))
        for tb in g.threadblocks:
            te = ET.SubElement(ge, 'tb')
            te.set('id', str(tb.rbid))
            te.set('send', str(tb.send))
            te.set('recv', str(tb.recv))
            te.set('chan', str(tb.channel))
            for op in tb.ops:
                if not use_scratch:
                    # scratch is addressed as the tail of the output buffer
                    if op.src_buffer == 's':
                        op.src_buffer, op.src_offset = 'o', op.src_offset + g.output_chunks
                    if op.dst_buffer == 's':
                        op.dst_buffer, op.dst_offset = 'o', op.dst_offset + g.output_chunks
                se = ET.SubElement(te, 'step')
                se.set('s', str(op.idx))
                se.set('type', op.op_type)
                se.set('srcbuf', op.src_buffer if op.src_buffer is not None else 'i')
                se.set('srcoff', str(op.src_offset) if op.src_buffer is not None else '-1')
                se.set('dstbuf', op.dst_buffer if op.dst_buffer is not None else 'o')
                se.set('dstoff', str(op.dst_offset) if op.dst_buffer is not None else '-1')
                se.set('cnt', str(op.cnt))
                assert len(op.depends) <= 1
                se.set('depid', str(op.depends[0].block_rbid) if op.depends else '-1')
                se.set('deps', str(op.depends[0].idx) if op.depends else '-1')
                se.set('hasdep', '1' if op.has_dependence else '0')
    if pretty_print:
        ET.indent(algo, space='  ')
    return ET.tostring(algo, encoding='unicode')
