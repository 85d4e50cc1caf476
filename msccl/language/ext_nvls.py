"""MSCCL-IR programs that use the in-switch (NVLS) extension instructions.

The classic instruction set moves data between pairs of GPUs.  An NVSwitch can also sum the same address
of every GPU on a load (``multimem.ld_reduce``) and replicate a store to every GPU (``multimem.st``).  Four
step types, additive to the XML schema and never produced by the classic tool chain, express that:

    bar    the k-th barrier of a channel on one GPU waits for the k-th barrier of that channel on all GPUs
    mmr    local dst  = sum over all GPUs of their (srcbuf, srcoff) slot
    mmb    (dstbuf, dstoff) of every GPU = local src
    mmar   the slot is replaced on every GPU by its sum over all GPUs

``in_switch_allreduce`` / ``in_switch_broadcast`` / ``in_switch_reduce`` add such steps to the
``MSCCLProgram`` in context (with ``Check()`` support); the builders ``allreduce_nvls`` / ``allgather_nvls`` /
``reduce_scatter_nvls`` return the XML text of the three collectives that map onto them.  The CPU interpreter
executes the steps (sum formed in fp32 and rounded once), the validator checks the barrier structure, and
``msccl.runtime.Executor.run`` hands such a program to the native kernel of the same shape on tensors from
``Communicator.symmetric_empty`` (the interpreter kernel itself does not execute these steps).

There is no counterpart in the reference: its instruction set ends at ``re`` (reference
``msccl/language/ir.py:69-83``).
"""
import xml.etree.ElementTree as ET

_KINDS = {'allreduce': 'mmar', 'allgather': 'mmb', 'reduce_scatter': 'mmr'}


def _program(collective, num_ranks, instances, name):
    if num_ranks < 2 or instances < 1:
        raise ValueError('need at least two ranks and one instance')
    per_rank = instances                                   # chunks owned by one rank
    total = num_ranks * per_rank
    inplace = collective != 'reduce_scatter'
    algo = ET.Element('algo')
    algo.set('name', name or f'{collective}_nvls_{num_ranks}')
    algo.set('proto', 'Simple')
    algo.set('nchannels', str(instances))
    algo.set('nchunksperloop', str(total))
    algo.set('ngpus', str(num_ranks))
    algo.set('coll', collective)
    algo.set('inplace', '1' if inplace else '0')
    for rank in range(num_ranks):
        gpu = ET.SubElement(algo, 'gpu')
        gpu.set('id', str(rank))
        if collective == 'allreduce':
            sizes = (total, total)
        elif collective == 'allgather':
            sizes = (per_rank, total)
        else:
            sizes = (total, per_rank)
        gpu.set('i_chunks', str(sizes[0]))
        gpu.set('o_chunks', str(sizes[1]))
        gpu.set('s_chunks', '0')
        for j in range(instances):
            tb = ET.SubElement(gpu, 'tb')
            tb.set('id', str(j))
            tb.set('send', '-1')
            tb.set('recv', '-1')
            tb.set('chan', str(j))
            mine = rank * per_rank + j                     # the chunk this threadblock is responsible for
            if collective == 'allreduce':
                src, dst = ('i', mine), ('i', mine)
            elif collective == 'allgather':
                src, dst = ('o', mine), ('o', mine)        # in place: the own part already sits in the output
            else:
                src, dst = ('i', mine), ('o', j)
            steps = [('bar', ('i', 0), ('i', 0), 0), (_KINDS[collective], src, dst, 1), ('bar', ('i', 0), ('i', 0), 0)]
            for s, (kind, (sbuf, soff), (dbuf, doff), cnt) in enumerate(steps):
                st = ET.SubElement(tb, 'step')
                st.set('s', str(s))
                st.set('type', kind)
                st.set('srcbuf', sbuf)
                st.set('srcoff', str(soff))
                st.set('dstbuf', dbuf)
                st.set('dstoff', str(doff))
                st.set('cnt', str(cnt))
                st.set('depid', '-1')
                st.set('deps', '-1')
                st.set('hasdep', '0')
    ET.indent(algo, space='  ')
    return ET.tostring(algo, encoding='unicode')


def allreduce_nvls(num_ranks, instances=1, name=None):
    """In-place all-reduce: rank r has its 1/n of the buffer summed by the switch and stored to everyone."""
    return _program('allreduce', num_ranks, instances, name)


def allgather_nvls(num_ranks, instances=1, name=None):
    """In-place all-gather: every rank's part of the output is stored to all ranks with one multicast store."""
    return _program('allgather', num_ranks, instances, name)


def reduce_scatter_nvls(num_ranks, instances=1, name=None):
    """Reduce-scatter: rank r reads the sum of everyone's part r through the switch into its own output."""
    return _program('reduce_scatter', num_ranks, instances, name)


# ------------------------------------------------------------------------ DSL surface
# Inside an ``MSCCLProgram`` the three functions below add in-switch steps.  A program is either classic
# (chunk.copy / chunk.reduce) or in-switch: the two kinds of step are ordered against each other only by
# cross-rank barriers, which the classic dependency analysis (per-GPU ``depid/deps``) cannot express, so
# mixing them in one program is refused.  Every rank's k-th in-switch step runs on channel k between two
# barriers; ``Check()`` works as usual because the symbolic buffers are updated.

def _program_in_context():
    from msccl.language import program as prog_module
    prog = prog_module._curr()
    if prog.instr_dag.all_ops:
        raise RuntimeError('in-switch steps cannot be mixed with copy/reduce steps in one program')
    return prog


def _slots(prog, rank, buffer, index, size):
    held, at = prog._resolved(rank, buffer, index)
    if at + size > len(held) or any(held[at + i] is None for i in range(size)):
        raise RuntimeError(f'rank {rank} {buffer}[{index}:{index + size}] holds no data yet')
    return held, at


def in_switch_allreduce(rank, buffer, index, size=1):
    """Issued by ``rank``: the slot is replaced on every rank by its sum over all ranks (``mmar``)."""
    prog = _program_in_context()
    everyone = [_slots(prog, r, buffer, index, size) for r in range(prog.num_ranks)]
    for i in range(size):
        total = everyone[0][0][everyone[0][1] + i]
        for held, at in everyone[1:]:
            total = total.reduce(rank, held[at + i])
        for held, at in everyone:
            held[at + i] = total
    prog.in_switch_ops.append(('mmar', rank, buffer, index, buffer, index, size))


def in_switch_broadcast(rank, buffer, index, size=1):
    """Issued by ``rank``: its slot is stored into the same slot of every rank (``mmb``)."""
    prog = _program_in_context()
    held, at = _slots(prog, rank, buffer, index, size)
    for r in range(prog.num_ranks):
        target, ti = prog._resolved(r, buffer, index)
        for i in range(size):
            target[ti + i] = held[at + i]
    prog.in_switch_ops.append(('mmb', rank, buffer, index, buffer, index, size))


def in_switch_reduce(rank, src_buffer, src_index, dst_buffer, dst_index, size=1):
    """Issued by ``rank``: its local destination becomes the sum over all ranks of the source slot (``mmr``)."""
    prog = _program_in_context()
    everyone = [_slots(prog, r, src_buffer, src_index, size) for r in range(prog.num_ranks)]
    target, ti = prog._resolved(rank, dst_buffer, dst_index)
    for i in range(size):
        total = everyone[0][0][everyone[0][1] + i]
        for held, at in everyone[1:]:
            total = total.reduce(rank, held[at + i])
        target[ti + i] = total
    prog.in_switch_ops.append(('mmr', rank, src_buffer, src_index, dst_buffer, dst_index, size))


def emit_in_switch_program(prog):
    """MSCCL-IR text of a program written with the functions above (called by ``MSCCLProgram.generate_xml``).
    Replication follows the classic compiler: chunk ``i`` of instance ``k`` is chunk ``i * instances + k``
    (interleaved) and runs on its own channel."""
    from msccl.language.mscclir import Buffer
    if not prog.interleaved_replication:
        raise RuntimeError('in-switch programs replicate interleaved only')
    n, inst = prog.num_ranks, prog.instances
    per_rank = [[op for op in prog.in_switch_ops if op[1] == r] for r in range(n)]
    width = max(len(ops) for ops in per_rank)
    if any(op[6] != 1 for op in prog.in_switch_ops):
        # a multi-chunk step is split so that instance replication stays a pure index map
        raise RuntimeError('in-switch steps take one chunk each; issue one step per chunk')
    algo = ET.Element('algo')
    algo.set('name', prog.name)
    algo.set('proto', prog.protocol)
    algo.set('nchannels', str(width * inst))
    sizes = [(len(prog.buffers[r][Buffer.input]) * inst, len(prog.buffers[r][Buffer.output]) * inst) for r in range(n)]
    algo.set('nchunksperloop', str(max(max(a, b) for a, b in sizes)))
    algo.set('ngpus', str(n))
    algo.set('coll', prog.collective.name)
    algo.set('inplace', '1' if prog.collective.inplace else '0')
    for r in range(n):
        gpu = ET.SubElement(algo, 'gpu')
        gpu.set('id', str(r))
        gpu.set('i_chunks', str(sizes[r][0]))
        gpu.set('o_chunks', str(sizes[r][1]))
        gpu.set('s_chunks', '0')
        tb_id = 0
        for j in range(width):
            for k in range(inst):
                tb = ET.SubElement(gpu, 'tb')
                tb.set('id', str(tb_id))
                tb.set('send', '-1')
                tb.set('recv', '-1')
                tb.set('chan', str(j * inst + k))
                tb_id += 1
                steps = [('bar', 'i', 0, 'i', 0, 0)]
                if j < len(per_rank[r]):
                    kind, _, sbuf, soff, dbuf, doff, _ = per_rank[r][j]
                    sbuf, soff = prog.collective.get_buffer_index(r, sbuf, soff)
                    dbuf, doff = prog.collective.get_buffer_index(r, dbuf, doff)
                    steps.append((kind, sbuf.value, soff * inst + k, dbuf.value, doff * inst + k, 1))
                steps.append(('bar', 'i', 0, 'i', 0, 0))
                for s_idx, (kind, sbuf, soff, dbuf, doff, cnt) in enumerate(steps):
                    st = ET.SubElement(tb, 'step')
                    for key, value in (('s', s_idx), ('type', kind), ('srcbuf', sbuf), ('srcoff', soff), ('dstbuf', dbuf),
                                       ('dstoff', doff), ('cnt', cnt), ('depid', -1), ('deps', -1), ('hasdep', 0)):
                        st.set(key, str(value))
    ET.indent(algo, space='  ')
    return ET.tostring(algo, encoding='unicode')


def classify(algo):
    """``'allreduce' | 'allgather' | 'reduce_scatter'`` if ``algo`` (an ``AlgoIR``) is exactly one of the programs
    above (any instance count), else None.  The executor uses it to pick the native kernel."""
    kind = _KINDS.get(algo.coll)
    if kind is None:
        return None
    for gpu in algo.gpus:
        per_rank = len(gpu.tbs)
        if per_rank == 0:
            return None
        for j, tb in enumerate(gpu.tbs):
            if [st.type for st in tb.steps] != ['bar', kind, 'bar'] or tb.send != -1 or tb.recv != -1:
                return None
            st = tb.steps[1]
            mine = gpu.id * per_rank + j
            want = {'mmar': (('i', mine), ('i', mine)), 'mmb': (('o', mine), ('o', mine)), 'mmr': (('i', mine), ('o', j))}[kind]
            if st.cnt != 1 or ((st.srcbuf, st.srcoff), (st.dstbuf, st.dstoff)) != want:
                return None
    return algo.coll
