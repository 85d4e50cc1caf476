"""MSCCL-IR programs that use the in-switch (NVLS) extension instructions.

The classic instruction set moves data between pairs of GPUs.  An NVSwitch can also sum the same address
of every GPU on a load (``multimem.ld_reduce``) and replicate a store to every GPU (``multimem.st``).  Four
step types, additive to the XML schema and never produced by the classic tool chain, express that:

    bar    the k-th barrier of a channel on one GPU waits for the k-th barrier of that channel on all GPUs
    mmr    local dst  = sum over all GPUs of their (srcbuf, srcoff) slot
    mmb    (dstbuf, dstoff) of every GPU = local src
    mmar   the slot is replaced on every GPU by its sum over all GPUs

The builders below return the XML text of the three collectives that map onto them; the CPU interpreter
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
