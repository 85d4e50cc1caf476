"""Instance replication: run ``instances`` copies of the program side by side, each on its
own channels and on its own fraction of every chunk.

Index mapping for copy ``i`` of an op at ``index`` (``size`` chunks):
  scratch slice  -> ``slice_len * i + index``                       (always batched)
  input/output   -> ``index * instances + i * size``   (interleaved: A0 A1 .. B0 B1 ..)
                 or ``len(buffer) * i + index``        (batched:     A0 B0 .. A1 B1 ..)
Channels become ``max_channels * i + channel`` and threadblock ids ``tbid * instances + i``.

Parity: reference ``msccl/language/rank_dag.py:318-378``.
"""
from msccl.language.mscclir import Buffer, ChunkRef, Op, Threadblock


def mixed_size_accesses(dag):
    """Pairs of accesses to the input/output buffers that overlap without covering the same chunks, as
    ``(rank, buffer, (index, size), (index, size))``.  Interleaved replication maps copy ``i`` of an access to
    ``index * instances + i * size``: two accesses of different extent to the same chunks then give their
    copy ``i`` different sub-chunks, and the dependency between them (kept per copy) no longer orders the data
    they share."""
    ranges = {}
    for tbs in dag.tbs:
        for tb in tbs.values():
            for op in tb.ops:
                for ref in (op.src, op.dst):
                    if ref is not None and (ref.buffer is Buffer.input or ref.buffer is Buffer.output):
                        ranges.setdefault((ref.rank, ref.buffer), set()).add((ref.index, ref.size))
    clashes = []
    for (rank, buffer), found in ranges.items():
        ordered = sorted(found)
        for a, (ia, sa) in enumerate(ordered):
            for ib, sb in ordered[a + 1:]:
                if ib >= ia + sa:
                    break
                clashes.append((rank, buffer, (ia, sa), (ib, sb)))
    return clashes


def replicate(dag, instances, interleaved):
    if instances == 1:
        dag.instanced_tbs = dag.tbs
        return
    if interleaved:
        clashes = mixed_size_accesses(dag)
        if clashes:
            rank, buffer, first, second = clashes[0]
            raise RuntimeError(
                f'interleaved replication needs every access to a chunk to have the same extent, but rank {rank} '
                f'{buffer} is accessed as chunks [{first[0]}, {first[0] + first[1]}) and [{second[0]}, {second[0] + second[1]}) '
                f'({len(clashes)} such pairs); use interleaved_replication=False for this program')

    def moved(ref, i):
        if ref is None:
            return None
        if ref.buffer is not Buffer.input and ref.buffer is not Buffer.output:
            index = dag.buffers[ref.rank][ref.buffer].instance_size() * i + ref.index
        elif interleaved:
            index = ref.index * instances + i * ref.size
        else:
            index = len(dag.buffers[ref.rank][ref.buffer]) * i + ref.index
        return ChunkRef(ref.rank, ref.buffer, index, ref.size)

    width = max(dag.num_channels)
    out = [dict() for _ in range(dag.num_ranks)]
    for i in range(instances):
        for rank, tbs in enumerate(dag.tbs):
            for tbid, tb in tbs.items():
                new_id = tbid * instances + i
                clone = Threadblock(width * i + tb.channel, tb.send, tb.recv)
                clone.ops = [Op(op.inst, op.rank, moved(op.src, i), moved(op.dst, i), [], op.step, new_id)
                             for op in tb.ops]
                out[rank][new_id] = clone
    for rank, tbs in enumerate(dag.tbs):
        for tbid, tb in tbs.items():
            for i in range(instances):
                clone = out[rank][tbid * instances + i]
                for op, cop in zip(tb.ops, clone.ops):
                    cop.depends = [out[rank][d.tb * instances + i].ops[d.step] for d in op.depends]
    dag.instanced_tbs = out
