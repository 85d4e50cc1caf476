"""Cross-threadblock dependency inference and scratch placement.

Parity: reference ``msccl/language/rank_dag.py:262-294``.
"""
from msccl.language.mscclir import Buffer, Instruction


def infer_dependencies(dag):
    """An op depends on its DAG predecessors.  Per predecessor threadblock only the latest
    step matters because a threadblock runs its steps in order."""
    for op in dag.all_ops:
        latest = {}
        for before in op.prev:
            if before.inst == Instruction.start:
                continue
            held = latest.get(before.tb)
            if held is None or before.step > held.step:
                latest[before.tb] = before
        op.depends = list(latest.values())


def place_scratch_slices(dag, instances):
    """Lay the named scratch slices of each rank end to end in one scratch buffer, leaving
    room for ``instances`` copies of each."""
    for per_rank in dag.buffers:
        offset = 0
        for key, piece in per_rank.items():
            if key is Buffer.input or key is Buffer.output:
                continue
            piece.set_offset(offset)
            offset += piece.instance_size() * instances
