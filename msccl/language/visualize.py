"""Instruction-DAG export as Graphviz DOT text (nothing is rendered).

The reference ships igraph plotting helpers that are never imported
(``msccl/language/visualize.py:8-102``); text export is the equivalent here.
"""
from msccl.language.mscclir import Instruction


def instruction_dag_dot(dag):
    lines = ['digraph mscclang {', '  rankdir=LR;']
    ids = {}

    def node(op):
        if op not in ids:
            ids[op] = f'n{len(ids)}'
            label = f'{op.inst} r{op.rank}'
            if op.inst != Instruction.start:
                label += f'\\n{op.src.buffer}[{op.src.index}]->{op.dst.buffer}[{op.dst.index}] x{op.cnt()}'
            else:
                label += f'\\n{op.dst.buffer}[{op.dst.index}]'
            lines.append(f'  {ids[op]} [label="{label}"];')
        return ids[op]

    for op in list(dag.start_ops()) + list(dag.all_ops):
        a = node(op)
        for succ in op.next:
            lines.append(f'  {a} -> {node(succ)};')
        if op.is_send() and op.recv_match is not None:
            lines.append(f'  {a} -> {node(op.recv_match)} [style=dashed];')
    lines.append('}')
    return '\n'.join(lines)
