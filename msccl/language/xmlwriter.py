"""MSCCL-IR XML emission for lowered MSCCLang programs.

Output format parity: reference ``msccl/language/ir.py:211-395`` - the same element and
attribute names in the same order, so files are interchangeable:

    <algo name proto nchannels nchunksperloop ngpus coll inplace>
      <gpu id i_chunks o_chunks s_chunks>
        <tb id send recv chan>
          <step s type srcbuf srcoff dstbuf dstoff cnt depid deps hasdep/>
"""
import xml.etree.ElementTree as ET
from collections import defaultdict

from msccl.language.mscclir import (Buffer, Instruction, LOCAL_DST_INSTS, LOCAL_SRC_INSTS, Op,
                                    Program)


def _buffer_extents(program):
    """Largest index+size touched on each (rank, buffer) by ops that address local memory."""
    extent = defaultdict(int)
    for gpu in program.gpus:
        for tb in gpu.threadblocks:
            for op in tb.ops:
                if op.inst in LOCAL_SRC_INSTS and op.src is not None:
                    key = (gpu.rank, op.src.buffer)
                    extent[key] = max(extent[key], op.src.index + op.src.size)
                if op.inst in LOCAL_DST_INSTS and op.dst is not None:
                    key = (gpu.rank, op.dst.buffer)
                    extent[key] = max(extent[key], op.dst.index + op.dst.size)
    return extent


def _prune_dependencies(program, tb_id):
    """Drop dependencies on the own threadblock and those already implied by an earlier op of
    the same threadblock waiting on the same op."""
    home = {op: tb_id[tb] for gpu in program.gpus for tb in gpu.threadblocks for op in tb.ops}
    for gpu in program.gpus:
        for tb in gpu.threadblocks:
            waited = set()
            for op in tb.ops:
                kept = [d for d in op.depends if home[d] != tb_id[tb] and d not in waited]
                waited.update(kept)
                op.depends = kept
    return home


def _hoist_reduce_dependencies(program):
    """``dependence_nop`` mode: move every cross-threadblock dependency of the local reduces
    of a threadblock in front of the first reduce (as nops), so that the run of reduces
    itself is dependency-free and can be batched by the executor."""
    for gpu in program.gpus:
        for tb in gpu.threadblocks:
            head, tail = [], []
            first_reduce = None
            first_dep = None
            for op in tb.ops:
                if op.inst is Instruction.reduce:
                    for dep in op.depends:
                        if first_dep is None:
                            first_dep = dep
                        else:
                            head.append(Op(Instruction.nop, -1, None, None, [dep]))
                    op.depends = []
                    if first_reduce is None:
                        first_reduce = op
                (tail if first_reduce is not None else head).append(op)
            if first_dep is not None:
                first_reduce.depends = [first_dep]
            tb.ops = head + tail


def _expand_extra_dependencies(program):
    """A step can wait on one (tb, step) only: extra waits become preceding nops.  Returns the
    final step index of every op."""
    position = {}
    for gpu in program.gpus:
        for tb in gpu.threadblocks:
            laid_out = []
            for op in tb.ops:
                if len(op.depends) > 1:
                    for extra in op.depends[1:]:
                        laid_out.append(Op(Instruction.nop, -1, None, None, [extra]))
                    op.depends = op.depends[:1]
                laid_out.append(op)
            for i, op in enumerate(laid_out):
                position[op] = i
            tb.ops = laid_out
    return position


def ir_to_xml(program: Program, old_format=True, use_scratch=True, pretty_print=True,
              dependence_nop=False):
    extent = _buffer_extents(program)

    # Threadblocks that drive the same connection sit next to each other.
    tb_id = {}
    for gpu in program.gpus:
        gpu.threadblocks = sorted(gpu.threadblocks, key=lambda tb: (tb.send, tb.recv, tb.channel))
        for i, tb in enumerate(gpu.threadblocks):
            tb_id[tb] = i

    home = _prune_dependencies(program, tb_id)
    waited_on = {d for gpu in program.gpus for tb in gpu.threadblocks for op in tb.ops for d in op.depends}
    if dependence_nop:
        _hoist_reduce_dependencies(program)
    position = _expand_extra_dependencies(program)

    nchannels = max((tb.channel + 1 for gpu in program.gpus for tb in gpu.threadblocks), default=0)
    algo = ET.Element('algo')
    algo.set('name', program.name)
    algo.set('proto', program.protocol)
    algo.set('nchannels', str(nchannels))
    if old_format:
        per_loop = max((max(extent[(g.rank, Buffer.input)], extent[(g.rank, Buffer.output)])
                        for g in program.gpus), default=0)
        algo.set('nchunksperloop', str(per_loop))
    algo.set('ngpus', str(len(program.gpus)))
    algo.set('coll', program.collective)
    algo.set('inplace', '1' if program.inplace else '0')

    step_tag, index_attr = ('step', 's') if old_format else ('op', 'step')
    for gpu in program.gpus:
        g = ET.SubElement(algo, 'gpu')
        g.set('id', str(gpu.rank))
        g.set('i_chunks', str(max(extent[(gpu.rank, Buffer.input)], gpu.input_chunks)))
        g.set('o_chunks', str(max(extent[(gpu.rank, Buffer.output)], gpu.output_chunks)))
        g.set('s_chunks', str(max(extent[(gpu.rank, Buffer.scratch)], gpu.scratch_size())))
        out_extent = extent[(gpu.rank, Buffer.output)]
        for tb in gpu.threadblocks:
            t = ET.SubElement(g, 'tb')
            t.set('id', str(tb_id[tb]))
            t.set('send', str(tb.send))
            t.set('recv', str(tb.recv))
            t.set('chan', str(tb.channel))
            for op in tb.ops:
                e = ET.SubElement(t, step_tag)
                e.set(index_attr, str(position[op]))
                e.set('type', str(op.inst))
                if not use_scratch:
                    # runtimes without a scratch buffer keep scratch behind the output buffer
                    for ref in (op.src, op.dst):
                        if ref is not None and ref.buffer == Buffer.scratch:
                            ref.buffer = Buffer.output
                            ref.index += out_extent
                if old_format:
                    e.set('srcbuf', str(op.src.buffer) if op.src is not None else 'i')
                    e.set('srcoff', str(op.src.index) if op.src is not None else '-1')
                    e.set('dstbuf', str(op.dst.buffer) if op.dst is not None else 'o')
                    e.set('dstoff', str(op.dst.index) if op.dst is not None else '-1')
                else:
                    ref = op.src if op.is_send() else op.dst
                    if ref is not None:
                        e.set('buf', str(ref.buffer))
                        e.set('off', str(ref.index))
                if old_format or op.cnt() > 1:
                    e.set('cnt', str(op.cnt()))
                assert len(op.depends) <= 1
                if op.depends:
                    e.set('depid', str(home[op.depends[0]]))
                    e.set('deps', str(position[op.depends[0]]))
                elif old_format:
                    e.set('depid', '-1')
                    e.set('deps', '-1')
                if op in waited_on:
                    e.set('hasdep', '1')
                elif old_format:
                    e.set('hasdep', '0')
    if pretty_print:
        ET.indent(algo, space='  ')
    return ET.tostring(algo, encoding='unicode')
