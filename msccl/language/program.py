"""The MSCCLang surface: ``MSCCLProgram`` context, ``chunk()``, ``Ref.copy/reduce/split/group``,
``XML()``, ``Check()``.

A program is written by moving chunk references between ranks; every move updates a symbolic
copy of all buffers (used by ``Check()``) and adds nodes to the instruction DAG that the
compiler lowers to MSCCL-IR.

Parity: reference ``msccl/language/__init__.py:16-269``.
"""
import os
import sys
import time
from dataclasses import dataclass

from msccl.language.compiler.schedule import auto_assign_tbs, manual_assign_tbs
from msccl.language.compiler.verify import check_dependency_cycles, check_threadblock_ordering
from msccl.language.dag import InstructionDAG
from msccl.language.mscclir import Buffer, ChunkRef, Program, ThreadblockPolicy
from msccl.language.symbolic import BufferSlice
from msccl.language.xmlwriter import ir_to_xml

_PROTOCOLS = ('Simple', 'LL', 'LL128')
_current_program = None


def _curr():
    if _current_program is None:
        raise RuntimeError('No Program in context')
    return _current_program


class MSCCLProgram:
    def __init__(self, name, topo, collective, instances, protocol='Simple',
                 threadblock_policy=ThreadblockPolicy.auto, interleaved_replication=True,
                 instr_fusion=True, check_xml=True, dependence_nop=False):
        assert protocol in _PROTOCOLS, f'Given protocol: {protocol}. Must be either Simple, LL, LL128'
        self.name = name
        self.topo = topo
        self.collective = collective
        self.num_ranks = topo.num_nodes()
        self.instances = instances
        self.protocol = protocol
        self.threadblock_policy = threadblock_policy
        self.interleaved_replication = interleaved_replication
        self.instr_fusion = instr_fusion
        self.check_xml = check_xml
        self.dependence_nop = dependence_nop
        self.run_opt = True
        self.buffers = collective.init_buffers()
        self.instr_dag = InstructionDAG(self.num_ranks, self.buffers)
        self._lowered = None
        self.in_switch_ops = []       # (kind, rank, src buffer, src index, dst buffer, dst index, size), see ext_nvls
        self.pass_times = {}          # compiler pass -> seconds (filled by lower / generate_xml)
        for rank in range(self.num_ranks):
            for index in range(len(self.buffers[rank][Buffer.input])):
                buffer, where = collective.get_buffer_index(rank, Buffer.input, index)
                self.instr_dag.add_start(rank, buffer, where, self.get_ref(rank, buffer, where, 1))

    # ------------------------------------------------------------ context
    def __enter__(self):
        global _current_program
        if _current_program is not None:
            raise RuntimeError('There is already a MSCCL Program in context')
        _current_program = self
        return self

    def __exit__(self, exc_type, exc_value, exc_traceback):
        global _current_program
        if _current_program is not self:
            raise RuntimeError('This program is not currently in context')
        _current_program = None

    # ------------------------------------------------- symbolic execution
    def _resolved(self, rank, buffer, index):
        buffer, index = self.collective.get_buffer_index(rank, buffer, index)
        return self.buffers[rank][buffer], index

    def apply_send(self, src, src_buffer, src_index, dst, dst_buffer, dst_index, size):
        source, si = self._resolved(src, src_buffer, src_index)
        target, di = self._resolved(dst, dst_buffer, dst_index)
        for i in range(size):
            target[di + i] = source[si + i]

    def apply_reduce(self, src, src_buffer, src_index, dst, dst_buffer, dst_index, size):
        source, si = self._resolved(src, src_buffer, src_index)
        target, di = self._resolved(dst, dst_buffer, dst_index)
        for i in range(size):
            target[di + i] = target[di + i].reduce(dst, source[si + i])

    def get_ref(self, rank, buffer, index, size):
        buffer, index = self.collective.get_buffer_index(rank, buffer, index)
        return Ref(rank, buffer, index, size, self)

    def get_chunks(self, rank, buffer, index, size=1):
        held = self.buffers[rank].get(buffer)
        return [held[index + i] if held and index + i < len(held) else None for i in range(size)]

    def check_buffer_exists(self, rank, name):
        if name is not None and name not in self.buffers[rank]:
            self.buffers[rank][name] = BufferSlice(Buffer.scratch, name)

    def _refuse_after_in_switch(self):
        if self.in_switch_ops:
            raise RuntimeError('copy/reduce steps cannot be mixed with in-switch steps in one program')

    def check(self):
        """True iff the symbolic buffers satisfy the collective's postcondition."""
        return self.collective.check(self)

    # ------------------------------------------------------------ lowering
    def _timed(self, name, fn, *args):
        t0 = time.perf_counter()
        out = fn(*args)
        self.pass_times[name] = self.pass_times.get(name, 0.0) + time.perf_counter() - t0
        return out

    def lower(self):
        dag = self.instr_dag
        self._timed('order edges', dag.convert_set_list)
        if self.instr_fusion:
            self._timed('fuse instructions', dag.optimize)
        self._timed('chunk steps and priorities', dag._complete_metadata)
        if self.threadblock_policy == ThreadblockPolicy.manual:
            self._timed('assign threadblocks (manual)', manual_assign_tbs, dag)
        else:
            self._timed('assign threadblocks and channels', auto_assign_tbs, dag)
        self._timed('infer dependencies, place scratch', dag.lower_pt1, self.instances)
        gpus = self._timed('replicate instances', dag.lower_pt2, self.instances, self.interleaved_replication)
        if self.check_xml:
            self._timed('check dependency cycles', check_dependency_cycles, dag.tbs)
            self._timed('check threadblock ordering', check_threadblock_ordering, dag)
        return Program(self.name, self.collective.name, self.collective.inplace, self.protocol, gpus)

    def generate_xml(self):
        # Lowering rewrites the instruction DAG in place, so it runs once and the text is kept.
        if self._lowered is None and self.in_switch_ops:
            from msccl.language.ext_nvls import emit_in_switch_program
            self._lowered = self._timed('write XML', emit_in_switch_program, self)
        if self._lowered is None:
            program = self.lower()
            self._lowered = self._timed('write XML', lambda: ir_to_xml(program, dependence_nop=self.dependence_nop))
            if os.environ.get('MSCCL_PROFILE'):
                print(self.format_pass_times(), file=sys.stderr)
        return self._lowered

    def format_pass_times(self):
        """Wall-clock seconds per compiler pass of the last lowering, one line per pass."""
        total = sum(self.pass_times.values())
        lines = [f'MSCCL: compile passes of {self.name} ({total * 1e3:.1f} ms)']
        lines += [f'  {name:<36} {seconds * 1e3:9.2f} ms' for name, seconds in self.pass_times.items()]
        return '\n'.join(lines)

    def to_dot(self):
        """Graphviz text of the instruction DAG (no rendering)."""
        from msccl.language.visualize import instruction_dag_dot
        return instruction_dag_dot(self.instr_dag)


def chunk(rank, buffer, index, size=1):
    """Reference to ``size`` chunks at (rank, buffer, index), or None if nothing is there yet."""
    prog = _curr()
    if prog.buffers[rank][buffer][index] is None:
        return None
    return prog.get_ref(rank, buffer, index, size)


def create_scratch(rank, name):
    """Create an (empty) named scratch slice on ``rank``."""
    _curr().check_buffer_exists(rank, name)
    return name


def XML():
    print(_curr().generate_xml())


def Check():
    return _curr().check()


def Print():
    """Print the instruction DAG of the current program as Graphviz text."""
    print(_curr().to_dot())


@dataclass
class Ref(ChunkRef):
    prog: MSCCLProgram

    def __hash__(self):
        return hash((self.rank, self.buffer, self.index, self.size))

    def __repr__(self):
        return f'Ref(Buffer:{self.buffer}, Index:{self.index}, Size:{self.size}, Rank:{self.rank})'

    def _end(self):
        return self.index + self.size

    def _get_chunk(self, index):
        return self.prog.buffers[self.rank][self.buffer][index]

    def split(self, num):
        assert self.size % num == 0, f'Trying to split a chunk of {self.size} elements into {num} parts'
        piece = self.size // num
        return [self.prog.get_ref(self.rank, self.buffer, self.index + i * piece, piece)
                for i in range(num)]

    def group(self, other):
        assert self.rank == other.rank, f'Trying to concatenate chunks on ranks {self.rank} and {other.rank}'
        assert self.buffer == other.buffer, f'Trying to concatenate chunks in {self.buffer} and {other.buffer}'
        low = min(self.index, other.index)
        high = max(self._end(), other._end())
        return Ref(self.rank, self.buffer, low, high - low, self.prog)

    def copy(self, dst, buffer=None, index=-1, sendtb=-1, recvtb=-1, ch=-1):
        """Copy these chunks to (dst, buffer, index).  With neither buffer nor index given the
        chunks land in the same place on ``dst``; for a scratch buffer without index they are
        appended.  Returns the destination reference (None for a copy onto itself)."""
        prog = self.prog
        prog._refuse_after_in_switch()
        prog.check_buffer_exists(dst, buffer)
        if index == -1 and buffer is None:
            buffer, index = self.buffer, self.index
        elif index == -1 and buffer is not Buffer.input and buffer is not Buffer.output:
            index = prog.buffers[dst][buffer].instance_size()
        # in-place collectives alias buffers; the alias is resolved from the sender's side
        buffer, index = prog.collective.get_buffer_index(self.rank, buffer, index)
        assert prog.topo.link(self.rank, dst) or dst == self.rank, f'No link from {self.rank} to {dst}'
        target = prog.get_ref(dst, buffer, index, self.size)
        if target == self:
            return None
        prog.apply_send(self.rank, self.buffer, self.index, dst, buffer, index, self.size)
        dag = prog.instr_dag
        if dst != self.rank:
            send = dag.add_send(self.rank, self, target, sendtb, ch)
            recv = dag.add_recv(dst, self, target, recvtb, ch, send)
            send.recv_match = recv
        else:
            dag.add_copy(self.rank, self, target, sendtb, ch)
        return target

    def reduce(self, other_chunkref, sendtb=-1, recvtb=-1, ch=-1):
        """Fold ``other_chunkref`` into these chunks (self is the accumulator); returns self."""
        prog = self.prog
        prog._refuse_after_in_switch()
        src, dst = other_chunkref.rank, self.rank
        assert prog.topo.link(src, dst) or src == dst, f'No link from {src} to {dst}'
        prog.apply_reduce(src, other_chunkref.buffer, other_chunkref.index,
                          dst, self.buffer, self.index, self.size)
        dag = prog.instr_dag
        if src != dst:
            send = dag.add_send(src, other_chunkref, self, sendtb, ch)
            recv = dag.add_recv_reduce_copy(dst, other_chunkref, self, recvtb, ch, send)
            send.recv_match = recv
        else:
            dag.add_reduce(src, other_chunkref, self, sendtb, ch)
        return self

    def get_origin_index(self, index=0):
        return self._get_chunk(index + self.index).origin_index

    def get_origin_rank(self, index=0):
        return self._get_chunk(index + self.index).origin_rank

    def get_dst_index(self, index=0):
        return self._get_chunk(index + self.index).dst_index

    def get_dst_rank(self, index=0):
        return self._get_chunk(index + self.index).dst_rank

    def print_chunk_info(self, index=0):
        print(self._get_chunk(index + self.index))
