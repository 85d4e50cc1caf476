"""Instruction DAG built while an MSCCLang program is written.

Every (rank, buffer, index) slot tracks its last writer and the readers since that
write, which yields read-after-write, write-after-read and write-after-write edges.
The compiler passes (``msccl.language.compiler``) then fuse, schedule and lower it.

Parity: reference ``msccl/language/rank_dag.py:30-174`` for construction; the passes
that the reference keeps as methods of its DAG class are separate modules here and
are reachable through same-named methods for compatibility.
"""
from collections import defaultdict

from msccl.language.mscclir import Buffer, ChunkRef, Gpu, Instruction, Op, link


class InstructionDAG:
    def __init__(self, num_ranks, buffers):
        self.num_ranks = num_ranks
        self.buffers = buffers
        self.operations = {}                 # slot -> first op that wrote the slot
        self.last_writer = {}                # slot -> op
        self.last_readers = defaultdict(list)
        self.all_ops = []                    # every non-start op in program order
        self.tbs = [dict() for _ in range(num_ranks)]
        self.tb_mapping = {}
        self.num_channels = [1] * num_ranks
        self.instanced_tbs = None

    # ------------------------------------------------------------- tracking
    def _note_write(self, rank, buffer, index, size, op, also_reads=False):
        before = []
        for i in range(index, index + size):
            slot = (rank, buffer, i)
            if also_reads:
                assert slot in self.last_writer, f'Destination slot has never been written before a reduce {op}'
            self.operations.setdefault(slot, op)
            readers = self.last_readers[slot]
            if readers:
                before.extend(readers)
            elif slot in self.last_writer:
                before.append(self.last_writer[slot])
            self.last_writer[slot] = op
            self.last_readers[slot] = []
        for b in before:
            if b is not op:
                link(b, op)

    def _note_read(self, rank, buffer, index, size, op):
        for i in range(index, index + size):
            slot = (rank, buffer, i)
            assert slot in self.last_writer, f'Slot has never been written before a read-type {op}'
            link(self.last_writer[slot], op)
            self.last_readers[slot].append(op)

    def _new(self, inst, rank, src, dst, tb, ch):
        op = Op(inst, rank, src, dst, tb=tb, channel=ch)
        self.all_ops.append(op)
        return op

    # ---------------------------------------------------------- node makers
    def add_start(self, rank, buffer, index, ref):
        op = Op(Instruction.start, rank, ref, ref, chunk_step=-1)
        self.operations[(rank, buffer, index)] = op
        self.last_writer[(rank, buffer, index)] = op
        return op

    def add_copy(self, rank, send_ref, recv_ref, tb, ch):
        op = self._new(Instruction.copy, rank, send_ref, recv_ref, tb, ch)
        self._note_read(rank, send_ref.buffer, send_ref.index, recv_ref.size, op)
        self._note_write(rank, recv_ref.buffer, recv_ref.index, recv_ref.size, op)
        return op

    def add_reduce(self, rank, send_ref, recv_ref, tb, ch):
        op = self._new(Instruction.reduce, rank, send_ref, recv_ref, tb, ch)
        self._note_read(rank, send_ref.buffer, send_ref.index, recv_ref.size, op)
        self._note_write(rank, recv_ref.buffer, recv_ref.index, recv_ref.size, op, also_reads=True)
        return op

    def add_send(self, rank, send_ref, recv_ref, tb, ch):
        op = self._new(Instruction.send, rank, send_ref, recv_ref, tb, ch)
        self._note_read(rank, send_ref.buffer, send_ref.index, send_ref.size, op)
        return op

    def add_recv(self, rank, send_ref, recv_ref, tb, ch, send_op):
        op = self._new(Instruction.recv, rank, send_ref, recv_ref, tb, ch)
        self._note_write(rank, recv_ref.buffer, recv_ref.index, recv_ref.size, op)
        op.send_match = send_op
        return op

    def add_recv_reduce_copy(self, rank, send_ref, recv_ref, tb, ch, send_op):
        op = self._new(Instruction.recv_reduce_copy, rank, send_ref, recv_ref, tb, ch)
        self._note_write(rank, recv_ref.buffer, recv_ref.index, recv_ref.size, op, also_reads=True)
        op.send_match = send_op
        return op

    def start_ops(self):
        seen = set()
        for op in self.operations.values():
            if op.inst == Instruction.start and op not in seen:
                seen.add(op)
                yield op

    # ------------------------------------------- compatibility entry points
    def convert_set_list(self):
        """Edges are already ordered lists; kept because callers of the reference API invoke it."""

    def optimize(self):
        from msccl.language.compiler.fusion import fuse_instructions
        fuse_instructions(self)

    def _complete_metadata(self):
        from msccl.language.compiler.schedule import annotate_depths
        annotate_depths(self)

    def infer_dependencies(self):
        from msccl.language.compiler.deps import infer_dependencies
        infer_dependencies(self)

    def lower_buffers(self, instances):
        from msccl.language.compiler.deps import place_scratch_slices
        place_scratch_slices(self, instances)

    def lower_pt1(self, instances):
        self.infer_dependencies()
        self.lower_buffers(instances)

    def replicate(self, instances, interleaved):
        from msccl.language.compiler.replicate import replicate
        replicate(self, instances, interleaved)

    def lower_chunk(self, ref):
        if ref is None or ref.buffer is Buffer.input or ref.buffer is Buffer.output:
            return ref
        piece = self.buffers[ref.rank][ref.buffer]
        return ChunkRef(ref.rank, piece.get_buffer(), piece.get_global_index(ref.index), ref.size)

    def lower_tbs(self):
        gpus = []
        for rank, tbs in enumerate(self.instanced_tbs):
            for tb in tbs.values():
                for op in tb.ops:
                    op.src = self.lower_chunk(op.src)
                    op.dst = self.lower_chunk(op.dst)
            gpus.append(Gpu(rank, list(tbs.values())))
        return gpus

    def lower_pt2(self, instances, interleaved):
        self.replicate(instances, interleaved)
        return self.lower_tbs()
