"""MSCCL-IR data model: instructions, buffers, chunk references, ops, threadblocks.

Parity: reference ``msccl/language/ir.py:10-200`` (the XML writer lives in
``msccl.language.xmlwriter``).  The instruction mnemonics are the on-disk ``type``
attribute values of MSCCL-IR XML and are therefore fixed.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from enum import Enum
from typing import List, Optional


class _StrEnum(Enum):
    def __str__(self):
        return self.value


class ThreadblockPolicy(_StrEnum):
    auto = 'auto'
    manual = 'manual'


class ChunkInstruction(_StrEnum):
    """Legacy chunk-level opcodes (kept for API compatibility; unused by the compiler)."""
    start = 'start'
    reduce = 'reduce'
    send = 'send'


class Instruction(_StrEnum):
    nop = 'nop'
    send = 's'
    recv = 'r'
    recv_copy_send = 'rcs'
    recv_reduce_send = 'rrs'
    recv_reduce_copy = 'rrc'
    recv_reduce_copy_send = 'rrcs'
    copy = 'cpy'
    reduce = 're'
    delete = 'd'
    start = 'st'
    # --- additive extensions executed by the B200 runtime (never produced by the
    # classic DSL surface; see msccl.language.ext_nvls) ---
    mm_reduce = 'mmr'        # multimem.ld_reduce over all ranks' slot -> local dst
    mm_broadcast = 'mmb'     # local src -> multimem.st into all ranks' slot
    mm_allreduce = 'mmar'    # ld_reduce + st on the same slot (in-switch all-reduce)
    barrier = 'bar'          # cross-rank barrier of the TB's channel


class Buffer(_StrEnum):
    input = 'i'
    output = 'o'
    scratch = 's'

    def __lt__(self, other):
        return self.value < other.value

    def __gt__(self, other):
        return self.value > other.value


_SENDERS = frozenset({Instruction.send, Instruction.recv_copy_send,
                      Instruction.recv_reduce_send, Instruction.recv_reduce_copy_send})
_RECEIVERS = frozenset({Instruction.recv, Instruction.recv_copy_send, Instruction.recv_reduce_send,
                        Instruction.recv_reduce_copy, Instruction.recv_reduce_copy_send})
_FUSED = frozenset({Instruction.recv_copy_send, Instruction.recv_reduce_send,
                    Instruction.recv_reduce_copy_send})
_LOCAL = frozenset({Instruction.copy, Instruction.reduce})
# which side of an op addresses memory of the GPU that executes it
LOCAL_SRC_INSTS = frozenset({Instruction.send, Instruction.copy, Instruction.reduce,
                             Instruction.mm_broadcast})
LOCAL_DST_INSTS = frozenset(_RECEIVERS | _LOCAL | {Instruction.mm_reduce, Instruction.mm_allreduce})


@dataclass
class ChunkRef:
    rank: int
    buffer: object      # Buffer or the name of a scratch slice
    index: int
    size: int

    def __hash__(self):
        return hash((self.rank, self.buffer, self.index, self.size))


_op_serial = itertools.count()


@dataclass(eq=False)
class Op:
    inst: Instruction
    rank: int
    src: Optional[ChunkRef]
    dst: Optional[ChunkRef]
    depends: list = field(default_factory=list)
    step: int = -1            # position inside its threadblock
    tb: int = -1              # threadblock id (user-chosen under the manual policy)
    prev: list = field(default_factory=list)   # DAG predecessors, insertion ordered, unique
    next: list = field(default_factory=list)   # DAG successors, insertion ordered, unique
    num: int = -1
    chunk_step: int = -1      # longest distance from a start op
    priority: int = -1        # longest distance to a sink
    channel: int = -1
    recv_match: Optional['Op'] = None   # for sending ops: the op that receives the data
    send_match: Optional['Op'] = None   # for receiving ops: the op that sent the data
    serial: int = field(default_factory=lambda: next(_op_serial))

    # identity semantics: ops are graph nodes
    def __hash__(self):
        return id(self)

    def __eq__(self, other):
        return self is other

    def cnt(self):
        if self.src is not None:
            if self.dst is not None:
                assert self.src.size == self.dst.size
            return self.src.size
        return self.dst.size if self.dst is not None else 0

    def is_send(self):
        return self.inst in _SENDERS

    def is_recv(self):
        return self.inst in _RECEIVERS

    def is_fused(self):
        return self.inst in _FUSED

    def is_local(self):
        return self.inst in _LOCAL

    def peer(self):
        if self.inst == Instruction.send:
            return self.dst.rank
        if self.inst == Instruction.recv:
            return self.src.rank
        return None

    def send_peer(self):
        return self.dst.rank if self.is_send() else -1

    def recv_peer(self):
        return self.src.rank if self.is_recv() else -1

    def _order_key(self):
        # earlier chunk step first, then higher priority, then lower source index
        return (self.chunk_step, -self.priority, self.src.index if self.src is not None else -1)

    def __lt__(self, other):
        return self._order_key() < other._order_key()

    def __gt__(self, other):
        return not self < other

    def __repr__(self):
        return f'Op({self.inst}, {self.rank}, {self.src}, {self.dst}, step:{self.step}, tb:{self.tb})'


def link(before: Op, after: Op):
    """Add the DAG edge before -> after (idempotent)."""
    if after not in before.next:
        before.next.append(after)
    if before not in after.prev:
        after.prev.append(before)


@dataclass(eq=False)
class Threadblock:
    channel: int = -1
    send: int = -1
    recv: int = -1
    ops: list = field(default_factory=list)
    rbid: int = -1

    def __hash__(self):
        return id(self)

    def __eq__(self, other):
        return self is other


@dataclass
class Gpu:
    rank: int
    threadblocks: list = field(default_factory=list)
    # bookkeeping used by the ncclize lowering
    precopies: list = field(default_factory=list)
    postcopies: list = field(default_factory=list)
    inputs: dict = field(default_factory=dict)
    outputs: dict = field(default_factory=dict)
    input_chunks: int = 0
    output_chunks: int = 0
    scratch: dict = field(default_factory=dict)

    def scratch_size(self):
        return max(self.scratch.values(), default=-1) + 1


@dataclass
class Program:
    name: str
    collective: str
    inplace: bool
    protocol: str
    gpus: List[Gpu] = field(default_factory=list)
