"""Symbolic chunks that the DSL moves around while a program is being written.

A ``Chunk`` remembers where it started (and, for collectives that say so, where it
should end up); a ``ReduceChunk`` is the multiset of chunks folded into one value.
``BufferSlice`` is a named, growable scratch region.

Parity: reference ``msccl/language/chunk.py:8-61`` and ``msccl/language/buffer.py:5-40``.
"""
from dataclasses import dataclass, field


@dataclass
class Chunk:
    origin_rank: int
    origin_index: int
    dst_rank: int = -1
    dst_index: int = -1

    def reduce(self, dst, other):
        if isinstance(other, ReduceChunk):
            return other.reduce(dst, self)
        if isinstance(other, Chunk):
            return ReduceChunk(dst, [self, other])
        raise TypeError('Trying to reduce with chunk of None')

    def _key(self):
        return (self.origin_rank, self.origin_index)

    def __hash__(self):
        return hash(self._key())

    def __eq__(self, other):
        return type(other) is Chunk and self._key() == other._key()

    def __lt__(self, other):
        return self._key() < other._key()


@dataclass
class ReduceChunk:
    creation_rank: int
    chunks: list = field(default_factory=list)

    def reduce(self, dst, other):
        if isinstance(other, ReduceChunk):
            return ReduceChunk(self.creation_rank, self.chunks + other.chunks)
        if isinstance(other, Chunk):
            return ReduceChunk(self.creation_rank, self.chunks + [other])
        raise TypeError('Trying to reduce with chunk of None')

    def sort(self):
        self.chunks.sort()

    def __hash__(self):
        return hash((self.creation_rank,) + tuple(sorted(self.chunks)))

    def __eq__(self, other):
        # equality ignores where and in which order the pieces were combined
        return isinstance(other, ReduceChunk) and sorted(self.chunks) == sorted(other.chunks)


class BufferSlice:
    """A named scratch region; indices are local until ``set_offset`` places the slice
    inside the GPU's single scratch buffer."""

    def __init__(self, buf, name):
        self.name = name
        self.buf = buf
        self.offset = -1
        self.chunks = []

    def get_buffer(self):
        return self.buf

    def instance_size(self):
        return len(self.chunks)

    def set_offset(self, offset):
        self.offset = offset

    def get_global_index(self, index):
        assert self.offset > -1, 'set_offset needs to be called first'
        return self.offset + index

    def __getitem__(self, index):
        return self.chunks[index]

    def __setitem__(self, index, value):
        if index >= len(self.chunks):
            self.chunks.extend([None] * (index + 1 - len(self.chunks)))
        self.chunks[index] = value

    def __len__(self):
        return len(self.chunks)
