"""Collectives as seen by MSCCLang programs: initial symbolic buffers, the expected final
buffers, and the aliasing rule of the in-place variants.

In-place aliasing (``get_buffer_index``):
  AllReduce      output[k] is input[k]
  AllGather      input[k]  is output[rank * chunk_factor + k]
  ReduceScatter  output[k] is input[rank * chunk_factor + k]
  AllToAll       input and output are the same list

Parity: reference ``msccl/language/collectives.py:5-225``.
"""
from msccl.language.mscclir import Buffer
from msccl.language.symbolic import Chunk, ReduceChunk


class Collective:
    """Base class; subclass it (``name`` stays 'custom') to describe any other data movement."""

    def __init__(self, num_ranks, chunk_factor, inplace):
        self.num_ranks = num_ranks
        self.chunk_factor = chunk_factor
        self.inplace = inplace
        self.name = 'custom'

    def init_buffers(self):
        pass

    def check(self, prog):
        pass

    def get_buffer_index(self, rank, buffer, index):
        return buffer, index


def _sum_over_ranks(num_ranks, index):
    return ReduceChunk(-1, [Chunk(r, index) for r in range(num_ranks)])


class AllToAll(Collective):
    def __init__(self, num_ranks, chunk_factor, inplace):
        super().__init__(num_ranks, chunk_factor, inplace)
        self.name = 'alltoall'

    def init_buffers(self):
        cf, width = self.chunk_factor, self.num_ranks * self.chunk_factor
        per_rank = []
        for r in range(self.num_ranks):
            # chunk i goes to rank i // cf and lands at slot (i % cf) + r * cf there
            sendbuf = [Chunk(r, i, i // cf, i % cf + r * cf) for i in range(width)]
            recvbuf = sendbuf if self.inplace else [None] * width
            per_rank.append({Buffer.input: sendbuf, Buffer.output: recvbuf})
        return per_rank

    def check(self, prog):
        cf, ok = self.chunk_factor, True
        for r in range(self.num_ranks):
            out = prog.buffers[r][Buffer.output]
            for peer in range(self.num_ranks):
                for k in range(cf):
                    slot, want = peer * cf + k, r * cf + k
                    got = out[slot]
                    if got is None or got.origin_rank != peer or got.origin_index != want:
                        print(f'Rank {r} chunk {slot} is incorrect should be chunk({peer},{want}) given {got}')
                        ok = False
        return ok


class AllGather(Collective):
    def __init__(self, num_ranks, chunk_factor, inplace):
        super().__init__(num_ranks, chunk_factor, inplace)
        self.name = 'allgather'

    def init_buffers(self):
        cf = self.chunk_factor
        per_rank = []
        for r in range(self.num_ranks):
            mine = [Chunk(r, k, -1, r * cf + k) for k in range(cf)]
            gathered = [None] * (self.num_ranks * cf)
            if self.inplace:
                gathered[r * cf:(r + 1) * cf] = mine
                # the input view is a snapshot used only to find out what a rank starts with
                per_rank.append({Buffer.input: list(mine), Buffer.output: gathered})
            else:
                per_rank.append({Buffer.input: mine, Buffer.output: gathered})
        return per_rank

    def check(self, prog):
        cf, ok = self.chunk_factor, True
        for r in range(self.num_ranks):
            out = prog.buffers[r][Buffer.output]
            for peer in range(self.num_ranks):
                for k in range(cf):
                    slot = peer * cf + k
                    got = out[slot]
                    if got is None:
                        print(f'Rank {r} chunk {slot} is incorrect should be ({peer}, {k}) given None')
                        ok = False
                    elif got.origin_rank != peer or got.origin_index != k:
                        print(f'Rank {r} chunk {slot} is incorrect should be ({peer}, {k}) given '
                              f'({got.origin_rank}, {got.origin_index})')
                        ok = False
        return ok

    def get_buffer_index(self, rank, buffer, index):
        if self.inplace and buffer == Buffer.input:
            return Buffer.output, index + rank * self.chunk_factor
        return buffer, index


class AllReduce(Collective):
    def __init__(self, num_ranks, chunk_factor, inplace):
        super().__init__(num_ranks, chunk_factor, inplace)
        self.name = 'allreduce'

    def init_buffers(self):
        per_rank = []
        for r in range(self.num_ranks):
            data = [Chunk(r, k, -1, k) for k in range(self.chunk_factor)]
            result = data if self.inplace else [None] * self.chunk_factor
            per_rank.append({Buffer.input: data, Buffer.output: result})
        return per_rank

    def check(self, prog):
        where = Buffer.input if self.inplace else Buffer.output
        ok = True
        for r in range(self.num_ranks):
            out = prog.buffers[r][where]
            for k in range(self.chunk_factor):
                got = out[k]
                if got is None or got != _sum_over_ranks(self.num_ranks, k):
                    print(f'Rank {r} chunk {k} is incorrect should be ReduceChunk index {k} from all ranks, given {got}')
                    ok = False
        return ok

    def get_buffer_index(self, rank, buffer, index):
        if self.inplace and buffer == Buffer.output:
            return Buffer.input, index
        return buffer, index


class ReduceScatter(Collective):
    def __init__(self, num_ranks, chunk_factor, inplace):
        super().__init__(num_ranks, chunk_factor, inplace)
        self.name = 'reduce_scatter'

    def init_buffers(self):
        cf = self.chunk_factor
        per_rank = []
        for r in range(self.num_ranks):
            data = [Chunk(r, owner * cf + k, owner, k) for owner in range(self.num_ranks) for k in range(cf)]
            if self.inplace:
                per_rank.append({Buffer.input: data})
            else:
                per_rank.append({Buffer.input: data, Buffer.output: [None] * cf})
        return per_rank

    def check(self, prog):
        cf, ok = self.chunk_factor, True
        where = Buffer.input if self.inplace else Buffer.output
        for r in range(self.num_ranks):
            out = prog.buffers[r][where]
            for k in range(cf):
                which = r * cf + k
                slot = which if self.inplace else k
                got = out[slot]
                if got is None or got != _sum_over_ranks(self.num_ranks, which):
                    print(f'Rank {r} chunk {slot} is incorrect should be index {which} from all ranks given {got}')
                    ok = False
        return ok

    def get_buffer_index(self, rank, buffer, index):
        if self.inplace and buffer == Buffer.output:
            return Buffer.input, index + rank * self.chunk_factor
        return buffer, index
