"""Defining a collective of your own: subclass ``Collective``, say where chunks start
(``init_buffers``) and what the final buffers must hold (``check``).  Here chunk 0 of rank 0 is
broadcast into the output of ranks 1 and 2, first as two direct copies, then as a chain."""
from _common import emit, parser
from msccl.language import Buffer, chunk
from msccl.language.collectives import Collective
from msccl.language.symbolic import Chunk


class FromRankZero(Collective):
    def init_buffers(self):
        return [{Buffer.input: [Chunk(r, c, -1, c) if r == 0 else None for c in range(self.chunk_factor)],
                 Buffer.output: [None] * self.chunk_factor} for r in range(self.num_ranks)]

    def check(self, prog):
        return all(ch is not None and ch.origin_rank == 0 and ch.origin_index == 0
                   for r in range(1, self.num_ranks) for ch in prog.buffers[r][Buffer.output])


def direct():
    c = chunk(0, Buffer.input, 0)
    c.copy(1, buffer=Buffer.output, index=0, sendtb=1, recvtb=1, ch=0)      # explicit threadblocks and channels
    c.copy(2, buffer=Buffer.output, index=0, sendtb=2, recvtb=1, ch=1)


def chained():
    c = chunk(0, Buffer.input, 0).copy(1, buffer=Buffer.output, index=0, sendtb=1, recvtb=1, ch=0)
    c.copy(2, buffer=Buffer.output, index=0, sendtb=2, recvtb=1, ch=1)       # copy() returns the chunk at its new place


args = parser(__doc__).parse_args()
emit('broadcast_direct', FromRankZero(3, 1, inplace=False), direct, execute=args.execute)
emit('broadcast_chained', FromRankZero(3, 1, inplace=False), chained, execute=args.execute)
