"""All-reduce programs.

``allreduce_ring`` and ``allreduce_allpairs`` express the same algorithms as the reference's
``msccl/programs/allreduce_a100_ring.py:10-26`` and ``msccl/programs/allreduce_allpairs.py:6-28``
(identical DSL call sequences, hence identical XML).  ``allreduce_one_shot`` and
``allreduce_two_shot`` are the NVSwitch-era algorithms: every GPU reaches every peer at full
port bandwidth, so one or two fully parallel exchange steps replace the ring's 2(n-1) hops.
"""
from msccl.language import Buffer, chunk


def allreduce_ring(size, channels):
    """In-place ring all-reduce over ``size`` ranks and ``size`` chunks.  Chunk ``i`` rides on
    channel/threadblock ``i % channels``: channels=1 is the classic single ring, channels=size
    gives every chunk its own connection."""
    def lane(i):
        return dict(ch=i % channels, sendtb=i % channels, recvtb=i % channels)

    for hop in range(size - 1):                       # reduce-scatter phase
        for i in range(size):
            holder, nxt = (i + hop) % size, (i + hop + 1) % size
            chunk(nxt, Buffer.input, i).reduce(chunk(holder, Buffer.input, i), **lane(i))
    for hop in range(-1, size - 2):                   # all-gather phase
        for i in range(size):
            holder, nxt = (i + hop) % size, (i + hop + 1) % size
            chunk(holder, Buffer.input, i).copy(nxt, Buffer.input, i, **lane(i))


def allreduce_allpairs(size):
    """In-place all-pairs all-reduce on ``size*size`` chunks: rank r owns block r (``size``
    chunks).  Everybody ships block r to rank r's scratch, rank r reduces the ``size-1``
    received copies into its block using ``size`` threadblocks, then broadcasts the block."""
    for src in range(size):
        for owner in range(size):
            if src != owner:
                chunk(src, Buffer.input, owner * size, size=size).copy(owner, 'scratch', sendtb=owner, recvtb=src)
    for r in range(size):
        for k in range(size * (size - 1)):
            chunk(r, Buffer.input, r * size + k % size).reduce(chunk(r, 'scratch', k), sendtb=k % size)
    for owner in range(size):
        for dst in range(size):
            if owner != dst:
                chunk(owner, Buffer.input, owner * size, size).copy(dst, Buffer.input, owner * size,
                                                                     sendtb=dst, recvtb=owner)


def allreduce_one_shot(size, lanes=1):
    """Latency-optimal all-reduce for small messages (chunk_factor = ``lanes``, in place).
    Every rank pushes its whole buffer into a private scratch slot of every peer (one step, all
    n(n-1) transfers in parallel through NVSwitch) and then sums the n-1 received copies into
    its own buffer.  Sends (n-1)*B per rank, so only worthwhile while latency dominates."""
    for lane in range(lanes):
        for src in range(size):
            for dst in range(size):
                if src != dst:
                    chunk(src, Buffer.input, lane).copy(dst, ('from', src), lane,
                                                        sendtb=dst * lanes + lane, recvtb=src * lanes + lane,
                                                        ch=lane)
    for lane in range(lanes):
        for r in range(size):
            acc = chunk(r, Buffer.input, lane)
            for src in range(size):
                if src != r:
                    # reduce on the threadblock that received the copy: no cross-TB wait needed
                    acc.reduce(chunk(r, ('from', src), lane), sendtb=src * lanes + lane, ch=lane)


def allreduce_two_shot(size, lanes=1):
    """Bandwidth-optimal two-step all-reduce (chunk_factor = ``size*lanes``, in place): a direct
    reduce-scatter (rank r receives block r from every peer and sums it) followed by a direct
    all-gather (rank r writes its reduced block straight into every peer's buffer).  Moves
    2(n-1)/n * B per rank like a ring but in 2 steps instead of 2(n-1)."""
    for lane in range(lanes):
        for owner in range(size):
            for src in range(size):
                if src != owner:
                    idx = owner * lanes + lane
                    chunk(src, Buffer.input, idx).copy(owner, ('from', src), lane,
                                                       sendtb=owner * lanes + lane, recvtb=src * lanes + lane,
                                                       ch=lane)
    for lane in range(lanes):
        for owner in range(size):
            acc = chunk(owner, Buffer.input, owner * lanes + lane)
            for src in range(size):
                if src != owner:
                    acc.reduce(chunk(owner, ('from', src), lane), sendtb=src * lanes + lane, ch=lane)
    for lane in range(lanes):
        for owner in range(size):
            for dst in range(size):
                if dst != owner:
                    idx = owner * lanes + lane
                    chunk(owner, Buffer.input, idx).copy(dst, Buffer.input, idx,
                                                         sendtb=dst * lanes + lane, recvtb=owner * lanes + lane,
                                                         ch=lane)
