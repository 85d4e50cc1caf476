"""All-gather programs for a single NVSwitch box."""
from msccl.language import Buffer, chunk


def allgather_direct(size, lanes=1):
    """Every rank writes its ``lanes`` input chunks straight into every peer's output (and its
    own).  One step; the algorithm the synthesizer also finds for a fully connected box."""
    for src in range(size):
        for lane in range(lanes):
            c = chunk(src, Buffer.input, lane)
            for dst in range(size):
                c.copy(dst, Buffer.output, src * lanes + lane, ch=lane)


def allgather_ring(size, channels=1):
    """Classic ring all-gather; chunk of rank r travels r -> r+1 -> ... on channel r % channels."""
    for r in range(size):
        c = chunk(r, Buffer.input, 0)
        c = c.copy(r, Buffer.output, r, ch=r % channels)
        for hop in range(1, size):
            c = c.copy((r + hop) % size, Buffer.output, r, ch=r % channels)


def reduce_scatter_direct(size, lanes=1):
    """Direct reduce-scatter (chunk_factor = ``lanes``, out of place): rank r receives block r
    from every peer into scratch and sums it into its output."""
    for owner in range(size):
        for lane in range(lanes):
            idx = owner * lanes + lane
            chunk(owner, Buffer.input, idx).copy(owner, Buffer.output, lane, ch=lane)
            for src in range(size):
                if src != owner:
                    chunk(src, Buffer.input, idx).copy(owner, ('from', src), lane, ch=lane)
            for src in range(size):
                if src != owner:
                    chunk(owner, Buffer.output, lane).reduce(chunk(owner, ('from', src), lane), ch=lane)
