"""Helpers shared by the Alltoall distributors."""


def pair_chunk(src, dst, idx, nodes, chunks):
    """Chunk number, in Alltoall(nodes) split ``chunks`` ways, of piece ``idx`` of the data that
    ``src`` sends to ``dst`` (precondition ``chunk // chunks % nodes == src``, postcondition
    ``chunk // chunks // nodes == dst``)."""
    return (src + dst * nodes) * chunks + idx


def require_plain(*algorithms):
    if any(a.is_pipelined() for a in algorithms):
        raise ValueError('Pipelining is not supported.')
