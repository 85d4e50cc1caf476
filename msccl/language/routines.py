"""Reusable MSCCLang building blocks over a contiguous group of GPUs.

Parity: reference ``msccl/language/routines.py:8-27``.
"""
from msccl.language.mscclir import Buffer
from msccl.language.program import chunk


def allgather_ring_inplace(gpus, gpu_offset=0, index_offset=0, ch=0):
    """Ring all-gather among ranks [gpu_offset, gpu_offset+gpus): each rank's input chunk 0
    travels once around the ring into output[index_offset + position] of every member."""
    for pos in range(gpus):
        rank = gpu_offset + pos
        c = chunk(rank, Buffer.input, 0)
        for hop in range(1, gpus):
            c = c.copy(gpu_offset + (rank + hop) % gpus, Buffer.output, index_offset + pos, ch=0)


def allreduce_ring_inplace(gpus, gpu_offset=0, index_offset=0, ch=0):
    """Ring all-reduce among ranks [gpu_offset, gpu_offset+gpus) on input chunks
    [index_offset, index_offset+gpus): chunk p is reduced around the ring starting at member p,
    then the result is passed around once more."""
    for pos in range(gpus):
        rank = gpu_offset + pos
        index = index_offset + pos
        c = chunk(rank, Buffer.input, index)
        for hop in range(1, gpus):
            c = chunk(gpu_offset + (rank + hop) % gpus, Buffer.input, index).reduce(c, ch=ch)
        for hop in range(gpus - 1):
            c = c.copy(gpu_offset + (rank + hop) % gpus, Buffer.input, index, ch=ch)
