"""``torch.distributed``-shaped entry points backed by the native executor.

    import torch.distributed as dist, msccl, msccl.torch as mt
    dist.init_process_group('nccl'); torch.cuda.set_device(local_rank)
    msccl.init('b200', 1, (msccl.Collective.allreduce, (0, None)))      # optional: registers MSCCL-IR plans
    mt.init(arena_bytes=2 << 30)
    grads = mt.symmetric_empty((n,), torch.bfloat16)                     # registered memory: every path can use it
    mt.all_reduce(grads)

The reference hands its plans to an NCCL fork and the application keeps calling ``torch.distributed``
(reference README.md:20-38); here the same plan table (``MSCCL_CONFIG``) is installed into this
process's ``Executor`` and the calls below dispatch by size and placement: one-shot LL kernels for small
blocks, kernels on symmetric memory for large ones, the registered MSCCL-IR plan otherwise.  Sums only.

A call that no kernel or plan of this process can run (no plan registered for the size, a size that does not divide
into the plan's chunks) is refused on the host before anything is launched; like the reference outside its registered
ranges ("Falling back to NCCL baseline", reference msccl/autosynth/__init__.py:167-168) it then runs on
``torch.distributed``.  ``msccl.torch.init(nccl_fallback=False)`` turns that into the ``PlanError``.
"""
import math
import os

import torch

from msccl.runtime import Communicator, Executor
from msccl.runtime.plan import PlanError

_state = {'comm': None, 'executor': None, 'group': None, 'nccl_fallback': True, 'told': set()}


def init(group=None, arena_bytes=1 << 30, fifo_bytes=256 << 20, load_plans=True, nccl_fallback=True):
    """Create this process's communicator and executor (collective: every rank of ``group`` calls it)."""
    if _state['comm'] is not None:
        raise RuntimeError('msccl.torch is already initialised; call shutdown() first')
    comm = Communicator.from_process_group(group, fifo_bytes=fifo_bytes, arena_bytes=arena_bytes)
    ex = Executor(comm)
    if load_plans and os.environ.get('MSCCL_CONFIG'):
        ex.load_plan_table()
    _state.update(comm=comm, executor=ex, group=group, nccl_fallback=nccl_fallback, told=set())
    return ex


def is_initialized():
    return _state['executor'] is not None


def executor():
    if _state['executor'] is None:
        raise RuntimeError('call msccl.torch.init() after torch.distributed.init_process_group()')
    return _state['executor']


def communicator():
    executor()
    return _state['comm']


def shutdown():
    if _state['comm'] is not None:
        _state['comm'].close()
    _state.update(comm=None, executor=None, group=None)


def symmetric_empty(shape, dtype=torch.bfloat16):
    """A tensor in registered memory at the same offset on every rank (all ranks call this in the same order)."""
    shape = (shape,) if isinstance(shape, int) else tuple(shape)
    flat, _ = communicator().symmetric_empty(math.prod(shape), dtype)
    return flat.view(shape)


def _or_nccl(name, native, library, stream):
    """Run ``native``; a PlanError (raised on the host, before any launch, the same on every rank) sends the call to
    ``library`` on torch.distributed instead."""
    try:
        native()
        return
    except PlanError as err:
        if not _state['nccl_fallback']:
            raise
        if name not in _state['told']:
            _state['told'].add(name)
            print(f'MSCCL: {name}: {err}. Falling back to NCCL baseline.')
    if stream is None:
        library()
    else:
        with torch.cuda.stream(stream):
            library()


def all_reduce(tensor, stream=None):
    """In-place sum over all ranks."""
    import torch.distributed as dist
    if not tensor.is_contiguous():
        raise ValueError('all_reduce needs a contiguous tensor')
    ex, group = executor(), _state['group']
    _or_nccl('all_reduce', lambda: ex.all_reduce(tensor.view(-1), stream=stream),
             lambda: dist.all_reduce(tensor, group=group), stream)
    return tensor


def all_gather_into_tensor(output, input, stream=None):
    """``output`` = concatenation of every rank's ``input`` along dimension 0."""
    import torch.distributed as dist
    ex, group = executor(), _state['group']
    _or_nccl('all_gather_into_tensor', lambda: ex.all_gather(output.view(-1), input.contiguous().view(-1), stream=stream),
             lambda: dist.all_gather_into_tensor(output, input.contiguous(), group=group), stream)
    return output


def reduce_scatter_tensor(output, input, stream=None):
    """``output`` = this rank's slice (along dimension 0) of the sum of every rank's ``input``."""
    import torch.distributed as dist
    ex, group = executor(), _state['group']
    _or_nccl('reduce_scatter_tensor', lambda: ex.reduce_scatter(output.view(-1), input.contiguous().view(-1), stream=stream),
             lambda: dist.reduce_scatter_tensor(output, input.contiguous(), group=group), stream)
    return output


def all_to_all_single(output, input, stream=None):
    """Equal splits along dimension 0: slice ``s`` of ``output`` = slice ``rank`` of rank ``s``'s ``input``."""
    import torch.distributed as dist
    ex, group = executor(), _state['group']
    _or_nccl('all_to_all_single', lambda: ex.all_to_all(output.view(-1), input.contiguous().view(-1), stream=stream),
             lambda: dist.all_to_all_single(output, input.contiguous(), group=group), stream)
    return output


def check():
    """Synchronise and raise if a kernel of this rank reported a timeout."""
    executor().check()


def require_peers(max_age=None):
    """Host-side check before the next step: raises ``PeerLostError`` if a rank has left the job."""
    executor().require_peers(max_age)
