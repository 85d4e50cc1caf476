"""Pipeline-parallel hand-over of activations (forward) and gradients (backward) between consecutive stages.

Point-to-point pipeline traffic stays on the process group's send/recv (NCCL on GPUs; it is a plain copy
with nothing to fuse) and is issued on a side stream so that it overlaps the stage's compute.  The
all-to-next MSCCLang programs (``msccl.programs.classic.alltonext``, reference
``examples/mscclang/alltonext_forward.py`` / ``alltonext_backward.py``) express the same pattern for
multi-node hand-over through all NICs and run on the interpreter.
"""
import torch
import torch.distributed as dist


class _Done:
    """Stands in for a CUDA event when the tensors live on the host: the transfer has already finished."""

    def wait(self, stream=None):
        return None

    def synchronize(self):
        return None


class PipelineP2P:
    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.stream = torch.cuda.Stream() if torch.cuda.is_available() else None

    def _global(self, rank):
        return dist.get_global_rank(self.group, rank) if self.group is not None else rank

    def _exchange(self, send_tensor, send_to, recv_tensor, recv_from):
        ops = []
        if send_tensor is not None and 0 <= send_to < self.world:
            ops.append(dist.P2POp(dist.isend, send_tensor, self._global(send_to), self.group))
        if recv_tensor is not None and 0 <= recv_from < self.world:
            ops.append(dist.P2POp(dist.irecv, recv_tensor, self._global(recv_from), self.group))
        on_gpu = any(t is not None and t.is_cuda for t in (send_tensor, recv_tensor))
        if not on_gpu or self.stream is None:
            for work in (dist.batch_isend_irecv(ops) if ops else []):
                work.wait()
            return _Done()
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            for work in (dist.batch_isend_irecv(ops) if ops else []):
                work.wait()
            done = torch.cuda.Event()
            done.record(self.stream)
        return done

    def send_next_recv_prev(self, send_tensor, recv_tensor):
        """Forward pass: send activations to stage + 1, receive from stage - 1 (the first stage receives
        nothing, the last sends nothing).  Returns an event; ``event.wait()`` before using ``recv_tensor``."""
        return self._exchange(send_tensor, self.rank + 1, recv_tensor, self.rank - 1)

    def send_prev_recv_next(self, send_tensor, recv_tensor):
        """Backward pass: send gradients to stage - 1, receive from stage + 1."""
        return self._exchange(send_tensor, self.rank - 1, recv_tensor, self.rank + 1)
