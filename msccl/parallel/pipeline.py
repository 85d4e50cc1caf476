"""Pipeline-parallel hand-over of activations between consecutive stages.

Point-to-point pipeline traffic stays on NCCL send/recv (it is a plain copy with nothing to fuse) and
is issued on a side stream so that it overlaps the stage's compute.  The all-to-next MSCCLang program
(``msccl.programs.classic.alltonext``) expresses the same pattern for multi-node hand-over through all
NICs and runs on the interpreter.
"""
import torch
import torch.distributed as dist


class PipelineP2P:
    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.stream = torch.cuda.Stream()

    def send_next_recv_prev(self, send_tensor, recv_tensor):
        """Send to stage+1 and receive from stage-1 on the side stream; returns an event to wait on."""
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            ops = []
            if self.rank + 1 < self.world and send_tensor is not None:
                ops.append(dist.P2POp(dist.isend, send_tensor, self.rank + 1, self.group))
            if self.rank > 0 and recv_tensor is not None:
                ops.append(dist.P2POp(dist.irecv, recv_tensor, self.rank - 1, self.group))
            for work in (dist.batch_isend_irecv(ops) if ops else []):
                work.wait()
            done = torch.cuda.Event()
            done.record(self.stream)
        return done
