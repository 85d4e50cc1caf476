"""gloo ranks on CPU for tests/test_host_side_ops.py: a forward and a backward hand-over through all stages."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from msccl.parallel.pipeline import PipelineP2P  # noqa: E402


def main():
    dist.init_process_group('gloo')
    rank, n = dist.get_rank(), dist.get_world_size()
    pipe = PipelineP2P()
    act = torch.full((4,), float(rank))
    prev = torch.full((4,), -1.0)
    pipe.send_next_recv_prev(act if rank + 1 < n else None, prev if rank > 0 else None).wait()
    assert prev[0].item() == (rank - 1 if rank > 0 else -1.0)
    grad = torch.full((4,), 10.0 * rank)
    nxt = torch.full((4,), -1.0)
    pipe.send_prev_recv_next(grad if rank > 0 else None, nxt if rank + 1 < n else None).wait()
    assert nxt[0].item() == (10.0 * (rank + 1) if rank + 1 < n else -1.0)
    dist.barrier()
    print(f'PIPELINE_OK {rank}', flush=True)
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
