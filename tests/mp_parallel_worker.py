"""NCCL ranks (one per GPU) for tests/test_multigpu.py: the pipeline hand-over helper and the flat gradient buckets
on real devices.

* ``PipelineP2P``: activations forward and gradients backward through all stages, issued on the helper's side
  stream while a GEMM runs on the main stream; the received values and the GEMM result are both checked.
* ``FlatGradients``: a small model whose gradients live in one registered bucket; ``all_reduce_gradients`` through
  ``msccl.torch.all_reduce`` must agree with ``torch.distributed.all_reduce`` of the same gradients.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import msccl.torch as mt  # noqa: E402
from msccl.parallel.data_parallel import FlatGradients  # noqa: E402
from msccl.parallel.pipeline import PipelineP2P  # noqa: E402


def pipeline(rank, n):
    pipe = PipelineP2P()
    a = torch.randn(2048, 2048, device='cuda')
    b = torch.randn(2048, 2048, device='cuda')
    want = a @ b
    torch.cuda.synchronize()
    for step in range(3):
        act = torch.full((1 << 20,), float(rank + step), device='cuda')
        prev = torch.full((1 << 20,), -1.0, device='cuda')
        done = pipe.send_next_recv_prev(act if rank + 1 < n else None, prev if rank > 0 else None)
        c = a @ b                                   # main stream: overlaps the transfer on the side stream
        done.wait()
        torch.cuda.synchronize()
        assert torch.equal(c, want)
        assert prev[0].item() == (rank - 1 + step if rank > 0 else -1.0) and prev[-1].item() == prev[0].item()
        grad = torch.full((1 << 20,), 10.0 * rank + step, device='cuda')
        nxt = torch.full((1 << 20,), -1.0, device='cuda')
        done = pipe.send_prev_recv_next(grad if rank > 0 else None, nxt if rank + 1 < n else None)
        c = a @ b
        done.wait()
        torch.cuda.synchronize()
        assert torch.equal(c, want)
        assert nxt[0].item() == (10.0 * (rank + 1) + step if rank + 1 < n else -1.0)
    dist.barrier()


def gradients(rank, n):
    torch.manual_seed(0)                            # the same model on every rank
    model = torch.nn.Sequential(torch.nn.Linear(512, 1024), torch.nn.GELU(), torch.nn.Linear(1024, 256)).cuda()
    flat = FlatGradients(model.parameters(), lambda numel, dtype: mt.symmetric_empty(numel, dtype))
    assert len(flat.buckets) == 1
    gen = torch.Generator(device='cuda').manual_seed(100 + rank)
    for step in range(3):
        flat.zero()
        x = torch.randn(64, 512, device='cuda', generator=gen)
        model(x).square().mean().backward()
        reference = [p.grad.clone() for p in model.parameters()]
        for g in reference:
            dist.all_reduce(g)
            g.div_(n)
        flat.all_reduce_gradients(mt.all_reduce, n)
        mt.check()
        for p, g in zip(model.parameters(), reference):
            assert torch.allclose(p.grad, g, rtol=1e-5, atol=1e-6), (step, (p.grad - g).abs().max().item())
    dist.barrier()


def main():
    local = int(os.environ['LOCAL_RANK'])
    torch.cuda.set_device(local)
    dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    rank, n = dist.get_rank(), dist.get_world_size()
    pipeline(rank, n)
    if rank == 0:
        print('PIPELINE_GPU_OK', flush=True)
    mt.init(arena_bytes=64 << 20, fifo_bytes=16 << 20, load_plans=False)
    gradients(rank, n)
    mt.shutdown()
    if rank == 0:
        print('GRADIENTS_GPU_OK', flush=True)
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
