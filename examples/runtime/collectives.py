"""Collectives through the native executor, in ``torch.distributed`` form (one process per GPU):

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/runtime/collectives.py

Small blocks run on the one-shot LL kernels (any memory), large tensors from ``symmetric_empty`` on the
in-switch two-shot all-reduce and the peer-store all-gather / all-to-all, everything else on the MSCCL-IR plans
that ``msccl.init`` registered.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import msccl  # noqa: E402
import msccl.torch as mt  # noqa: E402


def main():
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    rank, n = dist.get_rank(), dist.get_world_size()
    if rank == 0:                                   # plans for tensors that are not in registered memory
        msccl.init('b200' if n == 8 else f'b200x{n}', 1, (msccl.Collective.allreduce, (0, None)), ('allgather', (0, None)))
    config = [os.environ.get('MSCCL_CONFIG')]
    dist.broadcast_object_list(config, src=0)
    if config[0]:
        os.environ['MSCCL_CONFIG'] = config[0]
    ex = mt.init(arena_bytes=512 << 20)

    small = torch.full((1024,), float(rank + 1), device='cuda')
    mt.all_reduce(small)                            # 4 KB: one-shot LL
    big = mt.symmetric_empty(64 << 20, torch.bfloat16)
    big.fill_(1.0)
    mt.all_reduce(big)                              # 128 MB in registered memory: two-shot
    which = ex.last_algorithm
    shard = torch.full((1 << 20,), float(rank), device='cuda', dtype=torch.bfloat16)
    gathered = mt.symmetric_empty(n << 20, torch.bfloat16)
    mt.all_gather_into_tensor(gathered, shard)      # peer stores straight into every rank's `gathered`
    mt.check()
    assert small[0].item() == n * (n + 1) / 2 and big[0].item() == n
    assert gathered.view(n, -1)[:, 0].tolist() == list(range(n))
    if rank == 0:
        print(f'all_reduce 4 KB and 128 MB ({which}), all_gather 2 MB per rank: ok on {n} GPUs')
    mt.shutdown()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
