"""A rank leaves a running job between two steps (one process per GPU, launched by tests/test_multigpu.py
with the in-switch reduction off and plain peer loads/stores).  Nothing of the leaving rank is in flight:
all ranks finish their step, synchronise the device and meet at a barrier first.  The others learn of
the departure on the host, from the rendezvous store, and refuse to launch the next step."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from msccl.runtime import Communicator, Executor, PeerLostError  # noqa: E402


def main():
    local = int(os.environ['LOCAL_RANK'])
    torch.cuda.set_device(local)
    dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    rank, n = dist.get_rank(), dist.get_world_size()
    comm = Communicator.from_process_group(fifo_bytes=16 << 20, multicast=False)
    assert not comm.mc_base
    ex = Executor(comm)
    t = torch.full((4096,), float(rank + 1), device='cuda', dtype=torch.float32)
    for _ in range(3):                                   # healthy steps
        ex.require_peers()
        t.fill_(float(rank + 1))
        ex.all_reduce(t, algorithm='oneshot')
        ex.check()
        assert t[0].item() == n * (n + 1) / 2
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    code = 1
    if rank == n - 1:
        comm.leave('preempted')
        print(f'LEFT {rank}', flush=True)
        code = 0
    else:
        gone = comm.liveness.wait_for_departure(30.0)
        try:
            ex.require_peers()                           # what a training loop calls before its next step
        except PeerLostError as e:
            assert e.lost == {n - 1: 'preempted'} and gone == e.lost
            print(f'DETECTED {rank}: {e}', flush=True)
            code = 0
    comm.close()                                         # local: unmaps, frees; no collective
    sys.stdout.flush()
    os._exit(code)                                       # skip NCCL's collective teardown: a peer is gone


if __name__ == '__main__':
    main()
