"""gloo ranks on CPU for tests/test_liveness.py.  Scenario (argv[1]):

  leave   the last rank announces its departure between two steps and exits; the others learn it from
          the store before their next collective and do not start it
  raise   the last rank raises inside ``guard()``; the others see the exception text
  silent  the last rank stops reporting (a rank that hangs or never joins); the others flag it by age
"""
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from msccl.runtime.liveness import Liveness, PeerLostError  # noqa: E402


def main():
    scenario = sys.argv[1]
    dist.init_process_group('gloo')
    rank, n = dist.get_rank(), dist.get_world_size()
    live = Liveness.from_default_store()
    last = n - 1
    t = torch.ones(4)
    for _ in range(2):                       # two healthy steps
        live.beat()
        live.require_all(max_age=30.0)
        dist.all_reduce(t)
    assert t[0].item() == n * n
    dist.barrier()
    reporting = dist.new_group(list(range(n - 1)))   # the ranks that keep reporting in the 'silent' scenario
    if scenario == 'leave':
        if rank == last:
            live.leave('shutting down')
            print(f'LEFT {rank}', flush=True)
            return                            # no further collective: nothing of this rank is in flight
        gone = live.wait_for_departure(20.0)
        assert gone == {last: 'shutting down'}, gone
    elif scenario == 'raise':
        if rank == last:
            try:
                with live.guard():
                    raise ValueError('bad batch')
            except ValueError:
                print(f'RAISED {rank}', flush=True)
                return
        gone = live.wait_for_departure(20.0)
        assert gone == {last: 'ValueError: bad batch'}, gone
    elif scenario == 'silent':
        if rank == last:
            time.sleep(4.5)                   # alive, but not reporting
            print(f'SILENT {rank}', flush=True)
            return
        for _ in range(16):
            live.beat()
            time.sleep(0.15)
        live.beat()
        dist.barrier(group=reporting)         # both reporting ranks have just reported
        quiet = live.silent(max_age=1.5)
        assert list(quiet) == [last] and quiet[last].startswith('silent for'), quiet
    try:
        live.require_all(max_age=1.5 if scenario == 'silent' else None)
    except PeerLostError as e:
        assert list(e.lost) == [last]
        print(f'DETECTED {rank}: {e}', flush=True)    # and the next collective is never started
        return
    raise AssertionError('the lost peer was not detected')


if __name__ == '__main__':
    main()
