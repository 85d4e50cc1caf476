"""Host-side failure detection (msccl/runtime/liveness.py): unit tests against an in-memory store and
three gloo ranks on CPU where one rank leaves, raises, or falls silent between steps."""
import os
import socket
import subprocess
import sys

import pytest

from msccl.runtime.liveness import Liveness, PeerLostError

HERE = os.path.dirname(os.path.abspath(__file__))


class FakeStore:
    def __init__(self):
        self.data = {}

    def set(self, key, value):
        self.data[key] = value.encode() if isinstance(value, str) else value

    def get(self, key):
        return self.data[key]

    def check(self, keys):
        return all(k in self.data for k in keys)


def test_departure_and_silence_against_a_fake_store():
    store, now = FakeStore(), [100.0]
    ranks = [Liveness(store, r, 3, clock=lambda: now[0]) for r in range(3)]
    for lv in ranks:
        lv.beat()
    ranks[0].require_all(max_age=5.0)
    now[0] = 103.0
    ranks[0].beat()
    ranks[1].beat()
    now[0] = 107.0
    assert list(ranks[0].silent(5.0)) == [2]
    with pytest.raises(PeerLostError) as e:
        ranks[0].require_all(max_age=5.0)
    assert list(e.value.lost) == [2] and 'silent for 7.0 s' in str(e.value)
    late = Liveness(store, 0, 4, clock=lambda: now[0])          # rank 3 never reports
    assert 3 not in late.silent(5.0)
    now[0] = 113.0
    assert late.silent(5.0)[3] == 'never reported'
    ranks[1].leave('node drained')
    assert ranks[0].departed() == {1: 'node drained'}
    assert ranks[1].departed() == {}                      # a rank does not list itself
    with pytest.raises(PeerLostError) as e:
        ranks[2].require_all()
    assert e.value.lost == {1: 'node drained'}


def test_guard_reports_the_exception_and_reraises():
    store = FakeStore()
    a, b = Liveness(store, 0, 2), Liveness(store, 1, 2)
    with pytest.raises(KeyError):
        with a.guard():
            raise KeyError('missing shard')
    assert b.departed() == {0: "KeyError: 'missing shard'"}


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


@pytest.mark.parametrize('scenario', ['leave', 'raise', 'silent'])
def test_three_gloo_ranks(scenario):
    port, world = _free_port(), 3
    procs = []
    for rank in range(world):
        env = dict(os.environ, MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                   LOCAL_RANK=str(rank), OMP_NUM_THREADS='1')
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, 'mp_liveness_worker.py'), scenario], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    assert [p.returncode for p in procs] == [0] * world, '\n'.join(outs)
    assert all(f'DETECTED {r}' in outs[r] for r in range(world - 1)), '\n'.join(outs)
    assert 'DETECTED' not in outs[world - 1]
