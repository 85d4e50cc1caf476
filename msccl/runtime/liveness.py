"""Host-side failure detection between the ranks of one job.

The device side bounds every wait, so a peer that has gone away shows up as a timeout status a few
seconds later.  This module lets the surviving ranks learn about it *before* their next launch:
every rank records in the job's key-value store (the ``torch.distributed`` rendezvous store) that it
is alive (``beat``), that it is leaving on purpose (``leave``) or that it failed (``guard``), and
``require_all`` raises ``PeerLostError`` naming the ranks that left or fell silent.

Nothing here touches a GPU; it is exercised with ``gloo`` ranks on CPU (tests/test_liveness.py) and,
between steps, with NCCL ranks (tests/mp_leave_worker.py).
"""
import contextlib
import time


class PeerLostError(RuntimeError):
    def __init__(self, lost):
        self.lost = dict(lost)
        what = ', '.join(f'rank {r} ({why})' for r, why in sorted(self.lost.items()))
        super().__init__(f'peers are gone: {what}')


class Liveness:
    def __init__(self, store, rank, world, prefix='msccl/live', clock=time.time):
        self.store, self.rank, self.world, self.prefix, self.clock = store, rank, world, prefix, clock
        self.started = clock()

    @classmethod
    def from_default_store(cls, group=None):
        import torch.distributed as dist
        from torch.distributed import distributed_c10d as c10d
        return cls(c10d._get_default_store(), dist.get_rank(group), dist.get_world_size(group))

    def _key(self, kind, rank):
        return f'{self.prefix}/{kind}/{rank}'

    # ---------------------------------------------------------------- what this rank reports
    def beat(self):
        """Record that this rank is alive now."""
        self.store.set(self._key('beat', self.rank), repr(self.clock()))

    def leave(self, reason='left'):
        """Record that this rank stops taking part.  Call it between steps, with nothing in flight."""
        self.store.set(self._key('left', self.rank), str(reason))

    @contextlib.contextmanager
    def guard(self):
        """Report an exception that escapes the block to the other ranks, then re-raise it."""
        try:
            yield self
        except BaseException as e:       # noqa: BLE001 - reported and re-raised
            self.leave(f'{type(e).__name__}: {e}')
            raise

    # ---------------------------------------------------------------- what it learns about others
    def departed(self):
        """{rank: reason} of the ranks that announced their departure (does not block)."""
        out = {}
        for r in range(self.world):
            if r != self.rank and self.store.check([self._key('left', r)]):
                out[r] = self.store.get(self._key('left', r)).decode()
        return out

    def silent(self, max_age):
        """{rank: reason} of the ranks whose last ``beat`` is older than ``max_age`` seconds, or that have
        never reported although this object has existed for longer than that."""
        now, out = self.clock(), {}
        for r in range(self.world):
            if r == self.rank:
                continue
            key = self._key('beat', r)
            if not self.store.check([key]):
                if now - self.started > max_age:       # a peer gets max_age to report for the first time
                    out[r] = 'never reported'
                continue
            age = now - float(self.store.get(key).decode())
            if age > max_age:
                out[r] = f'silent for {age:.1f} s'
        return out

    def require_all(self, max_age=None):
        """Raise ``PeerLostError`` if a peer left, or (with ``max_age``) has not reported in that time."""
        lost = self.departed()
        if max_age is not None:
            for r, why in self.silent(max_age).items():
                lost.setdefault(r, why)
        if lost:
            raise PeerLostError(lost)

    def wait_for_departure(self, timeout, poll=0.05):
        """Poll until some peer has left or ``timeout`` seconds passed; returns ``departed()``."""
        deadline = self.clock() + timeout
        while True:
            gone = self.departed()
            if gone or self.clock() >= deadline:
                return gone
            time.sleep(poll)
