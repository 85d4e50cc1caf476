"""Abstract collective model used by the synthesizer.

A collective is a table of chunks.  Every chunk records the set of ranks that
hold it before the collective runs (``precondition``), the set of ranks that
must hold it afterwards (``postcondition``) and an integer ``address``.  Two
chunks with the same address are *combined* (reduced) when they meet, which is
what makes a collective "combining".

Parity: reference ``msccl/collectives.py:7-155`` (Chunk, Collective,
build_collective and the twelve constructors).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Tuple


@dataclass
class Chunk:
    precondition: set
    postcondition: set
    address: int


class Collective:
    """Pre/postcondition description of a collective over ``num_nodes`` ranks."""

    def __init__(self, name: str, num_nodes: int, chunks: List[Chunk],
                 triggers: Optional[Dict[Tuple[int, int], int]] = None,
                 runtime_name: str = 'custom'):
        self.name = name
        self.num_nodes = num_nodes
        self._chunks = list(chunks)
        self.num_chunks = len(self._chunks)
        self._triggers = dict(triggers) if triggers else {}
        self.runtime_name = runtime_name
        addresses = [c.address for c in self._chunks]
        distinct = set(addresses)
        self.num_addresses = len(distinct)
        # combining <=> at least two chunks alias one address
        self.is_combining = len(distinct) < len(addresses)

    # -- queries ---------------------------------------------------------
    def ranks(self) -> range:
        return range(self.num_nodes)

    def chunks(self) -> range:
        return range(self.num_chunks)

    def precondition(self, rank: int, chunk: int) -> bool:
        return rank in self._chunks[chunk].precondition

    def postcondition(self, rank: int, chunk: int) -> bool:
        return rank in self._chunks[chunk].postcondition

    def address(self, chunk: int) -> int:
        return self._chunks[chunk].address

    def trigger(self, rank: int, chunk: int) -> Optional[int]:
        return self._triggers.get((rank, chunk))

    def has_triggers(self) -> bool:
        return bool(self._triggers)

    # -- transformations -------------------------------------------------
    def chunk_up(self, div: int) -> 'Collective':
        """Split every chunk into ``div`` pieces; piece ``i`` of a chunk at
        address ``a`` lives at address ``a * div + i``."""
        if div < 1:
            raise ValueError('Divisor must be greater or equal to one (and one is a no-op).')
        if div == 1:
            return self
        pieces = [Chunk(c.precondition, c.postcondition, c.address * div + i)
                  for c in self._chunks for i in range(div)]
        return Collective(f'{self.name},chunks={div}', self.num_nodes, pieces)

    def __repr__(self):
        return f'Collective({self.name!r}, nodes={self.num_nodes}, chunks={self.num_chunks})'


def build_collective(name: str, num_nodes: int, num_chunks: int,
                     precondition: Callable[[int, int], bool],
                     postcondition: Callable[[int, int], bool],
                     address: Callable[[int], int] = lambda c: c,
                     trigger: Callable[[int, int], Optional[int]] = lambda r, c: None,
                     runtime_name: str = 'custom') -> Collective:
    """Build a collective from predicate functions over (rank, chunk)."""
    everyone = range(num_nodes)
    chunks = []
    for c in range(num_chunks):
        pre = {r for r in everyone if precondition(r, c)}
        post = {r for r in everyone if postcondition(r, c)}
        chunks.append(Chunk(pre, post, address(c)))
    triggers = {}
    for r in everyone:
        for c in range(num_chunks):
            t = trigger(r, c)
            if t is not None:
                triggers[(r, c)] = t
    return Collective(name, num_nodes, chunks, triggers, runtime_name)


# ---- predicate factories ------------------------------------------------
def _owner_is(n: int, group: int = 1):
    """Chunk c lives on rank (c // group) mod n."""
    return lambda rank, chunk: rank == (chunk // group) % n


def _block_owner(n: int):
    """Chunk c lives on rank c // n (transpose layout)."""
    return lambda rank, chunk: rank == chunk // n


def _everywhere(rank, chunk):
    return True


def _only(root: int):
    return lambda rank, chunk: rank == root


def _cycled(roots):
    return lambda rank, chunk: rank == roots[chunk % len(roots)]


def _fold_address(n: int):
    """All n per-rank contributions of one buffer element share an address."""
    return lambda chunk: chunk // n


def _fmt_roots(roots: Iterable[int]) -> str:
    return ','.join(str(r) for r in roots)


# ---- non-combining ------------------------------------------------------
def broadcast(num_nodes, root):
    return build_collective(f'Broadcast(n={num_nodes},root={root})', num_nodes, 1,
                            _only(root), _everywhere)


def scatter(num_nodes, root):
    return build_collective(f'Scatter(n={num_nodes},root={root})', num_nodes, num_nodes,
                            _only(root), _owner_is(num_nodes))


def gather(num_nodes, root):
    return build_collective(f'Gather(n={num_nodes},root={root})', num_nodes, num_nodes,
                            _owner_is(num_nodes), _only(root))


def allgather(num_nodes):
    return build_collective(f'Allgather(n={num_nodes})', num_nodes, num_nodes,
                            _owner_is(num_nodes), _everywhere, runtime_name='allgather')


def alltoall(num_nodes):
    return build_collective(f'Alltoall(n={num_nodes})', num_nodes, num_nodes * num_nodes,
                            _owner_is(num_nodes), _block_owner(num_nodes),
                            runtime_name='alltoall')


# ---- combining ----------------------------------------------------------
def reduce(num_nodes, root):
    return build_collective(f'Reduce(n={num_nodes},root={root})', num_nodes, num_nodes,
                            _owner_is(num_nodes), _only(root), _fold_address(num_nodes))


def allreduce(num_nodes):
    return build_collective(f'Allreduce(n={num_nodes})', num_nodes, num_nodes,
                            _owner_is(num_nodes), _everywhere, _fold_address(num_nodes),
                            runtime_name='allreduce')


def reduce_scatter(num_nodes):
    return build_collective(f'ReduceScatter(n={num_nodes})', num_nodes, num_nodes * num_nodes,
                            _owner_is(num_nodes), _block_owner(num_nodes),
                            _fold_address(num_nodes), runtime_name='reduce_scatter')


def scan(num_nodes):
    return build_collective(f'Scan(n={num_nodes})', num_nodes, num_nodes,
                            _owner_is(num_nodes),
                            lambda rank, chunk: rank >= chunk % num_nodes,
                            _fold_address(num_nodes))


# ---- multi-root generalisations ------------------------------------------
def multiroot_broadcast(num_nodes, roots):
    return build_collective(f'MultirootBroadcast(n={num_nodes},roots=({_fmt_roots(roots)}))',
                            num_nodes, len(roots), _cycled(roots), _everywhere)


def multiroot_scatter(num_nodes, roots):
    return build_collective(f'MultirootScatter(n={num_nodes},roots=({_fmt_roots(roots)}))',
                            num_nodes, num_nodes * len(roots), _cycled(roots),
                            _owner_is(num_nodes, len(roots)))


def multiroot_gather(num_nodes, roots):
    return build_collective(f'MultirootGather(n={num_nodes},roots=({_fmt_roots(roots)}))',
                            num_nodes, num_nodes * len(roots),
                            _owner_is(num_nodes, len(roots)), _cycled(roots))
