"""Synthesized algorithm = ordered steps of (address, src, dst) sends.

Parity: reference ``msccl/algorithm.py:7-137``: ``Step``, ``Algorithm``,
``make_implementation`` (derives the per-rank input/output address maps and
verifies the algorithm against the collective and the topology bandwidth).
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass
from typing import Dict, List, Optional, Set


@dataclass
class Step:
    rounds: int
    sends: list  # [(address, src, dst), ...]


class Algorithm:
    def __init__(self, name, collective, topology, instance, steps,
                 input_map: Optional[Dict[int, Set[int]]] = None,
                 output_map: Optional[Dict[int, Set[int]]] = None):
        self.name = name
        self.collective = collective
        self.topology = topology
        self.instance = instance
        self.steps = steps
        self.input_map = input_map if input_map is not None else {}
        self.output_map = output_map if output_map is not None else {}
        for step in self.steps:
            step.sends = sorted(tuple(s) for s in step.sends)
        self._assert_bandwidth()

    # ---------------------------------------------------------------- build
    @classmethod
    def make_implementation(cls, collective, topology, instance, steps):
        """Wrap ``steps`` as an algorithm for ``collective`` and verify it."""
        chunked = collective.chunk_up(instance.chunks)
        input_map: Dict[int, Set[int]] = {}
        output_map: Dict[int, Set[int]] = {}
        for rank in chunked.ranks():
            ins = {chunked.address(c) for c in chunked.chunks() if chunked.precondition(rank, c)}
            outs = {chunked.address(c) for c in chunked.chunks() if chunked.postcondition(rank, c)}
            if ins:
                input_map[rank] = ins
            if outs:
                output_map[rank] = outs
        name = f'{collective.name}-{topology.name}-{instance}'
        algo = cls(name, collective, topology, instance, steps, input_map, output_map)
        algo.check_implements(chunked)
        if instance.extra_rounds > 0:
            used = algo.extra_rounds()
            if used > instance.extra_rounds:
                raise ValueError(f'steps use {used} extra rounds but only '
                                 f'{instance.extra_rounds} were allowed')
        return algo

    # -------------------------------------------------------------- queries
    def ranks(self):
        return range(self.topology.num_nodes())

    def num_steps(self):
        return len(self.steps)

    def extra_rounds(self):
        return sum(step.rounds for step in self.steps) - len(self.steps)

    def is_pipelined(self):
        return self.instance.pipeline is not None

    # --------------------------------------------------------- verification
    def check_implements(self, collective):
        """Symbolically run the sends on have/have-not state and check the postcondition."""
        if self.topology.num_nodes() != collective.num_nodes:
            raise RuntimeError('topology and collective have different number of nodes')
        by_address = defaultdict(list)
        for c in collective.chunks():
            by_address[collective.address(c)].append(c)
        have = [{c for c in collective.chunks() if collective.precondition(r, c)}
                for r in collective.ranks()]
        for step in self.steps:
            arrivals = [set() for _ in collective.ranks()]
            for addr, src, dst in step.sends:
                for c in by_address[addr]:
                    if c in have[src]:
                        arrivals[dst].add(c)
            for r, new in enumerate(arrivals):
                have[r] |= new
        for r in collective.ranks():
            for c in collective.chunks():
                if collective.postcondition(r, c) and c not in have[r]:
                    raise RuntimeError(f'rank {r} does not get chunk {c} as required by the postcondition')

    def _assert_bandwidth(self):
        n = self.topology.num_nodes()
        usage = []
        for step in self.steps:
            table = [[0] * n for _ in range(n)]
            for _addr, src, dst in step.sends:
                table[dst][src] += 1
            usage.append(table)
        self._link_utilizations = usage
        stride = self.instance.pipeline if self.is_pipelined() else None
        for srcs, dsts, bw, name in self.topology.bandwidth_constraints():
            for i, step in enumerate(self.steps):
                overlapped = range(i, len(self.steps), stride) if stride else (i,)
                used = sum(usage[j][d][s] for j in overlapped for d in dsts for s in srcs)
                assert used <= bw * step.rounds, (
                    f'Step {i} uses {used} bandwidth but constraint {name} only allows for '
                    f'{bw * step.rounds} bandwidth (when rounds={step.rounds}).')

    def __str__(self):
        lines = []
        for i, step in enumerate(self.steps, start=1):
            head = f'(step {i}, rounds={step.rounds}) ' if step.rounds > 1 else f'(step {i}) '
            lines.append(head + ', '.join(f'{c}:{s}→{d}' for c, s, d in step.sends))
        return '\n'.join(lines)
