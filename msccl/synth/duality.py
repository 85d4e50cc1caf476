"""Non-combining dual of a combining collective.

A combining collective with a single root per address (Reduce, ReduceScatter) is
the time-reversal of a non-combining one (Broadcast, Allgather-like scatter) on the
reversed topology: swap pre- and postconditions per address, solve, then replay
the steps backwards with sources and destinations exchanged.

Parity: reference ``msccl/ncd_reduction.py:9-69``.
"""
from collections import defaultdict

from msccl.algorithm import Algorithm, Step
from msccl.collectives import build_collective
from msccl.topologies import reverse_topology


class ReductionNotApplicableError(ValueError):
    pass


def non_combining_dual(primal):
    if not primal.is_combining:
        raise ReductionNotApplicableError('The collective is already non-combining.')
    if primal.has_triggers():
        raise ReductionNotApplicableError('The collective has triggers.')
    holders_after = defaultdict(set)   # address -> ranks in some postcondition
    holders_before = defaultdict(set)  # address -> ranks in some precondition
    for c in primal.chunks():
        a = primal.address(c)
        holders_after[a]   # touch so that every address is present
        for r in primal.ranks():
            if primal.postcondition(r, c):
                holders_after[a].add(r)
            if primal.precondition(r, c):
                holders_before[a].add(r)
    if any(len(roots) > 1 for roots in holders_after.values()):
        raise ReductionNotApplicableError(
            'The non-combining reduction is only applicable to collectives with a unique root per address.')
    return build_collective(f'Dual{primal.name}', primal.num_nodes, len(holders_after),
                            lambda r, c: r in holders_after[c],
                            lambda r, c: r in holders_before[c])


def recover_primal_algorithm(dual_algorithm, primal, original_topology, instance):
    steps = [Step(st.rounds, [(addr, dst, src) for addr, src, dst in st.sends])
             for st in reversed(dual_algorithm.steps)]
    return Algorithm.make_implementation(primal, original_topology, instance, steps)


def wrap_try_ncd_reduction(solver_cls):
    """Class decorator: solve the dual on the reversed topology whenever it exists."""

    class NonCombiningReductionWrapper(solver_cls):
        def __init__(self, topology, collective):
            self.primal = collective
            self.original_topology = topology
            try:
                self.dual = non_combining_dual(collective)
            except ReductionNotApplicableError:
                self.dual = None
            if self.dual is not None:
                super().__init__(reverse_topology(topology), self.dual)
            else:
                super().__init__(topology, collective)

        def solve(self, instance):
            found = super().solve(instance)
            if found is None or self.dual is None:
                return found
            return recover_primal_algorithm(found, self.primal, self.original_topology, instance)

    return NonCombiningReductionWrapper
