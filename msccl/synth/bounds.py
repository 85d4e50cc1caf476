"""Lower bounds on steps (graph distance) and on rounds per chunk (fractional flow LP).

Parity: reference ``msccl/steps_bound.py:6-44`` and ``msccl/rounds_bound.py:12-76``.
"""
import math
from fractions import Fraction

import z3

from msccl.synth.duality import non_combining_dual
from msccl.topologies import reverse_topology


def _hop_distances(topology):
    """All-pairs hop counts; BFS from every node (links are unweighted for this purpose)."""
    n = topology.num_nodes()
    out_edges = [list(topology.destinations(s)) for s in range(n)]
    table = []
    for origin in range(n):
        dist = [math.inf] * n
        dist[origin] = 0
        wave = [origin]
        while wave:
            nxt = []
            for u in wave:
                for v in out_edges[u]:
                    if dist[v] == math.inf:
                        dist[v] = dist[u] + 1
                        nxt.append(v)
            wave = nxt
        table.append(dist)
    return table


def lower_bound_steps(topology, collective):
    """max over (chunk, required rank) of the distance from the nearest initial holder;
    ``None`` when some requirement is unreachable."""
    dist = _hop_distances(topology)
    bound = 0
    for c in collective.chunks():
        holders = [r for r in collective.ranks() if collective.precondition(r, c)]
        for dst in collective.ranks():
            if collective.postcondition(dst, c):
                nearest = min((dist[src][dst] for src in holders), default=math.inf)
                bound = max(bound, nearest)
    return None if bound == math.inf else bound


def lower_bound_rounds(topology, collective, logging=False):
    """Minimum ``rounds`` such that every chunk can flow (fractionally) from its holders to
    every rank that needs it within ``bw * rounds`` on each link/switch.  Returns a Fraction,
    or ``None`` if infeasible/unknown.  Combining collectives are bounded through their dual
    (raises ``ReductionNotApplicableError`` when none exists, e.g. Allreduce)."""
    shown_collective, shown_topology = collective.name, topology.name
    if collective.is_combining:
        collective = non_combining_dual(collective)
        topology = reverse_topology(topology)

    def flow(c, s, d):
        return z3.Real(f'flow_{c}_from_{s}_to_{d}')

    opt = z3.Optimize()
    for c in collective.chunks():
        for r in collective.ranks():
            outs = [flow(c, r, d) for d in topology.destinations(r)]
            for f in outs:
                opt.add(f >= 0, f <= 1)
            if collective.precondition(r, c):
                continue
            inflow = z3.Sum([flow(c, s, r) for s in topology.sources(r)]) \
                if any(True for _ in topology.sources(r)) else z3.RealVal(0)
            for f in outs:
                opt.add(f <= inflow)       # a relay cannot emit more than it received
            if collective.postcondition(r, c):
                opt.add(inflow == 1)

    rounds = z3.Real('rounds')
    for srcs, dsts, bw, _name in topology.bandwidth_constraints():
        terms = [flow(c, s, d) for s in srcs for d in dsts for c in collective.chunks()]
        if terms:
            opt.add(z3.Sum(terms) <= bw * rounds)
    objective = opt.minimize(rounds)
    verdict = opt.check()
    if verdict == z3.sat:
        value = opt.lower(objective)
        if isinstance(value, z3.IntNumRef):
            bound = Fraction(value.as_long(), 1)
        elif isinstance(value, z3.RatNumRef):
            bound = value.as_fraction()
        else:
            raise RuntimeError(f'Unhandled Z3 numeral type: {type(value)}')
        if logging:
            print(f'{shown_collective} algorithms need at least {bound} rounds in {shown_topology} topology.')
        return bound
    if logging:
        if verdict == z3.unsat:
            print(f'Unsat. {shown_collective} is not implementable in {shown_topology} topology.')
        else:
            print('Unknown. Z3 was not able to solve the lower bound.')
    return None
