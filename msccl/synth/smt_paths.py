"""SMT encoding of collective algorithms as per-chunk paths through the topology.

Unknowns, for every chunk ``c`` and rank ``r``: the step ``arrive[c,r]`` at which the chunk
becomes available on the rank (0 = held from the start, > steps = never), and for every
link a Boolean ``hop[c,s,d]`` saying the chunk travels ``s -> d``.  A send happens in step
``t`` iff ``hop[c,s,d]`` and ``arrive[c,d] == t + 1``.  Each step additionally has an
integer number of bandwidth ``rounds``.

Behavioural parity: reference ``msccl/path_encoding.py:35-222`` (correctness, combining,
triggers, rounds budget, pipelining, per-group pseudo-Boolean bandwidth limits, optional
memory model), including the sat/unsat boundaries its tests pin down.
"""
from collections import defaultdict

import z3

from msccl.algorithm import Algorithm, Step
from msccl.synth.duality import wrap_try_ncd_reduction


class _Vars:
    """Z3 constants, created on demand and named for readable models."""

    @staticmethod
    def arrive(c, r):
        return z3.Int(f'start_{c}_at_{r}')

    @staticmethod
    def leave(c, r):
        return z3.Int(f'end_{c}_at_{r}')

    @staticmethod
    def hop(c, s, d):
        return z3.Bool(f'send_{c}_from_{s}_to_{d}')

    @staticmethod
    def rounds(t):
        return z3.Int(f'rounds_{t}')

    @staticmethod
    def slot(a, r):
        return z3.Int(f'idx_{a}_at_{r}')

    @staticmethod
    def live_from(a, r):
        return z3.Int(f'addr_start_{a}_at_{r}')

    @staticmethod
    def live_to(a, r):
        return z3.Int(f'addr_end_{a}_at_{r}')


def _sent_in_step(c, s, d, t):
    return z3.And(_Vars.hop(c, s, d), _Vars.arrive(c, d) == t + 1)


class PathEncodingBase:
    def __init__(self, topology, collective):
        self.topology = topology
        self.collective = collective

    # ------------------------------------------------------------ constraints
    def _paths(self, add, inst, coll):
        V = _Vars
        same_address = defaultdict(list)
        for c in coll.chunks():
            same_address[coll.address(c)].append(c)
        for c in coll.chunks():
            siblings = [o for o in same_address[coll.address(c)] if o != c] if coll.is_combining else []
            for r in coll.ranks():
                feeders = list(self.topology.sources(r))
                if coll.precondition(r, c):
                    add(V.arrive(c, r) == 0)
                else:
                    one_feeder = z3.PbEq([(V.hop(c, s, r), 1) for s in feeders], 1)
                    add(z3.Implies(V.arrive(c, r) <= inst.steps, one_feeder))
                if coll.postcondition(r, c):
                    add(V.arrive(c, r) <= inst.steps)
                for s in feeders:
                    h = V.hop(c, s, r)
                    add(z3.Implies(h, V.arrive(c, s) < V.arrive(c, r)))
                    if inst.extra_memory is not None:
                        # the sender must still hold the chunk in the step it sends it
                        add(z3.Implies(h, V.leave(c, s) >= V.arrive(c, r) - 1))
                    for o in siblings:
                        # whatever has already been folded into this address travels along
                        add(z3.Implies(z3.And(h, V.arrive(o, s) < V.arrive(c, r)),
                                       z3.And(V.hop(o, s, r), V.arrive(o, r) == V.arrive(c, r))))
                    for owner in (r, s):
                        t = coll.trigger(owner, c)
                        if t is not None:
                            # a triggered chunk moves in the opposite direction in the same step
                            add(z3.Implies(h, z3.And(V.hop(t, r, s), V.arrive(t, s) == V.arrive(c, r))))

    def _rounds(self, add, inst, period):
        V = _Vars
        for t in range(inst.steps):
            add(V.rounds(t) >= 1)
        add(z3.Sum([V.rounds(t) for t in range(inst.steps)]) <= inst.rounds())
        for t in range(period):
            for twin in range(t + period, inst.steps, period):
                add(V.rounds(t) == V.rounds(twin))

    def _bandwidth(self, add, inst, coll, period):
        V = _Vars
        for srcs, dsts, bw, _name in self.topology.bandwidth_constraints():
            for t in range(period):
                together = range(t, inst.steps, period)
                terms = []
                for s in srcs:
                    for d in dsts:
                        per_address = defaultdict(list)
                        for c in coll.chunks():
                            for tt in together:
                                per_address[coll.address(c)].append(_sent_in_step(c, s, d, tt))
                        # chunks combined at one address cost one unit on the link
                        terms.extend((z3.Or(group), 1) for group in per_address.values())
                for k in range(1, inst.extra_rounds + 2):
                    add(z3.Implies(V.rounds(t) == k, z3.PbLe(terms, bw * k)))

    def _memory(self, add, inst, coll):
        V = _Vars
        for c in coll.chunks():
            for r in coll.ranks():
                if coll.postcondition(r, c):
                    add(V.leave(c, r) > inst.steps)
                else:
                    add(V.leave(c, r) >= V.arrive(c, r))
        for r in coll.ranks():
            every, ins, outs = set(), set(), set()
            for c in coll.chunks():
                a = coll.address(c)
                every.add(a)
                if coll.precondition(r, c):
                    ins.add(a)
                if coll.postcondition(r, c):
                    outs.add(a)
                add(V.live_from(a, r) <= V.arrive(c, r))
                add(V.live_to(a, r) >= V.leave(c, r))
            fixed = [a for a in sorted(ins) if a not in outs] + sorted(outs)
            for position, a in enumerate(fixed):
                add(V.slot(a, r) == position)
            capacity = len(ins) + len(outs) + inst.extra_memory
            pad = 0 if inst.allow_exchange else 1

            def overlap(a, b):
                return z3.And(V.live_from(a, r) - pad < V.live_to(b, r) + pad,
                              V.live_from(b, r) - pad < V.live_to(a, r) + pad)

            for a in every - ins - outs:
                for b in every:
                    if b != a:
                        add(z3.Implies(V.slot(a, r) == V.slot(b, r), z3.Not(overlap(a, b))))
                inside = z3.And(0 <= V.slot(a, r), V.slot(a, r) < capacity)
                add(z3.Implies(V.live_from(a, r) <= inst.steps, inside))

    def _encode(self, solver, inst, coll):
        if inst.pipeline is not None:
            if inst.pipeline <= 0:
                raise ValueError('instance.pipeline must be strictly positive.')
            period = inst.steps - max(inst.steps - inst.pipeline, 0)
        else:
            period = inst.steps
        add = solver.add
        self._paths(add, inst, coll)
        self._rounds(add, inst, period)
        self._bandwidth(add, inst, coll, period)
        if inst.extra_memory is not None:
            self._memory(add, inst, coll)

    # ------------------------------------------------------------------ solve
    def solve(self, instance):
        coll = self.collective.chunk_up(instance.chunks)
        solver = z3.Solver()
        self._encode(solver, instance, coll)
        if solver.check() != z3.sat:
            return None
        model = solver.model()
        per_step = [set() for _ in range(instance.steps)]
        for c in coll.chunks():
            a = coll.address(c)
            for d in coll.ranks():
                for s in self.topology.sources(d):
                    if z3.is_true(model.eval(_Vars.hop(c, s, d))):
                        t = model.eval(_Vars.arrive(c, d), model_completion=True).as_long() - 1
                        if 0 <= t < instance.steps:      # drop sends outside the schedule
                            per_step[t].add((a, s, d))
        steps = [Step(model.eval(_Vars.rounds(t), model_completion=True).as_long(), sorted(per_step[t]))
                 for t in range(instance.steps)]
        return Algorithm.make_implementation(self.collective, self.topology, instance, steps)


PathEncoding = wrap_try_ncd_reduction(PathEncodingBase)
