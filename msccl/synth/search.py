"""Search strategies over synthesis instances.

Parity: reference ``msccl/strategies.py:15-159`` including the log lines
(``Solving instance ... synthesized! (x.xs)``) that users and tests read.
"""
import itertools
import math
import time
from collections import defaultdict
from fractions import Fraction

from msccl.instance import Instance
from msccl.synth.bounds import lower_bound_rounds, lower_bound_steps
from msccl.synth.cache import active_cache
from msccl.synth.smt_paths import PathEncoding


def _attempt(encoding, instance, logging):
    if logging:
        print(f'Solving instance {instance}... ', end='', flush=True)
    t0 = time.time()
    cache = active_cache()
    known = False
    # the problem as the caller posed it (a combining collective is solved as its dual on the reversed topology)
    topology = getattr(encoding, 'original_topology', encoding.topology)
    collective = getattr(encoding, 'primal', encoding.collective)
    if cache is not None:
        known, algo = cache.lookup(topology, collective, instance)
    if not known:
        algo = encoding.solve(instance)
        if cache is not None:
            cache.store(topology, collective, instance, algo)
    if logging:
        verdict = 'synthesized!' if algo is not None else 'unsatisfiable.'
        print(f'{verdict} ({time.time() - t0:.1f}s)')
    return algo


def solve_instance(topology, collective, instance, logging=False):
    return _attempt(PathEncoding(topology, collective), instance, logging)


def solve_least_steps(topology, collective, initial_steps=1, base_instance=Instance(None), logging=False):
    """Find an algorithm with the fewest steps.  Starts from max(initial_steps, distance bound);
    if a larger initial guess works, walks down towards the bound, otherwise walks up."""
    if initial_steps < 1:
        raise ValueError('initial_steps must be strictly positive')
    encoding = PathEncoding(topology, collective)
    floor = lower_bound_steps(topology, collective)
    if floor is None:
        raise ValueError('The collective is unimplementable in this topology.')
    if logging:
        print(f'Algorithms need at least {floor} steps.')
    steps = max(initial_steps, floor)
    if steps > floor:
        best = _attempt(encoding, base_instance.set(steps=steps), logging)
        if best is not None:
            if logging:
                print('Synthesized on initial guess. Checking for fewer steps.')
            while steps > floor:
                steps -= 1
                better = _attempt(encoding, base_instance.set(steps=steps), logging)
                if better is None:
                    break
                best = better
            return best
        steps += 1
    while True:
        algo = _attempt(encoding, base_instance.set(steps=steps), logging)
        if algo is not None:
            return algo
        steps += 1


def solve_all_latency_bandwidth_tradeoffs(topology, collective, min_chunks=1, max_chunks=None,
                                          assume_rounds_per_chunk_lb=None,
                                          assume_monotonic_feasibility=False,
                                          base_instance=Instance(None), logging=False):
    """Generator over the latency/bandwidth frontier: for growing chunk counts, the smallest
    rounds-per-chunk fraction (in lowest terms) that is feasible with the fewest steps."""
    if min_chunks < 1:
        raise ValueError('min_chunks must be strictly positive.')
    if max_chunks is not None and max_chunks < min_chunks:
        raise ValueError('max_chunks must be greater or equal to min_chunks.')
    if assume_rounds_per_chunk_lb is not None and assume_rounds_per_chunk_lb < 0:
        raise ValueError('assume_rounds_per_chunk_lb must be positive.')

    steps_floor = lower_bound_steps(topology, collective)
    if logging:
        print(f'Algorithms need at least {steps_floor} steps.')
    if assume_rounds_per_chunk_lb is not None:
        rpc_floor = assume_rounds_per_chunk_lb
        if logging:
            print(f'Assuming algorithms need at least {rpc_floor} rounds per chunk.')
    else:
        rpc_floor = lower_bound_rounds(topology, collective)
        if logging:
            print(f'Algorithms need at least {rpc_floor} rounds per chunk.')

    infeasible_below = defaultdict(Fraction)   # steps -> largest rpc known to be insufficient
    chunk_counts = itertools.count(min_chunks) if max_chunks is None else range(min_chunks, max_chunks + 1)
    for chunks in chunk_counts:
        encoding = PathEncoding(topology, collective)
        rounds = math.ceil(rpc_floor * chunks) - 1
        hit = None
        while hit is None:
            rounds += 1
            if math.gcd(chunks, rounds) != 1:
                continue        # the reduced fraction was covered with fewer chunks
            rpc = Fraction(rounds, chunks)
            for steps in range(steps_floor, rounds + 1):
                if assume_monotonic_feasibility and rpc < infeasible_below[steps]:
                    continue
                inst = base_instance.set(steps=steps, extra_rounds=rounds - steps, chunks=chunks)
                algo = _attempt(encoding, inst, logging)
                if algo is not None:
                    assert rpc >= infeasible_below[steps], 'Monotonic feasibility assumption would have been violated.'
                    hit = rpc
                    yield algo
                    break
                infeasible_below[steps] = max(infeasible_below[steps], rpc)
                if logging and assume_monotonic_feasibility:
                    print(f'Assuming {steps} step algorithms need at least {rpc} rounds per chunk.')
        if hit <= rpc_floor:
            assert hit == rpc_floor, 'Rounds per chunk lower bound did not hold.'
            if logging:
                print('Bandwidth optimal algorithm found!')
            return
    if logging:
        print('Reached the limit for chunks.')


def _cost(algo):
    steps = len(algo.steps)
    return steps, Fraction(steps + algo.extra_rounds(), algo.instance.chunks)


def prune_pareto_optimal(algorithms):
    """Keep the algorithms not dominated in (steps, rounds per chunk)."""
    costs = [_cost(a) for a in algorithms]
    keep = []
    for a, (sa, ra) in zip(algorithms, costs):
        dominated = any(so <= sa and ro <= ra and (so < sa or ro < ra) for so, ro in costs)
        if not dominated:
            keep.append(a)
    return keep
