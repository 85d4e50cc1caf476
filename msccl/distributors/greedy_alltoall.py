"""Distributed Alltoall from a local Alltoall: run one copy of the local algorithm per machine
and squeeze the cross-machine sends into the local steps as far as the remote bandwidth allows;
what is left goes into the last step, which gets the extra rounds it needs.

Parity: reference ``msccl/distributors/greedy_alltoall.py:20-177``.
"""
import math

from msccl.algorithm import Algorithm, Step
from msccl.collectives import alltoall
from msccl.distributors._common import pair_chunk, require_plain


class _Budget:
    def __init__(self, srcs, dsts, bw):
        self.srcs, self.dsts, self.left, self.bw, self.used = set(srcs), set(dsts), bw, bw, 0

    def covers(self, src, dst):
        return src in self.srcs and dst in self.dsts


def synthesize_greedy_distributed_alltoall(topology, local_algorithm, logging=False):
    require_plain(local_algorithm)
    chunks = local_algorithm.instance.chunks
    n_local = local_algorithm.topology.num_nodes()
    local_coll = alltoall(n_local).chunk_up(chunks)
    try:
        local_algorithm.check_implements(local_coll)
    except Exception:
        raise ValueError(f'Given local Alltoall algorithm "{local_algorithm.name}" does not implement '
                         'Alltoall in the local topology.')
    if topology.num_nodes() % n_local != 0:
        raise ValueError('Number of nodes in topology is not a multiple of ranks in local_algorithm.')
    copies = topology.num_nodes() // n_local
    nodes = topology.num_nodes()

    def remote(a, b):
        return a // n_local != b // n_local

    # every bandwidth group must be purely local or purely remote
    remote_groups = []
    for srcs, dsts, bw, _name in topology.bandwidth_constraints():
        kinds = {remote(s, d) for s in srcs for d in dsts}
        if kinds == {True, False}:
            raise NotImplementedError('Support for switches with mixed local and remote connections is not implemented.')
        if True in kinds:
            if bw == 0:
                raise ValueError('All remote pairs must have direct connectivity.')
            remote_groups.append((srcs, dsts, bw))
    for s in range(nodes):
        for d in range(nodes):
            if remote(s, d) and topology.link(s, d) == 0:
                raise ValueError('All remote pairs must have direct connectivity.')

    if logging:
        print('Generating sends for remote pairs')
    backlog = {(s, d): [(pair_chunk(s, d, i, nodes, chunks), s, d) for i in range(chunks)]
               for s in range(nodes) for d in range(nodes) if remote(s, d)}

    def take(rounds):
        """Pop as many backlog sends as fit into ``rounds`` rounds of remote bandwidth."""
        budgets = [_Budget(srcs, dsts, bw * rounds) for srcs, dsts, bw in remote_groups]
        taken = []
        for pair in list(backlog):
            queue_ = backlog[pair]
            mine = [b for b in budgets if b.covers(*pair)]
            room = min([len(queue_)] + [b.left for b in mine])
            taken.extend(queue_[:room])
            del queue_[:room]
            for b in mine:
                b.left -= room
            if not queue_:
                del backlog[pair]
        return taken

    if logging:
        print('Overlapping remote sends with local algorithm')
    steps = []
    for t, local_step in enumerate(local_algorithm.steps, start=1):
        sends = []
        for chunk, src, dst in local_step.sends:
            origin = (chunk // chunks) % n_local
            target = (chunk // chunks) // n_local
            assert local_coll.precondition(origin, chunk) and local_coll.postcondition(target, chunk)
            for c in range(copies):
                base = c * n_local
                sends.append((pair_chunk(base + origin, base + target, chunk % chunks, nodes, chunks),
                              base + src, base + dst))
        extra = take(local_step.rounds)
        if logging:
            print(f'Packed {len(extra)} remote sends into step {t}')
        steps.append(Step(local_step.rounds, sends + extra))

    added = 0
    if backlog:
        budgets = [_Budget(srcs, dsts, bw) for srcs, dsts, bw in remote_groups]
        leftovers = len(backlog)
        for pair, queue_ in backlog.items():
            for b in budgets:
                if b.covers(*pair):
                    b.used += len(queue_)
            steps[-1].sends.extend(queue_)
        added = max(math.ceil(b.used / b.bw) for b in budgets)
        steps[-1].rounds += added
        if logging:
            print(f'Packed remaining {leftovers} remote sends into step {len(steps)} by adding {added} additional rounds')
    elif logging:
        print('All remote sends fit into the rounds of the local algorithm')

    instance = local_algorithm.instance.set(extra_rounds=local_algorithm.instance.extra_rounds + added)
    return Algorithm.make_implementation(alltoall(nodes), topology, instance, steps)
