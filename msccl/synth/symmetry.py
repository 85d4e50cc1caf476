"""Enumerate node permutations mapping one topology's link matrix onto another's.

Parity: reference ``msccl/isomorphisms.py:8-88`` (``Permutation``, ``find_isomorphisms``).
The search is an all-SAT loop over an integer permutation, blocking each found model.
"""
from dataclasses import dataclass

import z3


@dataclass
class Permutation:
    nodes: list

    def __str__(self):
        return f'Permutation(nodes={self.nodes})'


def find_isomorphisms(topology, target_topology, limit=None, logging=False):
    if len(topology.switches) > 0:
        print('MSCCL Warning: Topologies with switches are not supported. import msccl will be ignored.')
        return []
    if limit is not None and limit <= 0:
        raise ValueError('MSCCL error: limit was set improperly.')
    n = topology.num_nodes()
    if n != target_topology.num_nodes():
        raise ValueError('MSCCL error: target topology does not match with the given topology.')
    if logging:
        print(f'Encoding {topology.name} - {target_topology.name} isomorphisms to Z3')

    image = [z3.Int(f'perm_node_{i}') for i in range(n)]
    solver = z3.Solver()
    for p in image:
        solver.add(p >= 0, p < n)
    solver.add(z3.Distinct(*image) if n > 1 else z3.BoolVal(True))
    # For each ordered pair, forbid images whose target link count differs.
    for s in range(n):
        for d in range(n):
            want = topology.link(s, d)
            for ts in range(n):
                for td in range(n):
                    if target_topology.link(ts, td) != want:
                        solver.add(z3.Not(z3.And(image[s] == ts, image[d] == td)))
    if logging:
        print('Solving isomorphisms incrementally...')
    found = []
    while solver.check() == z3.sat:
        model = solver.model()
        perm = Permutation([model.eval(p, model_completion=True).as_long() for p in image])
        found.append(perm)
        if logging:
            print(perm)
        if limit is not None and len(found) >= limit:
            break
        solver.add(z3.Or([p != v for p, v in zip(image, perm.nodes)]))
    if logging:
        print(f'{len(found)} isomorphisms found.')
    return found
