"""Distributed Alltoall as local Gather -> root-to-root transpose -> local Scatter.

Every machine gathers all outgoing data on its gather root(s), the roots exchange it (one
send per chunk, scheduled right after the step in which the chunk reached the root), and the
scatter root(s) distribute what arrived.  Multi-root Gather/Scatter inputs multiply the chunk
count by the number of roots.

Parity: reference ``msccl/distributors/gather_scatter_alltoall.py:9-191``.
"""
from collections import defaultdict

from msccl.algorithm import Algorithm, Step
from msccl.collectives import alltoall, gather, multiroot_gather, multiroot_scatter, scatter
from msccl.distributors._common import pair_chunk, require_plain
from msccl.instance import Instance
from msccl.topologies import distributed_fully_connected


def _find_roots(algo, n_local, holds, what):
    roots = []
    for c in range(algo.collective.num_chunks // n_local):
        root = next((r for r in range(n_local) if holds(algo.collective, r, c)), None)
        if root is None:
            raise ValueError(f'Root number {c} not found for the {what} algorithm.')
        roots.append(root)
    if not roots:
        raise ValueError(f'No roots found for the {what} algorithm.')
    return roots


def _checked_collective(algo, n_local, chunks, roots, single, multi, what):
    if len(roots) > 1:
        coll, shown = multi(n_local, roots=roots).chunk_up(chunks), f'Multiroot{what} for the roots {roots}'
    else:
        coll, shown = single(n_local, root=roots[0]).chunk_up(chunks), f'{what} for the root {roots[0]}'
    try:
        algo.check_implements(coll)
    except Exception:
        raise ValueError(f'Given local {what} algorithm "{algo.name}" does not implement {shown}.')
    return coll


def synthesize_gather_scatter_distributed_alltoall(num_copies, gather_algo, scatter_algo, remote_bw=1,
                                                   logging=False):
    require_plain(gather_algo, scatter_algo)
    if gather_algo.instance.chunks != scatter_algo.instance.chunks:
        raise ValueError(f'Local gather and local scatter must have the same chunks (got '
                         f'{gather_algo.instance.chunks} and {scatter_algo.instance.chunks})')
    if gather_algo.topology.name != scatter_algo.topology.name:
        raise ValueError(f'Local gather and local scatter must have the same topology (got '
                         f'{gather_algo.topology.name} and {scatter_algo.topology.name})')
    local_topology = gather_algo.topology
    chunks = gather_algo.instance.chunks
    n_local = local_topology.num_nodes()
    nodes = n_local * num_copies

    g_roots = _find_roots(gather_algo, n_local, lambda c, r, k: c.postcondition(r, k), 'Gather')
    local_gather = _checked_collective(gather_algo, n_local, chunks, g_roots, gather, multiroot_gather, 'Gather')
    s_roots = _find_roots(scatter_algo, n_local, lambda c, r, k: c.precondition(r, k), 'Scatter')
    local_scatter = _checked_collective(scatter_algo, n_local, chunks, s_roots, scatter, multiroot_scatter, 'Scatter')
    if len(g_roots) != len(s_roots):
        raise ValueError(f'The number of roots for the Gather algorithm ({len(g_roots)}) does not match '
                         f'the number of roots for the Scatter algorithm ({len(s_roots)}).')
    if len(g_roots) > 1:
        chunks *= len(g_roots)
        print(f'Multiplying chunks by {len(g_roots)} to match the number of roots.')

    topology = distributed_fully_connected(local_topology, num_copies, remote_bw)
    steps = []
    reached_root_after = defaultdict(int)      # distributed chunk -> steps until it sits on its gather root

    # phase 1: every machine runs the gather once per final destination rank
    for t, local_step in enumerate(gather_algo.steps):
        sends = []
        for chunk, src, dst in local_step.sends:
            origin = (chunk // chunks) % n_local
            assert local_gather.precondition(origin, chunk)
            for target in range(nodes):
                for c in range(num_copies):
                    base = c * n_local
                    which = pair_chunk(base + origin, target, chunk % chunks, nodes, chunks)
                    sends.append((which, base + src, base + dst))
                    reached_root_after[which] = max(reached_root_after[which], t + 1)
        steps.append(Step(local_step.rounds * nodes, sends))

    # phase 2: transpose between roots, as early as each chunk allows
    transposes = [[] for _ in range(len(gather_algo.steps) + 1)]
    for src in range(nodes):
        for dst in range(nodes):
            same_machine = src // n_local == dst // n_local
            for k in range(chunks):
                g_root = g_roots[k % len(g_roots)]
                s_root = s_roots[k % len(s_roots)]
                if g_root != s_root and local_topology.link(g_root, s_root) == 0:
                    if same_machine:
                        raise ValueError(f'The local topology does not have a link from root {g_root} of the '
                                         f'Gather to root {s_root} of the Scatter.')
                if g_root == s_root and same_machine:
                    continue
                which = pair_chunk(src, dst, k, nodes, chunks)
                transposes[reached_root_after[which]].append(
                    (which, (src // n_local) * n_local + g_root, (dst // n_local) * n_local + s_root))
    transpose_rounds = chunks * n_local * n_local
    for t, sends in enumerate(transposes):
        if t < len(gather_algo.steps):
            steps[t].sends.extend(sends)
            steps[t].rounds = max(steps[t].rounds, transpose_rounds)
        else:
            steps.append(Step(transpose_rounds, sends))

    # phase 3: every machine runs the scatter once per original source rank
    for local_step in scatter_algo.steps:
        sends = []
        for chunk, src, dst in local_step.sends:
            target = (chunk // chunks) % n_local
            assert local_scatter.postcondition(target, chunk)
            for source in range(nodes):
                for c in range(num_copies):
                    base = c * n_local
                    sends.append((pair_chunk(source, base + target, chunk % chunks, nodes, chunks),
                                  base + src, base + dst))
        steps.append(Step(local_step.rounds * nodes, sends))

    instance = Instance(steps=len(steps), extra_rounds=sum(s.rounds - 1 for s in steps), chunks=chunks)
    return Algorithm.make_implementation(alltoall(nodes), topology, instance, steps)
