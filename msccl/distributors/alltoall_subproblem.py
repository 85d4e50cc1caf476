"""Distributed Alltoall through a one-machine sub-problem.

The sub-problem models one machine plus a single virtual "remote" node that stands for all
other machines.  Chunk numbering of the sub-problem collective:
  [0, L*L)                      local pairs (ordinary Alltoall on the machine),
  next (copies-1)*L*L           outgoing chunks: start on a local rank, must reach the remote node,
  last (copies-1)*L*L           incoming chunks: start on the remote node, must reach a local rank.
Triggers tie the k-th outgoing chunk to the k-th incoming one so that whenever the remote node
receives one it emits the other in the same step.  Stitching copies of a solved sub-problem
pairs each machine's sends-to-remote with the matching machine's receives-from-remote.

Parity: reference ``msccl/distributors/alltoall_subproblem.py:9-223``.  Unlike the reference the
``share_bw`` option works: it adds in/out switches over the relay links.
"""
from msccl.algorithm import Algorithm, Step
from msccl.collectives import alltoall, build_collective
from msccl.distributors._common import pair_chunk, require_plain
from msccl.instance import Instance
from msccl.topologies import Topology


def _layout(n_local, copies):
    local_end = n_local * n_local
    remote_pairs = (copies - 1) * n_local * n_local
    return local_end, remote_pairs, local_end + remote_pairs, local_end + 2 * remote_pairs


def _alltoall_subproblem(n_local, copies):
    remote = n_local
    local_end, remote_pairs, out_end, total = _layout(n_local, copies)

    def region(chunk):
        if chunk < local_end:
            return 0, chunk
        if chunk < out_end:
            return 1, chunk - local_end
        return 2, chunk - out_end

    def pre(rank, chunk):
        kind, c = region(chunk)
        if kind == 0:
            return rank == c % n_local
        if kind == 1:
            return rank == (c // (copies - 1)) % n_local
        return rank == remote

    def post(rank, chunk):
        kind, c = region(chunk)
        if kind == 0:
            return rank == c // n_local
        if kind == 1:
            return rank == remote
        return rank == (c // (copies - 1)) // n_local

    def trigger(rank, chunk):
        if rank != remote:
            return None
        kind, _ = region(chunk)
        if kind == 1:
            return chunk + remote_pairs
        if kind == 2:
            return chunk - remote_pairs
        return None

    return build_collective(f'AlltoallSubproblem(n={n_local},copies={copies})', n_local + 1, total,
                            pre, post, trigger=trigger)


def make_alltoall_subproblem_collective_and_topology(topology, num_copies, relay_nodes, bw=1, share_bw=False):
    n_local = topology.num_nodes()
    remote = n_local
    links = [[topology.link(s, d) if s < n_local and d < n_local else 0 for s in range(n_local + 1)]
             for d in range(n_local + 1)]
    for relay in relay_nodes:
        links[remote][relay] = bw
        links[relay][remote] = bw
    switches = list(topology.switches)
    if share_bw:
        switches.append((list(relay_nodes), [remote], bw, 'remote_out'))
        switches.append(([remote], list(relay_nodes), bw, 'remote_in'))
    name = f'Subtopo(local={topology.name},relays=({",".join(str(i) for i in relay_nodes)}))'
    return _alltoall_subproblem(n_local, num_copies), Topology(name, links, switches)


def synthesize_alltoall_subproblem(subproblem_algo, num_copies, logging=False):
    require_plain(subproblem_algo)
    sub_topology = subproblem_algo.topology
    sub_coll = subproblem_algo.collective
    chunks = subproblem_algo.instance.chunks
    n_local = sub_topology.num_nodes() - 1
    remote = n_local
    nodes = n_local * num_copies
    local_end, remote_pairs, out_end, total = _layout(n_local, num_copies)

    # Distributed topology: a relay reaches the relays of all other machines.
    links = [[0] * nodes for _ in range(nodes)]
    for dst in range(nodes):
        for src in range(nodes):
            ls, ld = src % n_local, dst % n_local
            if src // n_local == dst // n_local:
                links[dst][src] = sub_topology.link(ls, ld)
            else:
                links[dst][src] = min(sub_topology.link(ls, remote), sub_topology.link(remote, ld))
    switches = []
    for srcs, dsts, bw, name in sub_topology.switches:
        for c in range(num_copies):
            def spread(ranks):
                out = []
                for r in ranks:
                    if r < remote:
                        out.append(r + c * n_local)
                    else:       # the remote node stands for every rank of every other machine
                        out.extend(x for x in range(nodes) if x // n_local != c)
                return out
            switches.append((spread(srcs), spread(dsts), bw, f'copy_{c}_{name}_local'))
    topology = Topology(f'Stiched(sub={sub_topology.name},copies={num_copies})', links, switches)

    steps = []
    for sub_step in subproblem_algo.steps:
        sends = []
        waiting_out = {}   # distributed chunk -> sender that pushed it towards "remote"
        waiting_in = {}    # distributed chunk -> receiver that expects it from "remote"
        for chunk, src, dst in sub_step.sends:
            for c in range(num_copies):
                base = c * n_local

                def machine_of(rel):
                    other = rel % (num_copies - 1)
                    return (other + 1 if other >= c else other) * n_local

                if chunk < local_end:
                    assert src != remote and dst != remote
                    origin = base + (chunk // chunks) % n_local
                    target = base + (chunk // chunks) // n_local
                    assert sub_coll.precondition(origin % n_local, chunk)
                    assert sub_coll.postcondition(target % n_local, chunk)
                elif chunk < out_end:
                    rel = chunk - local_end
                    local_origin = ((rel // chunks) // (num_copies - 1)) % n_local
                    origin = base + local_origin
                    target = machine_of(rel) + (rel // (num_copies - 1)) // n_local
                    assert sub_coll.precondition(local_origin, chunk)
                    assert sub_coll.postcondition(target % n_local, chunk + remote_pairs)
                else:
                    assert chunk < total
                    rel = chunk - out_end
                    local_target = ((rel // chunks) // (num_copies - 1)) // n_local
                    target = base + local_target
                    origin = machine_of(rel) + (rel // (num_copies - 1)) % n_local
                    assert sub_coll.precondition(origin % n_local, chunk - remote_pairs)
                    assert sub_coll.postcondition(local_target, chunk)
                which = pair_chunk(origin, target, chunk % chunks, nodes, chunks)
                if dst == remote:
                    assert chunk < out_end
                    if which in waiting_in:
                        sends.append((which, base + src, waiting_in.pop(which)))
                    else:
                        waiting_out[which] = base + src
                elif src == remote:
                    if which in waiting_out:
                        sends.append((which, waiting_out.pop(which), base + dst))
                    else:
                        waiting_in[which] = base + dst
                else:
                    sends.append((which, base + src, base + dst))
        if waiting_out or waiting_in:
            raise ValueError('Subproblem algorithm has unpaired sends/recvs.')
        steps.append(Step(sub_step.rounds, sends))

    instance = Instance(steps=len(steps), extra_rounds=sum(s.rounds - 1 for s in steps), chunks=chunks)
    return Algorithm.make_implementation(alltoall(nodes), topology, instance, steps)
