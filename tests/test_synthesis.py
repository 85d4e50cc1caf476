"""SMT synthesis: sat/unsat boundaries, bounds, duality, isomorphisms, strategies, distributors."""
from fractions import Fraction

import pytest

from msccl.collectives import (allgather, allreduce, alltoall, build_collective, gather, reduce_scatter,
                               scatter)
from msccl.composers import compose_allreduce
from msccl.distributors import (make_alltoall_subproblem_collective_and_topology,
                                synthesize_alltoall_subproblem, synthesize_gather_scatter_distributed_alltoall,
                                synthesize_greedy_distributed_alltoall)
from msccl.instance import Instance
from msccl.isomorphisms import find_isomorphisms
from msccl.ncd_reduction import ReductionNotApplicableError, non_combining_dual
from msccl.path_encoding import PathEncoding
from msccl.rounds_bound import lower_bound_rounds
from msccl.steps_bound import lower_bound_steps
from msccl.strategies import (prune_pareto_optimal, solve_all_latency_bandwidth_tradeoffs, solve_instance,
                              solve_least_steps)
from msccl.topologies import (Topology, dgx1, distributed_fully_connected, fully_connected, hub_and_spoke,
                              line, ring)


@pytest.mark.parametrize('make', [allgather, reduce_scatter, allreduce])
def test_fully_connected_pair_boundary(make):
    enc = PathEncoding(fully_connected(2), make(2))
    assert enc.solve(Instance(1, chunks=2)) is None
    assert enc.solve(Instance(2, chunks=2)) is not None


@pytest.mark.parametrize('make', [allgather, reduce_scatter, allreduce])
def test_dgx1_boundary(make):
    enc = PathEncoding(dgx1(), make(8))
    assert enc.solve(Instance(1)) is None
    algo = enc.solve(Instance(2))
    assert algo is not None
    algo.check_implements(make(8))


def test_memory_constraint():
    enc = PathEncoding(line(3), alltoall(3))
    assert enc.solve(Instance(2, extra_memory=0)) is None
    assert enc.solve(Instance(2, extra_memory=1)) is not None


def test_pipelined_instance():
    algo = PathEncoding(ring(4), allgather(4)).solve(Instance(2, pipeline=1))
    assert algo is None or algo.is_pipelined()
    with pytest.raises(ValueError):
        PathEncoding(ring(4), allgather(4)).solve(Instance(2, pipeline=0))


def test_bounds():
    assert lower_bound_steps(dgx1(), allgather(8)) == 2
    assert lower_bound_steps(Topology('U', [[0, 0], [0, 0]]), allgather(2)) is None
    assert lower_bound_rounds(dgx1(), allgather(8)) == Fraction(7, 6)
    assert lower_bound_rounds(dgx1(), gather(8, 0)) == Fraction(7, 6)
    assert lower_bound_rounds(hub_and_spoke(8), allgather(8)) == 7
    assert lower_bound_rounds(fully_connected(8), allgather(8)) == 1
    send = build_collective('Send', 2, 1, lambda r, c: r == 0, lambda r, c: r == 1)
    assert lower_bound_rounds(Topology('Unconnected', [[0, 0], [0, 0]]), send) is None
    with pytest.raises(ReductionNotApplicableError):
        lower_bound_rounds(fully_connected(4), allreduce(4))


def test_duality():
    dual = non_combining_dual(reduce_scatter(3))
    assert not dual.is_combining and dual.num_chunks == 3
    for c in dual.chunks():
        assert dual.precondition(c, c) and all(dual.postcondition(r, c) for r in range(3))
    with pytest.raises(ReductionNotApplicableError):
        non_combining_dual(allgather(3))
    with pytest.raises(ReductionNotApplicableError):
        non_combining_dual(allreduce(3))


def test_isomorphisms():
    assert len(find_isomorphisms(dgx1(), dgx1())) == 4
    assert len(find_isomorphisms(ring(4), ring(4), limit=3)) == 3
    assert find_isomorphisms(hub_and_spoke(3), hub_and_spoke(3)) == []
    with pytest.raises(ValueError):
        find_isomorphisms(ring(3), ring(4))


def test_strategies(capsys):
    algo = solve_least_steps(dgx1(), allgather(8), logging=True)
    assert len(algo.steps) == 2
    out = capsys.readouterr().out
    assert 'Algorithms need at least 2 steps.' in out and 'synthesized!' in out
    assert len(solve_least_steps(ring(2), allgather(2), initial_steps=2).steps) == 1
    assert solve_instance(ring(4), allgather(4), Instance(1)) is None
    found = list(solve_all_latency_bandwidth_tradeoffs(ring(4), allgather(4)))
    assert [str(a.instance) for a in found] == ['steps=2', 'steps=2,rounds=3,chunks=2']
    assert [str(a.instance) for a in prune_pareto_optimal(found)] == ['steps=2,rounds=3,chunks=2']
    nvs = list(solve_all_latency_bandwidth_tradeoffs(hub_and_spoke(8), allgather(8)))
    assert [str(a.instance) for a in nvs] == ['steps=1,rounds=7']


def test_greedy_distributor():
    local_topo = fully_connected(2)
    local = PathEncoding(local_topo, alltoall(2)).solve(Instance(1))
    dist = synthesize_greedy_distributed_alltoall(distributed_fully_connected(local_topo, 2, 1), local)
    dist.check_implements(alltoall(4))
    with pytest.raises(ValueError):
        synthesize_greedy_distributed_alltoall(distributed_fully_connected(ring(3), 1, 1), local)


def test_subproblem_distributor():
    sub_coll, sub_topo = make_alltoall_subproblem_collective_and_topology(ring(2), 2, [0])
    assert sub_coll.name == 'AlltoallSubproblem(n=2,copies=2)' and sub_coll.has_triggers()
    assert sub_topo.name == 'Subtopo(local=Ring(n=2),relays=(0))'
    sub = PathEncoding(sub_topo, sub_coll).solve(Instance(3, extra_rounds=1))
    synthesize_alltoall_subproblem(sub, 2).check_implements(alltoall(4))
    _, shared = make_alltoall_subproblem_collective_and_topology(ring(3), 2, [0, 1], bw=2, share_bw=True)
    assert [sw[3] for sw in shared.switches] == ['remote_out', 'remote_in']


def test_gather_scatter_distributor_and_composer():
    g = solve_least_steps(dgx1(), gather(8, 5))
    s = solve_least_steps(dgx1(), scatter(8, 5))
    dist = synthesize_gather_scatter_distributed_alltoall(2, g, s)
    dist.check_implements(alltoall(16))
    rs = PathEncoding(dgx1(), reduce_scatter(8)).solve(Instance(2, extra_rounds=1, chunks=2))
    ag = PathEncoding(dgx1(), allgather(8)).solve(Instance(2, extra_rounds=1, chunks=2))
    ar = compose_allreduce(rs, ag)
    assert ar.name == 'Allreduce(n=8)-DGX1-steps=4,rounds=6,chunks=2'
    with pytest.raises(ValueError):
        compose_allreduce(rs, PathEncoding(dgx1(), allgather(8)).solve(Instance(2)))


def test_synthesis_cache_round_trip(tmp_path, monkeypatch, capsys):
    # solved and unsatisfiable instances are stored once and answered from disk afterwards
    from msccl.collectives import allgather, reduce_scatter
    from msccl.instance import Instance
    from msccl.serialization import load_msccl_object
    from msccl.strategies import solve_instance
    from msccl.synth import cache as synth_cache
    from msccl.topologies import ring
    monkeypatch.setenv('MSCCL_SYNTH_CACHE', str(tmp_path))
    store = synth_cache.active_cache()
    first = solve_instance(ring(4), allgather(4), Instance(2), logging=True)
    assert first is not None and (store.hits, store.misses) == (0, 1)
    files = list(tmp_path.iterdir())
    assert len(files) == 1 and files[0].name.endswith('.msccl.json')
    assert load_msccl_object(str(files[0])).name == first.name            # an ordinary algorithm file
    again = solve_instance(ring(4), allgather(4), Instance(2), logging=True)
    assert (store.hits, store.misses) == (1, 1)
    assert [sorted(s.sends) for s in again.steps] == [sorted(s.sends) for s in first.steps]
    assert capsys.readouterr().out.count('synthesized!') == 2              # same log lines either way
    # unsatisfiable: one step is too few on a ring of four
    assert solve_instance(ring(4), allgather(4), Instance(1)) is None
    assert solve_instance(ring(4), allgather(4), Instance(1)) is None
    assert (store.hits, store.misses) == (2, 2)
    # a combining collective is keyed by the problem as posed, not by its dual
    rs = solve_instance(ring(4), reduce_scatter(4), Instance(3))
    assert rs is not None and solve_instance(ring(4), reduce_scatter(4), Instance(3)).name == rs.name
    assert (store.hits, store.misses) == (3, 3)
    # a damaged entry is solved again and replaced
    files[0].write_text('{not json')
    assert solve_instance(ring(4), allgather(4), Instance(2)) is not None
    assert load_msccl_object(str(files[0])).name == first.name
    monkeypatch.delenv('MSCCL_SYNTH_CACHE')
    assert synth_cache.active_cache() is None
