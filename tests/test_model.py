"""Problem model: collectives, topologies, instance, algorithm verification, JSON."""
import pytest

from helpers import impossible_collective, null_collective
from msccl.algorithm import Algorithm, Step
from msccl.collectives import (allgather, allreduce, alltoall, broadcast, build_collective, gather,
                               multiroot_gather, multiroot_scatter, reduce, reduce_scatter, scan, scatter)
from msccl.instance import Instance
from msccl.serialization import MSCCLDecoder, MSCCLEncoder, load_msccl_object, save_msccl_object
from msccl.topologies import (Topology, amd4, amd8, b200_nvswitch, binarize_topology, dgx1, dgx_a100,
                              distributed_fully_connected, distributed_hub_and_spoke, fully_connected,
                              hub_and_spoke, line, nvlink_only, reverse_topology, ring, star)

SMI_DGX1 = '\tGPU0\tGPU1\tGPU2\tGPU3\tGPU4\tGPU5\tGPU6\tGPU7\tmlx5_0\tCPU Affinity\n' + '\n'.join(
    f'GPU{i}\t' + '\t'.join(' X ' if i == j else (f'NV{dgx1().links[i][j]}' if dgx1().links[i][j] else 'SYS')
                           for j in range(8)) + '\tPIX\t0-19' for i in range(8)) + \
    '\nmlx5_0\t' + '\t'.join(['PIX'] * 8) + '\t X \t\n\nLegend:\n\n  X    = Self\n'


def test_collective_kinds():
    assert not allgather(4).is_combining and not alltoall(3).is_combining and not broadcast(3, 1).is_combining
    assert allreduce(4).is_combining and reduce_scatter(3).is_combining and reduce(3, 0).is_combining
    assert scan(3).is_combining
    a2a = alltoall(3)
    assert a2a.num_chunks == 9
    for c in a2a.chunks():
        assert a2a.precondition(c % 3, c) and a2a.postcondition(c // 3, c)
    rs = reduce_scatter(2)
    assert [rs.address(c) for c in rs.chunks()] == [0, 0, 1, 1]


def test_chunk_up_and_triggers():
    coll = allreduce(2).chunk_up(3)
    assert coll.num_chunks == 6 and coll.name.endswith(',chunks=3')
    assert sorted({coll.address(c) for c in coll.chunks()}) == [0, 1, 2]
    with pytest.raises(ValueError):
        allgather(2).chunk_up(0)
    trig = build_collective('T', 2, 2, lambda r, c: r == c, lambda r, c: r != c,
                            trigger=lambda r, c: 1 - c if r == 0 else None)
    assert trig.has_triggers() and trig.trigger(0, 0) == 1 and trig.trigger(1, 0) is None


def test_multiroot_names_and_layout():
    g = multiroot_gather(3, [0, 1])
    assert g.name == 'MultirootGather(n=3,roots=(0,1))' and g.num_chunks == 6
    s = multiroot_scatter(3, [1, 2])
    assert all(s.precondition([1, 2][c % 2], c) for c in s.chunks())
    assert gather(4, 2).postcondition(2, 3) and scatter(4, 1).precondition(1, 0)


def test_topologies():
    assert hub_and_spoke(4).num_nodes() == 4 and len(hub_and_spoke(4).switches) == 8
    assert fully_connected(6).link(0, 5) == 1 and fully_connected(6).link(3, 3) == 0
    assert list(ring(5).sources(0)) == [1, 4]
    assert list(line(5).destinations(0)) == [1]
    assert star(6).link(0, 3) == 1 and star(6).link(2, 3) == 0 and len(star(4, False).switches) == 2
    assert dgx1().link(0, 1) == 2 and dgx1().link(0, 5) == 0 and amd4().num_nodes() == 4
    assert amd8().link(0, 2) == 6 and amd8().link(0, 1) == 5
    assert dgx_a100().link(1, 2) == 12
    b = b200_nvswitch()
    assert b.num_nodes() == 8 and b.link(0, 7) == 18 and len(b.switches) == 16
    with pytest.raises(ValueError):
        Topology('bad', [[0, 1], [1, 0]], [([0], [1], 0, 'zero')])
    assert len(list(ring(3).bandwidth_constraints())) == 6


def test_distributed_and_transformed_topologies():
    d = distributed_fully_connected(ring(4), 2, 1)
    assert d.num_nodes() == 8 and d.link(0, 4) == 1 and d.link(0, 2) == 0
    h = distributed_hub_and_spoke(star(6), 4, 2)
    assert h.num_nodes() == 24 and sum(1 for sw in h.switches if 'remote' in sw[3]) == 8
    rev = reverse_topology(star(4, False))
    assert rev.name == 'ReverseStar(n=4)' and rev.switches[0][3] == 'to_points_reversed'
    binar = binarize_topology(dgx1())
    assert max(max(r) for r in binar.links) == 1 and binar.switches == []


def test_nvlink_only_parser():
    topo = nvlink_only(SMI_DGX1)
    assert topo.num_nodes() == 8 and topo.links == dgx1().links


def test_instance():
    inst = Instance(2, extra_rounds=1, chunks=2)
    assert str(inst) == 'steps=2,rounds=3,chunks=2' and inst.rounds() == 3
    assert str(Instance(3, pipeline=2, extra_memory=0, allow_exchange=True)) == \
        'steps=3,pipeline=2,extra_memory=0,allow_exchange'
    assert Instance(None).set(steps=4).steps == 4 and inst.set(chunks=None).chunks == 2


def test_algorithm_verification():
    topo = fully_connected(2)
    with pytest.raises(RuntimeError):
        Algorithm.make_implementation(impossible_collective(2), topo, Instance(1), [Step(1, [])])
    assert Algorithm.make_implementation(null_collective(2), topo, Instance(1), [Step(1, [])]) is not None
    good = Algorithm.make_implementation(allgather(2), topo, Instance(1), [Step(1, [(0, 0, 1), (1, 1, 0)])])
    assert good.name == 'Allgather(n=2)-FullyConnected(n=2)-steps=1'
    assert good.input_map == {0: {0}, 1: {1}} and good.output_map == {0: {0, 1}, 1: {0, 1}}
    assert str(good) == '(step 1) 0:0→1, 1:1→0'
    with pytest.raises(AssertionError):       # two chunks over a bandwidth-1 link in one round
        Algorithm.make_implementation(alltoall(2).chunk_up(2), topo, Instance(1, chunks=2),
                                      [Step(1, [(2, 0, 1), (3, 0, 1), (4, 1, 0), (5, 1, 0)])])
    with pytest.raises(ValueError):
        Algorithm.make_implementation(null_collective(2), topo, Instance(1, extra_rounds=1), [Step(3, [])])


def test_json_roundtrip(tmp_path):
    steps = [Step(1, [(0, 0, 1)]), Step(2, [(1, 1, 0), (1, 0, 1)]), Step(1, [(0, 1, 0)])]
    inst = Instance(3, pipeline=2)
    algo = Algorithm('test_algorithm', null_collective(2), fully_connected(2), inst, steps)
    back = MSCCLDecoder().decode(MSCCLEncoder().encode(algo))
    assert back.name == 'test_algorithm' and back.instance == inst
    assert [(s.rounds, s.sends) for s in back.steps] == [(s.rounds, s.sends) for s in algo.steps]
    path = tmp_path / 'topo.json'
    save_msccl_object(hub_and_spoke(3), path)
    again = load_msccl_object(path)
    assert again.links == hub_and_spoke(3).links and len(again.switches) == 6


def test_loads_reference_written_json(tmp_path):
    # a file in the exact layout the reference tool writes (Ring(4) Allgather, 2 steps)
    text = ('{"msccl_type":"algorithm","name":"Allgather(n=4)-Ring(n=4)-steps=2",'
            '"instance":{"msccl_type":"instance","steps":2,"extra_rounds":0,"chunks":1,"pipeline":null,'
            '"extra_memory":null,"allow_exchange":false},'
            '"input_map":{"0":[0],"1":[1],"2":[2],"3":[3]},'
            '"output_map":{"0":[0,1,2,3],"1":[0,1,2,3],"2":[0,1,2,3],"3":[0,1,2,3]},'
            '"steps":[{"msccl_type":"step","rounds":1,"sends":[[0,0,3],[1,1,0],[1,1,2],[2,2,1],[2,2,3],[3,3,2]]},'
            '{"msccl_type":"step","rounds":1,"sends":[[0,0,1],[0,3,2],[1,2,3],[2,1,0],[3,2,1],[3,3,0]]}],'
            '"collective":{"msccl_type":"collective","name":"Allgather(n=4)","nodes":4,"chunks":['
            + ','.join('{"msccl_type":"chunk","pre":[%d],"post":[0,1,2,3],"addr":%d}' % (i, i) for i in range(4)) +
            '],"triggers":{},"runtime_name":"allgather"},'
            '"topology":{"msccl_type":"topology","name":"Ring(n=4)","switches":[],'
            '"links":[[0,1,0,1],[1,0,1,0],[0,1,0,1],[1,0,1,0]]}}')
    path = tmp_path / 'ag.msccl.json'
    path.write_text(text)
    algo = load_msccl_object(path)
    algo.check_implements(allgather(4))
    assert algo.collective.runtime_name == 'allgather' and algo.topology.name == 'Ring(n=4)'
