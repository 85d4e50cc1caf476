"""Plans for the Azure SKUs the reference registers (8xV100 ``ndv2``, 8xA100 ``ndv4``).

Same plan names, machine predicates, byte ranges and protocols as reference
``msccl/autosynth/ndv2_plans.py:12-20`` and ``msccl/autosynth/ndv4_plans.py:12-48``.
"""
from msccl.autosynth.registry import register_msccl_program, register_synthesis_plan
from msccl.collectives import gather, scatter
from msccl.distributors.gather_scatter_alltoall import synthesize_gather_scatter_distributed_alltoall
from msccl.language.mscclir import ThreadblockPolicy
from msccl.ncclize import ncclize
from msccl.programs.allreduce import allreduce_allpairs, allreduce_ring
from msccl.programs.alltoall import alltoall_hierarchical, alltoall_three_step
from msccl.synth.search import solve_least_steps
from msccl.topologies import dgx1, fully_connected


def register_ndv2_plans():
    @register_synthesis_plan('alltoall', 'ndv2', sizes=('1MB', None), machines=lambda m: m >= 2)
    def synthesize_ndv2_relay_alltoall(machines):
        # gather on GPU 0, relay to GPU 1 of the other machines, scatter from there
        gather_algo = solve_least_steps(dgx1(), gather(8, 0))
        scatter_algo = solve_least_steps(dgx1(), scatter(8, 1))
        algo = synthesize_gather_scatter_distributed_alltoall(machines, gather_algo, scatter_algo)
        return ncclize(algo, instances=8)


def register_ndv4_plans():
    box = fully_connected(8)
    manual = ThreadblockPolicy.manual

    def single(m):
        return m == 1

    allpairs = dict(chunk_factor=64, inplace=True, protocol='LL', threadblock_policy=manual,
                    interleaved_replication=False, dependence_nop=True, machines=single)

    @register_msccl_program(box, 'allreduce', 'ndv4', instances=2, sizes=('512B', '82944B'), **allpairs)
    def ndv4_allpairs_allreduce_config1(prog, nodes):
        allreduce_allpairs(8)

    @register_msccl_program(box, 'allreduce', 'ndv4', instances=4, sizes=('82944B', '458752B'), **allpairs)
    def ndv4_allpairs_allreduce_config2(prog, nodes):
        allreduce_allpairs(8)

    ring = dict(chunk_factor=8, inplace=True, instances=8, threadblock_policy=manual, machines=single)

    @register_msccl_program(box, 'allreduce', 'ndv4', protocol='LL', sizes=('458752B', '2129920B'), **ring)
    def ndv4_ring_allreduce_config1(prog, nodes):
        allreduce_ring(size=8, channels=4)

    @register_msccl_program(box, 'allreduce', 'ndv4', protocol='LL128', sizes=('2129920B', '22806528B'), **ring)
    def ndv4_ring_allreduce_config2(prog, nodes):
        allreduce_ring(size=8, channels=4)

    @register_msccl_program(box, 'alltoall', 'ndv4', protocol='LL128', sizes=('1MB', '32MB'),
                            machines=lambda m: m in (8, 16, 32, 64))
    def ndv4_alltoall_hierarchical_config1(prog, nodes):
        alltoall_hierarchical(num_nodes=nodes, gpus_per_node=8)

    def ndv4_alltoall_hierarchical_config2(prog, nodes):
        alltoall_hierarchical(num_nodes=nodes, gpus_per_node=8)

    register_msccl_program(box, 'alltoall', 'ndv4', protocol='Simple', sizes=('32MB', None),
                           machines=lambda m: m in (8, 16, 32))(ndv4_alltoall_hierarchical_config2)

    @register_msccl_program(box, 'alltoall', 'ndv4', protocol='Simple', sizes=('32MB', None),
                            machines=lambda m: m == 64)
    def ndv4_alltoall_three_step(prog, nodes):
        alltoall_three_step(num_nodes=nodes, gpus_per_node=8)

    register_msccl_program(box, 'alltoall', 'ndv4', protocol='Simple', sizes=('1KB', None),
                           machines=lambda m: m in (2, 4))(ndv4_alltoall_hierarchical_config2)
