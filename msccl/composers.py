"""Algorithm composition.  Parity: reference ``msccl/composers.py:8-26``."""
from msccl.algorithm import Algorithm
from msccl.collectives import allreduce
from msccl.instance import Instance


def compose_allreduce(reducescatter_algo, allgather_algo, logging=False):
    """Allreduce = ReduceScatter followed by Allgather on the same topology and chunking."""
    if reducescatter_algo.is_pipelined() or allgather_algo.is_pipelined():
        raise ValueError('Pipelining is not supported.')
    rs_chunks, ag_chunks = reducescatter_algo.instance.chunks, allgather_algo.instance.chunks
    if rs_chunks != ag_chunks:
        raise ValueError(f'ReduceScatter and Allgather must have the same chunks (got {rs_chunks} and {ag_chunks})')
    if reducescatter_algo.topology.name != allgather_algo.topology.name:
        raise ValueError(f'ReduceScatter and Allgather must have the same topology (got '
                         f'{reducescatter_algo.topology.name} and {allgather_algo.topology.name})')
    topology = reducescatter_algo.topology
    steps = reducescatter_algo.steps + allgather_algo.steps
    instance = Instance(len(steps), chunks=rs_chunks,
                        extra_rounds=reducescatter_algo.instance.extra_rounds + allgather_algo.instance.extra_rounds)
    return Algorithm.make_implementation(allreduce(topology.num_nodes()), topology, instance, steps)
