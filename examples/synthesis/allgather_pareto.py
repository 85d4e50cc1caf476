"""Synthesis walk-through: lower bounds, one instance, the latency/bandwidth frontier, lowering to
MSCCL-IR and execution on the CPU interpreter (the flow of the reference's dgx1_allgather notebook)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from msccl.collectives import allgather  # noqa: E402
from msccl.instance import Instance  # noqa: E402
from msccl.interp import run_reference_check  # noqa: E402
from msccl.ncclize import ncclize  # noqa: E402
from msccl.rounds_bound import lower_bound_rounds  # noqa: E402
from msccl.steps_bound import lower_bound_steps  # noqa: E402
from msccl.strategies import prune_pareto_optimal, solve_all_latency_bandwidth_tradeoffs, solve_instance  # noqa: E402
from msccl.topologies import dgx1  # noqa: E402
from msccl.xml import load_xml  # noqa: E402

topo, coll = dgx1(), allgather(8)
print('steps >=', lower_bound_steps(topo, coll), ' rounds per chunk >=', lower_bound_rounds(topo, coll))
algo = solve_instance(topo, coll, Instance(steps=2), logging=True)
print(algo)
frontier = prune_pareto_optimal(list(solve_all_latency_bandwidth_tradeoffs(topo, coll, max_chunks=3, logging=True)))
alpha = beta = 1.0
for a in frontier:
    steps, rounds, chunks = len(a.steps), len(a.steps) + a.extra_rounds(), a.instance.chunks
    print(f'{a.name}: time(size=10) = {alpha * steps + beta * 10 * rounds / chunks:.2f}')
xml = ncclize(frontier[-1], instances=2)
print('interpreter:', run_reference_check(load_xml(xml), 4, race_check=True))
