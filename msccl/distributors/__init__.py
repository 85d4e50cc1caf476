"""Builders of multi-machine Alltoall algorithms from single-machine pieces."""
from .greedy_alltoall import synthesize_greedy_distributed_alltoall
from .gather_scatter_alltoall import synthesize_gather_scatter_distributed_alltoall
from .alltoall_subproblem import (make_alltoall_subproblem_collective_and_topology,
                                  synthesize_alltoall_subproblem)
