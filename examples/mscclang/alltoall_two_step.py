"""Hierarchical two-step all-to-all over several machines.  usage: alltoall_two_step.py NODES GPUS_PER_NODE"""
from _common import emit, parser
from msccl.language.collectives import AllToAll
from msccl.programs.alltoall import alltoall_hierarchical

args = parser(__doc__, ('nodes', 'number of machines'), ('gpus', 'GPUs per machine')).parse_args()
emit('hierarchical_all_to_all', AllToAll(args.nodes * args.gpus, 1, False), lambda: alltoall_hierarchical(args.nodes, args.gpus),
     1, args.protocol, execute=args.execute)
