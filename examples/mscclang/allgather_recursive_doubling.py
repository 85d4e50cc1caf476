"""Recursive doubling all-gather (in place).  usage: allgather_recursive_doubling.py GPUS INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllGather
from msccl.programs.classic import allgather_recursive_doubling

args = parser(__doc__, ('gpus', 'number of GPUs (power of two)'), ('instances', 'replication')).parse_args()
emit('allgather_recursive_doubling', AllGather(args.gpus, 1, True), lambda: allgather_recursive_doubling(args.gpus),
     args.instances, args.protocol, manual=True, execute=args.execute)
