"""Recursive halving / doubling all-reduce.  usage: allreduce_recursive_doubling_halving.py GPUS INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllReduce
from msccl.programs.classic import allreduce_recursive_halving_doubling

args = parser(__doc__, ('gpus', 'number of GPUs (power of two)'), ('instances', 'replication')).parse_args()
emit('allreduce_recursive_doubling_halving', AllReduce(args.gpus, args.gpus, True),
     lambda: allreduce_recursive_halving_doubling(args.gpus), args.instances, args.protocol, manual=True,
     execute=args.execute, interleaved_replication=False)
