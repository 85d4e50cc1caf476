"""All-reduce along a binomial tree (reduce towards rank 0, broadcast back).  usage: allreduce_binomial_tree.py GPUS INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllReduce
from msccl.programs.classic import allreduce_binomial_tree

ap = parser(__doc__, ('gpus', 'number of GPUs (any number)'), ('instances', 'replication'))
args = ap.parse_args()
emit('allreduce-binomial-tree', AllReduce(args.gpus, 1, True), lambda: allreduce_binomial_tree(args.gpus), args.instances,
     args.protocol, execute=args.execute)
