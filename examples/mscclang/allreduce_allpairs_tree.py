"""All-pairs all-reduce with a tree reduction on the owner.  usage: allreduce_allpairs_tree.py GPUS INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllReduce
from msccl.programs.classic import allreduce_allpairs_tree

args = parser(__doc__, ('gpus', 'number of GPUs (power of two)'), ('instances', 'replication')).parse_args()
emit('allreduce_pairs', AllReduce(args.gpus, args.gpus, True), lambda: allreduce_allpairs_tree(args.gpus),
     args.instances, args.protocol, manual=True, execute=args.execute, interleaved_replication=False)
