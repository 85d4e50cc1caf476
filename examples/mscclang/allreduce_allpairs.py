"""All-pairs all-reduce with a chain reduction on the owner (the small-message plan of the A100 registry).  usage: allreduce_allpairs.py GPUS INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllReduce
from msccl.programs.allreduce import allreduce_allpairs

args = parser(__doc__, ('gpus', 'number of GPUs'), ('instances', 'replication')).parse_args()
emit('allreduce_pairs', AllReduce(args.gpus, args.gpus * args.gpus, True), lambda: allreduce_allpairs(args.gpus),
     args.instances, args.protocol, manual=True, execute=args.execute, interleaved_replication=False, dependence_nop=True)
