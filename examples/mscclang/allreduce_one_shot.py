"""One-shot all-reduce for small messages on an NVSwitch box.  usage: allreduce_one_shot.py GPUS INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllReduce
from msccl.programs.allreduce import allreduce_one_shot

args = parser(__doc__, ('gpus', 'number of GPUs'), ('instances', 'replication')).parse_args()
emit('allreduce_one_shot', AllReduce(args.gpus, 1, True), lambda: allreduce_one_shot(args.gpus), args.instances, args.protocol,
     manual=True, execute=args.execute)
