"""Two-shot (direct reduce-scatter + direct all-gather) all-reduce on an NVSwitch box.  usage: allreduce_two_shot.py GPUS INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllReduce
from msccl.programs.allreduce import allreduce_two_shot

args = parser(__doc__, ('gpus', 'number of GPUs'), ('instances', 'replication')).parse_args()
emit('allreduce_two_shot', AllReduce(args.gpus, args.gpus, True), lambda: allreduce_two_shot(args.gpus), args.instances,
     args.protocol, manual=True, execute=args.execute)
