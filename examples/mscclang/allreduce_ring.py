"""Ring all-reduce (in place), chunk i on channel i % channels.  usage: allreduce_ring.py GPUS CHANNELS INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllReduce
from msccl.programs.allreduce import allreduce_ring

args = parser(__doc__, ('gpus', 'number of GPUs'), ('channels', 'channels of the ring'), ('instances', 'replication')).parse_args()
emit('allreduce_ring', AllReduce(args.gpus, args.gpus, True), lambda: allreduce_ring(args.gpus, args.channels),
     args.instances, args.protocol, manual=True, execute=args.execute)
