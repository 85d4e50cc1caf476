"""Ring all-gather (out of place).  usage: allgather_ring.py GPUS CHANNELS INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllGather
from msccl.programs.allgather import allgather_ring

args = parser(__doc__, ('gpus', 'number of GPUs'), ('channels', 'channels'), ('instances', 'replication')).parse_args()
emit('allgather_ring', AllGather(args.gpus, 1, False), lambda: allgather_ring(args.gpus, args.channels), args.instances,
     args.protocol, execute=args.execute)
