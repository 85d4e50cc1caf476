"""Direct all-gather on an NVSwitch box.  usage: allgather_direct.py GPUS INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllGather
from msccl.programs.allgather import allgather_direct

args = parser(__doc__, ('gpus', 'number of GPUs'), ('instances', 'replication')).parse_args()
emit('allgather_direct', AllGather(args.gpus, 1, False), lambda: allgather_direct(args.gpus), args.instances, args.protocol,
     execute=args.execute)
