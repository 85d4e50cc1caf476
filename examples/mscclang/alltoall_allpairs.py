"""Direct all-to-all.  usage: alltoall_allpairs.py GPUS INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllToAll
from msccl.programs.alltoall import alltoall_direct

args = parser(__doc__, ('gpus', 'number of GPUs'), ('instances', 'replication')).parse_args()
emit('alltoall_allpairs', AllToAll(args.gpus, 1, False), lambda: alltoall_direct(args.gpus), args.instances, args.protocol,
     execute=args.execute)
