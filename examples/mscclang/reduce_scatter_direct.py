"""Direct reduce-scatter on an NVSwitch box.  usage: reduce_scatter_direct.py GPUS INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import ReduceScatter
from msccl.programs.allgather import reduce_scatter_direct

args = parser(__doc__, ('gpus', 'number of GPUs'), ('instances', 'replication')).parse_args()
emit('reduce_scatter_direct', ReduceScatter(args.gpus, 1, False), lambda: reduce_scatter_direct(args.gpus), args.instances,
     args.protocol, execute=args.execute)
