"""Sum inside groups of GPUs, then gather every group's sums on every GPU (a custom collective).  usage: reduce_gather.py GROUPS GPUS_PER_GROUP INSTANCES"""
from _common import emit, parser
from msccl.programs.multistage import ReduceGather, reduce_gather

ap = parser(__doc__, ('groups', 'number of groups'), ('gpus_per_group', 'GPUs in a group'), ('instances', 'replication'))
args = ap.parse_args()
emit('reduce-gather', ReduceGather(args.groups, args.gpus_per_group), lambda: reduce_gather(args.groups, args.gpus_per_group),
     args.instances, args.protocol, execute=args.execute)
