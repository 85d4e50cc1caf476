"""Two-level all-reduce (rings inside nodes, rings across nodes).  usage: hierarchical_allreduce.py GPUS_PER_NODE NODES INSTANCES [--schedule manual]"""
from _common import emit, parser
from msccl.language.collectives import AllReduce
from msccl.programs.classic import hierarchical_allreduce

ap = parser(__doc__, ('gpus', 'GPUs per node'), ('nodes', 'number of nodes'), ('instances', 'replication'))
ap.add_argument('--schedule', default='auto', choices=['auto', 'manual'], help='let the compiler pick channels or pin them')
args = ap.parse_args()
n = args.gpus * args.nodes
emit('hierarchical_allreduce', AllReduce(n, n, True),
     lambda: hierarchical_allreduce(args.gpus, args.nodes, manual_channels=args.schedule == 'manual'), args.instances,
     args.protocol, execute=args.execute, interleaved_replication=False)
