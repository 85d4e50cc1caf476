"""One pipeline stage reduces, the next stage receives the sum: ring or all-pairs inside the stages.  usage: pipeline_allreduce.py GPUS_PER_STAGE INSTANCES [--allpairs] [--channels N]"""
from _common import emit, parser
from msccl.programs.multistage import StageAllReduce, pipeline_allreduce_allpairs, pipeline_allreduce_ring

ap = parser(__doc__, ('gpus', 'GPUs in one stage'), ('instances', 'replication'))
ap.add_argument('--allpairs', action='store_true', help='all-pairs instead of rings inside the stages')
ap.add_argument('--channels', type=int, default=1, help='channels one ring is spread over')
args = ap.parse_args()
if args.allpairs:
    emit('pipeline-allreduce-allpairs', StageAllReduce(args.gpus, args.gpus), lambda: pipeline_allreduce_allpairs(args.gpus),
         args.instances, args.protocol, execute=args.execute)
else:
    emit('pipeline-allreduce-ring', StageAllReduce(args.gpus, args.gpus), lambda: pipeline_allreduce_ring(args.gpus, args.channels),
         args.instances, args.protocol, execute=args.execute)
