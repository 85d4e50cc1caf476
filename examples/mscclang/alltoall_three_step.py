"""Three-step all-to-all (gather, one big cross-machine copy, scatter).  usage: alltoall_three_step.py NODES GPUS_PER_NODE INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllToAll
from msccl.programs.alltoall import alltoall_three_step

ap = parser(__doc__, ('nodes', 'number of machines'), ('gpus', 'GPUs per machine'), ('instances', 'logical instances'))
ap.add_argument('--ib_connections', type=int, default=1, help='parallel cross-machine connections per pair')
args = ap.parse_args()
emit('alltoall_a100_three_step', AllToAll(args.nodes * args.gpus, args.instances, False),
     lambda: alltoall_three_step(args.nodes, args.gpus, args.instances, args.ib_connections), 1, args.protocol,
     execute=args.execute)
