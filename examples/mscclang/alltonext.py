"""Pipeline hand-over: every GPU passes its chunks to the next (or previous) GPU; the hop between machines is spread over all NICs.  usage: alltonext.py NODES INSTANCES [--backward]"""
from _common import emit, parser
from msccl.programs.classic import AllToNext, alltonext

ap = parser(__doc__, ('nodes', 'number of machines (8 GPUs each)'), ('instances', 'replication'))
ap.add_argument('--backward', action='store_true')
args = ap.parse_args()
emit('alltonext-backward' if args.backward else 'alltonext-forward', AllToNext(args.nodes * 8, 8, False, forward=not args.backward),
     lambda: alltonext(args.nodes, 8, forward=not args.backward), args.instances, args.protocol, execute=args.execute)
