"""All-reduce on ROWS x COLS GPUs: reduce-scatter in the fast columns, then along the slow rows, and back.  usage: allreduce_2d.py ROWS COLS INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllReduce
from msccl.programs.multistage import allreduce_2d

ap = parser(__doc__, ('rows', 'GPUs per column (fast links)'), ('cols', 'number of columns (slow links)'), ('instances', 'replication'))
args = ap.parse_args()
emit('allreduce-2d', AllReduce(args.rows * args.cols, args.rows * args.cols, True), lambda: allreduce_2d(args.rows, args.cols),
     args.instances, args.protocol, execute=args.execute,
     interleaved_replication=False)       # the last phase moves a whole row's chunks at once: replicate in batches
