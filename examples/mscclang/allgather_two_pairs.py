"""All-gather on 4 GPUs made of two NVLink pairs: every chunk crosses between the pairs once.  usage: allgather_two_pairs.py INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllGather
from msccl.programs.multistage import allgather_two_pairs

ap = parser(__doc__, ('instances', 'replication'))
args = ap.parse_args()
emit('allgather-two-pairs', AllGather(4, 1, False), allgather_two_pairs, args.instances, args.protocol, execute=args.execute)
