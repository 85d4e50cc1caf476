"""All-reduce on 4 GPUs made of two NVLink pairs (reduce in the pair, exchange across, copy back).  usage: allreduce_two_pairs.py INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllReduce
from msccl.programs.multistage import allreduce_two_pairs

ap = parser(__doc__, ('instances', 'replication'))
args = ap.parse_args()
emit('allreduce-two-pairs', AllReduce(4, 2, True), allreduce_two_pairs, args.instances, args.protocol, execute=args.execute)
