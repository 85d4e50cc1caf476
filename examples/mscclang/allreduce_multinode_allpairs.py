"""All-reduce over several machines: all-pairs inside each machine, one cross-machine exchange per GPU.  usage: allreduce_multinode_allpairs.py GPUS_PER_NODE NODES INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllReduce
from msccl.programs.multistage import allreduce_multinode_allpairs

ap = parser(__doc__, ('gpus_per_node', 'GPUs in one machine'), ('nodes', 'number of machines'), ('instances', 'replication'))
args = ap.parse_args()
emit('allreduce-multinode-allpairs', AllReduce(args.gpus_per_node * args.nodes, args.gpus_per_node, True),
     lambda: allreduce_multinode_allpairs(args.gpus_per_node, args.nodes), args.instances, args.protocol, execute=args.execute)
