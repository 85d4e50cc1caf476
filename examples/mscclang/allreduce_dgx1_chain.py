"""One-chunk all-reduce over DGX-1 machines: sum along an NVLink path, exchange between machines, send back.  usage: allreduce_dgx1_chain.py NODES INSTANCES"""
from _common import emit, parser
from msccl.language.collectives import AllReduce
from msccl.programs.multistage import allreduce_dgx1_chain
from msccl.topologies import dgx1, distributed_fully_connected

ap = parser(__doc__, ('nodes', 'number of DGX-1 machines'), ('instances', 'replication'))
args = ap.parse_args()
emit('allreduce-dgx1-chain', AllReduce(8 * args.nodes, 1, True), lambda: allreduce_dgx1_chain(args.nodes), args.instances,
     args.protocol, execute=args.execute, topology=distributed_fully_connected(dgx1(), args.nodes, 1))
