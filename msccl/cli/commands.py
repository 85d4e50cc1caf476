"""Sub-commands of ``msccl``: solve, compose, distribute, analyze, ncclize, plans (parity with
reference ``msccl/cli/{solve,compose,distribute,analyze,ncclize,plans}.py``) plus ``check``,
``run`` and ``bench`` for the in-repo executor.

A command is a function ``register(subparsers) -> handler`` where ``handler(args)`` runs it.
"""
import sys
from pathlib import Path

from msccl.cli.options import (FileSink, KnownCollectives, KnownDistributedTopologies, KnownTopologies,
                               add_input_algorithm, add_instance, name_msccl_object, parse_fraction)


class Group:
    """``msccl <group> <subcommand> ...``."""

    def __init__(self, subparsers, name, title):
        self.name, self.title = name, title
        cmd = subparsers.add_parser(name)
        self.sub = cmd.add_subparsers(title=title, dest=title)
        self.sub.required = True
        self.handlers = {}

    def command(self, name):
        parser = self.sub.add_parser(name)

        def bind(handler):
            self.handlers[name] = handler
            return handler
        return parser, bind

    def __call__(self, args):
        if args.command != self.name:
            return False
        self.handlers[vars(args)[self.title]](args)
        return True


# ------------------------------------------------------------------------- solve
def make_solvers(subparsers):
    import msccl.synth.search as search
    group = Group(subparsers, 'solve', 'solver')

    def strategy(name, invoke, take_steps):
        parser, bind = group.command(name)
        instance = add_instance(parser, take_steps=take_steps)
        topos, colls, sink = KnownTopologies(parser), KnownCollectives(parser), FileSink(parser)

        @bind
        def run(args):
            sink.validate(args)
            topology = topos.create(args)
            collective = colls.create(args, topology.num_nodes())
            sink.write_algorithm(args, invoke(args, topology, collective, instance(args)))
        return parser

    strategy('instance', lambda a, t, c, i: search.solve_instance(t, c, i, logging=True), True)
    strategy('least-steps', lambda a, t, c, i: search.solve_least_steps(t, c, a.initial_steps, i, logging=True),
             False).add_argument('--initial-steps', type=int, default=1, metavar='N')

    parser, bind = group.command('pareto-optimal')
    topos, colls, sink = KnownTopologies(parser), KnownCollectives(parser), FileSink(parser, single_file=False)
    parser.add_argument('--min-chunks', type=int, default=1, metavar='N')
    parser.add_argument('--max-chunks', type=int, default=None, metavar='N')
    parser.add_argument('--assume-rpc-bound', default=None, metavar='N/N',
                        help='assume bandwidth optimality requires at least this many rounds per chunk')
    parser.add_argument('--no-monotonic-feasibility', action='store_true',
                        help='turn off an unproven assumption about monotonic feasibility of instances')
    parser.add_argument('--save-eagerly', action='store_true',
                        help='save algorithms as soon as they are found, without pruning non-Pareto optimal '
                             'algorithms at the end')
    instance = add_instance(parser, take_steps=False, take_rounds=False)

    @bind
    def pareto(args):
        sink.validate(args)
        topology = topos.create(args)
        base = instance(args)
        collective = colls.create(args, topology.num_nodes())
        bound = None
        if args.assume_rpc_bound:
            try:
                bound = parse_fraction(args.assume_rpc_bound)
            except ValueError:
                parser.error('could not parse --assume-rpc-bound as a fraction')
        found = []
        for algo in search.solve_all_latency_bandwidth_tradeoffs(
                topology, collective, args.min_chunks, args.max_chunks, bound,
                not args.no_monotonic_feasibility, base_instance=base, logging=True):
            found.append(algo)
            if args.save_eagerly:
                sink.write_object(args, algo, algo.name)
        if not args.save_eagerly:
            best = search.prune_pareto_optimal(found)
            print(f'Found {len(best)} Pareto optimal algorithms. Pruned {len(found) - len(best)} non-optimal algorithms.')
            for algo in best:
                sink.write_object(args, algo, algo.name)
    return group


# ----------------------------------------------------------------------- analyze
def make_analyses(subparsers):
    group = Group(subparsers, 'analyze', 'analysis')
    parser, bind = group.command('rounds')
    topos, colls = KnownTopologies(parser), KnownCollectives(parser)

    @bind
    def rounds(args):
        from msccl.synth.bounds import lower_bound_rounds
        topology = topos.create(args)
        lower_bound_rounds(topology, colls.create(args, topology.num_nodes()), logging=True)

    parser, bind = group.command('isomorphisms')
    first, second = KnownTopologies(parser, tag='1'), KnownTopologies(parser, tag='2')

    @bind
    def isomorphisms(args):
        from msccl.synth.symmetry import find_isomorphisms
        find_isomorphisms(first.create(args), second.create(args), logging=True)
    return group


# ----------------------------------------------------------------------- compose
def make_composers(subparsers):
    group = Group(subparsers, 'compose', 'composer')
    parser, bind = group.command('allreduce')
    read_rs = add_input_algorithm(parser, name='reducescatter-algorithm')
    read_ag = add_input_algorithm(parser, name='allgather-algorithm')
    sink = FileSink(parser)

    @bind
    def allreduce(args):
        from msccl.composers import compose_allreduce
        rs, ag = read_rs(args), read_ag(args)
        sink.validate(args)
        sink.write_algorithm(args, compose_allreduce(rs, ag, logging=True))
    return group


# -------------------------------------------------------------------- distribute
def make_distributors(subparsers):
    import msccl.distributors as dist
    group = Group(subparsers, 'distribute', 'distributor')

    parser, bind = group.command('alltoall-greedy')
    read = add_input_algorithm(parser)
    dtopos, sink = KnownDistributedTopologies(parser), FileSink(parser)

    @bind
    def greedy(args, read=read, dtopos=dtopos, sink=sink):
        local = read(args)
        sink.validate(args)
        topology = dtopos.create(args, local.topology)
        sink.write_algorithm(args, dist.synthesize_greedy_distributed_alltoall(topology, local, logging=True))

    parser, bind = group.command('alltoall-gather-scatter')
    read_g, read_s = add_input_algorithm(parser, name='gather'), add_input_algorithm(parser, name='scatter')
    parser.add_argument('--copies', type=int, metavar='N', required=True, help='copies of the local topology to be made')
    parser.add_argument('-bw', '--remote-bandwidth', type=int, default=1, metavar='N', help='remote bandwidth')
    sink_gs = FileSink(parser)

    @bind
    def gather_scatter(args):
        g, s = read_g(args), read_s(args)
        sink_gs.validate(args)
        sink_gs.write_algorithm(args, dist.synthesize_gather_scatter_distributed_alltoall(
            args.copies, g, s, args.remote_bandwidth, logging=True))

    parser, bind = group.command('alltoall-create-subproblem')
    topos = KnownTopologies(parser)
    parser.add_argument('--copies', type=int, metavar='N', required=True, help='copies of the local topology to be made')
    parser.add_argument('--relay-nodes', type=int, nargs='+', default=[0], help='relay nodes')
    parser.add_argument('-bw', '--remote-bandwidth', type=int, default=1, metavar='N', help='remote bandwidth')
    parser.add_argument('--share-bandwidth', action='store_true', help='share local bandwidth between relay nodes')
    sink_sub = FileSink(parser, single_file=False)

    @bind
    def create_subproblem(args):
        local = topos.create(args)
        sink_sub.validate(args)
        collective, topology = dist.make_alltoall_subproblem_collective_and_topology(
            local, args.copies, args.relay_nodes, args.remote_bandwidth, args.share_bandwidth)
        sink_sub.write_object(args, collective, collective.name)
        sink_sub.write_object(args, topology, topology.name)

    parser, bind = group.command('alltoall-stitch-subproblem')
    read_sub = add_input_algorithm(parser)
    parser.add_argument('--copies', type=int, metavar='N', required=True,
                        help='copies of the local topology made for the subproblem')
    sink_st = FileSink(parser)

    @bind
    def stitch(args):
        sub = read_sub(args)
        sink_st.validate(args)
        sink_st.write_algorithm(args, dist.synthesize_alltoall_subproblem(sub, args.copies, logging=True))
    return group


# ----------------------------------------------------------------------- ncclize
def make_handle_ncclize(subparsers):
    from msccl.ncclize import ChannelPolicy, ncclize
    parser = subparsers.add_parser('ncclize')
    read = add_input_algorithm(parser, multiple=True)
    sink = FileSink(parser)
    remap = parser.add_mutually_exclusive_group()
    remap.add_argument('--remap-scratch', action='store_true', default=None,
                       help='remap scratch buffer indices into free input/output indices')
    remap.add_argument('--no-remap-scratch', action='store_false', dest='remap_scratch',
                       help="don't remap scratch buffer indices into free input/output indices")
    parser.add_argument('--no-merge-contiguous', action='store_true',
                        help="don't merge sends/receives from/to contiguous memory")
    parser.add_argument('--no-pretty-print', action='store_true', help="don't pretty print the generated XML")
    parser.add_argument('--greedy-scratch-sorting', action='store_true',
                        help='sort scratch buffer indices greedily to increase contiguous operations')
    parser.add_argument('--no-scratch', action='store_true',
                        help='use extra space at the end of output buffer instead of the scratch buffer')
    parser.add_argument('--channel-policy', type=ChannelPolicy, choices=list(ChannelPolicy),
                        default=ChannelPolicy.MatchTopology, help='channel allocation policy')
    parser.add_argument('--instances', type=int, default=1,
                        help='number of interleaved instances of the algorithm to make')
    parser.add_argument('--copy-threadblocks', type=int, default=1,
                        help='threadblocks that share the local copies of a rank (1 = reference layout)')

    def handle(args):
        if args.command != 'ncclize':
            return False
        algorithms = read(args)
        sink.validate(args)
        for algo in algorithms:
            text = ncclize(algo, remap_scratch=args.remap_scratch, channel_policy=args.channel_policy,
                           pretty_print=not args.no_pretty_print, use_scratch=not args.no_scratch,
                           merge_contiguous=not args.no_merge_contiguous,
                           greedy_scratch_sorting=args.greedy_scratch_sorting, instances=args.instances,
                           copy_threadblocks=args.copy_threadblocks,
                           logging=True)
            sink.write(args, lambda: text, name_msccl_object(algo.name, ending='msccl.xml'))
        return True
    return handle


# ------------------------------------------------------------------------- plans
def make_plans(subparsers):
    group = Group(subparsers, 'plans', 'subcommand')
    _parser, bind = group.command('list')

    @bind
    def list_plans(args):
        from msccl.autosynth import print_plans
        print_plans()
    return group


# ------------------------------------------------- executor-facing additions (new)
def make_check(subparsers):
    """``msccl check algo.xml``: validate MSCCL-IR and run it on the CPU interpreter."""
    parser = subparsers.add_parser('check', help='validate an MSCCL-IR XML file and execute it on the CPU interpreter')
    parser.add_argument('xml', type=Path, nargs='+')
    parser.add_argument('--elems', type=int, default=0, help='elements per chunk for the numeric run (0: skip)')
    parser.add_argument('--race-check', action='store_true', help='prove every conflicting access pair is ordered')
    parser.add_argument('--cost', default=None, metavar='SIZE',
                        help='also print the depth of the longest dependent chain and a time estimate for a message of '
                             'SIZE (e.g. 1MB) on one NVSwitch box')

    def handle(args):
        if args.command != 'check':
            return False
        from msccl.xml.loader import load_xml_file
        from msccl.xml.validator import validate
        from msccl.interp.cpu import run_reference_check
        status = 0
        for path in args.xml:
            algo = load_xml_file(path)
            problems = validate(algo)
            for p in problems:
                print(f'{path}: {p}')
            if problems:
                status = 1
                continue
            summary = f'{path}: ok ({algo.ngpus} gpus, {algo.num_threadblocks()} tbs, {algo.num_steps()} steps)'
            if args.elems > 0 or args.race_check:
                verdict = run_reference_check(algo, max(args.elems, 1), race_check=args.race_check)
                summary += f'; interpreter: {verdict}'
                if not verdict.startswith('pass'):
                    status = 1
            print(summary)
            if args.cost is not None:
                from msccl.utils.sizes import parse_size
                from msccl.xml.analysis import estimate_us, summarize
                figures = summarize(algo)
                nbytes = parse_size(args.cost)
                busiest = max(figures.sent_chunks, key=figures.sent_chunks.get)
                print(f'{path}: longest chain {figures.depth} steps; gpu {busiest} sends {figures.sent_chunks[busiest]} chunks '
                      f'from {figures.sending_tbs[busiest]} threadblocks; estimate for {args.cost}: '
                      f'{estimate_us(algo, nbytes, summary=figures):.1f} us ({algo.proto})')
        sys.exit(status)
    return handle


def make_run(subparsers):
    """``msccl run`` / ``msccl bench``: execute on the GPUs of this box (under torchrun for >1 GPU)."""
    for name in ('run', 'bench'):
        parser = subparsers.add_parser(name, help='execute a collective with the native executor on this box')
        parser.add_argument('--collective', default='allreduce',
                            choices=['allreduce', 'allgather', 'alltoall', 'reduce_scatter'])
        parser.add_argument('--xml', type=Path, default=None, help='MSCCL-IR file to execute (default: registered plan)')
        parser.add_argument('--min-bytes', default='1KB')
        parser.add_argument('--max-bytes', default='64MB')
        parser.add_argument('--dtype', default='bf16', choices=['bf16', 'fp16', 'fp32'])
        parser.add_argument('--iters', type=int, default=20)
        parser.add_argument('--nccl', action='store_true', help='also time torch.distributed (NCCL) on the same sizes')
        parser.add_argument('--suite', action='store_true',
                            help='all four collectives, direct kernels and registered plans, each verified against NCCL')
        parser.add_argument('--algo', default='auto', choices=['auto', 'oneshot', 'twoshot', 'direct', 'xml', 'xmlsym'],
                            help='auto: size-based dispatch (one-shot LL, then kernels on symmetric memory); oneshot / twoshot '
                                 '(all-reduce) / direct: one native kernel; xml: the registered MSCCL-IR plan through the '
                                 'interpreter (also what auto means when --xml is given)')
        parser.add_argument('--emulate', action='store_true',
                            help='with --xml: run every rank of the program on ONE GPU (no torchrun), check the result '
                                 'against the CPU interpreter and print one row per size')
        parser.add_argument('--trace', type=Path, default=None, metavar='FILE',
                            help='with --emulate: write per-step device time stamps of the last size to FILE (JSON rows: '
                                 'rank, tb, step, type, start_ns, end_ns, wait_ns, move_ns, signal_ns; a FILE ending in .json '
                                 'gets one Trace Event document for chrome://tracing / Perfetto instead)')
        parser.add_argument('--no-direct', action='store_true',
                            help='with --emulate: every tile through the FIFOs (no stores into the receivers\' buffers)')

    def handle(args):
        if args.command not in ('run', 'bench'):
            return False
        if getattr(args, 'emulate', False):
            from msccl.runtime.bench import run_emulated
            run_emulated(args)
            return True
        from msccl.runtime.bench import main_from_args
        main_from_args(args, check=(args.command == 'run'))
        return True
    return handle
