"""Reusable argparse building blocks for the ``msccl`` command line.

Each ``add_*`` function adds arguments to a parser and returns a callable that turns parsed
arguments into an object (or writes one).  Flags and file naming have parity with reference
``msccl/cli/common.py:11-188``, ``known_collectives.py``, ``known_topologies.py``,
``known_distributed_topologies.py`` and ``known_transformers.py``.
"""
import re
import sys
from fractions import Fraction
from pathlib import Path

import msccl.collectives as collectives
import msccl.topologies as topologies
from msccl.instance import Instance
from msccl.serialization import MSCCLEncoder, load_msccl_object


def _die(message):
    print(message, file=sys.stderr)
    sys.exit(1)


def name_msccl_object(name, ending='msccl.json'):
    """'Allgather(n=4)-Ring(n=4)-steps=2' -> 'Allgather.n4-Ring.n4-steps2.msccl.json'."""
    legal = name.translate(str.maketrans({'(': '.', ',': '.', '=': None, ')': None}))
    return f'{legal}.{ending}'


def _load(path):
    if not path.exists():
        _die(f'error: input file not found: {path}')
    return load_msccl_object(path)


# ----------------------------------------------------------------------- outputs
class FileSink:
    """-o/--output | -d/--directory, -f/--force, --no-save."""

    def __init__(self, parser, single_file=True):
        self.single_file = single_file
        if single_file:
            group = parser.add_mutually_exclusive_group()
            group.add_argument('-o', '--output', type=Path, metavar='FILE', help='file to write the result to')
            group.add_argument('-d', '--directory', type=Path, default=Path(), metavar='DIR',
                               help='directory to write the result to')
        else:
            parser.add_argument('-d', '--directory', type=Path, default=Path(), metavar='DIR',
                                help='directory to write outputs to')
        parser.add_argument('-f', '--force', action='store_true', help='overwrite existing files')
        parser.add_argument('--no-save', action='store_true', help='do not save to file')

    def validate(self, args):
        output = getattr(args, 'output', None)
        if output is not None and output.is_dir():
            _die('error: output path is a directory, did you mean to use -d?')
        if args.directory is not None:
            if not args.directory.exists():
                _die('error: output directory does not exists')
            if not args.directory.is_dir():
                _die('error: output path is not a directory')

    def write(self, args, make_text, default_name):
        """Returns True when a file was written."""
        if args.no_save:
            return False
        target = getattr(args, 'output', None)
        explicit = target is not None
        if not explicit:
            target = args.directory / default_name
        if target.exists():
            if target.is_dir():
                _die('error: output path is a directory')
            if not args.force:
                print(f'file already exists, use -f/--force to overwrite {target}', file=sys.stderr)
                return False
            if not explicit:
                print(f'Overwriting {target}')
        target.write_text(make_text())
        print(f'Wrote to {target}')
        return True

    def write_object(self, args, obj, name):
        return self.write(args, lambda: MSCCLEncoder().encode(obj), name_msccl_object(name))

    def write_algorithm(self, args, algorithm):
        if algorithm is None:
            return              # the strategy already reported the failure
        if not self.write_object(args, algorithm, algorithm.name):
            print(f'\n{algorithm.name} algorithm:')
            print(algorithm)


# ------------------------------------------------------------------------ inputs
def add_input_algorithm(parser, multiple=False, name='algorithm'):
    parser.add_argument(name, type=Path, nargs='+' if multiple else 1, help='algorithm to operate on')

    def read(args):
        loaded = [_load(p) for p in vars(args)[name]]
        return loaded if multiple else loaded[0]
    return read


def add_instance(parser, take_steps=True, take_rounds=True, take_chunks=True):
    if take_steps:
        parser.add_argument('-s', '--steps', type=int, required=True)
    if take_rounds:
        parser.add_argument('-r', '--rounds', type=int, default=None, metavar='N')
    if take_chunks:
        parser.add_argument('-c', '--chunks', type=int, default=1, metavar='N')
    parser.add_argument('--pipeline', type=int, default=None, metavar='N')
    parser.add_argument('--extra-memory', type=int, default=None, metavar='N')
    parser.add_argument('--allow-exchange', action='store_true')

    def build(args):
        extra = 0
        if take_rounds and args.rounds is not None:
            if args.rounds < args.steps:
                parser.error(f'error: rounds cannot be less than steps ({args.rounds} < {args.steps})')
            extra = args.rounds - args.steps
        return Instance(steps=args.steps if take_steps else None, extra_rounds=extra,
                        chunks=args.chunks if take_chunks else 1, pipeline=args.pipeline,
                        extra_memory=args.extra_memory, allow_exchange=args.allow_exchange)
    return build


def parse_fraction(value):
    """'3' -> 3, '7/6' -> Fraction(7, 6)."""
    try:
        return int(value)
    except ValueError:
        m = re.fullmatch(r'(.+)/(.+)', value)
        if m is None:
            raise ValueError('value must be in format "<numerator>/<denominator>"')
        return Fraction(int(m.group(1)), int(m.group(2)))


# ------------------------------------------------------------------ known objects
_PLAIN, _ROOTED, _MULTIROOT = range(3)
_COLLECTIVES = {
    'Broadcast': (_ROOTED, collectives.broadcast), 'Reduce': (_ROOTED, collectives.reduce),
    'Scatter': (_ROOTED, collectives.scatter), 'Gather': (_ROOTED, collectives.gather),
    'Allgather': (_PLAIN, collectives.allgather), 'Allreduce': (_PLAIN, collectives.allreduce),
    'Alltoall': (_PLAIN, collectives.alltoall), 'ReduceScatter': (_PLAIN, collectives.reduce_scatter),
    'Scan': (_PLAIN, collectives.scan),
    'MultirootBroadcast': (_MULTIROOT, collectives.multiroot_broadcast),
    'MultirootScatter': (_MULTIROOT, collectives.multiroot_scatter),
    'MultirootGather': (_MULTIROOT, collectives.multiroot_gather),
}


class KnownCollectives:
    def __init__(self, parser):
        self.parser = parser
        parser.add_argument('collective', type=str, choices=list(_COLLECTIVES) + ['custom'], help='collective')
        parser.add_argument('--collective-file', type=Path, default=None, metavar='FILE', help='a serialized collective')
        parser.add_argument('--root', type=int, default=0, metavar='N', help='used by rooted collectives')
        parser.add_argument('--roots', type=int, nargs='+', default=[0], metavar='N',
                            help='used by multi-rooted collectives')

    def create(self, args, num_nodes):
        if args.collective == 'custom':
            if args.collective_file is None:
                self.parser.error('--collective-file is required for custom collectives')
            return _load(args.collective_file)
        kind, make = _COLLECTIVES[args.collective]
        if kind == _ROOTED:
            return make(num_nodes, args.root)
        if kind == _MULTIROOT:
            return make(num_nodes, args.roots)
        return make(num_nodes)


_SIZED = {'FullyConnected': topologies.fully_connected, 'HubAndSpoke': topologies.hub_and_spoke,
          'Ring': topologies.ring, 'Line': topologies.line, 'Star': topologies.star}
_FIXED = {'AMD4': topologies.amd4, 'AMD8': topologies.amd8, 'DGX1': topologies.dgx1,
          'DGX2': lambda: topologies.hub_and_spoke(16), 'DGXA100': topologies.dgx_a100,
          'B200': topologies.b200_nvswitch, 'NVLinkOnly': topologies.nvlink_only}
_TRANSFORMS = {'reverse': topologies.reverse_topology, 'binarize': topologies.binarize_topology}


class KnownTransformers:
    def __init__(self, parser, tag=''):
        self.key = f'transform{tag}'
        parser.add_argument(f'-t{tag}', f'--transform{tag}', action='append', default=[],
                            choices=list(_TRANSFORMS),
                            help='apply a topology transformer. may be used multiple times')

    def transform(self, args, topology):
        for name in vars(args)[self.key]:
            topology = _TRANSFORMS[name](topology)
        return topology


class KnownTopologies:
    def __init__(self, parser, tag=''):
        self.parser, self.tag = parser, tag
        parser.add_argument(f'topology{tag}', type=str, choices=list(_SIZED) + list(_FIXED) + ['custom'],
                            help=f'topology {tag}')
        parser.add_argument(f'--topology-file{tag}', type=Path, default=None, metavar='FILE',
                            help='a serialized topology')
        parser.add_argument(f'-n{tag}', f'--nodes{tag}', type=int, metavar='N',
                            help='required for non-fixed topologies')
        self.transformers = KnownTransformers(parser, tag)

    def create(self, args):
        opts = vars(args)
        name, nodes = opts[f'topology{self.tag}'], opts[f'nodes{self.tag}']
        if name == 'custom':
            path = opts[f'topology_file{self.tag}']
            if path is None:
                self.parser.error(f'--topology-file{self.tag} is required for custom topologies')
            topo = _load(path)
        elif name in _FIXED:
            topo = _FIXED[name]()
            if nodes is not None and nodes != topo.num_nodes():
                self.parser.error(f'fixed-size topology {name} has {topo.num_nodes()} nodes, but command line '
                                  f'specified {nodes} nodes')
        else:
            if nodes is None:
                self.parser.error(f'topology {name} requires -n/--nodes')
            topo = _SIZED[name](nodes)
        return self.transformers.transform(args, topo)


_DISTRIBUTED = {'DistributedFullyConnected': topologies.distributed_fully_connected,
                'DistributedHubAndSpoke': topologies.distributed_hub_and_spoke}


class KnownDistributedTopologies:
    def __init__(self, parser):
        self.parser = parser
        parser.add_argument('topology', type=str, choices=list(_DISTRIBUTED), help='the distributed topology')
        parser.add_argument('-n', '--nodes', type=int,
                            help='total nodes in the distributed topology, must be divisible by local topology')
        parser.add_argument('--copies', type=int, help='copies of the local topology to be made')
        parser.add_argument('-bw', '--remote-bandwidth', type=int, default=1, metavar='N',
                            help='bandwidth of links in the distributed topology')

    def create(self, args, local_topology):
        if args.nodes is not None and args.copies is not None:
            self.parser.error('please use only one of -n/--nodes, --copies')
        n_local = local_topology.num_nodes()
        if args.copies is not None:
            copies = args.copies
        elif args.nodes is not None:
            if args.nodes % n_local != 0:
                self.parser.error(f'total number of nodes must be divisible by the local number of nodes '
                                  f'{n_local}, but {args.nodes} was given')
            copies = args.nodes // n_local
        else:
            self.parser.error('one of the following arguments is required: --nodes, --copies')
        return _DISTRIBUTED[args.topology](local_topology, copies, args.remote_bandwidth)
