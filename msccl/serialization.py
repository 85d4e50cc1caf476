"""``msccl_type``-tagged JSON for algorithms and everything they reference.

File format parity: reference ``msccl/serialization.py:12-108`` - files written by
either implementation load in the other.
"""
import json
import warnings

from msccl.algorithm import Algorithm, Step
from msccl.collectives import Chunk, Collective
from msccl.instance import Instance
from msccl.topologies import Topology


def _enc_algorithm(a):
    return {'msccl_type': 'algorithm', 'name': a.name, 'instance': a.instance,
            'input_map': {k: sorted(v) for k, v in a.input_map.items()},
            'output_map': {k: sorted(v) for k, v in a.output_map.items()},
            'steps': a.steps, 'collective': a.collective, 'topology': a.topology}


def _enc_step(s):
    return {'msccl_type': 'step', 'rounds': s.rounds, 'sends': [list(x) for x in s.sends]}


def _enc_collective(c):
    nested = {}
    for (rank, chunk), value in c._triggers.items():
        nested.setdefault(rank, {})[chunk] = value
    return {'msccl_type': 'collective', 'name': c.name, 'nodes': c.num_nodes, 'chunks': c._chunks,
            'triggers': nested, 'runtime_name': c.runtime_name}


def _enc_chunk(c):
    return {'msccl_type': 'chunk', 'pre': sorted(c.precondition), 'post': sorted(c.postcondition),
            'addr': c.address}


def _enc_topology(t):
    return {'msccl_type': 'topology', 'name': t.name, 'switches': t.switches, 'links': t.links}


def _enc_instance(i):
    return {'msccl_type': 'instance', 'steps': i.steps, 'extra_rounds': i.extra_rounds,
            'chunks': i.chunks, 'pipeline': i.pipeline, 'extra_memory': i.extra_memory,
            'allow_exchange': i.allow_exchange}


_ENCODERS = ((Algorithm, _enc_algorithm), (Step, _enc_step), (Collective, _enc_collective),
             (Chunk, _enc_chunk), (Topology, _enc_topology), (Instance, _enc_instance))


class MSCCLEncoder(json.JSONEncoder):
    def __init__(self):
        super().__init__()

    def default(self, o):
        for cls, fn in _ENCODERS:
            if isinstance(o, cls):
                return fn(o)
        return super().default(o)


def _dec_algorithm(o):
    return Algorithm(o['name'], o['collective'], o['topology'], o['instance'], o['steps'],
                     {int(k): set(v) for k, v in o['input_map'].items()},
                     {int(k): set(v) for k, v in o['output_map'].items()})


def _dec_collective(o):
    triggers = {(int(r), int(c)): v for r, per_rank in o['triggers'].items() for c, v in per_rank.items()}
    return Collective(o['name'], o['nodes'], o['chunks'], triggers, o['runtime_name'])


_DECODERS = {
    'algorithm': _dec_algorithm,
    'step': lambda o: Step(o['rounds'], [tuple(s) for s in o['sends']]),
    'collective': _dec_collective,
    'chunk': lambda o: Chunk(set(o['pre']), set(o['post']), o['addr']),
    'topology': lambda o: Topology(o['name'], o['links'],
                                   [tuple(sw) for sw in o['switches']]),
    'instance': lambda o: Instance(o['steps'], o['extra_rounds'], o['chunks'], o['pipeline'],
                                   o['extra_memory'], o['allow_exchange']),
}


def _object_hook(o):
    tag = o.get('msccl_type')
    if tag is None:
        return o
    if tag in _DECODERS:
        return _DECODERS[tag](o)
    warnings.warn('Unhandled msccl_type in JSON')
    return o


def MSCCLDecoder():
    return json.JSONDecoder(object_hook=_object_hook)


def save_msccl_object(obj, filename):
    with open(filename, 'w') as f:
        f.write(MSCCLEncoder().encode(obj))


def load_msccl_object(filename):
    with open(filename) as f:
        return MSCCLDecoder().decode(f.read())
