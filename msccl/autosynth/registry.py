"""Plan registry: which algorithm to use for (collective, machine type, #machines, size range).

``synthesis_plans[(collective, machine_type)]`` is a list of entries
``(description, provider, machines_predicate, (low, high), protocol, priority)`` where
``provider(num_machines)`` returns the path of an MSCCL-IR XML file.

Parity: reference ``msccl/autosynth/registry.py:16-99``.
"""
import atexit
import math
import os
import tempfile
from collections import defaultdict

import msccl.language.collectives as lang_collectives
from msccl.language import MSCCLProgram
from msccl.language.mscclir import ThreadblockPolicy
from msccl.topologies import distributed_fully_connected
from msccl.utils.sizes import parse_size

synthesis_plans = defaultdict(list)


def _to_temp_file(text):
    fd, path = tempfile.mkstemp(suffix='.msccl.xml')
    with os.fdopen(fd, 'w') as f:
        f.write(text)
    atexit.register(lambda p=path: os.path.exists(p) and os.remove(p))
    return path


def _normalise_sizes(sizes):
    if sizes is None:
        return 0, math.inf
    low, high = sizes
    low = parse_size(low) if isinstance(low, str) else low
    high = math.inf if high is None else (parse_size(high) if isinstance(high, str) else high)
    return low, high


def _register_ef_provider(desc, fun, collective, machine_type, machines, sizes, protocol, priority):
    entry = (desc, fun, machines, _normalise_sizes(sizes), protocol, priority)
    for mtype in (machine_type if isinstance(machine_type, list) else [machine_type]):
        synthesis_plans[(collective, mtype)].append(entry)


def register_ef_file(path, collective, machine_type, num_machines, sizes=None, protocol='Simple', priority=0):
    """Register an existing XML file for exactly ``num_machines`` machines."""
    _register_ef_provider(f'load {path}', lambda machines: path, collective, machine_type,
                          lambda m: m == num_machines, sizes, protocol, priority)


def register_synthesis_plan(collective, machine_type, machines=lambda x: True, sizes=None, protocol='Simple',
                            priority=0):
    """Decorator for a function ``f(num_machines) -> XML text`` (typically synthesis + ncclize)."""
    def decorator(fun):
        _register_ef_provider(f'call {fun.__name__}', lambda m: _to_temp_file(fun(m)), collective,
                              machine_type, machines, sizes, protocol, priority)
        return fun
    return decorator


_LANGUAGE_COLLECTIVES = {'allreduce': lang_collectives.AllReduce, 'allgather': lang_collectives.AllGather,
                         'alltoall': lang_collectives.AllToAll, 'reduce_scatter': lang_collectives.ReduceScatter}


def register_msccl_program(local_topology, collective, machine_type, machines=lambda x: True, sizes=None,
                           protocol='Simple', chunk_factor=1, priority=0, collective_obj=None, instances=1,
                           inplace=False, threadblock_policy=ThreadblockPolicy.auto,
                           interleaved_replication=True, dependence_nop=False):
    """Decorator for an MSCCLang body ``f(program, num_machines)``; the program runs over
    ``num_machines`` copies of ``local_topology`` and is checked before its XML is emitted."""
    def decorator(fun):
        name = fun.__name__

        def provider(num_machines):
            topology = distributed_fully_connected(local_topology, num_machines, 1)
            coll = collective_obj
            if coll is None:
                if collective not in _LANGUAGE_COLLECTIVES:
                    raise RuntimeError(f'No collective_obj in msccl.language.collectives known for "{collective}"')
                coll = _LANGUAGE_COLLECTIVES[collective](topology.num_nodes(), chunk_factor, inplace)
            prog = MSCCLProgram(name, topology, coll, instances, protocol, threadblock_policy=threadblock_policy,
                                interleaved_replication=interleaved_replication, dependence_nop=dependence_nop)
            with prog:
                fun(prog, num_machines)
            prog.check()
            return _to_temp_file(prog.generate_xml())

        _register_ef_provider(f'run {name}', provider, collective, machine_type, machines, sizes, protocol, priority)
        return fun
    return decorator
