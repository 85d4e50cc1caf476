"""``msccl.init``: choose registered plans for the requested collectives and sizes, materialise
their MSCCL-IR XML, write the ``<msccl_algos>`` plan table and publish it through environment
variables (``MSCCL_CONFIG``, ``NCCL_ALGO``).  The in-repo executor (``msccl.runtime``) loads the
same plan table, so the call both stays compatible with an external MSCCL runtime and drives
the native one.

Parity: reference ``msccl/autosynth/__init__.py:24-284`` (messages are kept verbatim because
users grep them).
"""
import fcntl
import math
import os
import re
import subprocess
import tempfile
import xml.etree.ElementTree as ET
from enum import Enum

from tabulate import tabulate

from msccl.autosynth.plans_azure import register_ndv2_plans, register_ndv4_plans
from msccl.autosynth.plans_b200 import register_b200_plans
from msccl.autosynth.registry import synthesis_plans
from msccl.synth.symmetry import find_isomorphisms
from msccl.topologies import dgx1, dgx_a100, nvlink_only
from msccl.utils.sizes import format_size, parse_size

register_ndv2_plans()
register_ndv4_plans()
register_b200_plans()


class Collective(Enum):
    allreduce = 'allreduce'
    allgather = 'allgather'
    reduce = 'reduce'
    broadcast = 'broadcast'
    alltoall = 'alltoall'
    reduce_scatter = 'reduce_scatter'

    def __str__(self):
        return self.value


def _detect_machine_type():
    seen = nvlink_only()
    n = seen.num_nodes()
    if n == 8 and len(find_isomorphisms(dgx1(), seen)) == 4:
        return 'ndv2'
    if seen.links == dgx_a100().links:
        return 'ndv4'
    if n in (2, 4, 8) and all(seen.links[d][s] == 18 for d in range(n) for s in range(n) if s != d):
        return 'b200' if n == 8 else f'b200x{n}'      # NV18 everywhere: NVLink 5 behind NVSwitch
    return None


def _request_range(sizes):
    if isinstance(sizes, tuple):
        low, high = sizes
        low = parse_size(low) if isinstance(low, str) else low
        high = math.inf if high is None else (parse_size(high) if isinstance(high, str) else high)
        return low, high
    point = parse_size(sizes) if isinstance(sizes, str) else sizes
    return point, point + 1


def init(machine_type, num_machines, *collectives):
    """``init('ndv4', 1, ('allreduce', (512, '20MB')), (Collective.alltoall, '1MB'))``."""
    if machine_type == 'auto':
        machine_type = _detect_machine_type()
        if machine_type is None:
            print('Did not recognize the SKU type automatically. If you are sure about the SKU, try replacing '
                  '"auto" with your explicit SKU name. Falling back to NCCL.')
            return
        print(f'The auto-detected SKU is a {machine_type}.')

    chosen = {}
    for name, sizes in collectives:
        name = str(name) if isinstance(name, Collective) else name
        plans = _select_plans(name, synthesis_plans[(name, machine_type)], num_machines, _request_range(sizes))
        if plans:
            chosen[name] = plans

    table = ET.Element('msccl_algos')
    for plans in chosen.values():
        for provider, (low, high, proto) in plans:
            load = ET.SubElement(table, 'load')
            load.set('path', provider(num_machines))
            if low != 0:
                load.set('minBytes', str(low))
            if high != math.inf:
                load.set('maxBytes', str(high))
            load.set('proto', proto)
    if len(table) == 0:
        print('MSCCL: No algorithms were selected.')
        return
    ET.indent(table, space='  ')
    fd, path = tempfile.mkstemp(suffix='.msccl_algos.xml')
    with os.fdopen(fd, 'w') as f:
        f.write(ET.tostring(table, encoding='unicode'))

    env = {'MSCCL_CONFIG': path}
    current = os.environ.get('NCCL_ALGO', '')
    if current == '':
        env['NCCL_ALGO'] = 'MSCCL,RING,TREE'
    elif 'MSCCL' not in current.split(','):
        os.environ['NCCL_ALGO'] = 'MSCCL,' + current
    if machine_type == 'ndv4' and num_machines >= 8 and 'alltoall' in chosen:
        print('MSCCL: Setting NCCL_IB_AR_THRESHOLD=0 (reason: alltoall and at least 16 ndv4 machines)')
        env['NCCL_IB_AR_THRESHOLD'] = '0'
    if machine_type == 'ndv4':
        print('MSCCL: Setting relaxed orderin, topo file and visible devices order')
        env['NCCL_IB_PCI_RELAXED_ORDERING'] = '1'
        env['NCCL_TOPO_FILE'] = '/opt/msft/topo.xml'
        env['CUDA_VISIBLE_DEVICES'] = '0,1,2,3,4,5,6,7'
    os.environ.update(env)


def _format_size(size):
    return 'infinity' if size == math.inf else format_size(size)


def _select_plans(name, candidates, num_machines, sizes):
    """Cut the byte axis at every applicable candidate's bounds; on each piece that overlaps the
    request the highest-priority candidate wins (the later registration on ties)."""
    usable = [c for c in candidates if c[2](num_machines)]
    usable = [c for c in usable if c[3][0] < sizes[1] and sizes[0] < c[3][1]]
    cuts = sorted({0, math.inf} | {b for c in usable for b in c[3]})
    results = []
    for low, high in zip(cuts, cuts[1:]):
        if low >= sizes[1] or sizes[0] >= high:
            continue
        covering = [c for c in usable if c[3][0] <= low and high <= c[3][1]]
        described = f'{name} with sizes from {_format_size(low)} to {_format_size(high)}'
        if not covering:
            print(f'MSCCL: No plan found for {described}. Falling back to NCCL baseline.')
            continue
        desc, provider, _, _, proto, _ = sorted(covering, key=lambda c: c[5])[-1]
        print(f'MSCCL: Plan for {described} is {desc} with {proto} protocol.')
        previous = results[-1] if results else None
        if previous and previous[0] == provider and low == previous[1][1] + 1 and proto == previous[1][2]:
            previous[1][1] = high
        else:
            results.append((provider, [low, high, proto]))
    return results


# ------------------------------------------------------------------ NDv2 device order
_LOCK_FILE = '/var/lock/msccl_autosynth_inspector_topo.lock'


def ndv2_perm():  # pragma: no cover - needs an NDv2 machine with inspector-topo installed
    """Find the GPU order that makes an NDv2 look like the canonical DGX-1 with the NIC next to
    GPUs 0/2; the order is cached in a lock file that ``msccl_ndv2_launcher.sh`` exports as
    CUDA_VISIBLE_DEVICES."""
    isomorphisms = find_isomorphisms(dgx1(), nvlink_only())
    if len(isomorphisms) != 4:
        raise RuntimeError(f'Expected to find 4 isomorphisms to DGX1 topology, but found {len(isomorphisms)}.')
    return _select_isomorphism(isomorphisms)


def _select_isomorphism(isomorphisms, verbose=True, lock_file=_LOCK_FILE,
                        probe=('/usr/local/bin/inspector-topo',)):  # pragma: no cover
    with open(lock_file, 'a+') as f:
        fcntl.lockf(f, fcntl.LOCK_EX)
        try:
            f.seek(0)
            cached = f.read()
            if cached:
                if verbose:
                    print(f'MSCCL: Read IB placement from {f.name}')
                return cached
            print('MSCCL: Running inspector-topo to find the IB placement. This will take a couple of minutes...')
            env = dict(os.environ, CUDA_VISIBLE_DEVICES='0,1,2,3,4,5,6,7')
            run = subprocess.run(list(probe), stdout=subprocess.PIPE, stderr=subprocess.PIPE, env=env)
            print('MSCCL: Finished running inspector-topo. Finding the permutaion.')
            if run.returncode != 0:
                raise RuntimeError(f'inspector-topo had a failure:\n{run.stdout}\n{run.stderr}')
            found = re.search(r'GPU pair shared with NIC appears to be (\d) and (\d)', run.stdout.decode('utf-8'))
            if found is None:
                raise RuntimeError('expected to detect a pair of GPUs connected to IB but something went wrong!')
            nic_gpus = {int(found.group(1)), int(found.group(2))}
            for iso in isomorphisms:
                if not nic_gpus & {iso.nodes[0], iso.nodes[2]}:
                    order = ','.join(str(r) for r in iso.nodes)
                    f.write(order)
                    f.flush()
                    if verbose:
                        print(f'MSCCL: Wrote IB placement to {f.name}')
                    return order
            raise RuntimeError('expected an isomorphism to match our expectation but none of them did!')
        finally:
            fcntl.lockf(f, fcntl.LOCK_UN)


# ------------------------------------------------------------------------ plan listing
_MAX_DESCRIBED_MACHINES = 2048


def _describe_machines(machines):
    """'1', '2,4', '8,16,32', '>=2' ... from a predicate over machine counts."""
    accepted = [i for i in range(_MAX_DESCRIBED_MACHINES) if machines(i)]
    if not accepted:
        return '???'
    runs = []
    start = prev = accepted[0]
    for i in accepted[1:]:
        if i != prev + 1:
            runs.append((start, prev))
            start = i
        prev = i
    runs.append((start, prev))
    parts = []
    for lo, hi in runs:
        if hi == _MAX_DESCRIBED_MACHINES - 1:
            parts.append(f'>={lo}')
        else:
            parts.append(str(lo) if lo == hi else f'{lo}-{hi}')
    return ','.join(parts)


def _list_plan_parameters():
    headers = ['Machine', 'Collective', '# machines', 'From', 'To', 'Protocol', 'Priority', 'Plan name']
    keyed = []
    for (collective, machine_type), plans in synthesis_plans.items():
        for desc, _provider, machines, (low, high), protocol, priority in plans:
            keyed.append(((machine_type, collective, low, high, protocol, priority, desc),
                          (machine_type, collective, _describe_machines(machines), _format_size(low),
                           _format_size(high), protocol, priority, desc)))
    return headers, [row for _key, row in sorted(keyed, key=lambda kr: kr[0])]


def tabulate_plans():
    headers, rows = _list_plan_parameters()
    return tabulate(rows, headers=headers, tablefmt='github')


def print_plans():
    print(tabulate_plans())
