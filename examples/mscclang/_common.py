"""Shared command-line plumbing of the MSCCLang example scripts."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from msccl.language import MSCCLProgram, ThreadblockPolicy  # noqa: E402
from msccl.topologies import fully_connected  # noqa: E402


def parser(description, *positional):
    ap = argparse.ArgumentParser(description=description)
    for name, helptext in positional:
        ap.add_argument(name, type=int, help=helptext)
    ap.add_argument('--protocol', default='Simple', choices=['Simple', 'LL', 'LL128'])
    ap.add_argument('--execute', action='store_true',
                    help='also validate the XML and run it on the CPU reference interpreter')
    return ap


def emit(name, collective, body, instances=1, protocol='Simple', manual=False, execute=False, topology=None,
         **program_options):
    """Compile ``body`` into MSCCL-IR, print the XML, report the symbolic check on stderr."""
    policy = ThreadblockPolicy.manual if manual else ThreadblockPolicy.auto
    prog = MSCCLProgram(name, topology or fully_connected(collective.num_ranks), collective, instances, protocol=protocol,
                        threadblock_policy=policy, **program_options)
    with prog:
        body()
        ok = prog.check()
    xml = prog.generate_xml()
    print(xml)
    print(f'{name}: symbolic check {"passed" if ok else "FAILED"}', file=sys.stderr)
    if execute:
        from msccl.interp import run_reference_check
        from msccl.xml import load_xml, validate
        algo = load_xml(xml)
        print(f'{name}: validator {validate(algo) or "ok"}; interpreter: {run_reference_check(algo, 4, race_check=True)}',
              file=sys.stderr)
    return xml
