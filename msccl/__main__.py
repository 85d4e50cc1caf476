#!/usr/bin/env python
# PYTHON_ARGCOMPLETE_OK
"""``msccl`` / ``python -m msccl``: solve, compose, distribute, analyze, ncclize, plans, check, run, bench.

Parity: reference ``msccl/__main__.py:16-35``.
"""
import argparse

from msccl.cli import (make_analyses, make_check, make_composers, make_distributors, make_handle_ncclize,
                       make_plans, make_run, make_solvers)


def main(argv=None):
    parser = argparse.ArgumentParser('msccl')
    commands = parser.add_subparsers(title='command', dest='command')
    commands.required = True
    handlers = [make(commands) for make in (make_solvers, make_composers, make_distributors, make_analyses,
                                            make_handle_ncclize, make_plans, make_check, make_run)]
    try:
        import argcomplete          # optional shell completion
        argcomplete.autocomplete(parser)
    except ImportError:
        pass
    args = parser.parse_args(argv)
    for handle in handlers:
        if handle(args):
            break


if __name__ == '__main__':
    main()
