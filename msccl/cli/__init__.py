"""Command-line interface (entry point ``msccl.__main__:main``)."""
from msccl.cli.commands import (make_analyses, make_check, make_composers, make_distributors,
                                make_handle_ncclize, make_plans, make_run, make_solvers)
