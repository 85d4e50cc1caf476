"""CPU reference interpreter for MSCCL-IR (the oracle every executor run is compared against)."""
from msccl.interp.cpu import (DeadlockError, Interpreter, RaceError, expected_result, run_algorithm,  # noqa: F401
                              run_reference_check)
