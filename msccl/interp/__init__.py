"""CPU reference interpreter for MSCCL-IR (the oracle every executor run is compared against)."""
from msccl.interp.cpu import (DeadlockError, Interpreter, RaceError, expected_result, input_chunks_of,  # noqa: F401
                              run_algorithm,
                              run_reference_check)
