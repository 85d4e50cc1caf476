"""Define a collective by its pre- and postcondition, save it, and synthesise an algorithm for it:

    python examples/custom_collective_file.py send.json
    python -m msccl solve least-steps DGX1 custom --collective-file send.json
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from msccl.collectives import build_collective  # noqa: E402
from msccl.serialization import save_msccl_object  # noqa: E402

path = sys.argv[1] if len(sys.argv) > 1 else 'send.json'
# one chunk that starts on rank 2 and must reach rank 7
send = build_collective('Send', 8, 1, lambda rank, chunk: rank == 2, lambda rank, chunk: rank == 7)
save_msccl_object(send, path)
print(f'wrote {path}')
