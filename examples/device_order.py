"""Find the permutations of this machine's GPUs that make its NVLink topology equal to a DGX-1
(what ``msccl.init('auto', ...)`` does to recognise an NDv2 and to pick ``CUDA_VISIBLE_DEVICES``).
Needs ``nvidia-smi``; pass ``--demo`` to permute a DGX-1 instead of reading the machine."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from msccl.isomorphisms import find_isomorphisms  # noqa: E402
from msccl.topologies import Topology, dgx1, nvlink_only  # noqa: E402

if '--demo' in sys.argv:
    order = [3, 0, 5, 6, 1, 7, 2, 4]
    ref = dgx1()
    local = Topology('shuffled', [[ref.links[order[d]][order[s]] for s in range(8)] for d in range(8)])
else:
    local = nvlink_only()
found = find_isomorphisms(dgx1(), local, limit=4)
if not found:
    raise SystemExit('no isomorphism to DGX-1 found')
for perm in found:
    print(perm)
