"""Synthesise a one-step all-gather for N fully connected GPUs (one NVSwitch box), lower it to MSCCL-IR
and write the XML; run it with ``torchrun --nproc-per-node N -m msccl bench --collective allgather --xml FILE``.

    python examples/synthesis/allgather_b200.py --gpus 8 --instances 8 -o allgather_fc8.xml
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from msccl.collectives import allgather  # noqa: E402
from msccl.instance import Instance  # noqa: E402
from msccl.ncclize import ncclize  # noqa: E402
from msccl.path_encoding import PathEncoding  # noqa: E402
from msccl.topologies import fully_connected  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=8)
    ap.add_argument('--instances', type=int, default=8, help='parallel copies of the algorithm (one channel each)')
    ap.add_argument('-o', '--output', default=None)
    args = ap.parse_args()
    algo = PathEncoding(fully_connected(args.gpus), allgather(args.gpus)).solve(Instance(1))
    if algo is None:
        raise SystemExit('no one-step algorithm exists for this topology')
    text = ncclize(algo, instances=args.instances, copy_threadblocks=args.instances)
    path = args.output or f'allgather_fc{args.gpus}.xml'
    with open(path, 'w') as f:
        f.write(text)
    print(f'wrote {path}: {algo.name}, {args.instances} instances')


if __name__ == '__main__':
    main()
