"""NVIDIA machine topologies and the ``nvidia-smi topo -m`` parser.

Parity: reference ``msccl/topologies/nvidia.py:9-81``.  ``b200_nvswitch`` is new: an
HGX B200 baseboard is eight GPUs behind NVSwitch with 18 NVLink-5 links each.
"""
import subprocess

from .topology import Topology

# NVLink count between GPU pairs of the DGX-1 hybrid cube-mesh, upper triangle only
# (pair -> links).  Two quads {0,1,2,3} and {4,5,6,7}; doubled links form the
# chains 0-1-3-2 / 4-5-7-6 plus the quad bridges 0-4 and 2-6.
_DGX1_PAIRS = {
    (0, 1): 2, (0, 2): 1, (0, 3): 1, (0, 4): 2,
    (1, 2): 1, (1, 3): 2, (1, 5): 1,
    (2, 3): 2, (2, 6): 2,
    (3, 7): 1,
    (4, 5): 2, (4, 6): 1, (4, 7): 1,
    (5, 6): 1, (5, 7): 2,
    (6, 7): 2,
}


def dgx1():
    links = [[0] * 8 for _ in range(8)]
    for (a, b), bw in _DGX1_PAIRS.items():
        links[a][b] = links[b][a] = bw
    return Topology('DGX1', links)


def _uniform(n, bw):
    return [[0 if s == d else bw for s in range(n)] for d in range(n)]


def dgx_a100():
    return Topology('DGX_A100', _uniform(8, 12))


def b200_nvswitch(num_gpus=8, links_per_gpu=18):
    """HGX B200: every GPU reaches every peer through NVSwitch; the per-GPU port
    (``links_per_gpu`` NVLink-5 links in, the same out) is the shared resource."""
    switches = []
    for g in range(num_gpus):
        rest = [o for o in range(num_gpus) if o != g]
        switches.append(([g], rest, links_per_gpu, f'gpu_{g}_out'))
        switches.append((rest, [g], links_per_gpu, f'gpu_{g}_in'))
    return Topology(f'B200NVSwitch(n={num_gpus})', _uniform(num_gpus, links_per_gpu), switches)


def nvlink_only(nvidia_smi_topo=None):
    """Topology whose link matrix is the NV# count matrix reported by ``nvidia-smi topo -m``."""
    if nvidia_smi_topo is None:
        nvidia_smi_topo = _get_nvidia_smi_topo()
    return Topology('NVLinkOnly', _parse_nvidia_smi_topo(nvidia_smi_topo))


def _get_nvidia_smi_topo():
    return subprocess.check_output(['nvidia-smi', 'topo', '-m']).decode('utf-8')


def _nvlink_num(cell):
    cell = cell.strip()
    return int(cell[2:]) if cell.startswith('NV') else 0


def _parse_nvidia_smi_topo(output):
    """Rows after the header that start with "GPU" form the matrix; columns are tab
    separated and only the first len(rows) columns are GPUs."""
    rows = []
    for line in output.splitlines()[1:]:
        if not line.startswith('GPU'):
            break
        rows.append(line.split('\t')[1:])
    n = len(rows)
    return [[_nvlink_num(row[g]) for g in range(n)] for row in rows]
