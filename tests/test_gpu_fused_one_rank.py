"""The fused compute + collective kernels in their one-rank form (every block local, the reducers add one slab, the
MoE all-to-all stays on the GPU): the same workers as the multi-GPU tests, started with a world of one process, so a
single B200 exercises the tcgen05 pipelines, the CTA-pair kernels, the block-scaled fp8 variants and the MoE routing
kernels against their PyTorch fp32 references."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(worker, port, marker, timeout=600):
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node=1', '--master-addr', '127.0.0.1',
           '--master-port', str(port), os.path.join(ROOT, 'tests', worker)]
    run = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
    assert run.returncode == 0 and marker in run.stdout, run.stdout[-3000:] + run.stderr[-3000:]


def test_fused_tensor_parallel_kernels_one_rank():
    _run('mp_fused_worker.py', 29661, 'FUSED_TP_OK')


def test_fused_moe_kernels_one_rank():
    _run('mp_moe_worker.py', 29662, 'FUSED_MOE_OK')
