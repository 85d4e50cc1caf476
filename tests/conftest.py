import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run with -m gpu on a B200 box)')
    config.addinivalue_line('markers', 'multigpu: needs at least two CUDA devices')


def pytest_collection_modifyitems(config, items):
    import torch
    have = torch.cuda.is_available()
    count = torch.cuda.device_count() if have else 0
    for item in items:
        if 'gpu' in item.keywords and not have:
            item.add_marker(pytest.mark.skip(reason='no CUDA device'))
        if 'multigpu' in item.keywords and count < 2:
            item.add_marker(pytest.mark.skip(reason='needs >= 2 CUDA devices'))


@pytest.fixture
def in_tempdir(tmp_path):
    old = os.getcwd()
    os.chdir(tmp_path)
    try:
        yield tmp_path
    finally:
        os.chdir(old)


@pytest.fixture
def clean_env():
    keys = ('MSCCL_CONFIG', 'NCCL_ALGO', 'NCCL_IB_AR_THRESHOLD', 'NCCL_IB_PCI_RELAXED_ORDERING',
            'NCCL_TOPO_FILE', 'CUDA_VISIBLE_DEVICES')
    saved = {k: os.environ.pop(k, None) for k in keys}
    try:
        yield
    finally:
        for k, v in saved.items():
            os.environ.pop(k, None)
            if v is not None:
                os.environ[k] = v
