import os
import os.path as osp
import sys

import pytest

ROOT = osp.dirname(osp.dirname(osp.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run on a B200)')
    # The native libraries are git-ignored build products: compile them when a fresh checkout
    # runs the tests (nvcc cross-compiles without a GPU).
    pkg = osp.join(ROOT, 'pytorch_scatter_b200')
    if not (osp.exists(osp.join(pkg, 'libtsb200.so')) and osp.exists(osp.join(pkg, '_C.so'))):
        import __graft_entry__
        __graft_entry__.build()


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)
