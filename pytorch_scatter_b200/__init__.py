"""torch_scatter's reduction operators, rebuilt for NVIDIA B200 (sm_100a).

Same public names and signatures as ``torch_scatter`` (``torch_scatter/__init__.py:78-106`` upstream);
every operator runs as hand-written CUDA behind ``torch.ops.torch_scatter.*``.  There is no CPU path:
tensors must live on a CUDA device, and importing fails loudly if the native libraries are missing.
"""
import os.path as osp

import torch

__version__ = '2.1.2+b200'

_PKG_DIR = osp.dirname(osp.abspath(__file__))
_OPS_LIB = osp.join(_PKG_DIR, '_C.so')
_KERNEL_LIB = osp.join(_PKG_DIR, 'libtsb200.so')

for _lib in (_KERNEL_LIB, _OPS_LIB):
    if not osp.exists(_lib):
        raise ImportError(
            f"{_lib} not found. Build the native libraries first: "
            f"`python pytorch_scatter_b200/_build.py` (needs nvcc with sm_100a support).")
if not hasattr(torch.ops.torch_scatter, 'segment_sum_csr'):
    torch.ops.load_library(_OPS_LIB)

# Same compatibility gate as upstream (torch_scatter/__init__.py:49-65): the CUDA major version the
# kernels were compiled with must match PyTorch's.
cuda_version = torch.ops.torch_scatter.cuda_version()
if torch.version.cuda is not None and cuda_version != -1:  # pragma: no cover
    if cuda_version < 10000:
        _major = int(str(cuda_version)[0])
    else:
        _major = int(str(cuda_version)[0:2])
    _t_major = int(torch.version.cuda.split('.')[0])
    if _t_major != _major:
        raise RuntimeError(
            f'Detected that PyTorch and torch_scatter were compiled with different CUDA major '
            f'versions ({_t_major} vs {_major}).')

from . import _meta  # noqa  (fake kernels for tracing compilers)
from .scatter import scatter_sum, scatter_add, scatter_mul  # noqa
from .scatter import scatter_mean, scatter_min, scatter_max, scatter  # noqa
from .segment_csr import segment_sum_csr, segment_add_csr  # noqa
from .segment_csr import segment_mean_csr, segment_min_csr  # noqa
from .segment_csr import segment_max_csr, segment_csr, gather_csr  # noqa
from .segment_coo import segment_sum_coo, segment_add_coo  # noqa
from .segment_coo import segment_mean_coo, segment_min_coo  # noqa
from .segment_coo import segment_max_coo, segment_coo, gather_coo  # noqa
from .composite import scatter_std, scatter_logsumexp  # noqa
from .composite import scatter_softmax, scatter_log_softmax  # noqa

__all__ = [
    'scatter_sum',
    'scatter_add',
    'scatter_mul',
    'scatter_mean',
    'scatter_min',
    'scatter_max',
    'scatter',
    'segment_sum_csr',
    'segment_add_csr',
    'segment_mean_csr',
    'segment_min_csr',
    'segment_max_csr',
    'segment_csr',
    'gather_csr',
    'segment_sum_coo',
    'segment_add_coo',
    'segment_mean_coo',
    'segment_min_coo',
    'segment_max_coo',
    'segment_coo',
    'gather_coo',
    'scatter_std',
    'scatter_logsumexp',
    'scatter_softmax',
    'scatter_log_softmax',
    '__version__',
]
