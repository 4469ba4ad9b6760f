"""Host-side contract of the Python / operator layer, checked without a GPU: names, schemas,
TorchScript-ability, error behaviour, the index broadcasting helper and the `torch_scatter` name shim."""
import os.path as osp
import sys

import pytest
import torch

import pytorch_scatter_b200 as ts

ROOT = osp.dirname(osp.dirname(osp.abspath(__file__)))

UPSTREAM_NAMES = [
    'scatter_sum', 'scatter_add', 'scatter_mul', 'scatter_mean', 'scatter_min', 'scatter_max', 'scatter',
    'segment_sum_csr', 'segment_add_csr', 'segment_mean_csr', 'segment_min_csr', 'segment_max_csr', 'segment_csr',
    'gather_csr', 'segment_sum_coo', 'segment_add_coo', 'segment_mean_coo', 'segment_min_coo', 'segment_max_coo',
    'segment_coo', 'gather_coo', 'scatter_std', 'scatter_logsumexp', 'scatter_softmax', 'scatter_log_softmax',
]

# as printed from upstream's own build (csrc/scatter.cpp:272-277, segment_coo.cpp:240-246, segment_csr.cpp:233-239)
SCHEMAS = {
    'scatter_sum': 'torch_scatter::scatter_sum(Tensor _0, Tensor _1, int _2, Tensor? _3, int? _4) -> Tensor _0',
    'scatter_mul': 'torch_scatter::scatter_mul(Tensor _0, Tensor _1, int _2, Tensor? _3, int? _4) -> Tensor _0',
    'scatter_mean': 'torch_scatter::scatter_mean(Tensor _0, Tensor _1, int _2, Tensor? _3, int? _4) -> Tensor _0',
    'scatter_min': 'torch_scatter::scatter_min(Tensor _0, Tensor _1, int _2, Tensor? _3, int? _4) -> (Tensor _0, Tensor _1)',
    'scatter_max': 'torch_scatter::scatter_max(Tensor _0, Tensor _1, int _2, Tensor? _3, int? _4) -> (Tensor _0, Tensor _1)',
    'segment_sum_csr': 'torch_scatter::segment_sum_csr(Tensor _0, Tensor _1, Tensor? _2) -> Tensor _0',
    'segment_mean_csr': 'torch_scatter::segment_mean_csr(Tensor _0, Tensor _1, Tensor? _2) -> Tensor _0',
    'segment_min_csr': 'torch_scatter::segment_min_csr(Tensor _0, Tensor _1, Tensor? _2) -> (Tensor _0, Tensor _1)',
    'segment_max_csr': 'torch_scatter::segment_max_csr(Tensor _0, Tensor _1, Tensor? _2) -> (Tensor _0, Tensor _1)',
    'gather_csr': 'torch_scatter::gather_csr(Tensor _0, Tensor _1, Tensor? _2) -> Tensor _0',
    'segment_sum_coo': 'torch_scatter::segment_sum_coo(Tensor _0, Tensor _1, Tensor? _2, int? _3) -> Tensor _0',
    'segment_mean_coo': 'torch_scatter::segment_mean_coo(Tensor _0, Tensor _1, Tensor? _2, int? _3) -> Tensor _0',
    'segment_min_coo': 'torch_scatter::segment_min_coo(Tensor _0, Tensor _1, Tensor? _2, int? _3) -> (Tensor _0, Tensor _1)',
    'segment_max_coo': 'torch_scatter::segment_max_coo(Tensor _0, Tensor _1, Tensor? _2, int? _3) -> (Tensor _0, Tensor _1)',
    'gather_coo': 'torch_scatter::gather_coo(Tensor _0, Tensor _1, Tensor? _2) -> Tensor _0',
    'cuda_version': 'torch_scatter::cuda_version() -> int _0',
}


def test_public_names():
    for name in UPSTREAM_NAMES:
        assert callable(getattr(ts, name)), name
        assert name in ts.__all__


@pytest.mark.parametrize('op', sorted(SCHEMAS))
def test_operator_schemas(op):
    assert str(getattr(torch.ops.torch_scatter, op).default._schema) == SCHEMAS[op]


@pytest.mark.parametrize('name', UPSTREAM_NAMES)
def test_torchscript_compiles(name):
    scripted = torch.jit.script(getattr(ts, name))
    assert scripted is not None


def test_cpu_tensors_fail_loudly():
    src, index = torch.randn(4, 2), torch.tensor([0, 1, 0, 1])
    for fn in (lambda: ts.scatter(src, index, 0), lambda: ts.segment_coo(src, index),
               lambda: ts.segment_csr(src, torch.tensor([0, 2, 4])), lambda: ts.gather_coo(src, index),
               lambda: ts.gather_csr(src, torch.tensor([0, 1, 2, 3, 4]))):
        with pytest.raises(RuntimeError, match='must be CUDA tensor'):
            fn()


def test_bad_reduce_is_a_value_error():
    src, index = torch.randn(4), torch.tensor([0, 1, 0, 1])
    with pytest.raises(ValueError):
        ts.scatter(src, index, 0, reduce='median')
    with pytest.raises(ValueError):
        ts.segment_coo(src, index, reduce='median')
    with pytest.raises(ValueError):
        ts.segment_csr(src, torch.tensor([0, 4]), reduce='median')


def test_composites_reject_integers():
    src, index = torch.arange(4), torch.tensor([0, 1, 0, 1])
    for fn in (ts.scatter_softmax, ts.scatter_log_softmax, ts.scatter_logsumexp):
        with pytest.raises(ValueError):
            fn(src, index)


def test_broadcast_helper_is_a_view():
    from pytorch_scatter_b200.utils import broadcast
    other = torch.zeros(3, 5, 4)
    idx = broadcast(torch.arange(5), other, 1)
    assert idx.shape == other.shape and idx.stride() == (0, 1, 0)
    idx = broadcast(torch.zeros(3, 1, dtype=torch.long), other, -1)
    assert idx.shape == other.shape
    assert torch.equal(broadcast(torch.arange(5), other, -2), broadcast(torch.arange(5), other, 1))


def test_torch_scatter_name_shim():
    sys.path.insert(0, osp.join(ROOT, 'pytorch_scatter_b200', 'compat'))
    try:
        import torch_scatter
        from torch_scatter import scatter, segment_csr  # noqa: F401
        from torch_scatter.testing import dtypes, reductions  # noqa: F401
        from torch_scatter.utils import broadcast  # noqa: F401
        from torch_scatter.composite import scatter_softmax  # noqa: F401
        assert torch_scatter.scatter is ts.scatter and callable(scatter)
        assert torch_scatter.__version__ == ts.__version__
    finally:
        sys.path.pop(0)
