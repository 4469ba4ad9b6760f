"""Tracing-compiler support: every operator that touches tensor data has a shape-only ("fake") kernel, so the public
operators propagate shapes on fake tensors (checked here without a GPU) and `torch.compile(fullgraph=True)` traces
models that call them, forward and backward, without graph breaks (checked on a GPU against eager results)."""
import pytest
import torch

import pytorch_scatter_b200 as ts


def test_fake_tensor_shapes_without_a_gpu():
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        src = torch.empty(3, 100, 16, device='cuda', dtype=torch.bfloat16)
        index = torch.empty(100, dtype=torch.long, device='cuda')
        indptr = torch.empty(11, dtype=torch.long, device='cuda').view(1, 11)
        table = torch.empty(3, 10, 16, device='cuda')
        for reduce in ('sum', 'mean', 'min', 'max', 'mul'):
            out = ts.scatter(src, index, dim=1, dim_size=10, reduce=reduce)
            assert tuple(out.shape) == (3, 10, 16) and out.dtype == src.dtype and out.device.type == 'cuda'
        out, arg = ts.scatter_max(src, index, 1, None, 10)
        assert arg.dtype == torch.long and arg.shape == out.shape
        for reduce in ('sum', 'mean', 'min', 'max'):
            assert tuple(ts.segment_csr(src, indptr, reduce=reduce).shape) == (3, 10, 16)
            assert tuple(ts.segment_coo(src, index.view(1, -1), dim_size=10, reduce=reduce).shape) == (3, 10, 16)
        assert tuple(ts.gather_coo(table, index.view(1, -1)).shape) == (3, 100, 16)
        flat = torch.empty(100, 16, device='cuda')
        assert tuple(ts.scatter_softmax(flat, index, 0, dim_size=10).shape) == (100, 16)
        assert tuple(ts.scatter_log_softmax(flat, index, 0, dim_size=10).shape) == (100, 16)
        assert tuple(ts.scatter_std(flat, index, 0, dim_size=10).shape) == (10, 16)
        with pytest.raises(RuntimeError, match='cannot be traced'):
            ts.scatter(flat, index, dim=0, out=torch.empty(10, 16, device='cuda'))


@pytest.mark.gpu
def test_compile_fullgraph_forward_and_backward():
    torch.manual_seed(0)
    E, N, F = 5000, 300, 32
    index = torch.randint(0, N, (E,), device='cuda')
    sorted_index = index.sort()[0]
    indptr = torch.cat([torch.zeros(1, dtype=torch.long, device='cuda'), torch.bincount(sorted_index, minlength=N).cumsum(0)])

    def model(x, w):
        h = x * w
        agg = ts.scatter(h, index, dim=0, dim_size=N, reduce='sum') + ts.scatter(h, index, dim=0, dim_size=N, reduce='max')
        seg = ts.segment_csr(h, indptr, reduce='mean') + ts.segment_coo(h, sorted_index, dim_size=N, reduce='sum')
        att = ts.scatter_softmax(h, index, dim=0, dim_size=N)
        return (agg * seg).sum() + (att * h).sum()

    compiled = torch.compile(model, fullgraph=True)
    x = torch.randn(E, F, device='cuda')
    w1 = torch.randn(F, device='cuda', requires_grad=True)
    w2 = w1.detach().clone().requires_grad_()
    want = model(x, w1)
    got = compiled(x, w2)
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-3), (float(got), float(want))
    want.backward()
    got.backward()
    assert torch.allclose(w2.grad, w1.grad, rtol=1e-4, atol=1e-2)
