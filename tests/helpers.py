"""Shared test helpers: API-level adapters around the C oracle, tolerances, golden loading."""
import math
import os.path as osp
import sys

import torch

ROOT = osp.dirname(osp.dirname(osp.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import oracle  # noqa: E402  (test infrastructure)

GOLDEN = osp.join(ROOT, 'tests', 'golden')

# Tolerances of the parity contract: integers, min/max values and arg indices bit-exact; float
# sums/means rtol 1e-5 (fp32), 1e-2 (fp16/bf16); atol covers cancellation near zero (upstream's own
# cross-check uses atol=1e-4, benchmark/scatter_segment.py:52).
TOL = {
    torch.float32: dict(rtol=1e-5, atol=1e-4),
    torch.float64: dict(rtol=1e-10, atol=1e-10),
    torch.float16: dict(rtol=1e-2, atol=1e-2),
    torch.bfloat16: dict(rtol=1e-2, atol=1e-2),
}


def prod(xs):
    return int(math.prod(xs))


def assert_close(got, want, exact=False, what=''):
    got, want = got.cpu(), want.cpu()
    assert got.shape == want.shape, f'{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}'
    assert got.dtype == want.dtype, f'{what}: dtype {got.dtype} vs {want.dtype}'
    if exact or not got.dtype.is_floating_point:
        assert torch.equal(got, want), f'{what}: not bit-exact; max diff {(got.double() - want.double()).abs().max()}'
    else:
        tol = TOL[got.dtype]
        ok = torch.allclose(got.double(), want.double(), equal_nan=True, **tol)
        assert ok, f'{what}: max abs diff {(got.double() - want.double()).abs().max()} (tol {tol})'


def assert_sum_close(got, want64, mass64, what=''):
    """Float SUM/MEAN check that is fair to any summation order: the error against the float64 result
    must stay within rtol * (sum of |terms| behind that output), rtol = 1e-5 for fp32 and 1e-2 for
    fp16/bf16 (for 16-bit the final rounding of the result is allowed on top)."""
    got = got.cpu()
    rtol = TOL[got.dtype]['rtol']
    err = (got.double() - want64).abs()
    bound = rtol * mass64 + 1e-30
    if got.dtype in (torch.float16, torch.bfloat16):
        bound = bound + rtol * want64.abs()
    bad = err > bound
    assert not bool(bad.any()), f'{what}: {int(bad.sum())} outputs off; worst err {float(err.max())} vs bound {float(bound[err.argmax()] if bound.dim() == 0 else bound.flatten()[err.argmax()])}'


def load_golden(name):
    return torch.load(osp.join(GOLDEN, name), weights_only=False)


def _rows2d(t, lead_shape, B):
    """int64 [*lead?, L] -> [1 or B, L] for the oracle (leading dims broadcast against lead_shape)."""
    L = t.size(-1)
    if all(s == 1 for s in t.shape[:-1]):
        return t.reshape(1, L)
    return t.expand(*lead_shape, L).reshape(B, L)


def oracle_segment_csr(src, indptr, reduce):
    lead = indptr.dim() - 1
    lead_shape, E, feat = src.shape[:lead], src.size(lead), src.shape[lead + 1:]
    B, K, N = prod(lead_shape), prod(feat), indptr.size(-1) - 1
    out, arg = oracle.segment_csr(src.reshape(B, E, K), _rows2d(indptr, lead_shape, B), reduce)
    shape = (*lead_shape, N, *feat)
    return out.reshape(shape), (None if arg is None else arg.reshape(shape))


def oracle_gather_csr(src, indptr):
    lead = indptr.dim() - 1
    lead_shape, N, feat = src.shape[:lead], src.size(lead), src.shape[lead + 1:]
    B, K = prod(lead_shape), prod(feat)
    E = int(indptr.reshape(-1)[-1]) if indptr.numel() > 0 else 0
    out = oracle.gather_csr(src.reshape(B, N, K), _rows2d(indptr, lead_shape, B), E)
    return out.reshape(*lead_shape, E, *feat)


def oracle_segment_coo(src, index, dim_size, reduce, out=None):
    lead = index.dim() - 1
    lead_shape, E, feat = src.shape[:lead], src.size(lead), src.shape[lead + 1:]
    B, K = prod(lead_shape), prod(feat)
    if out is not None:
        N = out.size(lead)
    elif dim_size is not None:
        N = dim_size
    else:
        N = int(index[..., -1].max()) + 1 if index.numel() > 0 else 0
    o3 = None if out is None else out.reshape(B, N, K)
    res, extra = oracle.segment_coo(src.reshape(B, E, K), _rows2d(index, lead_shape, B), N, reduce, o3)
    shape = (*lead_shape, N, *feat)
    if extra is not None and reduce in ('min', 'max'):
        extra = extra.reshape(shape)
    return res.reshape(shape), extra


def oracle_gather_coo(src, index):
    lead = index.dim() - 1
    lead_shape, N, feat = src.shape[:lead], src.size(lead), src.shape[lead + 1:]
    B, K, E = prod(lead_shape), prod(feat), index.size(-1)
    out = oracle.gather_coo(src.reshape(B, N, K), _rows2d(index, lead_shape, B))
    return out.reshape(*lead_shape, E, *feat)


def broadcast_index(index, src, dim):
    if index.dim() == 1:
        for _ in range(dim):
            index = index.unsqueeze(0)
    for _ in range(index.dim(), src.dim()):
        index = index.unsqueeze(-1)
    return index.expand(src.size())


def oracle_scatter(src, index, dim, dim_size, reduce, out=None):
    dim = dim + src.dim() if dim < 0 else dim
    lead_shape, E, feat = src.shape[:dim], src.size(dim), src.shape[dim + 1:]
    B, K = prod(lead_shape), prod(feat)
    if out is not None:
        N = out.size(dim)
    elif dim_size is not None:
        N = dim_size
    else:
        N = int(index.max()) + 1 if index.numel() > 0 else 0
    ix = broadcast_index(index, src, dim).reshape(B, E, K).contiguous()
    # collapse dims the index does not vary in, so the oracle's count has the reference's shape
    if index.dim() == 1:
        ix = ix[:1, :, :1]
    o3 = None if out is None else out.reshape(B, N, K)
    res, arg = oracle.scatter(src.reshape(B, E, K), ix, N, reduce, o3)
    shape = (*lead_shape, N, *feat)
    return res.reshape(shape), (None if arg is None else arg.reshape(shape))
