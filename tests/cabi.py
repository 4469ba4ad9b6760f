"""ctypes binding of libtsb200.so used by the tests: torch CUDA tensors in, C ABI calls on the current stream."""
import ctypes
import os.path as osp

import torch

ROOT = osp.dirname(osp.dirname(osp.abspath(__file__)))
LIB_PATH = osp.join(ROOT, 'pytorch_scatter_b200', 'libtsb200.so')
DTYPE = {torch.float32: 0, torch.float64: 1, torch.float16: 2, torch.bfloat16: 3, torch.int32: 4, torch.int64: 5,
         torch.uint8: 6, torch.int8: 7, torch.int16: 8}
REDUCE = {'sum': 0, 'mean': 1, 'min': 2, 'max': 3, 'mul': 4, 'lse': 5}
_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.tsb_status_string.restype = ctypes.c_char_p
        _lib.tsb_cuda_version.restype = ctypes.c_int64
        for name in ('tsb_segment_csr_workspace_bytes', 'tsb_segment_coo_workspace_bytes', 'tsb_scatter_workspace_bytes'):
            getattr(_lib, name).restype = ctypes.c_size_t
    return _lib


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _i(v):
    return ctypes.c_int64(int(v))


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(st, what):
    assert st == 0, f'{what}: {lib().tsb_status_string(st).decode()}'


def _ws(nbytes, device):
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device)


def segment_csr(src, indptr, reduce, bstride=None):
    """src [B,E,K], indptr [Bi,N+1] (Bi in {1,B}) -> (out [B,N,K], arg or None)."""
    B, E, K = src.shape
    N = indptr.size(-1) - 1
    if bstride is None:
        bstride = 0 if indptr.size(0) == 1 else N + 1
    out = torch.empty(B, N, K, dtype=torch.float32 if reduce == 'lse' else src.dtype, device=src.device)
    arg = torch.empty(B, N, K, dtype=torch.int64, device=src.device) if reduce in ('min', 'max') else None
    d, r = DTYPE[src.dtype], REDUCE[reduce]
    nbytes = lib().tsb_segment_csr_workspace_bytes(_i(B), _i(E), _i(K), _i(N), d, r)
    ws = _ws(nbytes, src.device)
    _check(lib().tsb_segment_csr(_p(src), _p(indptr), _p(out), _p(arg), _i(B), _i(E), _i(K), _i(N), _i(bstride), d, r,
                                 _p(ws), ctypes.c_size_t(nbytes), _stream()), 'tsb_segment_csr')
    return out, arg


def gather_csr(src, indptr, E, divide=False, out=None):
    B, N, K = src.shape
    bstride = 0 if indptr.size(0) == 1 else N + 1
    if out is None:
        out = torch.zeros(B, E, K, dtype=src.dtype, device=src.device)
    _check(lib().tsb_gather_csr(_p(src), _p(indptr), _p(out), _i(B), _i(E), _i(K), _i(N), _i(bstride), DTYPE[src.dtype],
                                int(divide), _stream()), 'tsb_gather_csr')
    return out


def segment_coo(src, index, N, reduce, out=None):
    """src [B,E,K], index [Bi,E] -> (out, extra) with extra = arg (min/max) or count [B,N] (mean)."""
    B, E, K = src.shape
    bstride = 0 if index.size(0) == 1 else E
    seeded = out is not None
    if out is None:
        out = torch.empty(B, N, K, dtype=torch.float32 if reduce == 'lse' else src.dtype, device=src.device)
    arg = torch.empty(B, N, K, dtype=torch.int64, device=src.device) if reduce in ('min', 'max') else None
    count = torch.empty(B, N, dtype=src.dtype, device=src.device) if reduce == 'mean' else None
    d, r = DTYPE[src.dtype], REDUCE[reduce]
    nbytes = lib().tsb_segment_coo_workspace_bytes(_i(B), _i(E), _i(K), _i(N), d, r)
    ws = _ws(nbytes, src.device)
    _check(lib().tsb_segment_coo(_p(src), _p(index), _p(out), _p(arg), _p(count), _i(B), _i(E), _i(K), _i(N), _i(bstride),
                                 d, r, int(seeded), _p(ws), ctypes.c_size_t(nbytes), _stream()), 'tsb_segment_coo')
    return out, (arg if arg is not None else count)


def gather_coo(src, index, count=None):
    B, N, K = src.shape
    E = index.size(-1)
    bstride = 0 if index.size(0) == 1 else E
    out = torch.zeros(B, E, K, dtype=src.dtype, device=src.device)
    _check(lib().tsb_gather_coo(_p(src), _p(index), _p(out), _p(count), _i(B), _i(E), _i(K), _i(N), _i(bstride),
                                DTYPE[src.dtype], _stream()), 'tsb_gather_coo')
    return out


def gather_coo_apply(x, table, index, op):
    """x [B,E,K], table fp32 [B,N,K], index [Bi,E]; op 1: exp(x - table[index]), 2: x - table[index], 3: its square."""
    assert table.dtype == torch.float32
    B, E, K = x.shape
    bstride = 0 if index.size(0) == 1 else E
    out = torch.empty_like(x)
    _check(lib().tsb_gather_coo_apply(_p(x), _p(table), _p(index), _p(out), _i(B), _i(E), _i(K), _i(table.size(1)),
                                      _i(bstride), DTYPE[x.dtype], int(op), _stream()), 'tsb_gather_coo_apply')
    return out


def index_unsorted(index):
    flag = torch.full((1,), -1, dtype=torch.int32, device=index.device)
    _check(lib().tsb_index_unsorted(_p(index), _i(index.numel()), _p(flag), _stream()), 'tsb_index_unsorted')
    return bool(flag.item())


def scatter(src, index, N, reduce, strides, out=None):
    """src [B,E,K]; index addressed with strides (sb, se, sk) -> (out, arg or None, count or None)."""
    B, E, K = src.shape
    sb, se, sk = strides
    seeded = out is not None
    if out is None:
        out = torch.empty(B, N, K, dtype=src.dtype, device=src.device)
    arg = torch.empty(B, N, K, dtype=torch.int64, device=src.device) if reduce in ('min', 'max') else None
    count = None
    if reduce == 'mean':
        count = torch.empty((B if sb else 1) * N * (K if sk else 1), dtype=torch.int32, device=src.device)
    d, r = DTYPE[src.dtype], REDUCE[reduce]
    nbytes = lib().tsb_scatter_workspace_bytes(_i(B), _i(E), _i(K), _i(N), d, r)
    ws = _ws(nbytes, src.device)
    _check(lib().tsb_scatter(_p(src), _p(index), _p(out), _p(arg), _p(count), _i(B), _i(E), _i(K), _i(N), _i(sb), _i(se),
                             _i(sk), d, r, int(seeded), _p(ws), ctypes.c_size_t(nbytes), _stream()),
           'tsb_scatter')
    return out, arg, count


def scatter_backward(grad_out, index, E, strides, count=None):
    B, N, K = grad_out.shape
    sb, se, sk = strides
    grad_in = torch.empty(B, E, K, dtype=grad_out.dtype, device=grad_out.device)
    _check(lib().tsb_scatter_backward(_p(grad_out), _p(index), _p(grad_in), _p(count), _i(B), _i(E), _i(K), _i(N), _i(sb),
                                      _i(se), _i(sk), DTYPE[grad_out.dtype], _stream()), 'tsb_scatter_backward')
    return grad_in


def arg_backward(grad_out, arg, E):
    B, N, K = grad_out.shape
    grad_in = torch.empty(B, E, K, dtype=grad_out.dtype, device=grad_out.device)
    _check(lib().tsb_arg_backward(_p(grad_out), _p(arg), _p(grad_in), _i(B), _i(E), _i(K), _i(N), DTYPE[grad_out.dtype],
                                  _stream()), 'tsb_arg_backward')
    return grad_in
