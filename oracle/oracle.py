"""TEST INFRASTRUCTURE - not product code.

ctypes front-end of ``liboracle.so`` (the plain-C restatement in ``scatter_oracle.c`` of the upstream
CPU loops).  Only the tests, the smoke check and the CPU-baseline leg of the benchmark may import
this module; the shipped operators never do.

All functions take and return CPU ``torch`` tensors in the flattened layout of the upstream loops:
``src [B,E,K]``, ``out [B,N,K]``, ``indptr [Bi,N+1]`` / ``index [Bi,E]`` with ``Bi`` equal to ``B`` or 1
(one row shared by every batch).  fp16/bf16 inputs are computed in fp32 and rounded once at the end
(upstream accumulates them in fp32 for the segment ops, ``csrc/cpu/segment_csr_cpu.cpp:62``).
"""
import ctypes
import os
import os.path as osp
import subprocess

import torch

_HERE = osp.dirname(osp.abspath(__file__))
_LIB_PATH = osp.join(_HERE, 'liboracle.so')
REDUCE = {'sum': 0, 'add': 0, 'mean': 1, 'min': 2, 'max': 3, 'mul': 4}
_SUFFIX = {torch.float32: 'f32', torch.float64: 'f64', torch.int32: 'i32', torch.int64: 'i64',
           torch.uint8: 'u8', torch.int8: 'i8', torch.int16: 'i16'}
_lib = None


def build():
    """Compile liboracle.so with gcc if it is missing or older than its source."""
    src = osp.join(_HERE, 'scatter_oracle.c')
    if not osp.exists(_LIB_PATH) or osp.getmtime(_LIB_PATH) < osp.getmtime(src):
        subprocess.run([os.environ.get('CC', 'gcc'), '-O3', '-std=c11', '-fPIC', '-shared', '-o', _LIB_PATH, src, '-lm'],
                       check=True)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _i64(v):
    return ctypes.c_int64(int(v))


def _compute_dtype(t):
    return torch.float32 if t.dtype in (torch.float16, torch.bfloat16) else t.dtype


def _fn(name, dtype):
    return getattr(lib(), f'oracle_{name}_{_SUFFIX[dtype]}')


def _rows(t, B):
    """[Bi, L] int64 rows -> (contiguous tensor, batch stride)."""
    t = t.contiguous()
    assert t.dim() == 2 and t.dtype == torch.int64 and t.size(0) in (1, B)
    return t, (t.size(1) if (t.size(0) == B and B > 1) else 0)


def segment_csr(src, indptr, reduce):
    """Follows segment_csr_cpu (csrc/cpu/segment_csr_cpu.cpp:8-92).  Returns (out, arg_out or None)."""
    B, E, K = src.shape
    ct = _compute_dtype(src)
    s = src.to(ct).contiguous()
    ip, bs = _rows(indptr, B)
    N = ip.size(1) - 1
    out = torch.zeros(B, N, K, dtype=ct)
    arg = torch.full((B, N, K), E, dtype=torch.int64) if reduce in ('min', 'max') else None
    if s.numel() > 0 or N > 0:
        _fn('segment_csr', ct)(_p(s), _p(ip), _p(out), _p(arg), _i64(B), _i64(E), _i64(K), _i64(N), _i64(bs),
                               ctypes.c_int(REDUCE[reduce]))
    return out.to(src.dtype), arg


def gather_csr(src, indptr, E, out=None):
    """Follows gather_csr_cpu (csrc/cpu/segment_csr_cpu.cpp:94-162).  src [B,N,K] -> out [B,E,K]."""
    B, N, K = src.shape
    s = src.contiguous()
    ct = s.dtype if s.dtype in _SUFFIX else None
    ip, bs = _rows(indptr, B)
    if out is None:
        out = torch.zeros(B, E, K, dtype=src.dtype)
    if ct is None:  # 16-bit: a pure copy, route through fp32 losslessly
        o32, s32 = out.float(), s.float()
        _fn('gather_csr', torch.float32)(_p(s32), _p(ip), _p(o32), _i64(B), _i64(E), _i64(K), _i64(N), _i64(bs))
        out.copy_(o32.to(src.dtype))
    else:
        _fn('gather_csr', ct)(_p(s), _p(ip), _p(out), _i64(B), _i64(E), _i64(K), _i64(N), _i64(bs))
    return out


def segment_coo(src, index, N, reduce, out=None):
    """Follows segment_coo_cpu (csrc/cpu/segment_coo_cpu.cpp:8-141).

    Returns (out, extra): extra is arg_out for min/max, the clamped count [B,N] for mean, else None.
    A given ``out`` is accumulated into (a copy of) it, first run seeded the way upstream does.
    """
    B, E, K = src.shape
    ct = _compute_dtype(src)
    s = src.to(ct).contiguous()
    ix, bs = _rows(index, B)
    has_out = out is not None
    o = out.to(ct).contiguous().clone() if has_out else torch.empty(B, N, K, dtype=ct)
    arg = torch.full((B, N, K), E, dtype=torch.int64) if reduce in ('min', 'max') else None
    count = torch.zeros(B, N, dtype=ct) if reduce == 'mean' else None
    _fn('segment_coo', ct)(_p(s), _p(ix), _p(o), _p(arg), _p(count), _i64(B), _i64(E), _i64(K), _i64(N), _i64(bs),
                           ctypes.c_int(REDUCE[reduce]), ctypes.c_int(int(has_out)))
    if E == 0 and not has_out:
        o.zero_()
    extra = arg if arg is not None else (count.to(src.dtype) if count is not None else None)
    return o.to(src.dtype), extra


def gather_coo(src, index):
    """Follows gather_coo_cpu (csrc/cpu/segment_coo_cpu.cpp:143-215).  src [B,N,K] -> out [B,E,K]."""
    B, N, K = src.shape
    ix, bs = _rows(index, B)
    E = ix.size(1)
    ct = _compute_dtype(src)
    s = src.to(ct).contiguous()
    out = torch.zeros(B, E, K, dtype=ct)
    _fn('gather_coo', ct)(_p(s), _p(ix), _p(out), _i64(B), _i64(E), _i64(K), _i64(N), _i64(bs))
    return out.to(src.dtype)


def scatter(src, index, N, reduce, out=None):
    """Follows scatter_cpu (csrc/cpu/scatter_cpu.cpp:7-87); mean as torch_scatter/scatter.py:44-66.

    ``index`` is any int64 tensor expandable to ``src``'s [B,E,K] shape (e.g. [1,E,1] for a
    broadcast 1-D index, [B,E,K] for a full one).  Returns (out, arg_out or None).
    """
    B, E, K = src.shape
    ct = _compute_dtype(src)
    s = src.to(ct).contiguous()
    ix = index.contiguous()
    assert ix.dim() == 3 and ix.dtype == torch.int64
    sb = 0 if ix.size(0) == 1 else ix.stride(0)
    se = 0 if ix.size(1) == 1 else ix.stride(1)
    sk = 0 if ix.size(2) == 1 else ix.stride(2)
    has_out = out is not None
    o = out.to(ct).contiguous().clone() if has_out else torch.empty(B, N, K, dtype=ct)
    arg = torch.full((B, N, K), E, dtype=torch.int64) if reduce in ('min', 'max') else None
    count = torch.zeros((B if sb else 1) * N * (K if sk else 1), dtype=torch.int64) if reduce == 'mean' else None
    _fn('scatter', ct)(_p(s), _p(ix), _p(o), _p(arg), _p(count), _i64(B), _i64(E), _i64(K), _i64(N), _i64(sb),
                       _i64(se), _i64(sk), ctypes.c_int(REDUCE[reduce]), ctypes.c_int(int(has_out)),
                       ctypes.c_int(int(ct.is_floating_point)))
    return o.to(src.dtype), arg
