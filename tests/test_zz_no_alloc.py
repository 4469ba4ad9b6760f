"""The allocation-free segment_csr entry point (tsb_segment_csr_noalloc).

Some callers of libtsb200.so cannot allocate device memory when they call it - a server whose own pool
owns the whole GPU, a real-time loop that must not hit cudaMalloc's implicit synchronisation, a plug-in
that may only launch kernels - so this entry point keeps the reduction's scratch in a fixed 8 MiB array
inside the library.  The test drives it through the C ABI, twice in a row (the array is shared and keeps
the previous call's contents), and requires the same results as the workspace-taking entry point.
This file sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

import cabi
from helpers import assert_close, assert_sum_close
from oracle import oracle

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 8 << 20  # TSB_STATIC_SCRATCH_BYTES in include/tsb200.h


def _noalloc(src, indptr, reduce):
    B, E, K = src.shape
    N = indptr.size(-1) - 1
    out = torch.empty(B, N, K, dtype=src.dtype, device=src.device)
    arg = torch.empty(B, N, K, dtype=torch.int64, device=src.device) if reduce in ('min', 'max') else None
    I = ctypes.c_int64
    st = cabi.lib().tsb_segment_csr_noalloc(
        ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(indptr.data_ptr()), ctypes.c_void_p(out.data_ptr()),
        ctypes.c_void_p(0 if arg is None else arg.data_ptr()), I(B), I(E), I(K), I(N), I(0),
        cabi.DTYPE[src.dtype], cabi.REDUCE[reduce], ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0, cabi.lib().tsb_status_string(st).decode()
    return out, arg


def _problem(seed, rows, K, dtype):
    gen = torch.Generator().manual_seed(seed)
    lens = torch.exp(1.7 + 1.5 * torch.randn(rows, generator=gen)).floor().clamp_(0, 3000).long()
    lens[rows // 2] = 4000  # a row that spans several 512-entry chunks, so the scratch is really used
    indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).view(1, -1)
    src = torch.randn(1, int(indptr[0, -1]), K, generator=gen).to(dtype)
    return src.cuda(), indptr.cuda()


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    # two different problems back to back: the second call finds the first call's leftovers in the array
    for seed, rows, K, dtype in ((1, 3000, 64, torch.float32), (2, 1500, 16, torch.bfloat16)):
        src, indptr = _problem(seed, rows, K, dtype)
        need = cabi.lib().tsb_segment_csr_workspace_bytes(ctypes.c_int64(1), ctypes.c_int64(src.size(1)),
                                                          ctypes.c_int64(K), ctypes.c_int64(rows), cabi.DTYPE[dtype], 3)
        assert 512 < need <= STATIC_SCRATCH_BYTES
        for reduce in ('sum', 'mean', 'max'):
            want, want_arg = cabi.segment_csr(src, indptr, reduce)
            got, got_arg = _noalloc(src, indptr, reduce)
            torch.cuda.synchronize()
            assert_close(got, want, what=f'noalloc {reduce} {dtype}')
            assert torch.equal(got, want)  # both are deterministic: same chunks, same order
            if want_arg is not None:
                assert torch.equal(got_arg, want_arg)
            # and against the restatement of upstream's CPU loop directly
            ref, ref_arg = oracle.segment_csr(src.cpu(), indptr.cpu(), reduce)
            if reduce == 'max':
                assert torch.equal(got.cpu(), ref) and torch.equal(got_arg.cpu(), ref_arg)
            else:
                mass = oracle.segment_csr(src.cpu().double().abs(), indptr.cpu(), reduce)[0]
                assert_sum_close(got, oracle.segment_csr(src.cpu().double(), indptr.cpu(), reduce)[0], mass,
                                 what=f'noalloc {reduce} {dtype} vs oracle')


def test_noalloc_rejects_problems_beyond_its_scratch():
    I = ctypes.c_int64
    dummy = ctypes.c_void_p(256)  # never dereferenced: the size check comes before any launch
    E = 64 << 20  # fp32, K = 64: 131072 chunks, far more than 8 MiB of partial rows
    st = cabi.lib().tsb_segment_csr_noalloc(dummy, dummy, dummy, None, I(1), I(E), I(64), I(1000), I(0), 0, 0, None)
    assert st == 6  # TSB_ERR_TOO_LARGE
    assert b'limit' in cabi.lib().tsb_status_string(st)
