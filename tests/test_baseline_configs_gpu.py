"""The five benchmark configurations at (or near) their own sizes, through the public Python API with no
variant forced, against the C oracle (the restatement of upstream's CPU loops).

The small-size tests elsewhere force every kernel variant in turn; which variant runs in production is decided by
size (chunk length, bucket geometry, grouped versus atomic scatter, replicated outputs, the index probe), so these
tests repeat the comparison where those decisions are the production ones:

  C1  scatter sum fp32 [1,048,576 x 32] -> 65,536 targets, full size
  C2  segment_csr sum / mean / min / max (+arg) fp32 on the 1,048,576-row power-law CSR for F in {1, 16, 64},
      gather_csr, and the scatter of the same rows through a shuffled index (the benchmark's second operator)
  C3  segment_coo / gather_coo / the four composites on the sorted index, a quarter of the rows, bf16 / fp16 / fp32
  C4  scatter sum / min / max (+arg) fp32 [E x 16] under a Zipf(1.2) index over 100,000 targets, a quarter of the
      entries, plus the variant quantised to 1/8 steps (many exact ties: the arg must be the first occurrence)
  C5  bf16 F=128 aggregation: the whole problem at 1/64 scale, and one GPU's share of the 8-GPU job (25 M edges
      into 10 M rows) checked on sampled rows

Bar: integers, MIN/MAX values and every arg index bit-exact; float SUM/MEAN within rtol 1e-5 (fp32) / 1e-2 (16-bit).
fp32 sums are compared order-independently: |result - float64 result| <= rtol * sum|terms| (a sequential fp32 sum
over a 20,000-entry row is itself further than 1e-5 * |result| from the exact value); the oracle's own fp32 output
must agree with the same float64 result within four times that bound, which ties the float64 reference (computed by
ATen on the GPU) to the oracle.  Inputs are generated on the GPU from fixed seeds and copied to the host for the
oracle, so both sides see identical bits.
"""
import os

import pytest
import torch

from helpers import assert_close
from oracle import oracle

pytestmark = pytest.mark.gpu

DEV = 'cuda'
HOOKS = ('TSB_CSR_CHUNK_ENTRIES', 'TSB_CSR_FORCE_FLAT', 'TSB_SCATTER_SLICE_BYTES', 'TSB_SCATTER_REPLICAS',
         'TSB_SCATTER_CLUSTERED', 'TSB_SCATTER_GROUPED', 'TSB_SCATTER_GROUPED_SORT', 'TSB_SCATTER_CACHED', 'TSB_CSR_KERNEL')


@pytest.fixture(scope='module')
def ts():
    import pytorch_scatter_b200
    return pytorch_scatter_b200


@pytest.fixture(autouse=True)
def no_forced_variants():
    """Nothing may dictate a kernel variant here."""
    for k in HOOKS:
        assert k not in os.environ, f'{k} is set: these tests must run the variants the library picks itself'
    yield


def gen(seed):
    return torch.Generator(device=DEV).manual_seed(seed)


def power_law_rows(rows, seed, mean=16.0, force_long=8):
    from bench import row_lengths
    lens = row_lengths(rows, seed, force_long=force_long, mean=mean)
    indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
    return lens, indptr


def ref64(src, index, N, mean=False):
    """float64 sums (or means) and the sums of |terms| behind every output, by ATen on the GPU."""
    s64 = src.double()
    want = torch.zeros((N,) + tuple(src.shape[1:]), dtype=torch.float64, device=src.device).index_add_(0, index, s64)
    mass = torch.zeros_like(want).index_add_(0, index, s64.abs_())
    if mean:
        cnt = torch.bincount(index, minlength=N).clamp_(min=1).double().view((-1,) + (1,) * (src.dim() - 1))
        want, mass = want / cnt, mass / cnt
    return want, mass


def check_sum(got, oracle_out, want64, mass64, what):
    """`got` (GPU) within rtol * mass of the float64 result; the oracle's output within four times that."""
    rtol = 1e-5 if got.dtype == torch.float32 else 1e-2
    err = (got.double() - want64).abs()
    bound = rtol * mass64 + 1e-30
    if got.dtype != torch.float32:
        bound = bound + rtol * want64.abs()
    bad = err > bound
    assert not bool(bad.any()), f'{what}: {int(bad.sum())} outputs off, worst {float((err / bound).max()):.2f} x the bound'
    o_err = (oracle_out.to(got.device).double() - want64).abs()
    o_bad = o_err > 4 * bound + 1e-6
    assert not bool(o_bad.any()), f'{what}: the oracle and the float64 reference disagree on {int(o_bad.sum())} outputs'


def exact(got, want, what):
    assert got.shape == want.shape and got.dtype == want.dtype, what
    assert torch.equal(got.cpu(), want), f'{what}: not bit-exact'


# ---------------------------------------------------------------------------------------------------------------
def test_c1_scatter_sum_full_size(ts):
    E, F, N = 1 << 20, 32, 65536
    g = gen(20240601)
    src = torch.randn(E, F, device=DEV, generator=g)
    index = torch.randint(0, N, (E,), device=DEV, generator=g)
    got = ts.scatter(src, index, 0, dim_size=N, reduce='sum')
    want, _ = oracle.scatter(src.cpu().view(1, E, F), index.cpu().view(1, E, 1), N, 'sum')
    want64, mass64 = ref64(src, index, N)
    check_sum(got, want[0], want64, mass64, 'C1 scatter sum')
    got = ts.scatter(src, index, 0, dim_size=N, reduce='mean')
    want, _ = oracle.scatter(src.cpu().view(1, E, F), index.cpu().view(1, E, 1), N, 'mean')
    want64, mass64 = ref64(src, index, N, mean=True)
    check_sum(got, want[0], want64, mass64, 'C1 scatter mean')


@pytest.mark.parametrize('F', [1, 16, 64])
def test_c2_segment_csr_full_rows(ts, F):
    rows = 1 << 20
    lens, indptr_h = power_law_rows(rows, 20240602)
    nnz = int(indptr_h[-1])
    indptr = indptr_h.to(DEV)
    index = torch.repeat_interleave(torch.arange(rows, device=DEV), lens.to(DEV))
    g = gen(20240602 + F)
    src = torch.randn(nnz, F, device=DEV, generator=g) if F > 1 else torch.randn(nnz, device=DEV, generator=g)
    src_h = src.cpu().view(1, nnz, F)
    shape = (rows, F) if F > 1 else (rows,)
    for reduce in ('sum', 'mean', 'min', 'max'):
        got = ts.segment_csr(src, indptr, reduce=reduce) if reduce in ('sum', 'mean') else \
            getattr(ts, f'segment_{reduce}_csr')(src, indptr)
        want, want_arg = oracle.segment_csr(src_h, indptr_h.view(1, -1), reduce)
        what = f'C2 segment_csr {reduce} F={F}'
        if reduce in ('sum', 'mean'):
            want64, mass64 = ref64(src.view(nnz, F), index, rows, mean=reduce == 'mean')
            check_sum(got.view(rows, F), want[0], want64, mass64, what)
        else:
            exact(got[0], want.view(shape), what)
            exact(got[1], want_arg.view(shape), what + ' arg')
        del got
    # backward of sum: gather_csr
    table = torch.randn(shape, device=DEV, generator=g)
    got = ts.gather_csr(table, indptr)
    want = oracle.gather_csr(table.cpu().view(1, rows, F), indptr_h.view(1, -1), nnz)
    exact(got, want.view((nnz, F) if F > 1 else (nnz,)), f'C2 gather_csr F={F}')
    if F == 64:
        # the benchmark's second operator: the same rows through a shuffled index (output 268 MB: larger than L2)
        perm = torch.randperm(nnz, device=DEV, generator=g)
        shuffled = index[perm]
        for reduce in ('sum', 'max'):
            want, want_arg = oracle.scatter(src_h, shuffled.cpu().view(1, nnz, 1), rows, reduce)
            if reduce == 'sum':
                got = ts.scatter(src, shuffled, 0, dim_size=rows, reduce='sum')
                want64, mass64 = ref64(src, shuffled, rows)
                check_sum(got, want[0], want64, mass64, 'C2 scatter sum F=64 (shuffled index)')
            else:
                got, got_arg = ts.scatter_max(src, shuffled, 0, None, rows)
                exact(got, want[0], 'C2 scatter max F=64 (shuffled index)')
                exact(got_arg, want_arg[0], 'C2 scatter max F=64 (shuffled index) arg')


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16, torch.float16])
def test_c3_segment_coo_quarter(ts, dtype):
    rows, F = 1 << 18, 64
    lens, indptr_h = power_law_rows(rows, 20240603, force_long=2)
    nnz = int(indptr_h[-1])
    index = torch.repeat_interleave(torch.arange(rows, device=DEV), lens.to(DEV))
    index_h = index.cpu()
    g = gen(20240603)
    src = torch.randn(nnz, F, device=DEV, generator=g).to(dtype)
    src_h = src.cpu().view(1, nnz, F)
    for reduce in ('sum', 'mean', 'min', 'max'):
        res = getattr(ts, f'segment_{reduce}_coo')(src, index, None, rows)
        want, extra = oracle.segment_coo(src_h, index_h.view(1, -1), rows, reduce)
        what = f'C3 segment_coo {reduce} {dtype}'
        if reduce in ('sum', 'mean'):
            if dtype == torch.float32:
                want64, mass64 = ref64(src, index, rows, mean=reduce == 'mean')
                check_sum(res, want[0], want64, mass64, what)
            else:
                assert_close(res, want[0], what=what)
        else:
            exact(res[0], want[0], what)
            exact(res[1], extra[0], what + ' arg')
    # dim_size inferred from the index (host sync): the last rows may be empty, so the shape can be shorter
    inferred = ts.segment_coo(src, index, reduce='max')
    assert inferred.size(0) == int(index_h[-1]) + 1
    # gather_coo: the backward of sum
    table = torch.randn(rows, F, device=DEV, generator=g).to(dtype)
    exact(ts.gather_coo(table, index), oracle.gather_coo(table.cpu().view(1, rows, F), index_h.view(1, -1))[0],
          f'C3 gather_coo {dtype}')


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16, torch.float16])
def test_c3_composites_sorted_index(ts, dtype):
    """The fused two-pass forms (the index is ascending) against the composed arithmetic of upstream's composites
    (torch_scatter/composite/softmax.py:9-51, logsumexp.py:8-56, std.py:8-39) evaluated in float64 by ATen."""
    rows, F = 1 << 18, 64
    lens, _ = power_law_rows(rows, 20240603, force_long=2)
    nnz = int(lens.sum())
    index = torch.repeat_interleave(torch.arange(rows, device=DEV), lens.to(DEV))
    g = gen(20240613)
    src = torch.randn(nnz, F, device=DEV, generator=g).to(dtype)
    x = src.double()
    ix = index.view(-1, 1).expand(-1, F)
    gmax = torch.full((rows, F), float('-inf'), dtype=torch.float64, device=DEV).scatter_reduce_(0, ix, x, 'amax')
    shifted = x - gmax[index]
    gsum = torch.zeros(rows, F, dtype=torch.float64, device=DEV).index_add_(0, index, shifted.exp())
    rtol, atol = (1e-5, 1e-6) if dtype == torch.float32 else (1e-2, 1e-3)

    def close(got, want, what):
        ok = torch.allclose(got.double(), want, rtol=rtol, atol=atol)
        assert ok, f'{what} {dtype}: max abs diff {float((got.double() - want).abs().max())}'

    close(ts.scatter_softmax(src, index, 0, dim_size=rows), shifted.exp() / gsum[index], 'C3 scatter_softmax')
    close(ts.scatter_log_softmax(src, index, 0, dim_size=rows), shifted - gsum.log()[index], 'C3 scatter_log_softmax')
    lse = (gsum.log() + gmax).nan_to_num_(neginf=0.0)   # groups nobody names give 0 upstream
    close(ts.scatter_logsumexp(src, index, 0, dim_size=rows), lse, 'C3 scatter_logsumexp')
    if dtype == torch.float32:
        cnt = torch.bincount(index, minlength=rows).double().view(-1, 1)
        mean = torch.zeros(rows, F, dtype=torch.float64, device=DEV).index_add_(0, index, x) / cnt.clamp(min=1)
        ss = torch.zeros(rows, F, dtype=torch.float64, device=DEV).index_add_(0, index, (x - mean[index]) ** 2)
        want = (ss / ((cnt - 1).clamp(min=1) + 1e-6)).sqrt()
        got = ts.scatter_std(src, index, 0, dim_size=rows)
        assert torch.allclose(got.double(), want, rtol=1e-4, atol=1e-5), float((got.double() - want).abs().max())


def zipf_index(E, N, g):
    """E i.i.d. draws from p(k) ~ k^-1.2 over N targets, the targets passed through a random permutation so that the
    hot ones are not neighbours; unsorted."""
    prob = torch.arange(1, N + 1, device=DEV, dtype=torch.float64).pow(-1.2)
    ranks = torch.multinomial((prob / prob.sum()).float(), E, replacement=True, generator=g)
    return torch.randperm(N, device=DEV, generator=g)[ranks]


@pytest.mark.parametrize('quantised', [False, True], ids=['N(0,1)', 'steps-of-1/8'])
def test_c4_scatter_zipf_quarter(ts, quantised):
    E, F, N = 1 << 23, 16, 100000
    g = gen(20240604)
    index = zipf_index(E, N, g)
    src = torch.randn(E, F, device=DEV, generator=g)
    if quantised:   # many exact ties inside every hot target: the arg must be the smallest entry id
        src = (src * 8).round_() / 8
    src_h, index_h = src.cpu().view(1, E, F), index.cpu().view(1, E, 1)
    assert int(torch.bincount(index, minlength=N).max()) > E // 20   # one target holds a large share of all entries
    got = ts.scatter(src, index, 0, dim_size=N, reduce='sum')
    want, _ = oracle.scatter(src_h, index_h, N, 'sum')
    want64, mass64 = ref64(src, index, N)
    if quantised:   # multiples of 1/8 below 2^21: every fp32 partial sum is exact, in any order
        exact(got, want64.float().cpu(), 'C4 scatter sum (exact)')
        exact(want[0], want64.float().cpu(), 'C4 oracle sum (exact)')
    else:
        check_sum(got, want[0], want64, mass64, 'C4 scatter sum')
    for reduce in ('min', 'max'):
        got, got_arg = getattr(ts, f'scatter_{reduce}')(src, index, 0, None, N)
        want, want_arg = oracle.scatter(src_h, index_h, N, reduce)
        exact(got, want[0], f'C4 scatter {reduce}')
        exact(got_arg, want_arg[0], f'C4 scatter {reduce} arg')


def test_c5_whole_problem_at_one_64th(ts):
    nodes, F = 156_250, 128
    lens, indptr_h = power_law_rows(nodes, 20240605, mean=20.0, force_long=1)
    E = int(indptr_h[-1])
    g = gen(20240605)
    src = torch.randn(E, F, device=DEV, generator=g).bfloat16()
    src_h = src.cpu().view(1, E, F)
    indptr = indptr_h.to(DEV)
    for reduce in ('sum', 'mean'):
        got = ts.segment_csr(src, indptr, reduce=reduce)
        want, _ = oracle.segment_csr(src_h, indptr_h.view(1, -1), reduce)
        assert_close(got, want[0], what=f'C5 segment_csr {reduce} bf16')
    index = torch.repeat_interleave(torch.arange(nodes, device=DEV), lens.to(DEV))
    index = index[torch.randperm(E, device=DEV, generator=g)]   # the unsorted edge list
    index_h = index.cpu().view(1, E, 1)
    got = ts.scatter(src, index, 0, dim_size=nodes, reduce='sum')
    want, _ = oracle.scatter(src_h, index_h, nodes, 'sum')
    assert_close(got, want[0], what='C5 scatter sum bf16')
    got, got_arg = ts.scatter_max(src, index, 0, None, nodes)
    want, want_arg = oracle.scatter(src_h, index_h, nodes, 'max')
    exact(got, want[0], 'C5 scatter max bf16')
    exact(got_arg, want_arg[0], 'C5 scatter max bf16 arg')


def test_c5_one_gpu_share_sampled_rows(ts):
    """One GPU's share of the 8-GPU job at its real size: 1/8 of the edges (bf16 [~25 M x 128]) reduced over the
    shard's own 1.25 M rows (segment_csr) and scattered into all 10 M destination rows (the full-length partial the
    exchange consumes).  The oracle sees every entry of a sample of rows."""
    F = 128
    rows_csr, n_all = 1_250_000, 10_000_000
    lens, indptr_h = power_law_rows(rows_csr, 20240615, mean=20.0, force_long=8)
    E = int(indptr_h[-1])
    g = gen(20240615)
    src = torch.randn(E, F, device=DEV, generator=g).bfloat16()
    indptr = indptr_h.to(DEV)
    # --- segment_csr: a contiguous range of rows, cut so that it starts and ends inside streamed chunks
    r0, r1 = 400_000, 420_000
    e0, e1 = int(indptr_h[r0]), int(indptr_h[r1])
    for reduce in ('sum', 'mean'):
        got = ts.segment_csr(src, indptr, reduce=reduce)[r0:r1]
        want, _ = oracle.segment_csr(src[e0:e1].cpu().view(1, e1 - e0, F), (indptr_h[r0:r1 + 1] - e0).view(1, -1), reduce)
        assert_close(got, want[0], what=f'C5 shard segment_csr {reduce} rows [{r0}, {r1})')
    # --- scatter into 10 M rows: every edge of the power-law graph lands on this GPU with probability 1/8
    lens_all, _ = power_law_rows(n_all, 20240625, mean=20.0, force_long=8)
    here = torch.binomial(lens_all.to(DEV).float(), torch.full((n_all,), 0.125, device=DEV), generator=g).long()
    index = torch.repeat_interleave(torch.arange(n_all, device=DEV), here)
    index = index[torch.randperm(index.numel(), device=DEV, generator=g)][:E]
    src = src[:index.numel()]
    Es = index.numel()
    sample = torch.randperm(n_all, device=DEV, generator=g)[:40_000].sort().values   # includes rows nobody names
    sample = torch.cat([sample, torch.bincount(index, minlength=n_all).topk(8).indices]).unique()   # and the longest
    lut = torch.full((n_all,), -1, dtype=torch.long, device=DEV)
    lut[sample] = torch.arange(sample.numel(), device=DEV)
    local = lut[index]
    keep = torch.nonzero(local >= 0).view(-1)          # ascending entry ids: the oracle's order is the global order
    sub_src = src[keep].cpu().view(1, keep.numel(), F)
    sub_index = local[keep].cpu().view(1, -1, 1)
    got = ts.scatter(src, index, 0, dim_size=n_all, reduce='sum')[sample]
    want, _ = oracle.scatter(sub_src, sub_index, sample.numel(), 'sum')
    assert_close(got, want[0], what='C5 shard scatter sum (sampled rows)')
    del got
    got, got_arg = ts.scatter_max(src, index, 0, None, n_all)
    want, want_arg = oracle.scatter(sub_src, sub_index, sample.numel(), 'max')
    exact(got[sample], want[0], 'C5 shard scatter max (sampled rows)')
    keep_h = torch.cat([keep.cpu(), torch.tensor([Es])])   # the oracle's "none" (its own entry count) -> ours
    exact(got_arg[sample], keep_h[want_arg[0]], 'C5 shard scatter max arg (sampled rows)')
