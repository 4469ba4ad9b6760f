"""GPU parity proper: the C ABI of libtsb200.so against the C oracle on seeded inputs.

Integers, MIN/MAX values and arg indices must be bit-exact; float SUM/MEAN within rtol 1e-5 (fp32) /
1e-2 (fp16, bf16), atol as in helpers.TOL.  Sizes are chosen so that the oracle finishes in seconds
while every kernel variant runs: short chunks are forced so that rows straddle many chunk borders.
"""
import itertools
import os

import pytest
import torch

import cabi
from helpers import assert_close, assert_sum_close
from oracle import oracle

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int32, torch.int64,
          torch.uint8, torch.int8, torch.int16]


NARROW = (torch.uint8, torch.int8, torch.int16)


def rand_src(gen, shape, dtype):
    if dtype.is_floating_point:
        return torch.randn(shape, generator=gen, dtype=torch.float32).to(dtype)
    if dtype == torch.uint8:
        # never 0: it is MAX's identity in this type, and a row whose maximum equals the identity keeps whatever arg
        # upstream's loop last held (csrc/cpu/segment_csr_cpu.cpp:60: the arg scratch is not reset per row)
        return torch.randint(1, 5, shape, generator=gen).to(dtype)
    if dtype == torch.int8:     # small enough that no row sum leaves the type (a 5,000-entry row is not for int8)
        return torch.randint(-1, 2, shape, generator=gen).to(dtype)
    return torch.randint(-9, 10, shape, generator=gen).to(dtype)


def row_lengths(gen, rows, kind):
    if kind == 'lognormal':  # the benchmark's shape: many empty rows, a heavy tail
        lens = torch.exp(1.7 + 1.5 * torch.randn(rows, generator=gen)).floor().clamp_(0, 3000).long()
    elif kind == 'uniform':
        lens = torch.randint(0, 9, (rows,), generator=gen)
    elif kind == 'giant':    # one row holds nearly everything, the rest are empty or tiny
        lens = torch.randint(0, 2, (rows,), generator=gen)
        lens[rows // 3] = 5000
    elif kind == 'empty_ends':
        lens = torch.randint(1, 40, (rows,), generator=gen)
        lens[:40] = 0
        lens[-70:] = 0
    elif kind == 'gaps':     # runs of empty rows: shorter than, equal to and many times a 31-row window, also at both ends
        lens = torch.randint(1, 12, (rows,), generator=gen)
        for first, count in ((0, 33), (50, 5), (70, 31), (110, 62), (180, 100)):
            lens[first:first + count] = 0
        lens[-45:] = 0
    else:
        raise ValueError(kind)
    return lens


@pytest.fixture(params=[None, 32, 64, 'staged', 'walk', 'walk-32', 'stream', 'stream-32', 'rows'],
                ids=['chunk-default', 'chunk-32', 'chunk-64', 'staged-rows', 'walk', 'walk-chunk-32', 'stream', 'stream-chunk-32',
                     'row-parallel'])
def chunk(request):
    """Chunk lengths of the row-pointer reduction (short chunks make rows straddle many chunk borders), the kernel
    that stages chunks in shared memory (the default for K == 1 only) forced for every entry of up to 64 bytes, and
    each of the two chunk kernels (lane groups walking pieces / the warp streaming steps) dictated where the library
    would pick by shape, and the row-parallel kernel (a lane group per row, long rows by the whole CTA) that it picks
    for rows of a few entries."""
    names = ('TSB_CSR_CHUNK_ENTRIES', 'TSB_CSR_FORCE_FLAT', 'TSB_CSR_KERNEL')
    old = {k: os.environ.get(k) for k in names}
    for k in names:
        os.environ.pop(k, None)
    if request.param == 'staged':
        os.environ['TSB_CSR_FORCE_FLAT'] = '1'
        os.environ['TSB_CSR_CHUNK_ENTRIES'] = '64'
    elif isinstance(request.param, str):
        kernel, _, entries = request.param.partition('-')
        os.environ['TSB_CSR_KERNEL'] = kernel
        if entries:
            os.environ['TSB_CSR_CHUNK_ENTRIES'] = entries
    elif request.param is not None:
        os.environ['TSB_CSR_CHUNK_ENTRIES'] = str(request.param)
    yield request.param
    for k, v in old.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


@pytest.mark.parametrize('kind', ['lognormal', 'uniform', 'giant', 'empty_ends', 'gaps'])
@pytest.mark.parametrize('K', [1, 2, 3, 4, 16, 33, 64, 130])
def test_segment_csr_and_coo(chunk, kind, K):
    gen = torch.Generator().manual_seed(1000 + K)
    rows = 300
    lens = row_lengths(gen, rows, kind)
    indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).view(1, -1)
    E = int(indptr[0, -1])
    index = torch.repeat_interleave(torch.arange(rows), lens).view(1, -1)
    dtypes = DTYPES if K in (1, 4, 64) else [torch.float32, torch.int64, torch.bfloat16]
    for dtype in dtypes:
        src = rand_src(gen, (1, E, K), dtype)
        for reduce in ('sum', 'mean', 'min', 'max'):
            if reduce == 'mean' and dtype in NARROW and int(lens.max()) > 100:
                continue   # a count beyond the narrow type: upstream divides by the wrapped count
            want, want_arg = oracle.segment_csr(src, indptr, reduce)
            got, got_arg = cabi.segment_csr(src.cuda(), indptr.cuda(), reduce)
            got2, got_extra = cabi.segment_coo(src.cuda(), index.cuda(), rows, reduce)
            what = f'segment_csr {reduce} {dtype} K={K} {kind}'
            if dtype.is_floating_point and reduce in ('sum', 'mean'):
                # long rows: judge against float64 with a bound relative to the summed magnitudes
                want64 = oracle.segment_csr(src.double(), indptr, reduce)[0]
                mass64 = oracle.segment_csr(src.double().abs(), indptr, reduce)[0]
                assert_sum_close(got, want64, mass64, what=what)
                assert_sum_close(got2, want64, mass64, what=what.replace('csr', 'coo'))
            else:
                assert_close(got, want, what=what)
                assert_close(got2, oracle.segment_coo(src, index, rows, reduce)[0], what=what.replace('csr', 'coo'))
            if want_arg is not None:
                assert torch.equal(got_arg.cpu(), want_arg), what + ' arg'
            want_extra = oracle.segment_coo(src, index, rows, reduce)[1]
            what = f'segment_coo {reduce} {dtype} K={K} {kind}'
            if reduce in ('min', 'max'):
                assert torch.equal(got_extra.cpu(), want_extra), what + ' arg'
            elif reduce == 'mean':
                assert_close(got_extra, want_extra, what=what + ' count')


def test_segment_csr_batched(chunk):
    """Per-batch row pointers and a row pointer shared by all batches."""
    gen = torch.Generator().manual_seed(5)
    B, rows, K = 3, 50, 8
    lens = torch.stack([row_lengths(gen, rows, 'uniform') for _ in range(B)])
    E = int(lens.sum(1).max())
    lens[:, -1] += E - lens.sum(1)  # same total per batch
    indptr = torch.cat([torch.zeros(B, 1, dtype=torch.long), lens.cumsum(1)], 1)
    for dtype in (torch.float32, torch.int64):
        src = rand_src(gen, (B, E, K), dtype)
        for reduce in ('sum', 'mean', 'min', 'max'):
            for ip in (indptr, indptr[:1]):
                want, want_arg = oracle.segment_csr(src, ip, reduce)
                got, got_arg = cabi.segment_csr(src.cuda(), ip.contiguous().cuda(), reduce)
                assert_close(got, want, what=f'batched csr {reduce} {dtype}')
                if want_arg is not None:
                    assert torch.equal(got_arg.cpu(), want_arg)


def test_segment_csr_long_runs_of_empty_rows(chunk):
    """Thousands of consecutive rows without entries (node-id ranges without edges) are written as identity rows by all
    lanes side by side and skipped with a search, not closed one by one: results as for any other row structure, with
    and without seeds in the output."""
    gen = torch.Generator().manual_seed(31)
    rows = 20000
    lens = torch.randint(0, 6, (rows,), generator=gen)
    lens[:1500] = 0
    lens[4000:13007] = 0
    lens[13100:13131] = 0
    lens[-2600:] = 0
    indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).view(1, -1)
    index = torch.repeat_interleave(torch.arange(rows), lens).view(1, -1)
    E = int(indptr[0, -1])
    for K, dtype in ((64, torch.float32), (16, torch.float32), (64, torch.bfloat16), (4, torch.int64), (1, torch.float32)):
        src = rand_src(gen, (1, E, K), dtype)
        for reduce in ('sum', 'mean', 'max'):
            want, want_arg = oracle.segment_csr(src, indptr, reduce)
            got, got_arg = cabi.segment_csr(src.cuda(), indptr.cuda(), reduce)
            what = f'gaps csr {reduce} {dtype} K={K}'
            assert_close(got, want, what=what)
            if want_arg is not None:
                assert torch.equal(got_arg.cpu(), want_arg), what + ' arg'
            want, want_extra = oracle.segment_coo(src, index, rows, reduce)
            got, got_extra = cabi.segment_coo(src.cuda(), index.cuda(), rows, reduce)
            assert_close(got, want, what=what.replace('csr', 'coo'))
            if reduce == 'max':
                assert torch.equal(got_extra.cpu(), want_extra), what + ' coo arg'
            elif reduce == 'mean':
                assert_close(got_extra, want_extra, what=what + ' coo count')
        seeds = rand_src(gen, (1, rows, K), dtype)
        index0 = index.clone()   # upstream seeds the first run from row 0 of `out`: let the first run be row 0's
        index0[0, 0] = 0
        for reduce in ('sum', 'max'):
            if reduce == 'max':   # seeds no entry ties with or loses to: where a seed wins, upstream's arg is a stale
                seeds = seeds - 100 if dtype != torch.uint8 else seeds * 0   # value of an earlier run, ours is E
            want, want_extra = oracle.segment_coo(src, index0, rows, reduce, out=seeds.clone())
            got, got_extra = cabi.segment_coo(src.cuda(), index0.cuda(), rows, reduce, out=seeds.clone().cuda())
            assert_close(got, want, what=f'gaps coo seeded {reduce} {dtype} K={K}')
            if reduce == 'max':
                bad = (got_extra.cpu() != want_extra).nonzero()
                assert bad.numel() == 0, (f'gaps coo seeded {reduce} {dtype} K={K} arg: {bad.size(0)} differ, first at '
                                          f'{bad[0].tolist()}: got {int(got_extra.cpu()[tuple(bad[0])])}, '
                                          f'want {int(want_extra[tuple(bad[0])])}, row length {int(lens[bad[0][1]])}')


def test_segment_csr_deterministic(chunk):
    gen = torch.Generator().manual_seed(11)
    lens = row_lengths(gen, 2000, 'lognormal')
    indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).view(1, -1).cuda()
    src = torch.randn(1, int(indptr[0, -1]), 64, generator=gen).cuda()
    a, _ = cabi.segment_csr(src, indptr, 'sum')
    b, _ = cabi.segment_csr(src, indptr, 'sum')
    assert torch.equal(a, b)


@pytest.mark.parametrize('kind', ['lognormal', 'giant', 'empty_ends', 'gaps'])
@pytest.mark.parametrize('K', [1, 3, 4, 64])
def test_log_sum_exp_rows(chunk, kind, K):
    """TSB_LSE (the reduction behind the fused softmax composites) against float64 torch.logsumexp per row."""
    gen = torch.Generator().manual_seed(2000 + K)
    rows = 300
    lens = row_lengths(gen, rows, kind)
    indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).view(1, -1)
    index = torch.repeat_interleave(torch.arange(rows), lens).view(1, -1)
    E = int(indptr[0, -1])
    for dtype in (torch.float32, torch.float16, torch.bfloat16):   # the table is fp32 for all of them
        tol = 1e-5
        src = (4 * torch.randn(1, E, K, generator=gen)).to(dtype)
        src[0, ::7, 0] = float('-inf')       # entries that contribute nothing
        want = torch.full((1, rows, K), float('-inf'), dtype=torch.float64)
        for r in range(rows):
            lo, hi = int(indptr[0, r]), int(indptr[0, r + 1])
            if hi > lo:
                want[0, r] = torch.logsumexp(src[0, lo:hi].double(), dim=0)
        got = cabi.segment_csr(src.cuda(), indptr.cuda(), 'lse')[0].cpu().double()
        got2 = cabi.segment_coo(src.cuda(), index.cuda(), rows, 'lse')[0].cpu().double()
        for g, what in ((got, 'csr'), (got2, 'coo')):
            assert torch.equal(torch.isinf(g), torch.isinf(want)), f'lse {what} {dtype} K={K} {kind}: -inf rows'
            fin = torch.isfinite(want)
            assert torch.allclose(g[fin], want[fin], rtol=tol, atol=tol), f'lse {what} {dtype} K={K} {kind}'
    for dtype in (torch.float64, torch.int32):   # no such reduction outside fp32 accumulators
        d = torch.zeros(1, 4, 1).to(dtype).cuda()
        with pytest.raises(AssertionError, match='dtype'):
            cabi.segment_csr(d, torch.tensor([[0, 4]]).cuda(), 'lse')


def test_gather_coo_apply_and_sortedness():
    gen = torch.Generator().manual_seed(77)
    for K in (1, 3, 4, 16, 64):
        for dtype, tol in ((torch.float32, 1e-6), (torch.float16, 1e-2), (torch.bfloat16, 1e-2)):
            N, E = 200, 5000
            index = torch.randint(0, N, (1, E), generator=gen).sort(dim=1)[0]
            x = torch.randn(2, E, K, generator=gen).to(dtype)
            table = torch.randn(2, N, K, generator=gen)
            rows = table[:, index[0]]
            for op, want in ((1, (x.float() - rows).exp()), (2, x.float() - rows), (3, (x.float() - rows) ** 2)):
                got = cabi.gather_coo_apply(x.cuda(), table.cuda(), index.cuda(), op).cpu().float()
                assert torch.allclose(got, want, rtol=tol, atol=tol), f'apply op={op} {dtype} K={K}'
    asc = torch.arange(100000).cuda() // 3
    assert not cabi.index_unsorted(asc)
    assert not cabi.index_unsorted(asc[:1]) and not cabi.index_unsorted(asc[:0])
    bad = asc.clone()
    bad[99999] = 5
    assert cabi.index_unsorted(bad)
    bad = asc.clone()
    bad[0] = 1
    assert cabi.index_unsorted(bad)


def test_segment_csr_bad_pointers_do_not_fault():
    """Row pointers outside [0, E] or not ascending are clamped: garbage in, garbage out, no fault."""
    src = torch.randn(1, 100, 4).cuda()
    indptr = torch.tensor([[0, 50, 20, 1000, -5, 100]]).cuda()
    out, _ = cabi.segment_csr(src, indptr, 'sum')
    torch.cuda.synchronize()
    assert out.shape == (1, 5, 4)


@pytest.mark.parametrize('K', [1, 4, 16, 33, 64])
def test_gathers(K):
    gen = torch.Generator().manual_seed(77 + K)
    rows = 400
    for kind in ('lognormal', 'giant', 'empty_ends'):
        lens = row_lengths(gen, rows, kind)
        indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).view(1, -1)
        E = int(indptr[0, -1])
        index = torch.repeat_interleave(torch.arange(rows), lens).view(1, -1)
        for dtype in DTYPES:
            table = rand_src(gen, (1, rows, K), dtype)
            want = oracle.gather_csr(table, indptr, E)
            assert_close(cabi.gather_csr(table.cuda(), indptr.cuda(), E), want, exact=True, what=f'gather_csr {dtype} K={K}')
            want = oracle.gather_coo(table, index)
            assert_close(cabi.gather_coo(table.cuda(), index.cuda()), want, exact=True, what=f'gather_coo {dtype} K={K}')
        # fused mean backward: value / row length
        table = rand_src(gen, (1, rows, K), torch.float32)
        want = oracle.gather_csr(table / lens.clamp(min=1).view(1, -1, 1).float(), indptr, E)
        assert_close(cabi.gather_csr(table.cuda(), indptr.cuda(), E, divide=True), want, what='gather_csr divide')
        count = lens.clamp(min=1).view(1, -1).float()
        assert_close(cabi.gather_coo(table.cuda(), index.cuda(), count.cuda()), want, what='gather_coo divide')


@pytest.fixture(params=['one-pass', 'sliced', 'replicated', 'runs', 'runs-sliced', 'direct', 'grouped', 'grouped-chunk32',
                        'grouped-atomic', 'grouped-walk', 'grouped-walk-chunk32', 'grouped-stream', 'grouped-rows', 'cached',
                        'cached-replicated'])
def scatter_slices(request):
    """Forces the variants the launcher normally picks by size or by probing the index: sliced multi-pass
    accumulation (outputs larger than L2), accumulation into several copies of the output (small,
    contended outputs), the run-combining versus the direct kernels, and the atomics-free path that groups the
    entries by target row and reduces rows through the permutation (also with 32-entry chunks, so that rows
    straddle many chunk borders)."""
    names = ('TSB_SCATTER_SLICE_BYTES', 'TSB_SCATTER_REPLICAS', 'TSB_SCATTER_CLUSTERED', 'TSB_SCATTER_GROUPED',
             'TSB_CSR_CHUNK_ENTRIES', 'TSB_SCATTER_GROUPED_SORT', 'TSB_SCATTER_CACHED', 'TSB_CSR_KERNEL')
    old = {k: os.environ.get(k) for k in names}
    for k in names:
        os.environ.pop(k, None)
    if 'sliced' in request.param:
        os.environ['TSB_SCATTER_SLICE_BYTES'] = '4096'
    if request.param == 'replicated':
        os.environ['TSB_SCATTER_REPLICAS'] = '4'
    if request.param.startswith('runs'):   # the run-combining kernel on any index, clustered or not
        os.environ['TSB_SCATTER_CLUSTERED'] = '1'
    if request.param == 'direct':          # the one-update-per-entry kernels, even on a sorted index
        os.environ['TSB_SCATTER_CLUSTERED'] = '0'
    os.environ['TSB_SCATTER_GROUPED'] = '1' if request.param.startswith('grouped') else '0'
    if request.param.endswith('chunk32'):
        os.environ['TSB_CSR_CHUNK_ENTRIES'] = '32'
    if 'walk' in request.param or 'stream' in request.param:   # which chunk kernel reduces the grouped rows
        os.environ['TSB_CSR_KERNEL'] = 'walk' if 'walk' in request.param else 'stream'
    if request.param == 'grouped-rows':    # ... or the row-parallel kernel (a lane group per row)
        os.environ['TSB_CSR_KERNEL'] = 'rows'
    if request.param.startswith('cached'):  # fp32 sums through the shared-memory row cache (skewed indices)
        os.environ['TSB_SCATTER_CACHED'] = '1'
        os.environ['TSB_SCATTER_CLUSTERED'] = '0'
        if request.param == 'cached-replicated':
            os.environ['TSB_SCATTER_REPLICAS'] = '4'
    if request.param == 'grouped-atomic':  # the grouping by one global atomic per entry (huge row counts)
        os.environ['TSB_SCATTER_GROUPED_SORT'] = 'atomic'
    yield request.param
    for k, v in old.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


@pytest.mark.parametrize('K', [1, 3, 4, 16, 33, 64])
def test_scatter_rows(scatter_slices, K):
    """Index constant along the features (a broadcast 1-D index): the vectorised row kernels."""
    gen = torch.Generator().manual_seed(300 + K)
    B, E, N = 2, 3000, 97
    index = torch.randint(0, N, (1, E, 1), generator=gen)
    index[0, :200, 0] = 5  # a hot target
    ascending = index.sort(1).values  # an edge list sorted by destination: runs of equal targets
    for dtype in DTYPES:
        src = rand_src(gen, (B, E, K), dtype)
        for ix, order in ((index, 'shuffled'), (ascending, 'ascending')):
            for reduce in ('sum', 'mean', 'min', 'max'):
                if order == 'ascending' and dtype not in (torch.float32, torch.int64, torch.bfloat16):
                    continue
                if reduce == 'mean' and dtype in NARROW:
                    continue   # the hot target's count leaves the narrow type: upstream divides by the wrapped count
                want, want_arg = oracle.scatter(src, ix, N, reduce)
                got, got_arg, _ = cabi.scatter(src.cuda(), ix.cuda(), N, reduce, (0, 1, 0))
                what = f'scatter {reduce} {dtype} K={K} {order}'
                if dtype.is_floating_point and reduce in ('sum', 'mean'):
                    want64 = oracle.scatter(src.double(), ix, N, reduce)[0]
                    mass64 = oracle.scatter(src.double().abs(), ix, N, reduce)[0]
                    assert_sum_close(got, want64, mass64, what=what)
                else:
                    assert_close(got, want, what=what)
                if want_arg is not None:
                    assert torch.equal(got_arg.cpu(), want_arg), what + ' arg'


def test_scatter_elements_and_ties():
    """A full-shaped index (one target per element) and quantised values with many exact ties."""
    gen = torch.Generator().manual_seed(9)
    B, E, K, N = 2, 2000, 5, 31
    index = torch.randint(0, N, (B, E, K), generator=gen)
    for dtype in DTYPES:
        src = rand_src(gen, (B, E, K), dtype)
        if dtype.is_floating_point:
            src = (src.float() * 4).round().div(4).to(dtype)
        for reduce in ('sum', 'mean', 'min', 'max', 'mul'):
            s = src
            if reduce == 'mul':
                if dtype in (torch.float16, torch.bfloat16):
                    continue
                s = torch.where(torch.rand(src.shape, generator=gen) < 0.02, src.double().clamp(-2, 2).to(dtype),
                                torch.ones_like(src))
            want, want_arg = oracle.scatter(s, index, N, reduce)
            got, got_arg, _ = cabi.scatter(s.cuda(), index.cuda(), N, reduce, (E * K, K, 1))
            what = f'scatter elems {reduce} {dtype}'
            assert_close(got, want, what=what)
            if want_arg is not None:
                assert torch.equal(got_arg.cpu(), want_arg), what + ' arg'
                # seeded, the seeds on the same quarter-step grid as the entries: a tie keeps the seed, arg "none"
                seeds = rand_src(gen, (B, N, K), dtype)
                if dtype.is_floating_point:
                    seeds = (seeds.float() * 4).round().div(4).to(dtype)
                want, want_arg = oracle.scatter(s, index, N, reduce, seeds)
                got, got_arg, _ = cabi.scatter(s.cuda(), index.cuda(), N, reduce, (E * K, K, 1), out=seeds.clone().cuda())
                assert_close(got, want, what=what + ' seeded')
                assert torch.equal(got_arg.cpu(), want_arg), what + ' seeded arg'


def test_scatter_rows_ties(scatter_slices):
    """Quantised values, hot targets: many exact ties, the arg must be the smallest entry id; also seeded."""
    gen = torch.Generator().manual_seed(77)
    B, E, K, N = 2, 4000, 8, 50
    index = torch.randint(0, N, (1, E, 1), generator=gen)
    index[0, 100:1500, 0] = 7
    for dtype in (torch.float32, torch.int32, torch.float16, torch.float64):
        src = rand_src(gen, (B, E, K), dtype)
        base = rand_src(gen, (B, N, K), dtype)
        # Two sets of seeds: on the half-step grid of the entries, so that seeds tie with entries all the time
        # (the CPU loop's strict comparison lets the value already in `out` win: arg stays "none",
        # csrc/cpu/reducer.h:63-67), and off the grid (no seed ever equals an entry).
        if dtype.is_floating_point:
            src = (src.float() * 2).round().div(2).to(dtype)
            on_grid = (base.float() * 2).round().div(2).to(dtype)
            off_grid = (on_grid.float() + 0.25).to(dtype)
        else:
            src, on_grid = src * 2, base * 2
            off_grid = on_grid + 1
        for reduce in ('min', 'max'):
            want, want_arg = oracle.scatter(src, index, N, reduce)
            got, got_arg, _ = cabi.scatter(src.cuda(), index.cuda(), N, reduce, (0, 1, 0))
            assert_close(got, want, what=f'ties {reduce} {dtype}')
            assert torch.equal(got_arg.cpu(), want_arg), f'ties {reduce} {dtype} arg'
            for seeds, name in ((off_grid, 'seeded'), (on_grid, 'seeded, seeds tie with entries')):
                want, want_arg = oracle.scatter(src, index, N, reduce, seeds)
                got, got_arg, _ = cabi.scatter(src.cuda(), index.cuda(), N, reduce, (0, 1, 0), out=seeds.clone().cuda())
                assert_close(got, want, what=f'{name} {reduce} {dtype}')
                assert torch.equal(got_arg.cpu(), want_arg), f'{name} {reduce} {dtype} arg'
                if name != 'seeded':   # the case must really occur: some target keeps its seed against an equal entry
                    tied = (want == seeds) & (want_arg == E)
                    hit = torch.zeros_like(tied)
                    hit[:, index.view(-1)] = True
                    assert bool((tied & hit).any())


@pytest.mark.parametrize('sort', ['buckets', 'atomic'])
def test_scatter_grouped_many_buckets(sort):
    """The atomics-free path at a size with tens of buckets, one of them (a 40,000-entry row) larger than the
    shared-memory stage, entries that name no row, and a batch dimension sharing the index."""
    names = ('TSB_SCATTER_GROUPED', 'TSB_SCATTER_GROUPED_SORT')
    old = {k: os.environ.get(k) for k in names}
    os.environ['TSB_SCATTER_GROUPED'] = '1'
    os.environ['TSB_SCATTER_GROUPED_SORT'] = sort
    try:
        gen = torch.Generator().manual_seed(91)
        B, E, K, N = 2, 400000, 4, 300000
        index = torch.randint(0, N, (1, E, 1), generator=gen)
        index[0, 1000:41000, 0] = 123456
        index[0, ::97, 0] = N + 5
        index[0, 5::101, 0] = -3
        keep = ((index >= 0) & (index < N)).view(-1)
        src = torch.randint(-8, 9, (B, E, K), generator=gen).float()   # exact in fp32 in any order
        for reduce in ('sum', 'mean', 'max'):
            got, got_arg, count = cabi.scatter(src.cuda(), index.cuda(), N, reduce, (0, 1, 0))
            kept = torch.nonzero(keep).view(-1)
            want, want_arg = oracle.scatter(src[:, keep], index[:, keep], N, reduce)
            assert_close(got, want, what=f'grouped {sort} {reduce}')
            if want_arg is not None:   # the oracle saw the compacted entries: map its args back
                lut = torch.cat([kept, torch.tensor([E])])
                assert torch.equal(got_arg.cpu(), lut[want_arg.clamp(max=kept.numel())]), f'grouped {sort} {reduce} arg'
            if reduce == 'mean':
                assert torch.equal(count.cpu().long(), torch.bincount(index.view(-1)[keep], minlength=N))
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def test_scatter_rows_mul(scatter_slices):
    """Products over a broadcast 1-D index: compare-and-swap atomics, or (grouped variants) the atomics-free path."""
    gen = torch.Generator().manual_seed(78)
    B, E, K, N = 2, 3000, 8, 40
    index = torch.randint(0, N, (1, E, 1), generator=gen)
    for dtype in (torch.float32, torch.float64, torch.int32, torch.int64):
        src = rand_src(gen, (B, E, K), dtype)
        # mostly ones, a few factors in [-2, 2]: products stay finite and exact enough for the tolerance
        s = torch.where(torch.rand(src.shape, generator=gen) < 0.02, src.double().clamp(-2, 2).to(dtype), torch.ones_like(src))
        base = rand_src(gen, (B, N, K), dtype)
        want, _ = oracle.scatter(s, index, N, 'mul')
        got, _, _ = cabi.scatter(s.cuda(), index.cuda(), N, 'mul', (0, 1, 0))
        assert_close(got, want, what=f'scatter mul {dtype}')
        want, _ = oracle.scatter(s, index, N, 'mul', base)
        got, _, _ = cabi.scatter(s.cuda(), index.cuda(), N, 'mul', (0, 1, 0), out=base.clone().cuda())
        assert_close(got, want, what=f'scatter mul seeded {dtype}')


def test_scatter_seeded_and_out_of_range(scatter_slices):
    gen = torch.Generator().manual_seed(21)
    E, K, N = 500, 8, 20
    index = torch.randint(0, N, (1, E, 1), generator=gen)
    src = torch.randn(1, E, K, generator=gen)
    base = torch.randn(1, N, K, generator=gen)
    for reduce in ('sum', 'mean', 'min', 'max'):
        want, _ = oracle.scatter(src, index, N, reduce, base)
        got, _, _ = cabi.scatter(src.cuda(), index.cuda(), N, reduce, (0, 1, 0), out=base.clone().cuda())
        assert_close(got, want, what=f'scatter seeded {reduce}')
    # targets outside [0, N) are skipped, never written
    bad = index.clone()
    bad[0, ::7, 0] = N + 3
    bad[0, 1::11, 0] = -1
    keep = ((bad >= 0) & (bad < N)).view(-1)
    want, _ = oracle.scatter(src[:, keep], bad[:, keep], N, 'sum')
    got, _, _ = cabi.scatter(src.cuda(), bad.cuda(), N, 'sum', (0, 1, 0))
    assert_close(got, want, what='scatter out-of-range skipped')


def test_backward_kernels():
    gen = torch.Generator().manual_seed(33)
    B, E, K, N = 2, 700, 16, 40
    index = torch.randint(0, N, (1, E, 1), generator=gen)
    grad_out = torch.randn(B, N, K, generator=gen)
    want = grad_out[:, index.view(-1)]
    got = cabi.scatter_backward(grad_out.cuda(), index.cuda(), E, (0, 1, 0))
    assert_close(got, want, exact=True, what='scatter_backward')
    count = torch.bincount(index.view(-1), minlength=N).int()
    want = grad_out[:, index.view(-1)] / count.clamp(min=1)[index.view(-1)].view(1, -1, 1)
    got = cabi.scatter_backward(grad_out.cuda(), index.cuda(), E, (0, 1, 0), count.cuda())
    assert_close(got, want, what='scatter_backward mean')
    arg = torch.randint(0, E + 1, (B, N, K), generator=gen)  # E marks "no element"
    want = torch.zeros(B, E + 1, K).scatter_(1, arg, grad_out)[:, :E]
    # several outputs may name the same element: use distinct args per (b,k) column for a defined result
    arg = torch.stack([torch.stack([torch.randperm(E + 1, generator=gen)[:N] for _ in range(K)], 1) for _ in range(B)])
    want = torch.zeros(B, E + 1, K).scatter_(1, arg, grad_out)[:, :E]
    got = cabi.arg_backward(grad_out.cuda(), arg.cuda(), E)
    assert_close(got, want, exact=True, what='arg_backward')


def test_scatter_sum_slice():
    """The sharded building block: each call fills (only) its slice of target rows of the partial."""
    import pytorch_scatter_b200  # noqa: F401  (registers the operator)
    gen = torch.Generator().manual_seed(55)
    E, K, N = 5000, 64, 300
    index = torch.randint(0, N, (E,), generator=gen)
    for dtype in (torch.float32, torch.bfloat16, torch.int64):
        src = rand_src(gen, (E, K), dtype)
        acc = torch.float32 if dtype == torch.bfloat16 else dtype
        partial = torch.full((N, K), 7, dtype=acc).cuda()
        for lo, hi in ((0, 100), (100, 257), (257, 300)):
            torch.ops.torch_scatter.scatter_sum_slice(src.cuda(), index.cuda(), partial, lo, hi)
        want = oracle.scatter(src.to(acc).view(1, E, K), index.view(1, E, 1), N, 'sum')[0][0]
        assert_close(partial, want, what=f'scatter_sum_slice {dtype}')
        # a slice call leaves the other rows alone
        before = partial.clone()
        torch.ops.torch_scatter.scatter_sum_slice(src.cuda(), index.cuda(), partial, 10, 20)
        assert torch.equal(partial[:10], before[:10]) and torch.equal(partial[20:], before[20:])


@pytest.mark.parametrize('sort', ['buckets', 'atomic'])
def test_scatter_group_and_permuted_row_slices(sort, chunk):
    """The two halves of the atomics-free scatter as operators: one grouping, then the rows reduced slice by slice
    (what the sharded scatter does between collectives); rows outside a call's slice stay untouched."""
    import pytorch_scatter_b200  # noqa: F401  (registers the operators)
    old = os.environ.get('TSB_SCATTER_GROUPED_SORT')
    os.environ['TSB_SCATTER_GROUPED_SORT'] = sort
    try:
        gen = torch.Generator().manual_seed(56)
        E, K, N = 20000, 16, 3000
        index = torch.randint(0, N, (E,), generator=gen)
        index[100:4100] = 777                      # a row spread over many chunks
        index[::53] = N + 1                        # names no row
        keep = (index >= 0) & (index < N)
        rowptr, perm = torch.ops.torch_scatter.scatter_group(index.cuda(), N)
        counts = torch.bincount(index[keep], minlength=N)
        assert torch.equal(rowptr.cpu(), torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]))
        got_rows = index[perm[:int(rowptr[-1])].cpu().long()]
        assert torch.equal(got_rows, torch.repeat_interleave(torch.arange(N), counts))   # grouped by row
        assert torch.equal(perm[:int(rowptr[-1])].cpu().long().sort().values, torch.nonzero(keep).view(-1))
        for dtype in (torch.float32, torch.bfloat16, torch.int64):
            src = rand_src(gen, (E, K), dtype)
            partial = torch.full((N, K), 7, dtype=dtype).cuda()
            for lo, hi in ((0, 700), (700, 778), (778, 2999)):
                torch.ops.torch_scatter.segment_sum_perm(src.cuda(), rowptr, perm, partial, lo, hi)
            assert torch.all(partial[2999:] == 7)                                       # not in any slice
            want = oracle.scatter(src[keep].view(1, -1, K), index[keep].view(1, -1, 1), N, 'sum')[0][0]
            if dtype.is_floating_point:
                want64 = oracle.scatter(src[keep].double().view(1, -1, K), index[keep].view(1, -1, 1), N, 'sum')[0][0]
                mass64 = oracle.scatter(src[keep].double().abs().view(1, -1, K), index[keep].view(1, -1, 1), N, 'sum')[0][0]
                assert_sum_close(partial[:2999], want64[:2999], mass64[:2999], what=f'segment_sum_perm {dtype}')
            else:
                assert_close(partial[:2999], want[:2999], what=f'segment_sum_perm {dtype}')
    finally:
        if old is None:
            os.environ.pop('TSB_SCATTER_GROUPED_SORT', None)
        else:
            os.environ['TSB_SCATTER_GROUPED_SORT'] = old


@pytest.fixture(params=[None, 'rows'], ids=['kernel-by-shape', 'row-parallel'])
def routed_kernel(request):
    old = os.environ.get('TSB_CSR_KERNEL')
    os.environ.pop('TSB_CSR_KERNEL', None)
    if request.param is not None:
        os.environ['TSB_CSR_KERNEL'] = request.param
    yield request.param
    os.environ.pop('TSB_CSR_KERNEL', None)
    if old is not None:
        os.environ['TSB_CSR_KERNEL'] = old


def test_routed_rows_two_ranks_emulated(routed_kernel):
    """The sharded scatter's fused exchange on one GPU: two "ranks" (two edge shards, run one after the other) store
    their finished rows into the owners' staging buffers; adding each owner's slabs must give the full scatter."""
    import pytorch_scatter_b200  # noqa: F401  (registers the operators)
    gen = torch.Generator().manual_seed(57)
    world, N, K = 2, 1001, 16
    rows = -(-N // world)
    for dtype, wide in ((torch.float32, True), (torch.bfloat16, False), (torch.bfloat16, True), (torch.float16, True),
                        (torch.int64, True)):
        # wide: 16-bit partial sums are staged in fp32 and rounded once by the owner
        stage_dtype = torch.float32 if wide and dtype in (torch.float16, torch.bfloat16) else dtype
        staging = [torch.full((world, rows, K), 9, dtype=stage_dtype).cuda() for _ in range(world)]   # owner q's buffer
        ptrs = [t.data_ptr() for t in staging]
        shards = []
        for rank in range(world):
            E = 7000 + 500 * rank
            index = torch.randint(0, N, (E,), generator=gen)
            index[:900] = 500 + rank                    # long rows on both sides of the ownership border
            src = rand_src(gen, (E, K), dtype)
            shards.append((src, index))
            rowptr, perm = torch.ops.torch_scatter.scatter_group(index.cuda(), N)
            torch.ops.torch_scatter.segment_sum_perm_routed(src.cuda(), rowptr, perm, ptrs, rank, rows, N, wide)
        got = torch.cat([torch.ops.torch_scatter.sum_slabs(buf, dtype) for buf in staging])[:N]
        assert got.dtype == dtype
        src_all = torch.cat([s for s, _ in shards])
        index_all = torch.cat([i for _, i in shards])
        if dtype.is_floating_point:
            want64 = oracle.scatter(src_all.double().view(1, -1, K), index_all.view(1, -1, 1), N, 'sum')[0][0]
            mass64 = oracle.scatter(src_all.double().abs().view(1, -1, K), index_all.view(1, -1, 1), N, 'sum')[0][0]
            assert_sum_close(got, want64, mass64, what=f'routed {dtype}')
            if wide and dtype != torch.float32:   # unrounded partials: as good as the single-GPU operator
                want = oracle.scatter(src_all.view(1, -1, K), index_all.view(1, -1, 1), N, 'sum')[0][0]
                assert_close(got, want, what=f'routed {dtype}, fp32 partials')
        else:
            want = oracle.scatter(src_all.view(1, -1, K), index_all.view(1, -1, 1), N, 'sum')[0][0]
            assert_close(got, want, what=f'routed {dtype}')
        assert torch.all(staging[1][:, N - rows:] == 9)   # the padding row past N is nobody's

