"""Generates the golden fixtures in this directory from the upstream project itself.

Runs only where a checkout of rusty1s/pytorch_scatter is available (``--ref``) and its CPU operator libraries have been built by ``make -C oracle ref`` into
``oracle/_ref/``.  It assembles the upstream Python package in a temporary directory (symlinks to the
checkout's ``torch_scatter/*.py`` plus the built ``_*_cpu.so``), imports it, and records

* ``known_answers.pt``  every known-answer table of the upstream tests (``test/test_scatter.py:11-90``,
  ``test/test_segment.py:9-82``, ``test/test_gather.py:9-46``), after checking that the upstream build
  reproduces its own tables;
* ``random_cases.pt``   seeded random cases for every operator x reduction x dtype with the outputs
  (and, for float64, the input gradients) the upstream CPU implementation gives.

The fixtures are small (inputs stored next to the outputs); tests never need the checkout.
This process must not import pytorch_scatter_b200: both register the ``torch_scatter::*`` operators.
"""
import argparse
import ast
import os
import os.path as osp
import sys
import tempfile

import torch

HERE = osp.dirname(osp.abspath(__file__))
ROOT = osp.dirname(osp.dirname(HERE))

DTYPES = [torch.half, torch.bfloat16, torch.float, torch.double, torch.int, torch.long]


def import_upstream(ref):
    tmp = tempfile.mkdtemp(prefix='upstream_pkg_')
    pkg = osp.join(tmp, 'torch_scatter')
    os.makedirs(osp.join(pkg, 'composite'))
    for sub in ('', 'composite'):
        d = osp.join(ref, 'torch_scatter', sub)
        for f in os.listdir(d):
            if f.endswith('.py'):
                os.symlink(osp.join(d, f), osp.join(pkg, sub, f))
    built = osp.join(ROOT, 'oracle', '_ref')
    for f in os.listdir(built):
        if f.endswith('.so'):
            os.symlink(osp.join(built, f), osp.join(pkg, f))
    sys.path.insert(0, tmp)
    import torch_scatter
    return torch_scatter


def table_of(path):
    """The literal assigned to ``tests`` in an upstream test module, without importing it."""
    tree = ast.parse(open(path).read())
    for node in tree.body:
        if isinstance(node, ast.Assign) and any(getattr(t, 'id', None) == 'tests' for t in node.targets):
            # the tables contain constant arithmetic such as `1 * 3`, which literal_eval rejects
            return eval(compile(ast.Expression(node.value), path, 'eval'), {'__builtins__': {}})
    raise RuntimeError(f'no tests table in {path}')


def tens(x, dtype):
    return torch.tensor(x).to(dtype)


def known_answers(ts, ref):
    out = {'scatter': [], 'segment': [], 'gather': []}
    # scatter: test/test_scatter.py:93-112
    for case in table_of(osp.join(ref, 'test', 'test_scatter.py')):
        for dtype in DTYPES:
            src, index, dim = tens(case['src'], dtype), tens(case['index'], torch.long), case['dim']
            for reduce in ['sum', 'add', 'mul', 'mean', 'min', 'max']:
                expected = tens(case[reduce], dtype)
                res = getattr(ts, 'scatter_' + reduce)(src, index, dim)
                if isinstance(res, tuple):
                    assert torch.all(res[1] == tens(case['arg_' + reduce], torch.long))
                    res = res[0]
                assert torch.all(res == expected), (case, reduce, dtype)
        out['scatter'].append(case)
    # segment_coo / segment_csr: test/test_segment.py:85-117
    for case in table_of(osp.join(ref, 'test', 'test_segment.py')):
        for dtype in DTYPES:
            src = tens(case['src'], dtype)
            index, indptr = tens(case['index'], torch.long), tens(case['indptr'], torch.long)
            for reduce in ['sum', 'add', 'mean', 'min', 'max']:
                expected = tens(case[reduce], dtype)
                for fn, key in ((ts.segment_csr, indptr), (ts.segment_coo, index)):
                    assert torch.all(fn(src, key, reduce=reduce) == expected), (case, reduce, dtype)
                for name in ('min', 'max'):
                    for r in (getattr(ts, f'segment_{name}_csr')(src, indptr), getattr(ts, f'segment_{name}_coo')(src, index)):
                        assert torch.all(r[1] == tens(case['arg_' + name], torch.long))
        out['segment'].append(case)
    # gather_coo / gather_csr: test/test_gather.py:49-60
    for case in table_of(osp.join(ref, 'test', 'test_gather.py')):
        for dtype in DTYPES:
            src = tens(case['src'], dtype)
            index, indptr = tens(case['index'], torch.long), tens(case['indptr'], torch.long)
            expected = tens(case['expected'], dtype)
            assert torch.all(ts.gather_csr(src, indptr) == expected)
            assert torch.all(ts.gather_coo(src, index) == expected)
        out['gather'].append(case)
    return out


# ---------------------------------------------------------------------------------------------
def rand_src(gen, shape, dtype):
    if dtype.is_floating_point:
        return torch.randn(shape, generator=gen, dtype=torch.float32).to(dtype)
    return torch.randint(-9, 10, shape, generator=gen).to(dtype)


def rand_rows(gen, n_rows, total, long_row=None):
    """Row lengths summing to `total` with empty rows; optionally one row takes `long_row` entries."""
    lens = torch.zeros(n_rows, dtype=torch.long)
    rest = total
    if long_row is not None:
        lens[int(torch.randint(0, n_rows, (1,), generator=gen))] = long_row
        rest -= long_row
    if rest > 0:
        picks = torch.randint(0, n_rows, (rest,), generator=gen)
        picks = picks[picks % 3 != 1] if n_rows > 3 else picks  # leave a third of the rows mostly empty
        lens += torch.bincount(picks, minlength=n_rows)
        lens[-1] += rest - picks.numel()
    return lens


def grads_of(fn, src, *args):
    """d(sum(out * w))/d(src) in float64 through the upstream autograd."""
    s = src.clone().requires_grad_()
    out = fn(s, *args)
    out = out[0] if isinstance(out, tuple) else out
    w = torch.arange(out.numel(), dtype=out.dtype).reshape(out.shape) / max(out.numel(), 1) + 0.5
    (out * w).sum().backward()
    return s.grad


def random_cases(ts):
    cases = []
    gen = torch.Generator().manual_seed(20240601)

    def add(op, reduce, kwargs, fn, *args, grad=False):
        res = fn(*args)
        rec = {'op': op, 'reduce': reduce, 'args': kwargs}
        if isinstance(res, tuple):
            rec['out'], rec['arg'] = res[0].clone(), res[1].clone()
        else:
            rec['out'] = res.clone()
        if grad:
            rec['grad'] = grads_of(fn, *args)
        cases.append(rec)

    # ---- segment_csr / segment_coo / gathers: (leading batch dims, rows, entries, trailing feature dims)
    seg_shapes = [((), 7, 50, ()), ((), 9, 64, (3,)), ((), 5, 40, (4,)), ((), 12, 96, (16,)), ((), 6, 70, (33,)),
                  ((), 4, 300, (2, 4)), ((2,), 6, 30, (5,)), ((2, 3), 4, 12, ()), ((), 3, 600, (8,))]
    for (lead, rows, total, feat) in seg_shapes:
        for dtype in DTYPES:
            long_row = 520 if total == 600 else None
            lens = rand_rows(gen, rows, total, long_row)
            indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
            index = torch.repeat_interleave(torch.arange(rows), lens)
            if len(lead) == 1:  # one row structure shared by the leading batch (broadcast)
                indptr, index = indptr.unsqueeze(0), index.unsqueeze(0)
            if len(lead) == 2:  # a different row structure per leading batch
                ips, ixs = [], []
                for _ in range(lead[0] * lead[1]):
                    ln = rand_rows(gen, rows, total)
                    ips.append(torch.cat([torch.zeros(1, dtype=torch.long), ln.cumsum(0)]))
                    ixs.append(torch.repeat_interleave(torch.arange(rows), ln))
                indptr = torch.stack(ips).reshape(*lead, rows + 1)
                index = torch.stack(ixs).reshape(*lead, total)
            src = rand_src(gen, (*lead, total, *feat), dtype)
            dim = len(lead)
            for reduce in ['sum', 'mean', 'min', 'max']:
                want_grad = dtype == torch.double
                if reduce in ('min', 'max'):
                    add('segment_csr', reduce, {'src': src, 'indptr': indptr},
                        getattr(ts, f'segment_{reduce}_csr'), src, indptr, grad=want_grad)
                    # upstream cannot differentiate segment_coo through a broadcast index
                    add('segment_coo', reduce, {'src': src, 'index': index, 'dim_size': rows},
                        getattr(ts, f'segment_{reduce}_coo'), src, index, None, rows,
                        grad=want_grad and (len(lead) != 1 or reduce in ('min', 'max')))
                else:
                    add('segment_csr', reduce, {'src': src, 'indptr': indptr},
                        getattr(ts, f'segment_{reduce}_csr'), src, indptr, grad=want_grad)
                    # upstream cannot differentiate segment_coo through a broadcast index
                    add('segment_coo', reduce, {'src': src, 'index': index, 'dim_size': rows},
                        getattr(ts, f'segment_{reduce}_coo'), src, index, None, rows,
                        grad=want_grad and (len(lead) != 1 or reduce in ('min', 'max')))
            # dim_size inferred from the index
            add('segment_coo', 'sum', {'src': src, 'index': index, 'dim_size': None},
                ts.segment_sum_coo, src, index, None, None)
            # gathers: the row table has `rows` entries along dim
            table = rand_src(gen, (*lead, rows, *feat), dtype)
            add('gather_csr', None, {'src': table, 'indptr': indptr}, ts.gather_csr, table, indptr,
                grad=dtype == torch.double)
            gidx = index.expand(*lead, index.size(-1)) if lead else index  # gather_coo does not broadcast
            add('gather_coo', None, {'src': table, 'index': gidx}, ts.gather_coo, table, gidx,
                grad=dtype == torch.double)
    # segment_coo accumulating into a given out (index starts at row 0)
    for dtype in (torch.float, torch.double, torch.long):
        lens = torch.tensor([3, 0, 5, 1, 0, 4])
        index = torch.repeat_interleave(torch.arange(6), lens)
        src = rand_src(gen, (13, 4), dtype)
        for reduce in ['sum', 'mean', 'min', 'max']:
            base = rand_src(gen, (6, 4), dtype)
            fn = getattr(ts, f'segment_{reduce}_coo')
            res = fn(src, index, base.clone(), None)
            res = res[0] if isinstance(res, tuple) else res
            cases.append({'op': 'segment_coo_out', 'reduce': reduce,
                          'args': {'src': src, 'index': index, 'out': base}, 'out': res.clone()})

    # ---- scatter: (src shape, dim, index kind)
    sc_shapes = [((40,), 0, 'full', 7), ((30, 3), 0, '1d', 6), ((30, 4), 0, 'full', 5), ((64, 16), 0, '1d', 9),
                 ((20, 33), 0, '1d', 4), ((3, 25, 4), 1, '1d', 6), ((3, 25, 4), 1, 'full', 6), ((5, 12), 1, 'full', 4),
                 ((2, 3, 10, 2), 2, 'lead', 5), ((50, 8), 0, 'same', 3)]
    for (shape, dim, kind, n) in sc_shapes:
        for dtype in DTYPES:
            src = rand_src(gen, shape, dtype)
            if kind == '1d':
                index = torch.randint(0, n, (shape[dim],), generator=gen)
            elif kind == 'full':
                index = torch.randint(0, n, shape, generator=gen)
            elif kind == 'lead':  # varies over a leading and the reduced dim only
                index = torch.randint(0, n, (shape[0], 1, shape[2], 1), generator=gen)
            else:
                index = torch.full((shape[dim],), n - 1, dtype=torch.long)
            for reduce in ['sum', 'mean', 'min', 'max', 'mul']:
                if reduce == 'mul' and dtype in (torch.half, torch.bfloat16):
                    continue
                s = src
                if reduce == 'mul':  # keep products small
                    s = (src.double().clamp(-2, 2)).to(dtype)
                fn = getattr(ts, 'scatter_' + reduce)
                add('scatter', reduce, {'src': s, 'index': index, 'dim': dim, 'dim_size': n},
                    fn, s, index, dim, None, n, grad=(dtype == torch.double and reduce != 'mul'))
            add('scatter', 'sum', {'src': src, 'index': index, 'dim': dim, 'dim_size': None},
                ts.scatter_sum, src, index, dim, None, None)
    # scatter accumulating into a given out
    for dtype in (torch.float, torch.long):
        src = rand_src(gen, (30, 4), dtype)
        index = torch.randint(0, 6, (30,), generator=gen)
        for reduce in ['sum', 'mean', 'min', 'max']:
            base = rand_src(gen, (6, 4), dtype)
            res = getattr(ts, 'scatter_' + reduce)(src, index, 0, base.clone(), None)
            res = res[0] if isinstance(res, tuple) else res
            cases.append({'op': 'scatter_out', 'reduce': reduce,
                          'args': {'src': src, 'index': index, 'dim': 0, 'out': base}, 'out': res.clone()})

    # ---- composites (float only)
    for dtype in (torch.float, torch.double):
        for (shape, dim, n) in [((40,), 0, 6), ((30, 5), 0, 7), ((4, 20), 1, 5)]:
            src = rand_src(gen, shape, dtype)
            index = torch.randint(0, n, (shape[dim],), generator=gen)
            for name in ('scatter_softmax', 'scatter_log_softmax', 'scatter_logsumexp', 'scatter_std'):
                fn = getattr(ts, name)
                if name in ('scatter_softmax', 'scatter_log_softmax'):
                    res = fn(src, index, dim, dim_size=n)
                else:
                    res = fn(src, index, dim, None, n)
                cases.append({'op': name, 'reduce': None,
                              'args': {'src': src, 'index': index, 'dim': dim, 'dim_size': n}, 'out': res.clone()})

    # ---- composites over an ASCENDING 1-D index (an edge list sorted by destination; the last groups empty), with
    # the input gradients: a sorted index is what a fused implementation may special-case, so it is pinned separately.
    # A generator of its own keeps every case above unchanged.
    gen2 = torch.Generator().manual_seed(20240611)
    for dtype in (torch.float, torch.half, torch.bfloat16):
        for (shape, dim, n) in [((300,), 0, 23), ((257, 8), 0, 40), ((3, 190, 16), 1, 31), ((2, 64), -1, 9)]:
            src = rand_src(gen2, shape, dtype)
            index = torch.randint(0, n - 2, (shape[dim],), generator=gen2).sort()[0]
            for name in ('scatter_softmax', 'scatter_log_softmax', 'scatter_logsumexp', 'scatter_std'):
                fn = getattr(ts, name)
                if name in ('scatter_softmax', 'scatter_log_softmax'):
                    call = lambda s: fn(s, index, dim, dim_size=n)  # noqa: E731
                else:
                    call = lambda s: fn(s, index, dim, None, n)  # noqa: E731
                rec = {'op': name, 'reduce': None, 'sorted_index': True,
                       'args': {'src': src, 'index': index, 'dim': dim, 'dim_size': n}, 'out': call(src).clone()}
                if dtype == torch.float:
                    rec['grad'] = grads_of(call, src)
                cases.append(rec)

    # ---- the narrow integer types upstream dispatches too (uint8 / int8 / int16), small values and short rows so that
    # no sum or count leaves the type.  A generator of its own keeps every case above unchanged.
    gen3 = torch.Generator().manual_seed(20240621)
    for dtype in (torch.uint8, torch.int8, torch.int16):
        # uint8 never 0: it is MAX's identity there, and upstream's arg for a row whose maximum equals the identity is
        # whatever its loop last held
        lo, hi = (1, 5) if dtype == torch.uint8 else (-3, 4)
        for (rows, total, feat) in [(7, 40, ()), (6, 50, (5,)), (9, 64, (16,))]:
            lens = rand_rows(gen3, rows, total)
            indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
            index = torch.repeat_interleave(torch.arange(rows), lens)
            src = torch.randint(lo, hi, (total,) + feat, generator=gen3).to(dtype)
            for reduce in ['sum', 'mean', 'min', 'max']:
                add('segment_csr', reduce, {'src': src, 'indptr': indptr}, getattr(ts, f'segment_{reduce}_csr'), src, indptr)
                add('segment_coo', reduce, {'src': src, 'index': index, 'dim_size': rows},
                    getattr(ts, f'segment_{reduce}_coo'), src, index, None, rows)
            table = torch.randint(lo, hi, (rows,) + feat, generator=gen3).to(dtype)
            add('gather_csr', None, {'src': table, 'indptr': indptr}, ts.gather_csr, table, indptr)
            add('gather_coo', None, {'src': table, 'index': index}, ts.gather_coo, table, index)
            shuffled = index[torch.randperm(total, generator=gen3)]
            for reduce in ['sum', 'mul', 'mean', 'min', 'max']:
                s = src if reduce != 'mul' else src.clamp(-1, 1)
                add('scatter', reduce, {'src': s, 'index': shuffled, 'dim': 0, 'dim_size': rows},
                    getattr(ts, 'scatter_' + reduce), s, shuffled, 0, None, rows)
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--ref', required=True, help='checkout of the upstream project (rusty1s/pytorch_scatter)')
    a = ap.parse_args()
    ts = import_upstream(a.ref)
    ka = known_answers(ts, a.ref)
    torch.save(ka, osp.join(HERE, 'known_answers.pt'))
    rc = random_cases(ts)
    torch.save(rc, osp.join(HERE, 'random_cases.pt'))
    print(f"known-answer tables: {sum(len(v) for v in ka.values())}; random cases: {len(rc)}")
    for f in ('known_answers.pt', 'random_cases.pt'):
        print(f, osp.getsize(osp.join(HERE, f)), 'bytes')


if __name__ == '__main__':
    main()
