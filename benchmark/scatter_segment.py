"""Timing table of the reduction operators, the command-line twin of the upstream project's
``benchmark/scatter_segment.py`` (same flags: ``--reduce``, ``--with_backward``, ``--device``; same rows: ATen's
``scatter_add_`` on a sorted / shuffled index, ``scatter`` on both, ``segment_coo``, ``segment_csr`` and the two dense
reductions; same cross-check of the three operators against each other before anything is timed).

Upstream times four SuiteSparse matrices that it downloads; here the row structures are synthetic (seeded) stand-ins for
its two regimes - short rows (about 8 entries per row) and long rows (about 14 and 49 per row) - and ``--matrix`` adds any
local ``.mat`` file in SuiteSparse format.  Times are seconds for ``iters`` calls, as upstream prints them.

    python benchmark/scatter_segment.py --reduce sum [--with_backward] [--sizes 1,16,64]
"""
import argparse
import os.path as osp
import sys
import time

import torch

sys.path.insert(0, osp.dirname(osp.dirname(osp.abspath(__file__))))

# (name, rows, mean row length, sigma of the log-normal row lengths; 0 = all rows alike)
SHORT_ROWS = [('synthetic/short-even (268k rows, ~8.6 per row)', 268_495, 8.6, 0.0),
              ('synthetic/short-skewed (282k rows, ~8.2 per row, log-normal)', 281_903, 8.2, 1.5)]
LONG_ROWS = [('synthetic/long-even (1.47M rows, ~14.3 per row)', 1_465_137, 14.3, 0.3),
             ('synthetic/long-heavy (952k rows, ~48.9 per row)', 952_203, 48.9, 0.5)]


def bold(text, flag=True):
    return f'\033[1m{text}\033[0m' if flag else text


def synthetic_rows(rows, mean, sigma, seed):
    """Row lengths: log-normal with the given mean (sigma 0: Poisson-like around the mean), never above 20,000."""
    g = torch.Generator().manual_seed(seed)
    if sigma > 0:
        mu = torch.log(torch.tensor(mean + 0.5, dtype=torch.float64)) - sigma * sigma / 2
        lens = torch.exp(mu + sigma * torch.randn(rows, generator=g, dtype=torch.float64)).floor()
    else:
        lens = torch.poisson(torch.full((rows,), mean, dtype=torch.float64), generator=g)
    return lens.clamp_(0, 20000).long()


def load_structure(spec, device):
    """(name, rowptr, row, shuffled row, rows) of a synthetic spec or of a SuiteSparse .mat file."""
    if isinstance(spec, str):
        from scipy.io import loadmat
        mat = loadmat(spec)['Problem'][0][0][2].tocsr()
        rowptr = torch.from_numpy(mat.indptr).to(device, torch.long)
        name = osp.basename(spec)
    else:
        name, rows, mean, sigma = spec
        lens = synthetic_rows(rows, mean, sigma, seed=len(name))
        rowptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).to(device)
    rows = rowptr.numel() - 1
    row = torch.repeat_interleave(torch.arange(rows, device=device), rowptr[1:] - rowptr[:-1])
    row2 = row[torch.randperm(row.numel(), device=device)]
    return name, rowptr, row, row2, rows


@torch.no_grad()
def correctness(ops, structure, sizes, device):
    """scatter, segment_coo and segment_csr must agree on every reduction (atol 1e-4, as upstream checks)."""
    _, rowptr, row, _, rows = structure
    for size in sizes:
        x = torch.randn((row.numel(), size), device=device)
        x = x.squeeze(-1) if size == 1 else x
        for reduce in ('add', 'mean', 'min', 'max'):
            out1 = ops.scatter(x, row, dim=0, dim_size=rows, reduce=reduce)
            out2 = ops.segment_coo(x, row, dim_size=rows, reduce=reduce)
            out3 = ops.segment_csr(x, rowptr, reduce=reduce)
            assert torch.allclose(out1, out2, atol=1e-4), (reduce, size)
            assert torch.allclose(out1, out3, atol=1e-4), (reduce, size)


def time_func(func, x, iters, with_backward):
    try:
        torch.cuda.synchronize()
        t = time.perf_counter()
        if not with_backward:
            with torch.no_grad():
                for _ in range(iters):
                    func(x)
        else:
            x = x.requires_grad_()
            for _ in range(iters):
                out = func(x)
                out = out[0] if isinstance(out, tuple) else out
                torch.autograd.grad(out, x, out, only_inputs=True)
        torch.cuda.synchronize()
        return time.perf_counter() - t
    except RuntimeError as e:
        if 'out of memory' not in str(e):
            raise
        torch.cuda.empty_cache()
        return float('inf')


def timing(ops, structure, sizes, args, iters):
    name, rowptr, row, row2, rows = structure
    avg_row_len = row.numel() / rows
    reduce = args.reduce

    def aten_on(index):
        def fn(x):
            out = x.new_zeros(rows, *x.size()[1:])
            return out.scatter_add_(0, index.view(-1, 1).expand_as(x) if x.dim() > 1 else index, x)
        return fn

    funcs = [('SCA1_ROW', aten_on(row)), ('SCA1_COL', aten_on(row2)),
             ('SCA2_ROW', lambda x: ops.scatter(x, row, dim=0, dim_size=rows, reduce=reduce)),
             ('SCA2_COL', lambda x: ops.scatter(x, row2, dim=0, dim_size=rows, reduce=reduce)),
             ('SEG_COO ', lambda x: ops.segment_coo(x, row, reduce=reduce)),
             ('SEG_CSR ', lambda x: ops.segment_csr(x, rowptr, reduce=reduce))]
    dense = [('DENSE1  ', lambda x: getattr(torch, reduce)(x, dim=-2), lambda s: (rows, int(avg_row_len + 1), s)),
             ('DENSE2  ', lambda x: getattr(torch, reduce)(x, dim=-1), lambda s: (rows, s, int(avg_row_len + 1)))]
    table = {label: [] for label, *_ in funcs + dense}
    for size in sizes:
        x = torch.randn((row.numel(), size), device=args.device)
        x = x.squeeze(-1) if size == 1 else x
        for label, fn in funcs:
            time_func(fn, x, 2, args.with_backward)   # warm-up: allocator, one-time kernel attributes
            table[label].append(time_func(fn, x, iters, args.with_backward))
        del x
        for label, fn, shape in dense:
            try:
                x = torch.randn(shape(size), device=args.device)
                table[label].append(time_func(fn, x, iters, args.with_backward))
                del x
            except RuntimeError as e:
                if 'out of memory' not in str(e):
                    raise
                torch.cuda.empty_cache()
                table[label].append(float('inf'))
    times = torch.tensor([table[label] for label in table])
    best = times.argmin(dim=0).tolist()
    print(f'{bold(name)} (avg row length: {avg_row_len:.2f}):')
    print('\t'.join(['        '] + [f'{size:>5}' for size in sizes]))
    for i, label in enumerate(table):
        print('\t'.join([bold(label)] + [bold(f'{t:.5f}', best[j] == i) for j, t in enumerate(table[label])]))
    print()
    return table


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument('--reduce', type=str, required=True, choices=['sum', 'mean', 'min', 'max'])
    parser.add_argument('--with_backward', action='store_true')
    parser.add_argument('--device', type=str, default='cuda')
    parser.add_argument('--sizes', type=str, default='1,16,32,64,128,256,512', help='feature sizes, comma separated')
    parser.add_argument('--matrix', action='append', default=[], help='a SuiteSparse .mat file to add (may repeat)')
    parser.add_argument('--iters', type=int, default=20)
    args = parser.parse_args()
    if not args.device.startswith('cuda'):
        parser.error('this build has no CPU path: --device must be a CUDA device')
    import pytorch_scatter_b200 as ops
    sizes = [int(s) for s in args.sizes.split(',')]
    for _ in range(10):  # warm-up
        torch.randn(100, 100, device=args.device).sum()
    for spec in SHORT_ROWS + LONG_ROWS + args.matrix:
        structure = load_structure(spec, args.device)
        correctness(ops, structure, [s for s in sizes if s <= 64], args.device)
        timing(ops, structure, sizes, args, args.iters)


if __name__ == '__main__':
    main()
