"""Timing table of the gather operators, the command-line twin of the upstream project's ``benchmark/gather.py``
(same flags: ``--with_backward``, ``--device``; rows: ATen's ``index_select`` and ``gather``, ``gather_coo``,
``gather_csr``; same cross-check against ``index_select`` first), over the synthetic row structures of
``benchmark/scatter_segment.py``.  Times are seconds for ``iters`` calls.

    python benchmark/gather.py [--with_backward] [--sizes 1,16,64]
"""
import argparse
import os.path as osp
import sys

import torch

sys.path.insert(0, osp.dirname(osp.abspath(__file__)))
from scatter_segment import LONG_ROWS, SHORT_ROWS, bold, load_structure, time_func  # noqa: E402


@torch.no_grad()
def correctness(ops, structure, sizes, device):
    _, rowptr, row, _, rows = structure
    for size in sizes:
        x = torch.randn((rows, size), device=device)
        x = x.squeeze(-1) if size == 1 else x
        want = x.index_select(0, row)
        assert torch.allclose(want, ops.gather_coo(x, row), atol=1e-4), size
        assert torch.allclose(want, ops.gather_csr(x, rowptr), atol=1e-4), size


def timing(ops, structure, sizes, args):
    name, rowptr, row, _, rows = structure
    funcs = [('SELECT    ', lambda x: x.index_select(0, row)),
             ('GATHER    ', lambda x: x.gather(0, row.view(-1, 1).expand(-1, x.size(1)) if x.dim() > 1 else row)),
             ('GATHER_COO', lambda x: ops.gather_coo(x, row)),
             ('GATHER_CSR', lambda x: ops.gather_csr(x, rowptr))]
    table = {label: [] for label, _ in funcs}
    for size in sizes:
        x = torch.randn((rows, size), device=args.device)
        x = x.squeeze(-1) if size == 1 else x
        for label, fn in funcs:
            time_func(fn, x, 2, args.with_backward)
            table[label].append(time_func(fn, x, args.iters, args.with_backward))
        del x
    times = torch.tensor([table[label] for label in table])
    best = times.argmin(dim=0).tolist()
    print(f'{bold(name)} (avg row length: {row.numel() / rows:.2f}):')
    print('\t'.join(['          '] + [f'{size:>5}' for size in sizes]))
    for i, label in enumerate(table):
        print('\t'.join([bold(label)] + [bold(f'{t:.5f}', best[j] == i) for j, t in enumerate(table[label])]))
    print()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument('--with_backward', action='store_true')
    parser.add_argument('--device', type=str, default='cuda')
    parser.add_argument('--sizes', type=str, default='1,16,32,64,128,256,512')
    parser.add_argument('--matrix', action='append', default=[])
    parser.add_argument('--iters', type=int, default=20)
    args = parser.parse_args()
    if not args.device.startswith('cuda'):
        parser.error('this build has no CPU path: --device must be a CUDA device')
    import pytorch_scatter_b200 as ops
    sizes = [int(s) for s in args.sizes.split(',')]
    for _ in range(10):
        torch.randn(100, 100, device=args.device).sum()
    for spec in SHORT_ROWS + LONG_ROWS + args.matrix:
        structure = load_structure(spec, args.device)
        correctness(ops, structure, [s for s in sizes if s <= 64], args.device)
        timing(ops, structure, sizes, args)


if __name__ == '__main__':
    main()
