"""Host-side logic of bench.py that needs no GPU: the figures it reads from profiles/, the shards of the global
problem, the Zipf and row-length recipes and the command line."""
import importlib.util
import os.path as osp
import subprocess
import sys

import pytest
import torch

ROOT = osp.dirname(osp.dirname(osp.abspath(__file__)))


@pytest.fixture(scope='module')
def bench():
    spec = importlib.util.spec_from_file_location('bench_under_test', osp.join(ROOT, 'bench.py'))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_profiled_traffic_figures_are_found(bench):
    """`roofline.traffic` comes from named lines of the committed launch-list summary; both names bench.py asks for
    must be there, with the entry count of the full workload."""
    for name in ('csr_kernel_contiguous', 'scatter_all_kernels'):
        nbytes, entries = bench.profiled_dram_bytes(name)
        assert nbytes is not None and entries == 16898963, name
        assert 4.5e9 < nbytes < 6e9, (name, nbytes)
    assert bench.profiled_dram_bytes('no_such_kernel') == (None, None)


def test_row_lengths_recipe(bench):
    lens = bench.row_lengths(bench.ROWS, bench.SEED, force_long=8)
    assert lens.numel() == bench.ROWS and int(lens.max()) == 20000 and int(lens.min()) == 0
    assert int((lens == 20000).sum()) >= 8
    assert 15.0 < float(lens.double().mean()) < 17.5
    assert 0.10 < float((lens == 0).double().mean()) < 0.16          # "some empty rows"
    assert int(lens.sum()) == 16898963                                # the entry count every figure is quoted on


def test_algorithmic_bytes(bench):
    b_csr, b_sc = bench.algorithmic_bytes(bench.ROWS, 16898963)
    assert b_csr == 16898963 * 64 * 4 + (bench.ROWS + 1) * 8 + bench.ROWS * 64 * 4 == 4602958600
    assert b_sc == 16898963 * (64 * 4 + 8) + bench.ROWS * 64 * 4 == 4729761688


def test_shards_of_one_global_problem(bench):
    """At N ranks the problem has N x 1,048,576 rows from one seed, cut into contiguous ranges of (nearly) equal entry
    counts; every row belongs to exactly one rank."""
    from pytorch_scatter_b200.dist import balanced_row_cuts
    world = 4
    lens = bench.row_lengths(world * bench.ROWS, bench.SEED, force_long=8 * world)
    indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
    cuts = balanced_row_cuts(indptr, world)
    assert int(cuts[0]) == 0 and int(cuts[-1]) == world * bench.ROWS
    assert torch.all(cuts[1:] > cuts[:-1])
    nnz = [int(indptr[cuts[r + 1]] - indptr[cuts[r]]) for r in range(world)]
    assert max(nnz) / (sum(nnz) / world) < 1.001


def test_command_line_defaults():
    out = subprocess.run([sys.executable, osp.join(ROOT, 'bench.py'), '--help'], stdout=subprocess.PIPE, text=True, timeout=300)
    assert out.returncode == 0
    for flag in ('--gpus', '--steps', '--warmup', '--impl', '--suite', '--comparator', '--graph', '--exchange'):
        assert flag in out.stdout, flag
