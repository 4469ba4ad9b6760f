"""The C++ API (include/torchscatter/scatter.h): a small program written against the header is compiled with g++,
linked to the in-tree operator library the way an installed TorchScatter package would be linked, and run on cuda:0.
The compile-and-link half needs no GPU."""
import os
import os.path as osp
import subprocess
import sys

import pytest
import torch

ROOT = osp.dirname(osp.dirname(osp.abspath(__file__)))
PKG = osp.join(ROOT, 'pytorch_scatter_b200')
BIN = osp.join(ROOT, 'tests', 'cpp', 'api_smoke')


def _build():
    from torch.utils.cpp_extension import include_paths
    src = osp.join(ROOT, 'tests', 'cpp', 'api_smoke.cpp')
    libs = [osp.join(PKG, '_C.so'), osp.join(PKG, 'libtsb200.so'), osp.join(ROOT, 'include', 'torchscatter', 'scatter.h'), src]
    if osp.exists(BIN) and all(osp.getmtime(BIN) >= osp.getmtime(f) for f in libs):
        return BIN
    torch_lib = osp.join(osp.dirname(torch.__file__), 'lib')
    cmd = ['g++', '-O1', '-std=c++17', f'-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}',
           f'-I{osp.join(ROOT, "include")}'] + [f'-I{p}' for p in include_paths()] + [src, '-o', BIN,
           f'-L{PKG}', '-l:_C.so', '-ltsb200', f'-L{torch_lib}', '-ltorch', '-ltorch_cpu', '-ltorch_cuda', '-lc10', '-lc10_cuda',
           f'-Wl,-rpath,{PKG}', f'-Wl,-rpath,{torch_lib}', '-Wl,--no-as-needed']
    subprocess.run(cmd, check=True)
    return BIN


def test_cpp_api_program_compiles_and_links():
    exe = _build()
    # every function the header declares resolves against the library (no GPU needed to check that)
    syms = subprocess.run(['nm', '-D', '--defined-only', '-C', osp.join(PKG, '_C.so')], stdout=subprocess.PIPE, text=True).stdout
    for name in ('scatter_sum', 'scatter_mul', 'scatter_mean', 'scatter_min', 'scatter_max', 'segment_sum_coo',
                 'segment_mean_coo', 'segment_min_coo', 'segment_max_coo', 'gather_coo', 'segment_sum_csr',
                 'segment_mean_csr', 'segment_min_csr', 'segment_max_csr', 'gather_csr', 'scatter::cuda_version'):
        assert any(ln.split(' ', 2)[-1].startswith(name + '(') for ln in syms.splitlines()), name
    assert osp.exists(exe)


@pytest.mark.gpu
def test_cpp_api_program_runs():
    exe = _build()
    res = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert res.returncode == 0 and 'cpp api ok' in res.stdout, res.stdout
