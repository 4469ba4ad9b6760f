"""In-tree build of the two native libraries.

``libtsb200.so``  the CUDA kernel library with the plain C ABI declared in ``include/tsb200.h``
                  (nvcc, sm_100a only, no torch dependency).
``_C.so``         the host side: the ``torch_scatter::*`` operator registry and autograd functions
                  (g++ against libtorch), linked to ``libtsb200.so``.

Both land next to this file so that they travel with the source tree.  Run
``python pytorch_scatter_b200/_build.py`` (add ``--force`` to rebuild everything).
"""
from __future__ import annotations

import os
import os.path as osp
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = osp.dirname(osp.abspath(__file__))
ROOT_DIR = osp.dirname(PKG_DIR)
KERNEL_DIR = osp.join(PKG_DIR, 'csrc', 'kernels')
OPS_DIR = osp.join(PKG_DIR, 'csrc', 'ops')
OBJ_DIR = osp.join(PKG_DIR, 'csrc', 'build')
INCLUDE_DIR = osp.join(ROOT_DIR, 'include')
KERNEL_LIB = osp.join(PKG_DIR, 'libtsb200.so')
OPS_LIB = osp.join(PKG_DIR, '_C.so')

CUDA_HOME = os.environ.get('CUDA_HOME', '/usr/local/cuda')
NVCC = osp.join(CUDA_HOME, 'bin', 'nvcc')
NVCC_FLAGS = [
    '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
    '--expt-relaxed-constexpr', '-Xcompiler', '-fPIC', '-Xptxas', '-v',
]


def _sources(directory, ext):
    return sorted(osp.join(directory, f) for f in os.listdir(directory) if f.endswith(ext))


def _headers():
    hdrs = _sources(KERNEL_DIR, '.cuh') + _sources(OPS_DIR, '.h') + _sources(INCLUDE_DIR, '.h')
    return hdrs


def _stale(target, deps):
    if not osp.exists(target):
        return True
    t = osp.getmtime(target)
    return any(osp.getmtime(d) > t for d in deps)


def _run(cmd, log):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    with open(log, 'w') as f:
        f.write(' '.join(cmd) + '\n' + proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{proc.stdout}")
    return proc.stdout


def build_kernels(force=False, verbose=False):
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdrs = _headers()
    jobs, objs = [], []
    for src in _sources(KERNEL_DIR, '.cu'):
        obj = osp.join(OBJ_DIR, osp.basename(src)[:-3] + '.o')
        objs.append(obj)
        if force or _stale(obj, [src] + hdrs):
            jobs.append([NVCC] + NVCC_FLAGS + ['-c', src, '-o', obj])
    with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as pool:
        for out in pool.map(lambda c: _run(c, osp.join(OBJ_DIR, osp.basename(c[-1]) + '.log')), jobs):
            if verbose:
                print(out)
    if force or jobs or _stale(KERNEL_LIB, objs):
        _run([NVCC, '-shared', '-o', KERNEL_LIB] + objs + ['-cudart', 'static'], osp.join(OBJ_DIR, 'libtsb200.so.log'))
    return KERNEL_LIB


def build_ops(force=False, verbose=False):
    import torch
    from torch.utils.cpp_extension import include_paths
    os.makedirs(OBJ_DIR, exist_ok=True)
    torch_lib = osp.join(osp.dirname(torch.__file__), 'lib')
    cxx = os.environ.get('CXX', 'g++')
    flags = ['-O2', '-std=c++17', '-fPIC', '-Wno-sign-compare',
             f'-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}']
    incs = [f'-I{p}' for p in include_paths()] + [f'-I{osp.join(CUDA_HOME, "include")}']
    hdrs = _headers()
    jobs, objs = [], []
    for src in _sources(OPS_DIR, '.cpp'):
        obj = osp.join(OBJ_DIR, osp.basename(src)[:-4] + '.o')
        objs.append(obj)
        if force or _stale(obj, [src] + hdrs):
            jobs.append([cxx] + flags + incs + ['-c', src, '-o', obj])
    with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as pool:
        for out in pool.map(lambda c: _run(c, osp.join(OBJ_DIR, osp.basename(c[-1]) + '.log')), jobs):
            if verbose:
                print(out)
    if force or jobs or _stale(OPS_LIB, objs + [KERNEL_LIB]):
        _run([cxx, '-shared', '-o', OPS_LIB] + objs +
             [f'-L{PKG_DIR}', '-ltsb200', f'-L{torch_lib}', '-lc10', '-lc10_cuda', '-ltorch_cpu',
              '-ltorch_cuda', '-ltorch', '-Wl,-rpath,$ORIGIN', f'-Wl,-rpath,{torch_lib}'],
             osp.join(OBJ_DIR, '_C.so.log'))
    return OPS_LIB


def build(force=False, verbose=False):
    """Compile whatever is out of date; returns the two library paths."""
    return build_kernels(force, verbose), build_ops(force, verbose)


if __name__ == '__main__':
    paths = build(force='--force' in sys.argv, verbose='-v' in sys.argv)
    print('\n'.join(paths))
