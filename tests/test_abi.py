"""The C ABI library loads without a GPU and exports every symbol include/tsb200.h declares; argument
errors are reported as status codes before anything is launched."""
import ctypes
import os.path as osp
import re

import pytest

ROOT = osp.dirname(osp.dirname(osp.abspath(__file__)))
HEADER = osp.join(ROOT, 'include', 'tsb200.h')
LIB = osp.join(ROOT, 'pytorch_scatter_b200', 'libtsb200.so')


def declared_functions():
    text = re.sub(r'/\*.*?\*/', '', open(HEADER).read(), flags=re.S)
    return sorted(set(re.findall(r'\b(tsb_[a-z0-9_]+)\s*\(', text)))


@pytest.fixture(scope='module')
def lib():
    return ctypes.CDLL(LIB)


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ('tsb_segment_csr', 'tsb_gather_csr', 'tsb_segment_coo', 'tsb_gather_coo', 'tsb_scatter',
                 'tsb_scatter_backward', 'tsb_arg_backward', 'tsb_cuda_version', 'tsb_status_string'):
        assert must in names


def test_every_declared_symbol_is_exported(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f'{name} is declared in tsb200.h but not exported by libtsb200.so'


def test_version_and_status_strings(lib):
    lib.tsb_cuda_version.restype = ctypes.c_int64
    assert lib.tsb_cuda_version() >= 12000
    lib.tsb_status_string.restype = ctypes.c_char_p
    texts = {lib.tsb_status_string(i) for i in range(7)}
    assert len(texts) == 7 and lib.tsb_status_string(0) == b'ok'


def test_argument_errors_are_status_codes(lib):
    I = ctypes.c_int64
    dummy = ctypes.c_void_p(256)  # never dereferenced: the checks below fail before any launch
    # negative size
    assert lib.tsb_segment_csr(dummy, dummy, dummy, None, I(-1), I(4), I(4), I(4), I(0), 0, 0, dummy,
                               ctypes.c_size_t(1 << 20), None) == 3
    # MIN without arg_out
    assert lib.tsb_segment_csr(dummy, dummy, dummy, None, I(1), I(4), I(4), I(4), I(0), 0, 2, dummy,
                               ctypes.c_size_t(1 << 20), None) == 3
    # unknown dtype / reduce
    assert lib.tsb_segment_csr(dummy, dummy, dummy, None, I(1), I(4), I(4), I(4), I(0), 99, 0, dummy,
                               ctypes.c_size_t(1 << 20), None) == 1
    assert lib.tsb_segment_csr(dummy, dummy, dummy, None, I(1), I(4), I(4), I(4), I(0), 0, 4, dummy,
                               ctypes.c_size_t(1 << 20), None) == 2
    # workspace too small / missing
    assert lib.tsb_segment_csr(dummy, dummy, dummy, None, I(1), I(4), I(4), I(4), I(0), 0, 0, None,
                               ctypes.c_size_t(0), None) == 4
    assert lib.tsb_segment_coo(dummy, dummy, dummy, None, None, I(1), I(4), I(4), I(4), I(0), 0, 0, 0, None,
                               ctypes.c_size_t(0), None) == 4
    assert lib.tsb_scatter(dummy, dummy, dummy, None, None, I(1), I(4), I(4), I(4), I(0), I(1), I(0), 2, 0, 0, None,
                           ctypes.c_size_t(0), None) == 4  # fp16 needs its fp32 workspace
    # empty problems succeed without touching the device
    assert lib.tsb_segment_csr(None, None, None, None, I(0), I(0), I(4), I(0), I(0), 0, 0, None,
                               ctypes.c_size_t(0), None) == 0
    assert lib.tsb_gather_coo(None, None, None, None, I(1), I(0), I(4), I(4), I(0), 0, None) == 0


def test_workspace_queries(lib):
    I = ctypes.c_int64
    for name in ('tsb_segment_csr_workspace_bytes', 'tsb_segment_coo_workspace_bytes', 'tsb_scatter_workspace_bytes'):
        getattr(lib, name).restype = ctypes.c_size_t
    # fp32 K=64: 512-entry chunks, two partial rows of 64 floats + one row id per chunk
    n = lib.tsb_segment_csr_workspace_bytes(I(1), I(512 * 100), I(64), I(1000), 0, 0)
    assert n >= 100 * (2 * 64 * 4 + 8) and n % 256 == 0
    n_arg = lib.tsb_segment_csr_workspace_bytes(I(1), I(512 * 100), I(64), I(1000), 0, 3)
    assert n_arg >= n + 100 * 2 * 64 * 8
    assert lib.tsb_segment_coo_workspace_bytes(I(1), I(512 * 100), I(64), I(1000), 0, 0) >= n + 1001 * 8
    # a flag header, then (small output) 16 copies of the fp32 accumulators
    assert lib.tsb_scatter_workspace_bytes(I(2), I(100), I(8), I(10), 0, 0) == 256 + 16 * 2 * 10 * 8 * 4
    assert lib.tsb_scatter_workspace_bytes(I(2), I(100), I(8), I(10), 3, 0) == 256 + 16 * 2 * 10 * 8 * 4
    # a large output: no copies; 16-bit dtypes still get their fp32 accumulators
    assert lib.tsb_scatter_workspace_bytes(I(1), I(1000), I(64), I(1 << 19), 0, 0) == 256
    assert lib.tsb_scatter_workspace_bytes(I(1), I(1000), I(64), I(1 << 19), 3, 0) == 256 + (1 << 19) * 64 * 4
