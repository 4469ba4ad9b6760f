"""Pins the C oracle (oracle/scatter_oracle.c) to the upstream project: every known-answer table of
its test-suite and every recorded output of its CPU libraries must be reproduced."""
import pytest
import torch

from helpers import (assert_close, load_golden, oracle_gather_coo, oracle_gather_csr, oracle_scatter,
                     oracle_segment_coo, oracle_segment_csr)

DTYPES = [torch.half, torch.bfloat16, torch.float, torch.double, torch.int, torch.long, torch.uint8, torch.int8, torch.int16]


def tens(x, dtype):
    return torch.tensor(x).to(dtype)


@pytest.mark.parametrize('dtype', DTYPES)
def test_known_answers_scatter(dtype):
    for case in load_golden('known_answers.pt')['scatter']:
        src, index, dim = tens(case['src'], dtype), tens(case['index'], torch.long), case['dim']
        for reduce in ['sum', 'add', 'mul', 'mean', 'min', 'max']:
            out, arg = oracle_scatter(src, index, dim, None, reduce)
            assert torch.equal(out, tens(case[reduce], dtype)), (case, reduce)
            if reduce in ('min', 'max'):
                assert torch.equal(arg, tens(case['arg_' + reduce], torch.long)), (case, reduce)


@pytest.mark.parametrize('dtype', DTYPES)
def test_known_answers_segment(dtype):
    for case in load_golden('known_answers.pt')['segment']:
        src = tens(case['src'], dtype)
        index, indptr = tens(case['index'], torch.long), tens(case['indptr'], torch.long)
        for reduce in ['sum', 'add', 'mean', 'min', 'max']:
            want = tens(case[reduce], dtype)
            out, arg = oracle_segment_csr(src, indptr, reduce)
            assert torch.equal(out, want), (case, reduce)
            out2, arg2 = oracle_segment_coo(src, index, None, reduce)
            assert torch.equal(out2, want), (case, reduce)
            if reduce in ('min', 'max'):
                want_arg = tens(case['arg_' + reduce], torch.long)
                assert torch.equal(arg, want_arg) and torch.equal(arg2, want_arg), (case, reduce)


@pytest.mark.parametrize('dtype', DTYPES)
def test_known_answers_gather(dtype):
    for case in load_golden('known_answers.pt')['gather']:
        src = tens(case['src'], dtype)
        index, indptr = tens(case['index'], torch.long), tens(case['indptr'], torch.long)
        want = tens(case['expected'], dtype)
        assert torch.equal(oracle_gather_csr(src, indptr), want)
        assert torch.equal(oracle_gather_coo(src, index), want)


def _run_oracle(case):
    op, reduce, a = case['op'], case['reduce'], case['args']
    if op == 'segment_csr':
        return oracle_segment_csr(a['src'], a['indptr'], reduce)
    if op == 'segment_coo':
        return oracle_segment_coo(a['src'], a['index'], a['dim_size'], reduce)
    if op == 'segment_coo_out':
        return oracle_segment_coo(a['src'], a['index'], None, reduce, a['out'])
    if op == 'gather_csr':
        return oracle_gather_csr(a['src'], a['indptr']), None
    if op == 'gather_coo':
        return oracle_gather_coo(a['src'], a['index']), None
    if op == 'scatter':
        return oracle_scatter(a['src'], a['index'], a['dim'], a['dim_size'], reduce)
    if op == 'scatter_out':
        return oracle_scatter(a['src'], a['index'], a['dim'], None, reduce, a['out'])
    return None


def test_recorded_upstream_outputs():
    """Every recorded upstream output: integers and arg indices exact, floats within tolerance
    (the oracle keeps 16-bit accumulators in fp32 where upstream's scatter rounds every step)."""
    n = 0
    for case in load_golden('random_cases.pt'):
        res = _run_oracle(case)
        if res is None:
            continue
        out, extra = res
        what = f"{case['op']} {case['reduce']} {case['out'].dtype} {tuple(case['args']['src'].shape)}"
        assert_close(out, case['out'], what=what)
        if 'arg' in case:
            assert torch.equal(extra, case['arg']), what
        n += 1
    assert n > 500
