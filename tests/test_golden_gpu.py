"""GPU parity against the upstream project's own outputs (tests/golden/): every known-answer table of
its test-suite and ~1000 recorded seeded cases, run through the public Python API on cuda:0."""
import pytest
import torch

from helpers import assert_close, load_golden

pytestmark = pytest.mark.gpu

DTYPES = [torch.half, torch.bfloat16, torch.float, torch.double, torch.int, torch.long, torch.uint8, torch.int8, torch.int16]


def tens(x, dtype, device='cuda'):
    return torch.tensor(x, device=device).to(dtype)


@pytest.fixture(scope='module')
def ts():
    import pytorch_scatter_b200
    return pytorch_scatter_b200


@pytest.mark.parametrize('dtype', DTYPES)
def test_known_answers_scatter(ts, dtype):
    for case in load_golden('known_answers.pt')['scatter']:
        src, index, dim = tens(case['src'], dtype), tens(case['index'], torch.long), case['dim']
        for reduce in ['sum', 'add', 'mul', 'mean', 'min', 'max']:
            res = getattr(ts, 'scatter_' + reduce)(src, index, dim)
            if isinstance(res, tuple):
                assert torch.equal(res[1].cpu(), tens(case['arg_' + reduce], torch.long, 'cpu')), (case, reduce)
                res = res[0]
            assert torch.equal(res.cpu(), tens(case[reduce], dtype, 'cpu')), (case, reduce)


@pytest.mark.parametrize('dtype', DTYPES)
def test_known_answers_segment(ts, dtype):
    for case in load_golden('known_answers.pt')['segment']:
        src = tens(case['src'], dtype)
        index, indptr = tens(case['index'], torch.long), tens(case['indptr'], torch.long)
        for reduce in ['sum', 'add', 'mean', 'min', 'max']:
            want = tens(case[reduce], dtype, 'cpu')
            assert torch.equal(ts.segment_csr(src, indptr, reduce=reduce).cpu(), want), (case, reduce)
            assert torch.equal(ts.segment_coo(src, index, reduce=reduce).cpu(), want), (case, reduce)
        for name in ('min', 'max'):
            want_arg = tens(case['arg_' + name], torch.long, 'cpu')
            assert torch.equal(getattr(ts, f'segment_{name}_csr')(src, indptr)[1].cpu(), want_arg)
            assert torch.equal(getattr(ts, f'segment_{name}_coo')(src, index)[1].cpu(), want_arg)


@pytest.mark.parametrize('dtype', DTYPES)
def test_known_answers_gather(ts, dtype):
    for case in load_golden('known_answers.pt')['gather']:
        src = tens(case['src'], dtype)
        index, indptr = tens(case['index'], torch.long), tens(case['indptr'], torch.long)
        want = tens(case['expected'], dtype, 'cpu')
        assert torch.equal(ts.gather_csr(src, indptr).cpu(), want)
        assert torch.equal(ts.gather_coo(src, index).cpu(), want)


def _cuda(v):
    return v.cuda() if isinstance(v, torch.Tensor) else v


def _run(ts, case, with_grad=False):
    op, reduce = case['op'], case['reduce']
    a = {k: _cuda(v) for k, v in case['args'].items()}
    src = a['src']
    if with_grad:
        src = src.clone().requires_grad_()
    if op == 'segment_csr':
        fn = getattr(ts, f'segment_{reduce}_csr')
        res = fn(src, a['indptr'])
    elif op == 'segment_coo':
        res = getattr(ts, f'segment_{reduce}_coo')(src, a['index'], None, a['dim_size'])
    elif op == 'segment_coo_out':
        res = getattr(ts, f'segment_{reduce}_coo')(src, a['index'], a['out'].clone(), None)
    elif op == 'gather_csr':
        res = ts.gather_csr(src, a['indptr'])
    elif op == 'gather_coo':
        res = ts.gather_coo(src, a['index'])
    elif op == 'scatter':
        res = getattr(ts, 'scatter_' + reduce)(src, a['index'], a['dim'], None, a['dim_size'])
    elif op == 'scatter_out':
        res = getattr(ts, 'scatter_' + reduce)(src, a['index'], a['dim'], a['out'].clone(), None)
    elif op in ('scatter_softmax', 'scatter_log_softmax'):
        res = getattr(ts, op)(src, a['index'], a['dim'], dim_size=a['dim_size'])
    elif op in ('scatter_logsumexp', 'scatter_std'):
        res = getattr(ts, op)(src, a['index'], a['dim'], None, a['dim_size'])
    else:
        raise AssertionError(op)
    return res, src


def test_recorded_upstream_outputs(ts):
    cases = load_golden('random_cases.pt')
    for i, case in enumerate(cases):
        res, _ = _run(ts, case)
        out, arg = (res if isinstance(res, tuple) else (res, None))
        what = f"#{i} {case['op']} {case['reduce']} {case['out'].dtype} {tuple(case['args']['src'].shape)}"
        assert_close(out, case['out'], what=what)
        if 'arg' in case:
            assert torch.equal(arg.cpu(), case['arg']), what + ' arg'


def test_recorded_upstream_gradients(ts):
    n = 0
    for i, case in enumerate(load_golden('random_cases.pt')):
        if 'grad' not in case:
            continue
        res, src = _run(ts, case, with_grad=True)
        out = res[0] if isinstance(res, tuple) else res
        w = (torch.arange(out.numel(), dtype=out.dtype).reshape(out.shape) / max(out.numel(), 1) + 0.5).cuda()
        (out * w).sum().backward()
        what = f"#{i} grad {case['op']} {case['reduce']} {tuple(case['args']['src'].shape)}"
        assert_close(src.grad, case['grad'], what=what)
        n += 1
    assert n > 50
