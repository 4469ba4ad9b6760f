"""Two-GPU checks of the edge-sharded scatter (skipped on a single-GPU box): the exchange fused into the reduction
kernel (peer stores into the owners' staging buffers), the NCCL per-slice variant, and the plain one-collective
variant for sum / mean / min / max with global arg indices, all against the single-GPU operator on the concatenated
shards."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, dtype_name, results):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    try:
        import pytorch_scatter_b200 as ts
        from pytorch_scatter_b200.dist import (owned_rows, overlapped_layout, routed_exchange_available,
                                                scatter_sum_overlapped, scatter_sum_routed)
        dtype = getattr(torch, dtype_name)
        N, K = 50001, 32
        shards = []
        for r in range(world):   # every rank builds all shards (seeded) to know the expected result
            gen = torch.Generator().manual_seed(900 + r)
            E = 200000 + 1000 * r
            index = torch.randint(0, N, (E,), generator=gen)
            index[:3000] = 25000 + r
            src = torch.randint(-4, 5, (E, K), generator=gen).to(dtype)   # sums exact in any order
            shards.append((src, index))
        want = ts.scatter(torch.cat([s for s, _ in shards]).to(dev), torch.cat([i for _, i in shards]).to(dev), dim=0,
                          dim_size=N, reduce='sum')
        src, index = shards[rank][0].to(dev), shards[rank][1].to(dev)

        def same(a, b):   # 16-bit partials are rounded once per rank before they are added
            if dtype == torch.float32:
                return bool(torch.equal(a, b))
            return bool(torch.allclose(a.float(), b.float(), rtol=2e-2, atol=0.5))

        ok = []
        if routed_exchange_available(src, N):
            rows = -(-N // world)
            for _ in range(3):   # two staging buffers alternate: the third call reuses the first one
                got = scatter_sum_routed(src, index, N)
            lo, hi = rank * rows, min((rank + 1) * rows, N)
            ok.append(same(got[:hi - lo], want[lo:hi]) and bool((got[hi - lo:] == 0).all()))
        else:
            ok.append(None)
        got = scatter_sum_overlapped(src, index, N, pass_bytes=1 << 20)
        passes, sub = overlapped_layout(N, world, K * src.element_size(), 1 << 20)
        mine = owned_rows(N, world, rank, passes, sub, dev)
        valid = mine < N
        ok.append(same(got[valid], want[mine[valid]]))
        # plain variant with one collective per reduction: sum / mean / min / max with GLOBAL arg indices, against
        # the single-GPU operator on the concatenated shards (quantised values: ties across ranks, arg = first edge)
        from pytorch_scatter_b200.dist import scatter_sharded
        offsets = [0]
        for s_, _ in shards:
            offsets.append(offsets[-1] + s_.size(0))
        all_src = torch.cat([s_ for s_, _ in shards]).to(dev)
        all_index = torch.cat([i_ for _, i_ in shards]).to(dev)
        per = -(-N // world)
        lo, hi = rank * per, min((rank + 1) * per, N)
        for reduce in ('sum', 'mean', 'min', 'max'):
            res = scatter_sharded(src, index, N, reduce, edge_offset=offsets[rank], total_edges=offsets[-1])
            if reduce in ('min', 'max'):
                want, want_arg = getattr(ts, f'scatter_{reduce}')(all_src, all_index, 0, None, N)
                ok.append(bool(torch.equal(res[0][:hi - lo], want[lo:hi])) and bool(torch.equal(res[1][:hi - lo], want_arg[lo:hi])))
            else:
                want = ts.scatter(all_src, all_index, dim=0, dim_size=N, reduce=reduce)
                ok.append(same(res[:hi - lo], want[lo:hi]) if reduce == 'sum' else
                          bool(torch.allclose(res[:hi - lo].float(), want[lo:hi].float(), rtol=2e-2, atol=0.05)))
        results[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('dtype_name', ['float32', 'bfloat16'])
def test_sharded_scatter_two_gpus(dtype_name):
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    import torch.multiprocessing as mp
    ctx = mp.get_context('spawn')
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, dtype_name, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        if p.is_alive():   # never reached in a healthy run: end exactly the processes started here
            p.terminate()
            p.join()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    for rank in range(2):
        routed, overlapped, *plain = results[rank]
        assert routed in (True, None), f'rank {rank}: routed exchange wrong'
        assert overlapped, f'rank {rank}: overlapped exchange wrong'
        assert all(plain) and len(plain) == 4, f'rank {rank}: scatter_sharded sum/mean/min/max: {plain}'
