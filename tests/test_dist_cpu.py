"""Host-side logic of the multi-GPU path on two gloo ranks (CPU): the nnz-balanced row partitioner,
row-range sharding without a collective, and edge-sharded scatter + reduce-scatter including the
global arg indices.  The local reductions are done by the C oracle, so no GPU is needed."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import oracle_scatter, oracle_segment_csr


def test_balanced_row_cuts():
    from pytorch_scatter_b200.dist import balanced_row_cuts
    lens = torch.tensor([0, 5, 0, 100, 1, 1, 1, 40, 0, 0, 12])
    indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
    for parts in (1, 2, 3, 4, 8):
        cuts = balanced_row_cuts(indptr, parts)
        assert cuts.numel() == parts + 1 and int(cuts[0]) == 0 and int(cuts[-1]) == lens.numel()
        assert bool((cuts[1:] >= cuts[:-1]).all())
        sizes = indptr[cuts[1:]] - indptr[cuts[:-1]]
        assert int(sizes.sum()) == int(lens.sum())
        # no part exceeds its fair share by more than the longest row
        assert int(sizes.max()) <= int(lens.sum()) / parts + int(lens.max())


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _local_reduce(src, index, dim_size, reduce):
    out, arg = oracle_scatter(src, index, 0, dim_size, reduce)
    return out, arg


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from pytorch_scatter_b200.dist import scatter_sharded, shard_csr
        gen = torch.Generator().manual_seed(123)
        rows, feat = 37, 3
        lens = torch.randint(0, 9, (rows,), generator=gen)
        lens[5] = 60
        indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
        nnz = int(indptr[-1])
        src = torch.randn(nnz, feat, generator=gen)
        # --- CSR: row ranges are independent; gathering the shards gives the full result
        s_loc, ip_loc, (lo, hi) = shard_csr(src, indptr, rank, world)
        out_loc, _ = oracle_segment_csr(s_loc, ip_loc, 'sum')
        pieces = [None] * world
        dist.all_gather_object(pieces, (lo, hi, out_loc))
        full = torch.cat([p[2] for p in sorted(pieces, key=lambda p: p[0])])
        want, _ = oracle_segment_csr(src, indptr, 'sum')
        ok_csr = torch.allclose(full, want, rtol=1e-5, atol=1e-5) and full.shape == want.shape
        # --- scatter: edge shards + reduce-scatter
        n_targets = 11
        index = torch.randint(0, n_targets - 2, (nnz,), generator=gen)  # the last targets stay empty
        src_q = (src * 2).round() / 2  # ties across ranks
        per = (nnz + world - 1) // world
        e_lo, e_hi = rank * per, min(nnz, (rank + 1) * per)
        ok = {}
        for reduce in ('sum', 'mean', 'min', 'max'):
            res = scatter_sharded(src_q[e_lo:e_hi], index[e_lo:e_hi], n_targets, reduce, edge_offset=e_lo,
                                  total_edges=nnz, local_reduce=_local_reduce)
            blocks = [None] * world
            dist.all_gather_object(blocks, res)
            want, want_arg = oracle_scatter(src_q, index, 0, n_targets, reduce)
            if reduce in ('min', 'max'):
                got = torch.cat([b[0] for b in blocks])[:n_targets]
                got_arg = torch.cat([b[1] for b in blocks])[:n_targets]
                ok[reduce] = torch.equal(got, want) and torch.equal(got_arg, want_arg)
            else:
                got = torch.cat(blocks)[:n_targets]
                ok[reduce] = torch.allclose(got, want, rtol=1e-5, atol=1e-5)
        # --- the overlapped variant: slices of whole owner blocks, each reduced to its owner when final
        from pytorch_scatter_b200.dist import scatter_sum_overlapped

        def slice_reduce(s, ix, partial, lo, hi):
            keep = (ix >= lo) & (ix < hi)  # targets outside the slice (padding rows included) are ignored
            full, _ = oracle_scatter(s[keep], ix[keep], 0, partial.size(0), 'sum')
            partial[lo:hi] = full[lo:hi]
            return partial

        from pytorch_scatter_b200.dist import overlapped_layout, owned_rows
        for pass_bytes in (1, 40, 1 << 30):  # smallest slices / several / everything in one pass
            mine = scatter_sum_overlapped(src_q[e_lo:e_hi], index[e_lo:e_hi], n_targets, pass_bytes=pass_bytes,
                                          slice_reduce=slice_reduce)
            passes, sub = overlapped_layout(n_targets, world, feat * 4, pass_bytes)
            pieces = [None] * world
            dist.all_gather_object(pieces, (owned_rows(n_targets, world, rank, passes, sub), mine))
            want, _ = oracle_scatter(src_q, index, 0, n_targets, 'sum')
            got = torch.zeros(passes * sub * world, feat)
            for rows_r, vals in pieces:
                got[rows_r] = vals
            ok[f'overlapped-{pass_bytes}'] = torch.allclose(got[:n_targets], want, rtol=1e-5, atol=1e-5)
        results[rank] = (ok_csr, ok)
    finally:
        dist.destroy_process_group()


def test_sharded_paths_two_ranks():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        ok_csr, ok = results[rank]
        assert ok_csr, f'rank {rank}: sharded segment_csr differs from the full result'
        assert all(ok.values()), f'rank {rank}: {ok}'
