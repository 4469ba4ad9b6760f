"""Sharding the reductions over the GPUs of one node (one process per GPU, ``torch.distributed``).

Upstream has no distributed code; this follows how the reductions decompose:

* ``segment_csr`` / ``segment_coo`` / the gathers: every output row depends only on its own contiguous
  source range, so contiguous row ranges are independent units.  :func:`balanced_row_cuts` picks the
  cut points so that every rank gets about the same number of *entries* (not rows);
  :func:`shard_csr` slices and rebases.  No collective is needed.
* ``scatter`` on an unsorted index: shard the **edge** dimension.  Every rank reduces its edges into a
  full-length partial; one reduce-scatter (sum / min / max) leaves rank ``r`` with output rows
  ``[r*N/P, (r+1)*N/P)``.  ``mean`` reduce-scatters sums and counts and divides afterwards; the arg index
  of min/max is the smallest global edge position whose value equals the reduced value, found with a
  second (min) reduction over int64 candidates - the same first-occurrence rule as the single-GPU path.
"""
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def balanced_row_cuts(indptr: torch.Tensor, parts: int) -> torch.Tensor:
    """``parts + 1`` ascending row indices ``c`` with ``c[0] = 0`` and ``c[-1] = rows`` such that every range
    ``[c[p], c[p+1])`` holds about ``nnz / parts`` entries.  A row is never split."""
    assert indptr.dim() == 1 and indptr.numel() >= 1
    rows = indptr.numel() - 1
    nnz = int(indptr[-1])
    targets = torch.arange(1, parts, dtype=torch.float64, device=indptr.device) * (nnz / parts)
    inner = torch.searchsorted(indptr.to(torch.float64), targets, right=False).clamp_(0, rows)
    cuts = torch.cat([torch.zeros(1, dtype=torch.long, device=indptr.device), inner.long(),
                      torch.full((1,), rows, dtype=torch.long, device=indptr.device)])
    return torch.cummax(cuts, 0).values


def shard_csr(src: torch.Tensor, indptr: torch.Tensor, rank: int, world: int
              ) -> Tuple[torch.Tensor, torch.Tensor, Tuple[int, int]]:
    """The slice of a 1-D-indptr CSR problem that ``rank`` owns: ``(src_local, indptr_local, (row_lo, row_hi))``
    with ``indptr_local`` rebased to start at 0."""
    cuts = balanced_row_cuts(indptr, world)
    lo, hi = int(cuts[rank]), int(cuts[rank + 1])
    e_lo, e_hi = int(indptr[lo]), int(indptr[hi])
    return src[e_lo:e_hi], indptr[lo:hi + 1] - e_lo, (lo, hi)


def _padded_rows(n: int, world: int) -> int:
    return (n + world - 1) // world * world


def _reduce_scatter(full: torch.Tensor, op, group) -> torch.Tensor:
    """Row-blocked reduce-scatter of ``full`` [P*rows_per_rank, ...]; falls back to all-reduce + slice on
    backends without reduce_scatter_tensor (gloo)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    per = full.size(0) // world
    out = torch.empty((per,) + tuple(full.shape[1:]), dtype=full.dtype, device=full.device)
    if dist.get_backend(group) == 'nccl':
        dist.reduce_scatter_tensor(out, full.contiguous(), op=op, group=group)
        return out
    tmp = full.clone()
    dist.all_reduce(tmp, op=op, group=group)
    return tmp[rank * per:(rank + 1) * per].clone()


def scatter_sharded(src_local: torch.Tensor, index_local: torch.Tensor, dim_size: int, reduce: str = 'sum',
                    edge_offset: int = 0, total_edges: Optional[int] = None, group=None,
                    local_reduce: Optional[Callable] = None):
    """Edge-sharded ``scatter`` along dim 0 with a 1-D index.

    ``src_local`` [E_local, ...] and ``index_local`` [E_local] are this rank's edges; ``edge_offset`` is the
    global position of its first edge and ``total_edges`` the global edge count (both only matter for the arg
    indices of min/max).  Returns this rank's block of ``ceil(dim_size / P)`` output rows (the last rank's block
    may include padding rows past ``dim_size``), plus the arg block for min/max.

    ``local_reduce(src, index, dim_size, reduce) -> (out, arg_or_None)`` computes the local partial; it defaults
    to this package's CUDA operators (tests on CPU ranks inject a reference).
    """
    world = dist.get_world_size(group)
    n_pad = _padded_rows(dim_size, world)
    if local_reduce is None:
        local_reduce = _cuda_local_reduce
    if reduce in ('sum', 'add'):
        part, _ = local_reduce(src_local, index_local, n_pad, 'sum')
        return _reduce_scatter(part, dist.ReduceOp.SUM, group)
    if reduce == 'mean':
        part, _ = local_reduce(src_local, index_local, n_pad, 'sum')
        ones = torch.ones(index_local.numel(), dtype=torch.float32, device=src_local.device)
        count, _ = local_reduce(ones, index_local, n_pad, 'sum')
        total = _reduce_scatter(part, dist.ReduceOp.SUM, group)
        count = _reduce_scatter(count, dist.ReduceOp.SUM, group).clamp_(min=1)
        count = count.view((-1,) + (1,) * (total.dim() - 1))
        if total.is_floating_point():
            return total / count.to(total.dtype)
        return torch.div(total, count.to(total.dtype), rounding_mode='floor')
    if reduce in ('min', 'max'):
        op = dist.ReduceOp.MIN if reduce == 'min' else dist.ReduceOp.MAX
        if total_edges is None:
            t = torch.tensor([index_local.numel()], dtype=torch.long, device=src_local.device)
            dist.all_reduce(t, group=group)
            total_edges = int(t)
        part, arg = local_reduce(src_local, index_local, n_pad, reduce)
        # rows nobody on this rank wrote hold 0 with arg == E_local: give them the identity for the reduction
        untouched = arg >= index_local.numel()
        if part.is_floating_point():
            ident = torch.finfo(part.dtype).max if reduce == 'min' else torch.finfo(part.dtype).min
        else:
            ident = torch.iinfo(part.dtype).max if reduce == 'min' else torch.iinfo(part.dtype).min
        vals = torch.where(untouched, torch.full_like(part, ident), part)
        final = vals.clone()
        dist.all_reduce(final, op=op, group=group)
        cand = torch.where((vals == final) & ~untouched, arg + edge_offset, torch.full_like(arg, total_edges))
        arg_block = _reduce_scatter(cand, dist.ReduceOp.MIN, group)
        rank, per = dist.get_rank(group), n_pad // world
        out_block = final[rank * per:(rank + 1) * per].clone()
        out_block[arg_block >= total_edges] = 0  # targets no edge names, as in the single-GPU operator
        return out_block, arg_block
    raise ValueError(reduce)


def overlapped_layout(dim_size: int, world: int, row_bytes: int, pass_bytes: int = 128 << 20) -> Tuple[int, int]:
    """``(passes, sub)`` of :func:`scatter_sum_overlapped`: the output rows are processed in ``passes`` slices of
    ``sub * world`` rows each (about ``pass_bytes``), and within every slice rank ``r`` owns the ``r``-th run of
    ``sub`` rows."""
    rows_per_pass = max(world, min(max(dim_size, 1), pass_bytes // max(1, row_bytes)))
    passes = max(1, -(-dim_size // rows_per_pass))
    sub = -(-dim_size // (passes * world))
    return passes, sub


def owned_rows(dim_size: int, world: int, rank: int, passes: int, sub: int, device=None) -> torch.Tensor:
    """Global output rows behind the tensor :func:`scatter_sum_overlapped` returns on ``rank`` (ids past
    ``dim_size`` are padding)."""
    base = torch.arange(passes, device=device).view(-1, 1) * (sub * world) + rank * sub
    return (base + torch.arange(sub, device=device).view(1, -1)).reshape(-1)


def scatter_sum_overlapped(src_local: torch.Tensor, index_local: torch.Tensor, dim_size: int, group=None,
                           pass_bytes: int = 128 << 20, slice_reduce: Optional[Callable] = None) -> torch.Tensor:
    """Edge-sharded ``scatter(sum)`` along dim 0 whose collective overlaps the local accumulation.

    The local accumulation runs slice by slice over the output rows (a slice of about ``pass_bytes`` stays
    L2-resident, which is also how the single-GPU scatter treats large outputs).  As soon as a slice is final
    it is reduce-scattered over the ranks on a side stream - all links busy, every rank receiving its share of
    the slice - while the next slice is accumulated.  Ownership is therefore interleaved: within every slice,
    rank ``r`` owns the ``r``-th run of ``sub`` rows (see :func:`overlapped_layout` / :func:`owned_rows`).
    Returns this rank's ``passes * sub`` rows.  On CUDA the local accumulation is the atomics-free path (entry
    ids grouped by target row once, every slice a row range of one segmented reduction through that permutation)
    and partials travel in the source dtype; with an injected ``slice_reduce`` they are held in accumulation
    precision (fp32 for 16-bit sources).

    ``slice_reduce(src, index, partial, row_lo, row_hi)`` fills the slice; it defaults to this package's
    ``scatter_sum_slice`` operator (CPU tests inject a reference).
    """
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    feat = tuple(src_local.shape[1:])
    grouped = slice_reduce is None and src_local.is_cuda and 0 < src_local.size(0) < (1 << 30)
    acc_dtype = torch.float32 if src_local.dtype in (torch.float16, torch.bfloat16) and not grouped else src_local.dtype
    row_bytes = max(1, int(torch.tensor(feat).prod()) if feat else 1) * torch.empty((), dtype=acc_dtype).element_size()
    passes, sub = overlapped_layout(dim_size, world, row_bytes, pass_bytes)
    rows_per_pass = sub * world
    partial = torch.empty((passes * rows_per_pass,) + feat, dtype=acc_dtype, device=src_local.device)
    mine = torch.empty((passes * sub,) + feat, dtype=acc_dtype, device=src_local.device)
    if grouped:
        # group this rank's entry ids by target row once, then every slice is a row range of one
        # atomics-free segmented reduction through that permutation
        rowptr, perm = torch.ops.torch_scatter.scatter_group(index_local, passes * rows_per_pass)

        def slice_reduce(src, index, partial, row_lo, row_hi):
            return torch.ops.torch_scatter.segment_sum_perm(src, rowptr, perm, partial, row_lo, row_hi)
    elif slice_reduce is None:
        slice_reduce = torch.ops.torch_scatter.scatter_sum_slice
    on_gpu = src_local.is_cuda
    nccl = dist.get_backend(group) == 'nccl'
    comm = torch.cuda.Stream(device=src_local.device) if on_gpu else None
    work = []
    for j in range(passes):
        lo, hi = j * rows_per_pass, (j + 1) * rows_per_pass
        slice_reduce(src_local, index_local, partial, lo, hi)
        if on_gpu:
            done = torch.cuda.Event()
            done.record()
            comm.wait_event(done)
        piece, dst = partial[lo:hi], mine[j * sub:(j + 1) * sub]
        if nccl:
            with torch.cuda.stream(comm):
                work.append(dist.reduce_scatter_tensor(dst, piece, op=dist.ReduceOp.SUM, group=group, async_op=True))
        else:  # backends without reduce_scatter_tensor (gloo): all-reduce, keep the own share
            tmp = piece.clone()
            dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=group)
            dst.copy_(tmp[rank * sub:(rank + 1) * sub])
    for w in work:
        w.wait()
    if on_gpu:
        torch.cuda.current_stream().wait_stream(comm)
    return mine


_ROUTED_STAGING = {}


def _routed_staging(world: int, rows: int, feat: tuple, dtype: torch.dtype, device: torch.device, group):
    """Two symmetric staging buffers [2, world, rows, *feat] of this rank plus the device addresses of every rank's
    copy; allocated and exchanged once per shape (the rendezvous is a collective).  Returns a dict with the buffer,
    the rendezvous handle, the base addresses, the byte distance between the two buffers and a call counter."""
    import os
    import torch.distributed._symmetric_memory as symm_mem
    # plain peer stores are all this path needs: keep the buffers off NVLink multicast objects
    os.environ.setdefault('TORCH_SYMM_MEM_DISABLE_MULTICAST', '1')
    key = (id(group), world, rows, feat, dtype, device.index)
    if key not in _ROUTED_STAGING:
        buf = symm_mem.empty((2, world, rows) + feat, dtype=dtype, device=device)
        handle = symm_mem.rendezvous(buf, group if group is not None else dist.group.WORLD)
        _ROUTED_STAGING[key] = {'buf': buf, 'handle': handle, 'ptrs': [int(p) for p in handle.buffer_ptrs],
                                'half_bytes': buf[0].numel() * buf.element_size(), 'calls': 0}
    return _ROUTED_STAGING[key]


def routed_exchange_available(src_local: torch.Tensor, dim_size: int, group=None, wide_partials: bool = True) -> bool:
    """Sets up the staging buffers :func:`scatter_sum_routed` needs for this shape and says whether that worked on
    EVERY rank (a collective: all ranks must call it).  False means: use :func:`scatter_sum_overlapped`."""
    world = dist.get_world_size(group)
    ok = 1
    try:
        _routed_staging(world, -(-dim_size // world), tuple(src_local.shape[1:]),
                        _staging_dtype(src_local.dtype, wide_partials), src_local.device, group)
    except Exception as exc:  # noqa: BLE001  (no symmetric memory on this box, whatever the reason)
        print(f'[pytorch_scatter_b200.dist] routed exchange unavailable: {type(exc).__name__}: {exc}', flush=True)
        ok = 0
    flag = torch.tensor([ok], device=src_local.device, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(flag.item())


ROUTED_PHASES = ('grouping', 'reduction + peer stores', 'barrier', 'slab sum')


def _staging_dtype(dtype: torch.dtype, wide: bool) -> torch.dtype:
    return torch.float32 if wide and dtype in (torch.float16, torch.bfloat16) else dtype


def scatter_sum_routed(src_local: torch.Tensor, index_local: torch.Tensor, dim_size: int, group=None,
                       timeline: Optional[list] = None, wide_partials: bool = True) -> torch.Tensor:
    """Edge-sharded ``scatter(sum)`` along dim 0 with the exchange fused into the reduction kernel.

    Every rank groups its entry ids by target row and reduces all ``dim_size`` rows through that permutation in one
    launch; the kernel stores each finished row straight into the staging buffer of the rank that owns it (peer
    memory over NVLink, plain stores), so the transfer runs while the reduction is still going and no collective
    kernel competes for SMs.  After a barrier every rank adds the ``world`` partial slabs it received.  Rank ``r``
    owns the contiguous rows ``[r * rows, (r + 1) * rows)`` with ``rows = ceil(dim_size / world)`` and gets them
    back (zero rows beyond ``dim_size``), in the source dtype.  CUDA + NCCL only.

    Two staging buffers alternate from call to call, so one barrier per call is enough: a rank starts storing into
    buffer ``i % 2`` of its peers only after the barrier of call ``i - 1``, which every peer reaches after it has
    finished adding up call ``i - 2`` (the last reader of that buffer).

    ``wide_partials`` (default): fp16 / bf16 partial sums cross NVLink as fp32 and are rounded once, by the owner, so
    the result equals the single-GPU operator's up to summation order.  ``False`` halves the NVLink bytes of 16-bit
    sources at the price of one more rounding per rank (error up to ``world`` half-ulps of the largest partial).

    ``timeline``, if given, receives ``len(ROUTED_PHASES) + 1`` CUDA events recorded on the current stream at the
    phase borders (see :data:`ROUTED_PHASES`).
    """
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    feat = tuple(src_local.shape[1:])
    rows = -(-dim_size // world)
    wide = wide_partials and src_local.dtype in (torch.float16, torch.bfloat16)
    st = _routed_staging(world, rows, feat, _staging_dtype(src_local.dtype, wide), src_local.device, group)
    half = st['calls'] % 2
    st['calls'] += 1
    buf, handle = st['buf'][half], st['handle']
    ptrs = [p + half * st['half_bytes'] for p in st['ptrs']]

    def mark():
        if timeline is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            timeline.append(ev)

    mark()
    rowptr, perm = torch.ops.torch_scatter.scatter_group(index_local, dim_size)
    mark()
    torch.ops.torch_scatter.segment_sum_perm_routed(src_local, rowptr, perm, ptrs, rank, rows, dim_size, wide)
    valid = min(max(dim_size - rank * rows, 0), rows)   # rows of this rank's block that exist; the rest is padding
    if valid < rows:                                    # nobody writes padding rows: keep them zero
        buf[:, valid:].zero_()
    mark()
    # a bounded wait: a rank that never arrives ends the call with an error instead of hanging the GPUs
    handle.barrier(channel=half, timeout_ms=60000)      # every rank's rows have landed
    mark()
    out = torch.ops.torch_scatter.sum_slabs(buf, src_local.dtype)
    mark()
    return out


def _cuda_local_reduce(src, index, dim_size, reduce):
    from . import scatter_max, scatter_min, scatter_sum
    if reduce == 'sum':
        return scatter_sum(src, index, 0, None, dim_size), None
    fn = scatter_min if reduce == 'min' else scatter_max
    return fn(src, index, 0, None, dim_size)
