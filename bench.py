#!/usr/bin/env python
"""Benchmark of the reduction hot path: segment_csr(sum) and unsorted scatter(sum), fp32, F=64, on the
synthetic power-law CSR workload (1,048,576 rows, ~16.8M entries, log-normal row lengths).

One step = one segment_csr(sum) over the sorted rows + one scatter(sum) of the same source rows
through a shuffled (unsorted) copy of the row index.  The metric is effective HBM bandwidth:
algorithmic bytes (each of src, index/indptr and out counted once) divided by device time.

    python bench.py [--gpus N] [--steps K] [--warmup W]        this library, N GPUs (torchrun for N>1)
    python bench.py --impl reference [...]                     the upstream CPU implementation on the
                                                               host cores, on a bounded sample

Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import os.path as osp
import statistics
import subprocess
import sys
import time

import torch

ROOT = osp.dirname(osp.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS = 1 << 20
FEAT = 64
SEED = 20240602
METRIC = 'segment_csr+scatter sum effective HBM bandwidth (F=64, fp32, power-law CSR)'
UNIT = 'GB/s'
# Per-operator timings (--suite, --comparator, --profile-op) start from an idle GPU after a synchronize; without a lead the
# event pair would also span the host's own path to the first launch (tens of microseconds).  A spin kernel of this many
# cycles (about 1 ms) keeps the GPU busy while the host enqueues the operator; the start event follows it on the stream.
HOST_LEAD_CYCLES = 2_000_000


def row_lengths(rows, seed, force_long=8, mean=16.0):
    """Log-normal row lengths with the given mean (16 by default), clipped to 20,000, ~13% empty rows;
    `force_long` seeded rows are set to 20,000 so that the long-row path is always exercised."""
    g = torch.Generator().manual_seed(seed)
    sigma = 1.5
    mu = torch.log(torch.tensor(mean + 0.5, dtype=torch.float64)) - sigma * sigma / 2
    z = torch.randn(rows, generator=g, dtype=torch.float64)
    lens = torch.exp(mu + sigma * z).floor().clamp_(0, 20000).long()
    if force_long:
        where = torch.randperm(rows, generator=g)[:force_long]
        lens[where] = 20000
    return lens


def make_workload(rows, seed, feat=FEAT):
    """CPU tensors: indptr [rows+1], sorted index [nnz], shuffled index [nnz], src [nnz, feat]."""
    lens = row_lengths(rows, seed, force_long=max(1, 8 * rows // ROWS))
    indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
    nnz = int(indptr[-1])
    g = torch.Generator().manual_seed(seed + 1)
    sorted_index = torch.repeat_interleave(torch.arange(rows), lens)
    shuffled_index = sorted_index[torch.randperm(nnz, generator=g)]
    src = torch.randn(nnz, feat, generator=g, dtype=torch.float32)
    return indptr, sorted_index, shuffled_index, src


def algorithmic_bytes(rows, nnz, feat=FEAT, s=4):
    csr = nnz * feat * s + (rows + 1) * 8 + rows * feat * s
    scatter = nnz * feat * s + nnz * 8 + rows * feat * s
    return csr, scatter


def profiled_dram_bytes(name):
    """DRAM bytes per launch of one kernel as ncu counted them (dram__bytes_read.sum + dram__bytes_write.sum), from the
    line `dram_bytes_per_launch <name> <bytes> <entries>` of the committed launch-list summary, together with the
    entry count of the captured launch (traffic grows in proportion to it).  (None, None) if there is no such line."""
    path = osp.join(ROOT, 'profiles', 'bench_launch_list_csr_scatter_F64_fp32.md')
    try:
        with open(path) as f:
            for ln in f:
                parts = ln.split()
                if len(parts) >= 4 and parts[0] == 'dram_bytes_per_launch' and parts[1] == name:
                    return int(parts[2]), int(parts[3])
    except OSError:
        pass
    return None, None


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML (read-only) in a background thread
    while the timed region runs; falls back to one `nvidia-smi` query when NVML is not importable."""
    REASONS = {0x4: 'sw_power_cap', 0x8: 'hw_slowdown', 0x20: 'sw_thermal_slowdown', 0x40: 'hw_thermal_slowdown'}

    def __init__(self, device):
        import threading
        self.device, self.samples, self.reasons, self.max_mhz = device, [], set(), None
        self.stop_flag, self.thread, self.handle, self.nvml = threading.Event(), None, None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device).uuid)
            uuid = uuid if uuid.startswith('GPU-') else 'GPU-' + uuid
            self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self.nvml = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._run, daemon=True)
        except Exception:  # noqa: BLE001
            self.nvml = None

    def _run(self):
        n = self.nvml
        while not self.stop_flag.is_set():
            try:
                self.samples.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
                bits = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.005)

    def start(self):
        if self.thread is not None:
            self.thread.start()

    def stop(self):
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            return {'sm_mhz': statistics.median(self.samples) if self.samples else None, 'sm_max_mhz': self.max_mhz,
                    'reasons': sorted(self.reasons), 'samples': len(self.samples), 'source': 'nvml'}
        try:
            q = 'clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.sw_power_cap'
            out = subprocess.run(['nvidia-smi', f'--query-gpu={q}', '--format=csv,noheader,nounits'],
                                 stdout=subprocess.PIPE, text=True, timeout=10).stdout.strip().splitlines()[0].split(',')
            return {'sm_mhz': float(out[0]), 'sm_max_mhz': float(out[1]), 'reasons': [], 'samples': 1,
                    'source': 'nvidia-smi after the timed region'}
        except Exception:  # noqa: BLE001
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['clock query unavailable'], 'samples': 0}


# -------------------------------------------------------------------------------------------------
def run_reference(args):
    """Upstream CPU implementation (oracle/_ref when built, else the C port) on a bounded sample."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    rows = ROWS // args.ref_fraction
    indptr, _, shuffled, src = make_workload(rows, SEED)
    nnz = src.size(0)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ref_dir = osp.join(ROOT, 'oracle', '_ref')
    libs = sorted(f for f in os.listdir(ref_dir) if f.endswith('_cpu.so')) if osp.isdir(ref_dir) else []
    if len(libs) >= 3:
        kind = 'reference'
        for f in libs:
            torch.ops.load_library(osp.join(ref_dir, f))

        def step():
            out1 = torch.ops.torch_scatter.segment_sum_csr(src, indptr, None)
            # upstream's Python scatter_sum: zeros + ATen scatter_add_ (torch_scatter/scatter.py:8-25)
            idx = shuffled.view(-1, 1).expand(-1, src.size(1))
            out2 = torch.zeros(rows, src.size(1)).scatter_add_(0, idx, src)
            return out1, out2
    else:
        kind = 'port'
        cores = 1
        from oracle import oracle

        def step():
            out1 = oracle.segment_csr(src.view(1, nnz, -1), indptr.view(1, -1), 'sum')[0]
            out2 = oracle.scatter(src.view(1, nnz, -1), shuffled.view(1, -1, 1), rows, 'sum')[0]
            return out1, out2

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    b_csr, b_sc = algorithmic_bytes(rows, nnz)
    value = (b_csr + b_sc) / dt / 1e9
    sample = f'{rows} rows / {nnz} entries (1/{args.ref_fraction} of the workload), F={FEAT}, fp32'
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dt * 1e3, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': f'power-law CSR {ROWS} rows, F={FEAT}, fp32; reference arm timed on: {sample}',
                   'threads': torch.get_num_threads()},
        'cpu_baseline': {'value': value, 'unit': UNIT, 'cores': cores, 'kind': kind, 'sample': sample},
        'e2e': {'value': value, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
    }
    print(json.dumps(line), flush=True)


# -------------------------------------------------------------------------------------------------
def sharded_workload(world, rank, dev):
    """This rank's shard of ONE global problem, materialised on its device only.

    Global problem: world x 1,048,576 CSR rows whose lengths come from a single seed (at world == 1 exactly the
    single-GPU workload).  segment_csr: the rows are cut into `world` contiguous ranges holding about the same number of
    entries (`balanced_row_cuts`); rank r reduces range r, no collective.  scatter: the same entries as an unsorted edge
    list into 1,048,576 target rows (target = global row id modulo 1,048,576, so every rank's edges cover all targets
    with the single-GPU degree distribution; globally a graph whose mean in-degree grows with `world`); rank r holds the
    edges of its CSR range in shuffled order, reduces them for ALL target rows and the exchange leaves it with its
    block of 1,048,576 / world rows."""
    from pytorch_scatter_b200.dist import balanced_row_cuts
    lens = row_lengths(world * ROWS, SEED, force_long=8 * world)
    indptr_g = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
    cuts = balanced_row_cuts(indptr_g, world)
    lo, hi = int(cuts[rank]), int(cuts[rank + 1])
    e_lo, e_hi = int(indptr_g[lo]), int(indptr_g[hi])
    nnz_all = [int(indptr_g[cuts[r + 1]] - indptr_g[cuts[r]]) for r in range(world)]
    indptr = (indptr_g[lo:hi + 1] - e_lo).to(dev)
    g = torch.Generator(device=dev).manual_seed(SEED + 1 + rank)
    sorted_index = torch.repeat_interleave(torch.arange(lo, hi, device=dev), lens[lo:hi].to(dev))
    targets = sorted_index % ROWS
    shuffled = targets[torch.randperm(e_hi - e_lo, device=dev, generator=g)]
    src = torch.randn(e_hi - e_lo, FEAT, device=dev, generator=g)
    return {'indptr': indptr, 'sorted_local': sorted_index - lo, 'shuffled': shuffled, 'src': src, 'rows': hi - lo,
            'nnz': e_hi - e_lo, 'nnz_all': nnz_all, 'rows_all': [int(cuts[r + 1] - cuts[r]) for r in range(world)]}


def check_results(ts, w, world, rank, dev, scatter_step, interleaved=False):
    """After the timed region: both operators once more, compared with float64 results computed by ATen on the device
    (`index_add_`).  segment_csr: this rank's rows.  scatter: this rank's block of target rows against the same block
    of an NCCL reduce-scatter of the ranks' float64 partials.  Tolerance: |error| <= 1e-5 x the sum of |terms| behind
    an output (an fp32 sum in any order stays inside it).  Returns (csr worst error / bound, scatter worst, ok)."""
    import torch.distributed as dist
    src, rows = w['src'], w['rows']
    s64 = src.double()
    want = torch.zeros(rows, FEAT, dtype=torch.float64, device=dev).index_add_(0, w['sorted_local'], s64)
    mass = torch.zeros(rows, FEAT, dtype=torch.float64, device=dev).index_add_(0, w['sorted_local'], s64.abs())
    got = ts.segment_csr(src, w['indptr'], reduce='sum')
    csr_ratio = float(((got.double() - want).abs() / (1e-5 * mass + 1e-30)).max())
    del want, mass, got
    per = -(-ROWS // world)
    want = torch.zeros(per * world, FEAT, dtype=torch.float64, device=dev).index_add_(0, w['shuffled'], s64)
    mass = torch.zeros(per * world, FEAT, dtype=torch.float64, device=dev).index_add_(0, w['shuffled'], s64.abs_())
    del s64
    if world > 1:
        want_b, mass_b = torch.empty(per, FEAT, dtype=torch.float64, device=dev), torch.empty(per, FEAT, dtype=torch.float64, device=dev)
        dist.reduce_scatter_tensor(want_b, want)
        dist.reduce_scatter_tensor(mass_b, mass)
        want, mass = want_b, mass_b
    got = scatter_step(src, w['shuffled'])
    if world > 1 and interleaved:
        # the NCCL per-slice variant interleaves ownership: compare the rows this rank really holds
        from pytorch_scatter_b200.dist import overlapped_layout, owned_rows
        passes, sub = overlapped_layout(ROWS, world, FEAT * 4)
        mine = owned_rows(ROWS, world, rank, passes, sub, dev)
        ok_rows = mine < ROWS
        full_want = torch.zeros(per * world, FEAT, dtype=torch.float64, device=dev)
        full_mass = torch.zeros(per * world, FEAT, dtype=torch.float64, device=dev)
        gathered_w = [torch.empty_like(want) for _ in range(world)]
        gathered_m = [torch.empty_like(mass) for _ in range(world)]
        dist.all_gather(gathered_w, want)
        dist.all_gather(gathered_m, mass)
        full_want, full_mass = torch.cat(gathered_w), torch.cat(gathered_m)
        sc_ratio = float(((got[ok_rows].double() - full_want[mine[ok_rows]]).abs() / (1e-5 * full_mass[mine[ok_rows]] + 1e-30)).max())
    else:
        valid = min(max(ROWS - rank * per, 0), per)
        sc_ratio = float(((got[:valid].double() - want[:valid]).abs() / (1e-5 * mass[:valid] + 1e-30)).max())
        if got.size(0) > valid:   # padding rows of the last block stay zero
            sc_ratio = max(sc_ratio, float('inf') if bool((got[valid:] != 0).any()) else 0.0)
    worst = torch.tensor([csr_ratio, sc_ratio], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    csr_ratio, sc_ratio = float(worst[0]), float(worst[1])
    return csr_ratio, sc_ratio, bool(csr_ratio <= 1.0 and sc_ratio <= 1.0)


C5_NODES, C5_EDGES, C5_FEAT = 10_000_000, 200_000_000, 128


def c5_lengths(nodes=C5_NODES, edges=C5_EDGES, seed=SEED + 5):
    """In-degrees of the GNN-scale graph: the log-normal recipe with mean 20 (clip 20,000), rescaled to exactly
    `edges` edges."""
    lens = row_lengths(nodes, seed, mean=20.0, force_long=8)
    lens = (lens.double() * (edges / int(lens.sum()))).floor().long().clamp_(max=20000)
    diff = edges - int(lens.sum())
    if diff > 0:
        lens[torch.nonzero(lens < 20000).view(-1)[:diff]] += 1
    elif diff < 0:
        lens[torch.nonzero(lens > 0).view(-1)[:-diff]] -= 1
    assert int(lens.sum()) == edges
    return lens


def run_c5(ts, world, rank, dev, steps):
    """GNN-scale aggregation, ONE global problem at every GPU count (strong scaling): 10 M destination nodes, 200 M
    edges, bf16 messages [200 M x 128].  segment_csr sum / mean over nnz-balanced contiguous row ranges (no collective);
    scatter sum of the shuffled edge list, edge-sharded, with the exchange of the benchmark's scatter.  Messages are
    generated on the device, shard by shard (51 GB do not pass through the host).  Returns the `c5` block of the line."""
    import torch.distributed as dist
    from pytorch_scatter_b200.dist import balanced_row_cuts, routed_exchange_available, scatter_sum_overlapped, scatter_sum_routed
    nodes, E, F = C5_NODES, C5_EDGES, C5_FEAT
    lens = c5_lengths()
    indptr_g = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
    cuts = balanced_row_cuts(indptr_g, world)
    lo, hi = int(cuts[rank]), int(cuts[rank + 1])
    e_lo, e_hi = int(indptr_g[lo]), int(indptr_g[hi])
    nnz_all = [int(indptr_g[cuts[r + 1]] - indptr_g[cuts[r]]) for r in range(world)]
    n_here = e_hi - e_lo
    g = torch.Generator(device=dev).manual_seed(SEED + 50 + rank)
    src = torch.empty(n_here, F, dtype=torch.bfloat16, device=dev)
    for c0 in range(0, n_here, 1 << 23):   # fp32 noise in pieces: no 100 GB temporary
        c1 = min(n_here, c0 + (1 << 23))
        src[c0:c1] = torch.randn(c1 - c0, F, device=dev, generator=g)
    indptr = (indptr_g[lo:hi + 1] - e_lo).to(dev)
    # the unsorted edge list: destinations of all edges in one global shuffled order (same seed on every rank),
    # rank r holding the slice that matches its messages
    g_all = torch.Generator(device=dev).manual_seed(SEED + 49)
    dst = torch.repeat_interleave(torch.arange(nodes, device=dev), lens.to(dev))
    order = torch.randperm(E, device=dev, generator=g_all)
    index = dst[order[e_lo:e_hi]].clone()
    sorted_local = (dst[e_lo:e_hi] - lo).clone()
    del dst, order
    torch.cuda.empty_cache()

    routed = world > 1 and routed_exchange_available(src, nodes)

    def scatter_op():
        if world == 1:
            return ts.scatter(src, index, dim=0, dim_size=nodes, reduce='sum')
        if routed:
            return scatter_sum_routed(src, index, nodes)
        return scatter_sum_overlapped(src, index, nodes)

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    ms = {'segment_csr_sum': timed(lambda: ts.segment_csr(src, indptr, reduce='sum')),
          'segment_csr_mean': timed(lambda: ts.segment_csr(src, indptr, reduce='mean')),
          'scatter_sum': timed(scatter_op)}

    # ---- checks on samples (bf16 bar: |error| <= 1e-2 |result| + 1e-2), float64 by ATen
    def worst(got, want):
        return float(((got.double() - want).abs() / (1e-2 * want.abs() + 1e-2)).max()) if got.numel() else 0.0

    r0 = (hi - lo) // 3
    r1 = min(hi - lo, r0 + 20000)
    a, b = int(indptr[r0]), int(indptr[r1])
    want = torch.zeros(r1 - r0, F, dtype=torch.float64, device=dev).index_add_(0, sorted_local[a:b] - r0, src[a:b].double())
    csr_ratio = worst(ts.segment_csr(src, indptr, reduce='sum')[r0:r1], want)
    cnt = (indptr[r0 + 1:r1 + 1] - indptr[r0:r1]).clamp(min=1).double().view(-1, 1)
    mean_ratio = worst(ts.segment_csr(src, indptr, reduce='mean')[r0:r1], want / cnt)
    sample = torch.randperm(nodes, generator=torch.Generator().manual_seed(SEED + 51))[:50000].sort().values.to(dev)
    lut = torch.full((nodes,), -1, dtype=torch.long, device=dev)
    lut[sample] = torch.arange(sample.numel(), device=dev)
    local = lut[index]
    keep = torch.nonzero(local >= 0).view(-1)
    want = torch.zeros(sample.numel(), F, dtype=torch.float64, device=dev).index_add_(0, local[keep], src[keep].double())
    if world > 1:
        dist.all_reduce(want)
    got = scatter_op()
    per = -(-nodes // world) if world > 1 else nodes
    mine = (sample >= rank * per) & (sample < rank * per + got.size(0)) if world > 1 else torch.ones_like(sample, dtype=torch.bool)
    sc_ratio = worst(got[sample[mine] - (rank * per if world > 1 else 0)], want[mine])
    ratios = torch.tensor([csr_ratio, mean_ratio, sc_ratio], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ratios, op=dist.ReduceOp.MAX)
    del src, index, got, want, lut
    torch.cuda.empty_cache()

    peaks_path = osp.join(ROOT, 'MEASURED_PEAKS.json')
    peak = float(json.load(open(peaks_path))['hbm_gbs']) if osp.exists(peaks_path) else 6650.0
    b_csr = E * F * 2 + (nodes + 1) * 8 + nodes * F * 2
    b_sc = E * (F * 2 + 8) + nodes * F * 2

    def entry(name, nbytes):
        gbs = nbytes / (ms[name] * 1e-3) / 1e9
        return {'ms': ms[name], 'GB/s': gbs, 'frac_of_peak_per_gpu': gbs / world / peak,
                'elements_per_s': E * F / (ms[name] * 1e-3)}

    # what bounds the sharded scatter: every rank holds a partial of every node row (fp32 on the wire) and stores
    # (world - 1) / world of them into its peers; 770 GB/s is the peer-copy rate measured on this pool, per direction
    nvlink = None
    if world > 1 and routed:
        wire = nodes * F * 4 * (world - 1) / world
        nvlink = {'bytes_out_per_rank': int(wire), 'ms_at_770_GBps': wire / 770e9 * 1e3,
                  'frac': (wire / 770e9 * 1e3) / ms['scatter_sum']}
    return {'workload': f'{nodes} nodes / {E} edges (log-normal in-degree, mean 20, clip 20000), bf16 messages [{E} x {F}], '
                        'one global problem at every GPU count (strong scaling)', 'n_gpus': world, 'steps': steps,
            'shard_entries': nnz_all, 'nnz_imbalance_max_over_mean': max(nnz_all) / (E / world),
            'exchange': ('peer stores from the reduction kernel' if routed else 'NCCL reduce-scatter per slice') if world > 1 else None,
            'segment_csr_sum': entry('segment_csr_sum', b_csr), 'segment_csr_mean': entry('segment_csr_mean', b_csr),
            'scatter_sum': entry('scatter_sum', b_sc), 'scatter_nvlink_bound': nvlink,
            'check': {'segment_csr_sum': float(ratios[0]), 'segment_csr_mean': float(ratios[1]), 'scatter_sum': float(ratios[2]),
                      'what': 'worst |error| / (1e-2 |result| + 1e-2) over 20,000 rows per rank (csr) and 50,000 sampled '
                              'target rows (scatter), against float64 index_add_', 'ok': bool((ratios <= 1.0).all())}}


def run_ours(args):
    import torch.distributed as dist
    import pytorch_scatter_b200 as ts
    from pytorch_scatter_b200.dist import (ROUTED_PHASES, routed_exchange_available, scatter_sum_overlapped,
                                            scatter_sum_routed)

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    assert torch.cuda.is_available(), 'bench.py needs a CUDA device (no CPU fallback exists)'
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)

    w = sharded_workload(world, rank, dev)
    src, indptr, shuffled, rows_here = w['src'], w['indptr'], w['shuffled'], w['rows']
    nnz_all, rows_all = w['nnz_all'], w['rows_all']
    src_p = torch.empty(src.shape, dtype=src.dtype).pin_memory()
    indptr_p = torch.empty(indptr.shape, dtype=indptr.dtype).pin_memory()
    shuffled_p = torch.empty(shuffled.shape, dtype=shuffled.dtype).pin_memory()
    src_p.copy_(src), indptr_p.copy_(indptr), shuffled_p.copy_(shuffled)
    out_csr = torch.empty(rows_here, FEAT, device=dev)

    exchange = {'kind': None}   # how the sharded scatter exchanges rows; decided by the first call
    timeline = []               # CUDA events at the phase borders of the routed exchange (timed steps only)

    def scatter_step(s, ix, record=False):
        # Unsorted scatter shards the edge dimension.  One GPU: the plain operator.  Several: every rank reduces
        # its edges for all rows through one grouping and the kernel stores each finished row into its owner's
        # staging buffer over NVLink (peer stores), then the owners add the slabs.  If symmetric memory cannot be
        # set up on this box, the per-slice NCCL reduce-scatter variant runs instead.
        if world == 1:
            return ts.scatter(s, ix, dim=0, dim_size=ROWS, reduce='sum')
        if exchange['kind'] is None:   # decided once, by all ranks together
            if args.exchange != 'nccl' and routed_exchange_available(s, ROWS):
                exchange['kind'] = 'peer stores from the reduction kernel (symmetric memory), owners add the slabs'
            else:
                exchange['kind'] = 'NCCL reduce-scatter per output slice, overlapped with the next slice'
        if exchange['kind'].startswith('peer'):
            return scatter_sum_routed(s, ix, ROWS, timeline=timeline if record else None)
        return scatter_sum_overlapped(s, ix, ROWS)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        ts.segment_csr(src, indptr, out=out_csr, reduce='sum')
        scatter_step(src, shuffled)
    sync_all()

    sampler = ClockSampler(dev)
    if rank == 0:
        sampler.start()
    stream = torch.cuda.current_stream()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps + 1)]
    host_t0 = time.perf_counter()
    ev[0].record(stream)
    for i in range(args.steps):
        # CSR rows are independent: each rank reduces its own row range, no collective.
        ts.segment_csr(src, indptr, out=out_csr, reduce='sum')
        ev[2 * i + 1].record(stream)
        scatter_step(src, shuffled, record=True)
        ev[2 * i + 2].record(stream)
    host_ms = (time.perf_counter() - host_t0) * 1e3 / args.steps   # what the host needs to enqueue a step
    sync_all()

    total_ms = ev[0].elapsed_time(ev[-1])
    launch = 'eager (one operator call after the other from Python)'
    # Several ranks wait for one another in every step (the exchange's barrier), so a rank whose host falls behind with
    # its launches holds up all of them.  The step is therefore also captured in a CUDA graph (two steps: the exchange
    # alternates between two staging buffers) and replayed; if every rank could capture it, the replays are what
    # `value` reports, and the per-operator and per-phase times stay those of the eager loop above.
    graph = None
    if args.graph == 'on' or (args.graph == 'auto' and world > 1 and (exchange['kind'] or '').startswith('peer')):
        captured = 1
        try:
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(2):
                    ts.segment_csr(src, indptr, out=out_csr, reduce='sum')
                    scatter_step(src, shuffled)
        except Exception as exc:  # noqa: BLE001  (whatever refuses to be captured: time the eager loop instead)
            print(f'[bench] rank {rank}: CUDA graph capture failed, eager timing stands: {type(exc).__name__}: {exc}',
                  file=sys.stderr, flush=True)
            graph, captured = None, 0
        if world > 1:
            flag = torch.tensor([captured], device=dev, dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            captured = int(flag.item())
        if not captured:
            graph = None
    if graph is not None:
        for _ in range(2):
            graph.replay()
        sync_all()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        for _ in range(args.steps // 2):
            graph.replay()
        if args.steps % 2:   # exactly K steps: the odd one out runs eagerly
            ts.segment_csr(src, indptr, out=out_csr, reduce='sum')
            scatter_step(src, shuffled)
        g1.record(stream)
        sync_all()
        total_ms = g0.elapsed_time(g1)
        launch = 'CUDA graph of two steps, replayed (per-phase times: eager loop)'
    csr_ms = sum(ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(args.steps)) / args.steps
    sc_ms = sum(ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) for i in range(args.steps)) / args.steps
    csr_eager_ms, sc_eager_ms = csr_ms, sc_ms
    if graph is not None and args.steps >= 2:
        # the two operators on their own, replayed the same way (a graph of two calls each), so that the per-operator
        # times belong to the same kind of launch as `value`; if a capture fails here the eager times stand
        def replayed(fn):
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2):
                for _ in range(2):
                    fn()
            g2.replay()
            sync_all()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(args.steps // 2):
                g2.replay()
            b.record(stream)
            sync_all()
            return a.elapsed_time(b) / (2 * (args.steps // 2))
        ok_ops = 1
        try:
            csr_g = replayed(lambda: ts.segment_csr(src, indptr, out=out_csr, reduce='sum'))
            sc_g = replayed(lambda: scatter_step(src, shuffled))
        except Exception as exc:  # noqa: BLE001
            print(f'[bench] rank {rank}: per-operator graphs failed, eager times stand: {type(exc).__name__}: {exc}',
                  file=sys.stderr, flush=True)
            ok_ops = 0
        if world > 1:
            flag = torch.tensor([ok_ops], device=dev, dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok_ops = int(flag.item())
        if ok_ops:
            csr_ms, sc_ms = csr_g, sc_g
    clocks = sampler.stop() if rank == 0 else None
    n_ph = len(ROUTED_PHASES)
    phase_ms = [0.0] * n_ph
    if timeline:
        per_call = n_ph + 1
        calls = len(timeline) // per_call
        for c in range(calls):
            for k in range(n_ph):
                phase_ms[k] += timeline[c * per_call + k].elapsed_time(timeline[c * per_call + k + 1]) / calls

    # ---- end to end through the public API with host buffers: every step copies its inputs from pinned
    # host memory, runs both operators and copies both results back to pinned host memory, all inside
    # the timed region.  The three stages run on three streams with two sets of device input buffers,
    # so step i's read-back and step i+1's upload share the PCIe link's two directions.
    e2e_steps = max(1, min(args.steps, 5))
    per = -(-ROWS // world)
    out_csr_h = torch.empty(rows_here, FEAT).pin_memory()
    out_sc_h = [None]         # pinned landing buffer of the scatter result, sized by the first (untimed) step
    in_bufs = [(torch.empty_like(src), torch.empty_like(indptr), torch.empty_like(shuffled)) for _ in range(2)]
    up_s, down_s = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    consumed = [None, None]   # per buffer set: the step that last read it has finished computing
    read_back = [None]        # the previous step's results have left the pinned output buffers' way

    def e2e_step(i):
        s, ip, ix = in_bufs[i % 2]
        with torch.cuda.stream(up_s):
            if consumed[i % 2] is not None:
                up_s.wait_event(consumed[i % 2])
            s.copy_(src_p, non_blocking=True)
            ip.copy_(indptr_p, non_blocking=True)
            ix.copy_(shuffled_p, non_blocking=True)
            uploaded = torch.cuda.Event()
            uploaded.record(up_s)
        stream.wait_event(uploaded)
        o1 = ts.segment_csr(s, ip, reduce='sum')
        o2 = scatter_step(s, ix)
        consumed[i % 2] = torch.cuda.Event()
        consumed[i % 2].record(stream)
        with torch.cuda.stream(down_s):
            down_s.wait_event(consumed[i % 2])
            if out_sc_h[0] is None:
                out_sc_h[0] = torch.empty(o2.shape, dtype=o2.dtype).pin_memory()
            out_sc_h[0].copy_(o2, non_blocking=True)
            out_csr_h.copy_(o1, non_blocking=True)
            o1.record_stream(down_s)
            o2.record_stream(down_s)
            read_back[0] = torch.cuda.Event()
            read_back[0].record(down_s)

    def e2e_drain():
        stream.wait_event(read_back[0])

    e2e_step(0)
    e2e_drain()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    up_s.wait_event(e0)
    for i in range(e2e_steps):
        e2e_step(i + 1)
    e2e_drain()
    e1.record(stream)
    sync_all()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    del in_bufs

    # ---- what was timed is also checked (untimed)
    csr_ratio, sc_ratio, ok = check_results(ts, w, world, rank, dev, scatter_step,
                                            interleaved=world > 1 and not (exchange['kind'] or '').startswith('peer'))

    # ---- the GNN-scale configuration (bf16 F=128, 10 M nodes / 200 M edges) at this GPU count, untimed by the metric
    del src, indptr, shuffled, out_csr
    w.clear()
    torch.cuda.empty_cache()
    c5 = None if args.no_c5 else run_c5(ts, world, rank, dev, max(3, min(args.steps, 10)))

    # ---- max (and mean) over ranks
    times = torch.tensor([total_ms, csr_ms, sc_ms, e2e_ms] + phase_ms + [csr_eager_ms, sc_eager_ms, host_ms], device=dev,
                         dtype=torch.float64)
    if world > 1:
        gathered = [torch.empty_like(times) for _ in range(world)]
        dist.all_gather(gathered, times)
        allt = torch.stack(gathered)
    else:
        allt = times.unsqueeze(0)
    total_ms, csr_ms, sc_ms, e2e_ms = [float(allt[:, i].max()) for i in range(4)]

    if rank == 0:
        nnz_total = sum(nnz_all)
        # the global problem's bytes: every tensor counted once (the scatter's output exists once, on its owners)
        b_csr = nnz_total * FEAT * 4 + (sum(rows_all) + 1) * 8 + sum(rows_all) * FEAT * 4
        b_sc = nnz_total * (FEAT * 4 + 8) + ROWS * FEAT * 4
        ms_per_step = total_ms / args.steps
        value = (b_csr + b_sc) / (ms_per_step * 1e-3) / 1e9
        peaks_path = osp.join(ROOT, 'MEASURED_PEAKS.json')
        if osp.exists(peaks_path):
            peak, peak_src = float(json.load(open(peaks_path))['hbm_gbs']), 'measured (MEASURED_PEAKS.json hbm_gbs)'
        else:
            peak, peak_src = 6650.0, 'fallback'
        # per-GPU figures: the largest shard's own bytes over the slowest rank's time
        big = max(range(world), key=lambda r: nnz_all[r])
        b0_csr, b0_sc = algorithmic_bytes(rows_all[big], nnz_all[big])
        b0_sc = nnz_all[big] * (FEAT * 4 + 8) + per * FEAT * 4 if world > 1 else b0_sc
        csr_gbs = b0_csr / (csr_ms * 1e-3) / 1e9
        sc_gbs = b0_sc / (sc_ms * 1e-3) / 1e9
        h2d = nnz_all[0] * FEAT * 4 + (rows_all[0] + 1) * 8 + nnz_all[0] * 8
        d2h = rows_all[0] * FEAT * 4 + (per if world > 1 else ROWS) * FEAT * 4
        routed = world > 1 and exchange['kind'].startswith('peer')
        scatter_passes = -(-(ROWS * FEAT * 4) // (128 << 20))  # 128 MiB output slices (NCCL variant)

        def traffic_of(kernel, entries):
            t, e = profiled_dram_bytes(kernel)
            return None if t is None else int(round(t * entries / e))

        line = {
            'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
            'elements_per_s': 2 * nnz_total * FEAT / (ms_per_step * 1e-3),
            'config': {'workload': f'power-law CSR: ONE problem of {world} x {ROWS} rows / {nnz_total} entries (log-normal row '
                                   f'lengths, mean 16, clip 20000, {8 * world} rows forced to 20000), src fp32 [nnz x {FEAT}], '
                                   'int64 indptr/index; step = segment_csr(sum) over nnz-balanced contiguous row ranges + '
                                   f'scatter(sum) of the same entries (shuffled) into {ROWS} target rows'
                                   + (f'; exchange: {exchange["kind"]}' if world > 1 else ''),
                       'l2': 'inputs (4.3 GB per GPU) larger than L2, no flush needed',
                       'parallelism': f'{world} x nnz-balanced row ranges, no collective (csr); edge shards + exchange (scatter)',
                       'shard_entries': nnz_all, 'shard_rows': rows_all,
                       'nnz_imbalance_max_over_mean': max(nnz_all) / (nnz_total / world)},
            'ops': {'segment_csr_sum': {'ms': csr_ms, 'GB/s': csr_gbs, 'frac_of_peak': csr_gbs / peak,
                                        'elements_per_s': nnz_all[big] * FEAT / (csr_ms * 1e-3)},
                    'scatter_sum': {'ms': sc_ms, 'GB/s': sc_gbs, 'frac_of_peak': sc_gbs / peak,
                                    'elements_per_s': nnz_all[big] * FEAT / (sc_ms * 1e-3)},
                    'collective': f'inside scatter_sum ({exchange["kind"]})' if world > 1 else None},
            'roofline': {'bound': 'hbm', 'kernel': 'csr_walk_kernel<float,sum,VEC=8> (+ csr_fixup_kernel), segment_csr',
                         'achieved': csr_gbs, 'peak': peak, 'unit': 'GB/s', 'frac': csr_gbs / peak,
                         'traffic': traffic_of('csr_kernel_contiguous', nnz_all[big]),
                         'peak_source': peak_src, 'algorithmic_bytes_per_launch': b0_csr},
            'roofline_scatter': {'bound': 'hbm', 'kernel': 'scatter(sum): bucket_hist/scan/partition/finalize + '
                                                           'csr_stream_kernel<float,sum,VEC=4,perm> + csr_fixup_kernel'
                                                           + (' + sum_slabs_kernel' if routed else ''),
                                 'achieved': sc_gbs, 'peak': peak, 'unit': 'GB/s', 'frac': sc_gbs / peak,
                                 'traffic': traffic_of('scatter_all_kernels', nnz_all[big]),
                                 'peak_source': peak_src, 'algorithmic_bytes_per_launch': b0_sc},
            'e2e': {'value': (b_csr + b_sc) / (e2e_ms * 1e-3) / 1e9, 'unit': UNIT, 'ms_per_step': e2e_ms,
                    'steps': e2e_steps, 'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h},
            'check': {'csr_max_err_over_bound': csr_ratio, 'scatter_max_err_over_bound': sc_ratio,
                      'bound': '1e-5 x sum|terms| per output, against float64 index_add_ (N>1: reduce-scatter of the '
                               'float64 partials)', 'ok': ok},
            # per step, segment_csr: csr_walk_kernel + csr_fixup_kernel.  scatter on one GPU (output larger
            # than L2: the grouped path): bucket_hist, bucket_scan, bucket_partition, bucket_finalize, then
            # csr_stream_kernel + csr_fixup_kernel through the permutation.  Several GPUs with the routed exchange:
            # the same plus sum_slabs_kernel; with the NCCL variant: the grouping once plus stream + fix-up per slice.
            'gpu_launches': ((2 + 6) if world == 1 else (2 + 6 + 1) if routed else (2 + 4 + 2 * scatter_passes)) * args.steps,
            'launch': launch,
            'host_enqueue_ms_per_step': {'max': float(allt[:, -1].max()), 'per_rank': [round(float(x), 3) for x in allt[:, -1].tolist()]},
            'clocks': clocks,
        }
        if routed:
            line['ops']['scatter_phases_ms'] = {
                name: {'max': float(allt[:, 4 + k].max()), 'mean': float(allt[:, 4 + k].mean()),
                       'per_rank': [round(float(x), 4) for x in allt[:, 4 + k].tolist()]}
                for k, name in enumerate(ROUTED_PHASES)}
            line['ops']['per_rank_ms'] = {'segment_csr_sum': [round(float(x), 4) for x in allt[:, 1].tolist()],
                                          'scatter_sum': [round(float(x), 4) for x in allt[:, 2].tolist()]}
            line['ops']['eager_ms'] = {'segment_csr_sum': float(allt[:, -3].max()), 'scatter_sum': float(allt[:, -2].max())}
        if c5 is not None:
            line['c5'] = c5
        if world == 1 and not args.no_cpu_baseline:
            line['cpu_baseline'] = cpu_baseline(args)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if not ok or (c5 is not None and not c5['check']['ok']):
        sys.exit(3)


def cpu_baseline(args):
    """Times the upstream CPU path in a child process (it registers the same operator names)."""
    try:
        p = subprocess.run([sys.executable, osp.abspath(__file__), '--impl', 'reference', '--steps', '3', '--warmup', '1',
                            '--ref-fraction', str(args.ref_fraction)],
                           stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900,
                           env={k: v for k, v in os.environ.items() if k not in ('RANK', 'WORLD_SIZE', 'LOCAL_RANK')})
        for ln in reversed(p.stdout.strip().splitlines()):
            if ln.startswith('{'):
                return json.loads(ln)['cpu_baseline']
        return {'value': None, 'unit': UNIT, 'cores': None, 'kind': None, 'sample': 'failed: ' + p.stderr[-200:]}
    except Exception as e:  # noqa: BLE001
        return {'value': None, 'unit': UNIT, 'cores': None, 'kind': None, 'sample': f'failed: {e}'}


def zipf_index(E, N, dev, g):
    """E i.i.d. draws from p(k) ~ k^-1.2 over N targets, passed through a random permutation of the targets."""
    prob = torch.arange(1, N + 1, device=dev, dtype=torch.float64).pow(-1.2)
    ranks = torch.multinomial((prob / prob.sum()).float(), E, replacement=True, generator=g)
    return torch.randperm(N, device=dev, generator=g)[ranks]


def run_profile_op(args):
    """Profiling helper, meant to be wrapped in ncu on a small case: runs warmup+steps calls of ONE operator and exits.
    `csr` / `scatter` / `gather-csr`: the benchmark's operators (and the backward of the first) on a `--rows`-sized copy of
    its workload with `--feat` features in `--dtype`.  `c4-sum` / `c4-max`:
    scatter of fp32 [`--entries` x 16] under a Zipf(1.2) index over 100,000 targets.  `c3-*`: segment_coo / softmax on
    the sorted index of a `--rows`-sized workload in `--dtype`.  `c5-scatter`: bf16 F=128, `--entries` edges of a
    power-law graph into `--rows` target rows."""
    import pytorch_scatter_b200 as ts
    dev = torch.device('cuda')
    g = torch.Generator(device=dev).manual_seed(SEED)
    op = args.profile_op
    dtype = {'fp32': torch.float32, 'bf16': torch.bfloat16, 'fp16': torch.float16}[args.dtype]
    if op in ('csr', 'scatter', 'gather-csr'):
        indptr, _, shuffled, src = make_workload(args.rows, SEED, feat=args.feat)
        src, indptr, shuffled = src.to(dtype).cuda(), indptr.cuda(), shuffled.cuda()
        if args.feat == 1:
            src = src.view(-1)   # a 1-D source: the K == 1 kernel
        out = torch.empty((args.rows, args.feat) if args.feat > 1 else (args.rows,), device='cuda', dtype=dtype)
        fn = {'csr': lambda: ts.segment_csr(src, indptr, out=out, reduce='sum'),
              'scatter': lambda: ts.scatter(src, shuffled, dim=0, dim_size=args.rows, reduce='sum'),
              'gather-csr': lambda: ts.gather_csr(out, indptr, src)}[op]
        entries = src.size(0)
    elif op in ('c4-sum', 'c4-max'):
        entries, N = args.entries, 100000
        idx = zipf_index(entries, N, dev, g)
        src = torch.randn(entries, 16, device=dev, generator=g)
        fn = (lambda: ts.scatter_sum(src, idx, 0, None, N)) if op == 'c4-sum' else (lambda: ts.scatter_max(src, idx, 0, None, N))
    elif op.startswith('c3-'):
        lens = row_lengths(args.rows, SEED, force_long=max(1, 8 * args.rows // ROWS))
        index = torch.repeat_interleave(torch.arange(args.rows, device=dev), lens.to(dev))
        entries = index.numel()
        src = torch.randn(entries, args.feat, device=dev, generator=g).to(dtype)
        fn = {'c3-sum': lambda: ts.segment_sum_coo(src, index, None, args.rows),
              'c3-max': lambda: ts.segment_max_coo(src, index, None, args.rows),
              'c3-softmax': lambda: ts.scatter_softmax(src, index, 0, dim_size=args.rows)}[op]
    elif op == 'c5-scatter':
        entries, N = args.entries, args.rows
        lens = row_lengths(N, SEED + 6, mean=20.0, force_long=8).to(dev)
        here = torch.binomial(lens.float(), torch.full((N,), min(1.0, entries / float(lens.sum())), device=dev), generator=g).long()
        idx = torch.repeat_interleave(torch.arange(N, device=dev), here)
        idx = idx[torch.randperm(idx.numel(), device=dev, generator=g)]
        entries = idx.numel()
        src = torch.randn(entries, 128, device=dev, generator=g).bfloat16()
        fn = lambda: ts.scatter_sum(src, idx, 0, None, N)  # noqa: E731
    else:
        raise ValueError(op)
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda._sleep(HOST_LEAD_CYCLES)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    print(json.dumps({'profile_op': op, 'rows': args.rows, 'entries': entries, 'calls': args.warmup + args.steps,
                      'ms_per_call': e0.elapsed_time(e1) / max(1, args.steps)}))


def run_comparator(args):
    """`--comparator`: the upstream project's own CUDA kernels (compiled for sm_100 into oracle/_ref/ by
    `make -C oracle refcuda`), timed on this GPU in THIS process, which must not import pytorch_scatter_b200 (both
    register the torch_scatter::* operators).  One JSON line per operator; `python bench.py --suite` gives this
    library's times for the same shapes.  A comparator, not an oracle: upstream's float order and arg ties on the GPU
    are not deterministic."""
    ref_dir = osp.join(ROOT, 'oracle', '_ref')
    libs = sorted(f for f in os.listdir(ref_dir) if f.endswith('_cuda.so')) if osp.isdir(ref_dir) else []
    if len(libs) < 3:
        print(json.dumps({'comparator': 'unavailable', 'why': 'oracle/_ref/_*_cuda.so not built (make -C oracle refcuda REF=...)'}))
        return
    for f in libs:
        torch.ops.load_library(osp.join(ref_dir, f))
    ops = torch.ops.torch_scatter
    dev = torch.device('cuda')
    g = torch.Generator(device=dev).manual_seed(SEED)
    peaks_path = osp.join(ROOT, 'MEASURED_PEAKS.json')
    peak = float(json.load(open(peaks_path))['hbm_gbs']) if osp.exists(peaks_path) else 6650.0

    def timeit(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(args.steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(HOST_LEAD_CYCLES)  # the host enqueues the operator while the GPU is still busy
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        return statistics.median(times)

    def emit(config, op, ms, nbytes):
        gbs = nbytes / ms / 1e6
        print(json.dumps({'comparator': 'upstream csrc/cuda for sm_100', 'suite': config, 'op': op, 'ms': round(ms, 4),
                          'GB/s': round(gbs, 1), 'frac_of_measured_peak': round(gbs / peak, 3)}), flush=True)

    # C2 / C3 at F=64 fp32: the benchmark's workload
    lens = row_lengths(ROWS, SEED, force_long=8)
    indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).to(dev)
    nnz = int(indptr[-1])
    index = torch.repeat_interleave(torch.arange(ROWS, device=dev), lens.to(dev))
    shuffled = index[torch.randperm(nnz, device=dev, generator=g)]
    src = torch.randn(nnz, FEAT, device=dev, generator=g)
    b_csr, b_sc = algorithmic_bytes(ROWS, nnz)
    emit('C2', 'segment_csr sum fp32 F=64', timeit(lambda: ops.segment_sum_csr(src, indptr, None)), b_csr)
    emit('C2', 'segment_csr max fp32 F=64', timeit(lambda: ops.segment_max_csr(src, indptr, None)), b_csr + ROWS * FEAT * 8)
    emit('C3', 'segment_coo sum fp32 F=64', timeit(lambda: ops.segment_sum_coo(src, index, None, ROWS)), b_sc)
    wide = shuffled.view(-1, 1).expand(-1, FEAT)
    emit('bench', 'scatter sum fp32 F=64, shuffled index (upstream scatter_kernel)', timeit(lambda: ops.scatter_sum(src, wide, 0, None, ROWS)), b_sc)
    emit('bench', 'scatter sum fp32 F=64, shuffled index (ATen scatter_add_, what upstream\'s Python scatter_sum calls)',
         timeit(lambda: torch.zeros(ROWS, FEAT, device=dev).scatter_add_(0, wide, src)), b_sc)
    del src, wide, index, shuffled
    # C4: Zipf(1.2) index over 100,000 targets, fp32 [33.5 M x 16]
    E, F, N = 1 << 25, 16, 100000
    idx = zipf_index(E, N, dev, g).view(-1, 1).expand(-1, F)
    src = torch.randn(E, F, device=dev, generator=g)
    nb = E * F * 4 + E * 8 + N * F * 4
    emit('C4', 'scatter sum fp32 [33554432x16] Zipf(1.2)->100000 (ATen scatter_add_)',
         timeit(lambda: torch.zeros(N, F, device=dev).scatter_add_(0, idx, src)), nb)
    emit('C4', 'scatter max fp32 [33554432x16] Zipf(1.2)->100000 (upstream scatter_kernel + arg kernel)',
         timeit(lambda: ops.scatter_max(src, idx, 0, None, N)), nb + N * F * 8)


def run_suite(args):
    """`--suite`: device-time table over the other BASELINE configurations (one JSON line per operator):
    C1 scatter sum [1,048,576 x 32] -> 65,536; C2 segment_csr sum/mean/min/max at F in {1,16,64,128} and
    gather_csr; C3 segment_coo / gather_coo / scatter_softmax on the sorted index in fp32/bf16/fp16;
    C4 scatter sum/max/min with a Zipf(1.2) index over 100,000 targets, [33,554,432 x 16]; C5 one GPU's 1/8 shard
    of the 10M-node / 200M-edge bf16 F=128 aggregation."""
    import pytorch_scatter_b200 as ts
    dev = torch.device('cuda')
    peaks_path = osp.join(ROOT, 'MEASURED_PEAKS.json')
    peak = float(json.load(open(peaks_path))['hbm_gbs']) if osp.exists(peaks_path) else 6650.0
    l2_flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timeit(fn, nbytes, small):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(args.steps):
            if small:
                l2_flush.zero_()  # working set below ~250 MB: flush L2 between iterations
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(HOST_LEAD_CYCLES)  # the host enqueues the operator while the GPU is still busy
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        return ms, nbytes / ms / 1e6

    only = set(x for x in args.suite_only.split(',') if x)

    def emit(config, op, ms, gbs, **extra):
        if only and config not in only:
            return
        print(json.dumps({'suite': config, 'op': op, 'ms': round(ms, 4), 'GB/s': round(gbs, 1),
                          'frac_of_measured_peak': round(gbs / peak, 3), **extra}), flush=True)

    g = torch.Generator(device='cuda').manual_seed(SEED)

    def c1():
        E, F, N = 1 << 20, 32, 65536
        src = torch.randn(E, F, device=dev, generator=g)
        idx = torch.randint(0, N, (E,), device=dev, generator=g)
        nb = E * F * 4 + E * 8 + N * F * 4
        ms, gbs = timeit(lambda: ts.scatter(src, idx, 0, dim_size=N, reduce='sum'), nb, True)
        emit('C1', 'scatter sum fp32 [1048576x32]->65536', ms, gbs, l2_flushed=True)
        del src, idx

    def c2_c3():
        lens = row_lengths(ROWS, SEED, force_long=8)
        indptr_h = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
        nnz = int(indptr_h[-1])
        indptr = indptr_h.to(dev)
        index = torch.repeat_interleave(torch.arange(ROWS, device=dev), lens.to(dev))
        for F in (1, 16, 64, 128):
            src = torch.randn(nnz, F, device=dev, generator=g) if F > 1 else torch.randn(nnz, device=dev, generator=g)
            small = nnz * F * 4 < (250 << 20)
            for reduce in ('sum', 'mean', 'min', 'max'):
                nb = nnz * F * 4 + (ROWS + 1) * 8 + ROWS * F * 4 + (ROWS * F * 8 if reduce in ('min', 'max') else 0)
                fn = getattr(ts, f'segment_{reduce}_csr')
                ms, gbs = timeit(lambda: fn(src, indptr), nb, small)
                emit('C2', f'segment_csr {reduce} fp32 F={F}', ms, gbs, l2_flushed=small)
            if F == 64:
                table = torch.randn(ROWS, F, device=dev, generator=g)
                nb = ROWS * F * 4 + (ROWS + 1) * 8 + nnz * F * 4
                out = torch.empty(nnz, F, device=dev)
                ms, gbs = timeit(lambda: ts.gather_csr(table, indptr, out), nb, False)
                emit('C2', 'gather_csr fp32 F=64', ms, gbs)
            del src
        F = 64
        for dtype, name in ((torch.float32, 'fp32'), (torch.bfloat16, 'bf16'), (torch.float16, 'fp16')):
            s = 4 if dtype == torch.float32 else 2
            src = torch.randn(nnz, F, device=dev, generator=g).to(dtype)
            for reduce in ('sum', 'mean', 'max'):
                nb = nnz * F * s + nnz * 8 + ROWS * F * s + (ROWS * F * 8 if reduce == 'max' else 0) + (ROWS * s if reduce == 'mean' else 0)
                fn = getattr(ts, f'segment_{reduce}_coo')
                ms, gbs = timeit(lambda: fn(src, index, None, ROWS), nb, False)
                emit('C3', f'segment_coo {reduce} {name} F=64', ms, gbs)
            table = torch.randn(ROWS, F, device=dev, generator=g).to(dtype)
            out = torch.empty(nnz, F, device=dev, dtype=dtype)
            nb = ROWS * F * s + nnz * 8 + nnz * F * s
            ms, gbs = timeit(lambda: ts.gather_coo(table, index, out), nb, False)
            emit('C3', f'gather_coo {name} F=64', ms, gbs)
            # composites: bytes of the ideal single read + single write; the fused path reads src twice
            nb = 2 * nnz * F * s + nnz * 8
            ms, gbs = timeit(lambda: ts.scatter_softmax(src, index, 0, dim_size=ROWS), nb, False)
            emit('C3', f'scatter_softmax {name} F=64 (composite)', ms, gbs)
            if dtype == torch.float32:
                ms, gbs = timeit(lambda: ts.scatter_log_softmax(src, index, 0, dim_size=ROWS), nb, False)
                emit('C3', 'scatter_log_softmax fp32 F=64 (composite)', ms, gbs)
                nb = nnz * F * s + nnz * 8 + ROWS * F * s
                ms, gbs = timeit(lambda: ts.scatter_logsumexp(src, index, 0, dim_size=ROWS), nb, False)
                emit('C3', 'scatter_logsumexp fp32 F=64 (composite)', ms, gbs)
                ms, gbs = timeit(lambda: ts.scatter_std(src, index, 0, dim_size=ROWS), nb, False)
                emit('C3', 'scatter_std fp32 F=64 (composite)', ms, gbs)
            del src, table, out
        del index, indptr

    def c4():
        E, F, N = 1 << 25, 16, 100000
        prob = torch.arange(1, N + 1, device=dev, dtype=torch.float64).pow(-1.2)
        ranks = torch.multinomial((prob / prob.sum()).float(), E, replacement=True, generator=g)
        idx = torch.randperm(N, device=dev, generator=g)[ranks]
        del ranks
        src = torch.randn(E, F, device=dev, generator=g)
        for reduce in ('sum', 'max', 'min'):
            nb = E * F * 4 + E * 8 + N * F * 4 + (N * F * 8 if reduce != 'sum' else 0)
            fn = getattr(ts, f'scatter_{reduce}')
            ms, gbs = timeit(lambda: fn(src, idx, 0, None, N), nb, False)
            emit('C4', f'scatter {reduce} fp32 [33554432x16] Zipf(1.2)->100000', ms, gbs)

    def c5():
        # One GPU's share of the 8-GPU job: 1/8 of the 200M edges (bf16 [25M x 128]); segment_csr over the
        # shard's own row range (1.25M rows), scatter over all 10M destination rows (the full-length partial
        # that the exchange would consume).  Row lengths: the log-normal recipe with mean 20.
        rows_csr, n_all, F = 1_250_000, 10_000_000, 128
        lens = row_lengths(rows_csr, SEED + 5, mean=20.0, force_long=8)
        indptr = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).to(dev)
        E = int(indptr[-1])
        src = torch.randn(E, F, device=dev, generator=g).bfloat16()
        for reduce in ('sum', 'mean'):
            nb = E * F * 2 + (rows_csr + 1) * 8 + rows_csr * F * 2
            ms, gbs = timeit(lambda: ts.segment_csr(src, indptr, reduce=reduce), nb, False)
            emit('C5', f'segment_csr {reduce} bf16 F=128, {rows_csr} rows / {E} edges (1/8 shard)', ms, gbs)
        del indptr
        # the shard's edges: every edge of the power-law graph (in-degree log-normal, mean 20, clip 20,000) lands on
        # this GPU with probability 1/8, in random order
        lens_all = row_lengths(n_all, SEED + 6, mean=20.0, force_long=8).to(dev)
        lens_here = torch.binomial(lens_all.float(), torch.full((n_all,), 0.125, device=dev), generator=g).long()
        idx = torch.repeat_interleave(torch.arange(n_all, device=dev), lens_here)
        idx = idx[torch.randperm(idx.numel(), device=dev, generator=g)]
        Es = idx.numel()
        del lens_all, lens_here
        if Es > E:
            idx = idx[:E]
            Es = E
        src = src[:Es]
        for reduce in ('sum', 'max'):
            nb = Es * F * 2 + Es * 8 + n_all * F * 2 + (n_all * F * 8 if reduce == 'max' else 0)
            fn = getattr(ts, f'scatter_{reduce}')
            ms, gbs = timeit(lambda: fn(src, idx, 0, None, n_all), nb, False)
            emit('C5', f'scatter {reduce} bf16 F=128, {Es} edges -> {n_all} rows (1/8 shard of a power-law graph, full-length partial)', ms, gbs)

    if not only or 'C1' in only:
        c1()
    if not only or only & {'C2', 'C3'}:
        c2_c3()
    if not only or 'C4' in only:
        c4()
    if not only or 'C5' in only:
        c5()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=100)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--ref-fraction', type=int, default=4, help='reference arm runs on 1/this of the rows')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--graph', default='auto', choices=['auto', 'on', 'off'],
                    help="replay the step from a CUDA graph for the timed value: 'auto' = with more than one GPU")
    ap.add_argument('--exchange', default='auto', choices=['auto', 'nccl'],
                    help='N > 1: auto = peer stores from the reduction kernel when symmetric memory is available; nccl = '
                         'the per-slice NCCL reduce-scatter variant')
    ap.add_argument('--no-c5', action='store_true', help='skip the GNN-scale block (bf16 F=128, 10 M nodes / 200 M edges)')
    ap.add_argument('--comparator', action='store_true', help="upstream's own CUDA kernels (oracle/_ref/_*_cuda.so) on this GPU")
    ap.add_argument('--suite', action='store_true', help='per-operator table over the other configurations')
    ap.add_argument('--suite-only', default='', help='comma-separated configs to run, e.g. C3,C4')
    ap.add_argument('--profile-op', default=None,
                    choices=['csr', 'scatter', 'gather-csr', 'c4-sum', 'c4-max', 'c3-sum', 'c3-max', 'c3-softmax', 'c5-scatter'])
    ap.add_argument('--rows', type=int, default=ROWS, help='rows of the workload for --profile-op')
    ap.add_argument('--entries', type=int, default=1 << 22, help='entries for --profile-op c4-* / c5-scatter')
    ap.add_argument('--feat', type=int, default=64, help='features for --profile-op csr / scatter / gather-csr / c3-*')
    ap.add_argument('--dtype', default='fp32', choices=['fp32', 'bf16', 'fp16'], help='dtype for --profile-op csr / scatter / gather-csr / c3-*')
    args = ap.parse_args()
    if args.comparator:
        run_comparator(args)
        return
    if args.profile_op is not None:
        run_profile_op(args)
        return
    if args.suite:
        run_suite(args)
        return
    if args.warmup < 3 and args.impl == 'ours':
        args.warmup = 3
    if args.impl == 'reference':
        run_reference(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
