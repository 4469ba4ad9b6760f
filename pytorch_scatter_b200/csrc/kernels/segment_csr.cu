// segment_csr for sm_100a: row-pointer segmented reduction of src [B,E,K] into out [B,N,K].
//
// Merge-path style, balanced over ENTRIES rather than rows.  The rows of a CSR matrix are contiguous
// in src, so the whole reduced dimension is one byte stream; it is cut into fixed chunks of C entries
// (about 128 KiB) and every chunk is streamed by one warp (one single-warp CTA, so the hardware
// scheduler balances them and a finished warp frees its slot at once):
//   * the warp finds the first row that ends inside its chunk with a cooperative 32-ary search over
//     the row pointers (4 rounds for a million rows);
//   * an entry (K contiguous elements) is covered by L lanes holding one 16-byte pack each, so the
//     warp consumes 32/L entries (512 contiguous bytes for 16-byte packs) per step; loads run 16 steps
//     ahead of consumption through a shared-memory ring filled by per-lane cp.async copies (global ->
//     shared without passing through registers), so 8 KiB stay in flight per warp no matter how short
//     the rows are, the consuming loop is not unrolled and the kernel fits in 80 registers;
//   * row boundaries live in registers, 31 rows at a time (lane j holds row pointer j of the window);
//     all control flow that depends on them is warp-uniform.  When rows end inside a step, the lanes
//     whose entry belongs to the closing row feed a shuffle butterfly and the row is written;
//   * a row that straddles chunk borders is never written by the stream: the chunk where it ends
//     stores a HEAD partial, every chunk it runs out of stores a TAIL partial (workspace), and a
//     small fix-up kernel folds TAIL[c1..c2-1] and HEAD[c2] in a fixed order and writes the row.
//   * a run of rows without entries sits at one position of the stream and therefore in one chunk: after two
//     windows without any entry the warp searches for the next row that has one, and the fix-up kernel writes the
//     rows in between (every empty row that follows kEmptyRun or more empty rows), all of them in parallel.
// A 20,000-entry row is thus spread over 40 warps, a million-entry row over 2,000.  Nothing is
// atomic: results depend only on the shapes, never on scheduling.
// Two more kernels reduce the same problems where they are faster: the walking kernel (segment_csr_walk.cu: lane groups
// own pieces of a chunk) and the row-parallel kernel (segment_csr_rows.cu: a lane group per row, short narrow rows).
//
// Replaces segment_csr_kernel / segment_csr_broadcast_kernel of the upstream project
// (csrc/cuda/segment_csr_cuda.cu:15-95), which walk each row with a single thread per feature.
#include <mutex>

#include "csr_rows.cuh"

namespace tsb {

namespace {

// Streaming kernel: blockIdx.x = (batch, chunk); one warp.
// 16-bit MIN/MAX carry eight fp32 values and eight arg indices per lane: under the 80-register cap they spill, so
// those variants trade resident warps for registers (16 CTAs = 128 KiB in flight per SM still covers the latency).
template <typename T, int REDUCE, int VEC> constexpr int stream_ctas_per_sm() {
  if (sizeof(T) == 2 && VEC > 1 && REDUCE == kMean) return 20;   // the row count and its reciprocal on top of a sum's registers
  return (sizeof(T) == 2 && VEC > 1 && (REDUCE == kMin || REDUCE == kMax)) ? 16 : kMinCtasPerSm;
}

// MODE 0: contiguous source.  1: source through CsrParams::perm.  2: perm plus the sharded-scatter features (row
// slices, rows routed to their owners).  The features are compiled out of the other modes: as run-time branches
// they cost every variant registers (all of them spilled) and the 16-bit and MIN/MAX variants up to 60 % of their speed.
template <typename T, int REDUCE, int VEC, int MODE>
__global__ void __launch_bounds__(32, stream_ctas_per_sm<T, REDUCE, VEC>()) csr_stream_kernel(CsrParams p, CsrGeom g) {
  constexpr bool INDIRECT = MODE >= 1;
  constexpr bool EXTRAS = MODE == 2;
  using A = acc_t<T>;
  using Acc = RowAcc<T, REDUCE, VEC, int>;  // arg indices relative to the chunk start inside the stream
  constexpr bool kArg = Acc::kArg;

  const T *__restrict__ src = static_cast<const T *>(p.src);
  const int L = 1 << g.l_log2;
  const int lane = threadIdx.x;
  const int col = lane & (L - 1);
  const int sub = lane >> g.l_log2;
  const int eps = 32 >> g.l_log2;
  const int64_t Kv = p.K / VEC;

  int64_t chunk_id = blockIdx.x;
  if (EXTRAS && p.route_world > 1) {
    // Routed rows: chunks are scheduled roughly in order, so without a rotation every rank would store to owner 0
    // first, then to owner 1, ... and world-1 senders would share one GPU's NVLink ingress at any time.  Rank r
    // starts with the chunks that hold the rows of owner r+1: at any moment the ranks target distinct owners.
    // (Striding through the chunks instead, so that every rank stores to all owners all the time, measured no
    // faster on 4 GPUs.)
    int64_t first_row = (int64_t)((p.route_rank + 1) % p.route_world) * p.route_rows;
    if (first_row > p.N) first_row = p.N;
    chunk_id = (chunk_id + clamp64(p.indptr[first_row], 0, p.E) / g.chunk_entries) % g.chunks;  // single batch
  }
  const int64_t b = chunk_id / g.chunks;
  const int64_t w = chunk_id - b * g.chunks;
  const int64_t cs = w * g.chunk_entries;
  const int64_t ce = (cs + g.chunk_entries < p.E) ? cs + g.chunk_entries : p.E;
  const int t = (int)(ce - cs);
  const int64_t *ip = p.indptr + b * p.bstride;
  if (EXTRAS && p.skip_outside && (ce <= ip[0] || cs >= ip[p.N])) {  // warp-uniform
    if (lane == 0) g.head_row[chunk_id] = -1;
    return;
  }

  // ---- first row that ends after cs: 32-ary search over ends[r] = indptr[r + 1] -----------------
  int64_t r_first = 0;
  if (w > 0) {
    int64_t lo = 0, hi = p.N;  // answer in [lo, hi]; hi == N means "no such row"
    while (hi - lo > 32) {
      const int64_t step = (hi - lo + 31) / 32;
      int64_t probe = lo + (lane + 1) * step - 1;
      if (probe > hi - 1) probe = hi - 1;
      const unsigned gt = __ballot_sync(kFullMask, ip[probe + 1] > cs);
      if (gt == 0) { lo = hi; break; }
      const int f = __ffs((int)gt) - 1;
      const int64_t new_hi = lo + (int64_t)(f + 1) * step - 1;
      lo = lo + (int64_t)f * step;
      hi = new_hi < hi - 1 ? new_hi : hi - 1;  // ends[hi] > cs is known: the answer is <= hi
      if (hi < lo) hi = lo;
    }
    if (lo < p.N) {
      const bool in = lo + lane <= hi && lo + lane < p.N;
      const unsigned gt = __ballot_sync(kFullMask, in && ip[lo + lane + 1] > cs);
      r_first = gt ? lo + (__ffs((int)gt) - 1) : hi;  // ends[hi] > cs is known (or hi == N: no such row)
    } else {
      r_first = p.N;
    }
  }

  const T *bsrc = src + (b * p.E) * p.K;
  const int64_t step_stride = (int64_t)eps * p.K;  // elements between consecutive steps of a lane

  A *carry = static_cast<A *>(g.carry_val) + chunk_id * 2 * p.K;
  int64_t *carry_arg = Acc::kPair ? g.carry_arg + chunk_id * 2 * p.K : nullptr;  // arg indices / LSE sums

  for (int64_t cb = 0; cb < Kv; cb += L) {
    const int64_t c = cb + col;
    const bool col_ok = c < Kv;

    // ---- window of row pointers: lane j holds pointer j of rows [r_win, r_win + 31) -------------
    int64_t r_win = r_first;
    int rel = 0;            // this lane's pointer relative to cs, clamped to [0, kRelInf]
    bool head_pending = false;
    auto load_window = [&]() {
      const int64_t r = r_win + lane;
      int64_t v = (r <= p.N) ? ip[r] : (int64_t)1 << 62;
      if (lane == 0 && r_win == r_first) head_pending = (w > 0) && (r < p.N) && (v < cs);
      v -= cs;
      rel = v < 0 ? 0 : (v > kRelInf ? kRelInf : (int)v);
      if (r > p.N) rel = kRelInf;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {  // monotone, so that bad pointers stay harmless
        const int o = __shfl_up_sync(kFullMask, rel, off);
        if (lane >= off && o > rel) rel = o;
      }
    };
    load_window();
    head_pending = __shfl_sync(kFullMask, (int)head_pending, 0) != 0;

    int cur = 0;  // row r_win + cur is open: entries [cur_start, cur_end) relative to cs
    int cur_start = __shfl_sync(kFullMask, rel, 0);
    int cur_end = __shfl_sync(kFullMask, rel, 1);
    if (r_win >= p.N) { cur_start = kRelInf; cur_end = kRelInf; }
    Acc acc;
    acc.init(kRelInf);
    int empty_windows = 0;   // windows in a row without any entry

    // Closes every row that ends at or before `step_end`; `v` is this lane's entry `e` of the step.
    // `id` is what MIN/MAX record for the entry: its position, or with a permutation its source entry.
    auto close_rows = [&](const Pack<T, VEC> &v, int e, int id, int step_end) {
      while (cur_end <= step_end) {
        Acc tot = acc;
        if (kArg || cur_end != cur_start) {  // warp-uniform; an empty row's accumulators are still the identity
                                               // (MIN/MAX keep the plain path: the extra branch cost them 3-8 %)
          if (e >= cur_start && e < cur_end) tot.template update<INDIRECT>(v, id, kRelInf);
          tot.butterfly(L, 32);
        }
        const int64_t row = r_win + cur;
        if (head_pending) {
          // the row started in an earlier chunk: leave its last piece for the fix-up kernel
          if (sub == 0 && col_ok) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
              carry[c * VEC + i] = tot.val[i];
              if (kArg) carry_arg[c * VEC + i] = tot.arg[i] == kRelInf ? p.E : (INDIRECT ? 0 : cs) + tot.arg[i];
              if (Acc::kLseAcc) carry_arg[c * VEC + i] = tot.arg[i];
            }
          }
          if (lane == 0 && cb == 0) g.head_row[chunk_id] = row;
          head_pending = false;
        } else {
          const int64_t grow = b * p.N + row;
          if (sub == 0 && col_ok && !store_wide_routed<T, REDUCE, VEC, EXTRAS, int>(p, tot, grow, c * VEC)) {
            write_row<T, REDUCE, VEC, int>(tot, row_address<T, REDUCE, EXTRAS>(p, grow, c * VEC),
                                           kArg ? p.arg_out + grow * p.K + c * VEC : nullptr,
                                           (int64_t)(cur_end - cur_start), p.mode, p.E, INDIRECT ? 0 : cs, kRelInf);
          }
          if (lane == 0 && cb == 0 && p.count_out != nullptr) {
            const int len = cur_end - cur_start;
            static_cast<T *>(p.count_out)[grow] = from_acc<T>((A)(len > 0 ? len : 1));
          }
        }
        acc.init(kRelInf);
        ++cur;
        if (cur == kWindowRows) {
          r_win += kWindowRows;
          cur = 0;
          load_window();
          // Runs of rows without entries: closed one by one like any other row, a gap of thousands of rows would keep
          // this warp busy for longer than the rest of the launch takes.  When a second window in a row holds no entry at
          // all (every pointer at the position the last row ended), the warp searches for the next row that has one
          // and leaves the rows in between, each preceded by kEmptyRun or more empty rows, to the fix-up kernel.
          if (__all_sync(kFullMask, rel == cur_end)) {
            if (++empty_windows > 1) {
              empty_windows = 0;
              const int64_t r_next = first_row_ending_after_cold(ip, p.N, cs + cur_end, lane);  // the rows before it end here
              if (r_next > r_win) {
                r_win = r_next;
                load_window();
              }
            }
          } else {
            empty_windows = 0;
          }
        }
        cur_start = cur_end;
        cur_end = __shfl_sync(kFullMask, rel, cur + 1);
        if (r_win + cur >= p.N) cur_end = kRelInf;  // past the last row: nothing more closes
      }
    };

    if (lane == 0 && cb == 0) g.head_row[chunk_id] = -1;

    const T *next_ptr = bsrc + (cs + sub) * p.K + c * VEC;
    int next_rel = sub;
    // Load ring in shared memory, filled by per-lane asynchronous copies (global -> shared without
    // passing through registers).  Every lane reads back only the slot it copied itself, so the
    // per-thread completion of cp.async.wait_group is all the synchronisation the ring needs.
    constexpr int S = kRingDepth;
    __shared__ Pack<T, VEC> s_ring[S][32];
    __shared__ int s_id[(INDIRECT && kArg) ? S : 1][32];  // source entry of each slot, for the arg
    // INDIRECT: the permutation is read 32 positions at a time (lane j holds position 32 w + j of the
    // chunk), two windows ahead of the one the copies are issued from, and handed out by shuffle.
    int pw0 = 0, pw1 = 0, pw2 = 0;
    const int row_elems = (int)p.K;                 // K < 2^31 with a permutation (checked by the launcher)
    const T *perm_col = bsrc + c * VEC;             // this lane's columns of source entry 0
    auto load_perm_window = [&](int first) -> int {
      const int q = first + lane;
      int v = (q < t) ? p.perm[cs + q] : 0;
      const int last = (int)p.E - 1;
      return v < 0 ? 0 : (v > last ? last : v);  // a stale slot past the last row must stay a valid address
    };
    if (INDIRECT) { pw0 = load_perm_window(0); pw1 = load_perm_window(32); pw2 = load_perm_window(64); }
    auto issue = [&](int into) {
      if (INDIRECT) {
        const int step_first = next_rel - sub;  // warp-uniform, a multiple of eps
        if (step_first > 0 && (step_first & 31) == 0) { pw0 = pw1; pw1 = pw2; pw2 = load_perm_window(step_first + 64); }
        const int id = __shfl_sync(kFullMask, pw0, (step_first & 31) + sub);
        if (col_ok && next_rel < t) {
          async_copy_pack<T, VEC>(&s_ring[into][lane], perm_col + (int64_t)id * row_elems);  // one 32x32->64 multiply-add
          if (kArg) s_id[into][lane] = id;
        }
      } else {
        if (col_ok && next_rel < t) async_copy_pack<T, VEC>(&s_ring[into][lane], next_ptr);
        next_ptr += step_stride;
      }
      async_commit();
      next_rel += eps;
    };
#pragma unroll
    for (int j = 0; j < S; ++j) issue(j);
    int slot = 0;
    for (int pos = 0; pos < t; pos += eps) {
      async_wait_all_but<S - 1>();  // the oldest copy in flight, this slot's, has landed
      const int e = pos + sub;
      // A lane without an entry (past the chunk's end, or a column beyond K) reads a stale slot; its
      // value is never used: the updates below are predicated on e, such a column is never written.
      const Pack<T, VEC> v = s_ring[slot][lane];
      const int id = (INDIRECT && kArg) ? s_id[slot][lane] : e;
      const int step_end = (pos + eps < t) ? pos + eps : t;
      if (cur_end <= step_end) close_rows(v, e, id, step_end);
      if (e >= cur_start && e < t) acc.template update<INDIRECT>(v, id, kRelInf);  // the row still open after this step
      issue(slot);
      slot = (slot + 1) & (S - 1);
    }
    async_wait_all_but<0>();
    // rows that end exactly at the chunk's end, including rows without entries there
    close_rows(Pack<T, VEC>(), t, t, t);  // e == t belongs to no row: the value is not looked at

    // the row still open runs on into the next chunk: store what this chunk holds of it
    if (r_win + cur < p.N && cur_start < t) {
      acc.butterfly(L, 32);
      if (sub == 0 && col_ok) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          carry[p.K + c * VEC + i] = acc.val[i];
          if (kArg) carry_arg[p.K + c * VEC + i] = acc.arg[i] == kRelInf ? p.E : (INDIRECT ? 0 : cs) + acc.arg[i];
          if (Acc::kLseAcc) carry_arg[p.K + c * VEC + i] = acc.arg[i];
        }
      }
    }
  }
}

// K == 1 (a 1-D source; wider entries only through the tuning hook, where it loses): the streaming kernel would
// spend a whole warp step (about 70 instructions plus the row-close path) on 32 scalars.  Here a CTA stages
// its chunk (at most 32 KiB of entries) in shared memory with coalesced loads, finds the rows that end inside the
// chunk with two cooperative searches, and then a group of L lanes (one 16-byte pack of the entry each) reduces a
// whole row out of shared memory: a load, VEC adds and a loop counter per entry.  Rows with more than kFlatLongRow
// entries inside the chunk are queued and reduced by a warp each.  Rows that straddle chunk borders use the same
// HEAD / TAIL partials and the same fix-up kernel as the streaming kernel.
template <typename T, int REDUCE, int VEC>
__global__ void __launch_bounds__(kFlatThreads) csr_flat_kernel(CsrParams p, CsrGeom g) {
  using A = acc_t<T>;
  using Acc = RowAcc<T, REDUCE, VEC, int64_t>;  // arg: absolute position, p.E = none
  constexpr bool kArg = Acc::kArg;
  extern __shared__ __align__(16) unsigned char s_flat_raw[];
  T *s_src = reinterpret_cast<T *>(s_flat_raw);
  __shared__ int64_t s_rows[2];          // r_lo, r_hi
  __shared__ int s_nlong;
  __shared__ int64_t s_long[kFlatThreads];  // queued rows (at most one per lane group and sweep)
  const T *__restrict__ src = static_cast<const T *>(p.src);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = 1 << g.l_log2;             // lanes per entry
  const int col = lane & (L - 1);
  const int sub = lane >> g.l_log2;        // lane group inside the warp
  const int eps = 32 >> g.l_log2;          // lane groups per warp
  const int groups = kFlatThreads >> g.l_log2;
  const int group = tid >> g.l_log2;
  const int64_t Kv = p.K / VEC;
  const bool col_ok = col < Kv;
  const int64_t chunk_id = blockIdx.x;
  const int64_t b = chunk_id / g.chunks;
  const int64_t w = chunk_id - b * g.chunks;
  const int64_t cs = w * g.chunk_entries;
  const int64_t ce = (cs + g.chunk_entries < p.E) ? cs + g.chunk_entries : p.E;
  const int t = (int)(ce - cs);
  const int64_t *ip = p.indptr + b * p.bstride;
  const T *csrc = src + (b * p.E + cs) * p.K;

  // ---- stage the chunk ---------------------------------------------------------------------------
  constexpr int kPer16 = 16 / (int)sizeof(T);
  const int elems = t * (int)p.K;
  if ((reinterpret_cast<uintptr_t>(csrc) & 15u) == 0) {
    const int full = elems / kPer16;
    for (int i = tid; i < full; i += kFlatThreads)
      reinterpret_cast<int4 *>(s_src)[i] = __ldcs(reinterpret_cast<const int4 *>(csrc) + i);
    for (int i = full * kPer16 + tid; i < elems; i += kFlatThreads) s_src[i] = csrc[i];
  } else {
    for (int i = tid; i < elems; i += kFlatThreads) s_src[i] = csrc[i];
  }
  // ---- the rows that end inside (cs, ce] (chunk 0: also those that end at 0) ----------------------
  if (warp == 0) {
    const int64_t r_lo = w > 0 ? first_row_ending_after(ip, p.N, cs, lane) : 0;
    const int64_t r_hi = first_row_ending_after(ip, p.N, ce, lane);
    if (lane == 0) {
      s_rows[0] = r_lo;
      s_rows[1] = r_hi < r_lo ? r_lo : r_hi;
      s_nlong = 0;
      g.head_row[chunk_id] = -1;
    }
  }
  __syncthreads();
  const int64_t r_lo = s_rows[0], r_hi = s_rows[1];
  A *carry = static_cast<A *>(g.carry_val) + chunk_id * 2 * p.K;          // [HEAD, TAIL] of K values
  int64_t *carry_arg = Acc::kPair ? g.carry_arg + chunk_id * 2 * p.K : nullptr;

  // Finishes row r (this lane's VEC columns of it), whose part inside the chunk has been reduced into `acc`.
  auto finish = [&](int64_t r, int64_t rs, int64_t re, const Acc &acc) {
    if (r == r_lo && w > 0 && rs < cs) {  // began in an earlier chunk: the fix-up kernel adds the other pieces
      if (col_ok) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          carry[col * VEC + i] = acc.val[i];
          if (kArg) carry_arg[col * VEC + i] = acc.arg[i];
          if (Acc::kLseAcc) carry_arg[col * VEC + i] = acc.arg[i];
        }
      }
      if (col == 0) g.head_row[chunk_id] = r;
      return;
    }
    const int64_t grow = b * p.N + r;
    if (col_ok)
      write_row<T, REDUCE, VEC, int64_t>(acc, row_address<T, REDUCE, false>(p, grow, col * VEC),
                                         kArg ? p.arg_out + grow * p.K + col * VEC : nullptr, re - rs, p.mode, p.E, 0, p.E);
    if (col == 0 && p.count_out != nullptr) static_cast<T *>(p.count_out)[grow] = from_acc<T>((A)(re - rs > 0 ? re - rs : 1));
  };
  // Reduces this lane's columns of the staged entries lo + first, lo + first + stride, ... below hi.
  auto reduce_part = [&](Acc &acc, int lo, int hi, int first, int stride) {
    if (!col_ok) return;
    const T *base = s_src + col * VEC;
    for (int i = lo + first; i < hi; i += stride)
      acc.update(*reinterpret_cast<const Pack<T, VEC> *>(base + (size_t)i * p.K), cs + i);
  };

  for (int64_t first_row = r_lo; first_row < r_hi; first_row += groups) {  // CTA-uniform trip count
    const int64_t r = first_row + group;
    if (r < r_hi) {
      const int64_t re = clamp64(ip[r + 1], 0, ce);   // bad pointers stay harmless: 0 <= rs <= re <= ce
      const int64_t rs = clamp64(ip[r], 0, re);
      const int lo = (int)((rs > cs ? rs : cs) - cs), hi = (int)(re - cs);
      if (hi - lo > kFlatLongRow) {
        if (col == 0) s_long[atomicAdd(&s_nlong, 1)] = r;
      } else {
        Acc acc;
        acc.init(p.E);
        reduce_part(acc, lo, hi, 0, 1);
        finish(r, rs, re, acc);
      }
    }
    __syncthreads();
    const int nlong = s_nlong;
    for (int q = warp; q < nlong; q += kFlatThreads / 32) {  // warp-uniform
      const int64_t rr = s_long[q];
      const int64_t re = clamp64(ip[rr + 1], 0, ce);
      const int64_t rs = clamp64(ip[rr], 0, re);
      Acc acc;
      acc.init(p.E);
      reduce_part(acc, (int)((rs > cs ? rs : cs) - cs), (int)(re - cs), sub, eps);
      acc.butterfly(L, 32);
      if (sub == 0) finish(rr, rs, re, acc);
    }
    __syncthreads();
    if (tid == 0) s_nlong = 0;
    __syncthreads();
  }
  // ---- the row still open at the chunk's end: its part inside the chunk is this chunk's TAIL partial ----
  if (warp == 0 && r_hi < p.N) {
    const int64_t rs = clamp64(ip[r_hi], 0, p.E);
    if (rs < ce) {
      Acc acc;
      acc.init(p.E);
      reduce_part(acc, (int)((rs > cs ? rs : cs) - cs), t, sub, eps);
      acc.butterfly(L, 32);
      if (sub == 0 && col_ok) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          carry[p.K + col * VEC + i] = acc.val[i];
          if (kArg) carry_arg[p.K + col * VEC + i] = acc.arg[i];
          if (Acc::kLseAcc) carry_arg[p.K + col * VEC + i] = acc.arg[i];
        }
      }
    }
  }
}

// Fix-up kernel: one warp per chunk.  If the chunk closed a row that began in an earlier chunk,
// fold the TAIL partials of the chunks the row ran through and this chunk's HEAD partial, in a
// fixed order, and write the row.  With CsrGeom::fill_empty the first warps also write the rows the reduction kernels
// leave out: rows without entries deep inside a long run of such rows.
template <typename T, int REDUCE, int VEC, bool EXTRAS>
__global__ void __launch_bounds__(kThreads) csr_fixup_kernel(CsrParams p, CsrGeom g) {
  using A = acc_t<T>;
  using Acc = RowAcc<T, REDUCE, VEC>;
  constexpr bool kArg = Acc::kArg;
  const int L = 1 << g.l_log2;
  const int lane = threadIdx.x & 31;
  const int col = lane & (L - 1);
  const int sub = lane >> g.l_log2;
  const int eps = 32 >> g.l_log2;
  const int64_t Kv = p.K / VEC;
  const int64_t warp_id = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);

  // Rows without entries that follow at least kEmptyRun such rows: the reduction kernels stop closing a run there and
  // search for its end.  The first (rows / 32) warps look at 32 rows each: row n is such a row iff the pointers of rows
  // n - kEmptyRun and n + 1 are equal.
  if (g.fill_empty && warp_id * 32 < p.B * p.N) {
    const int64_t gr = warp_id * 32 + lane;
    bool todo_lane = false;
    if (gr < p.B * p.N) {
      const int64_t b = p.B == 1 ? 0 : gr / p.N;
      const int64_t n = gr - b * p.N;
      if (n >= kEmptyRun) {
        const int64_t *ip = p.indptr + b * p.bstride + n;
        todo_lane = clamp64(ip[1], 0, p.E) == clamp64(ip[-kEmptyRun], 0, p.E);
      }
    }
    const unsigned todo = __ballot_sync(kFullMask, todo_lane);
    if (todo != 0) {
      Acc idn;
      idn.init(p.E);
      for (int j = sub; j < 32; j += eps) {   // a lane group per row
        if (!((todo >> j) & 1u)) continue;
        const int64_t grow = warp_id * 32 + j;
        for (int64_t cb = 0; cb < Kv; cb += L) {
          const int64_t c = cb + col;
          if (c < Kv && !store_wide_routed<T, REDUCE, VEC, EXTRAS, int64_t>(p, idn, grow, c * VEC))
            write_row<T, REDUCE, VEC, int64_t>(idn, row_address<T, REDUCE, EXTRAS>(p, grow, c * VEC),
                                               kArg ? p.arg_out + grow * p.K + c * VEC : nullptr, (int64_t)0, p.mode, p.E,
                                               0, p.E);
        }
        if (col == 0 && p.count_out != nullptr) static_cast<T *>(p.count_out)[grow] = from_acc<T>((A)1);
      }
    }
  }

  // (One thread per chunk looking for such rows and the warps sharing out the hits, to launch fewer CTAs, was slower:
  // nearly every chunk of a short-row problem closes a row begun earlier, and eight warps then took 256 folds in turn.)
  const int64_t chunk_id = warp_id;
  if (chunk_id >= p.B * g.chunks) return;
  const int64_t row = g.head_row[chunk_id];
  if (row < 0 || row >= p.N) return;
  const int64_t b = chunk_id / g.chunks;
  const int64_t w = chunk_id - b * g.chunks;
  const int64_t *ip = p.indptr + b * p.bstride + row;
  const int64_t rs = clamp64(ip[0], 0, p.E);
  const int64_t re = clamp64(ip[1], rs, p.E);
  int64_t c1 = rs / g.chunk_entries;
  if (c1 > w) c1 = w;
  const A *carry = static_cast<const A *>(g.carry_val);
  const int64_t grow = b * p.N + row;
  for (int64_t cb = 0; cb < Kv; cb += L) {
    const int64_t c = cb + col;
    const bool col_ok = c < Kv;
    Acc acc;
    acc.init(p.E);
    if (col_ok) {
      // TAIL partials of the chunks run through, kFold loads in flight (a 20,000-entry row runs through 150 chunks:
      // one load per trip made this loop, and with it the kernel, a chain of 80 L2 latencies), merged in chunk order
      constexpr int kFold = 4;
      int64_t cc = c1 + sub;
      for (; cc + (kFold - 1) * eps < w; cc += kFold * eps) {
        A oval[kFold][VEC];
        int64_t oarg[kFold][Acc::kPair ? VEC : 1];
#pragma unroll
        for (int f = 0; f < kFold; ++f) {
          const int64_t at = ((b * g.chunks + cc + f * eps) * 2 + 1) * p.K + c * VEC;
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            oval[f][i] = __ldg(carry + at + i);
            if (Acc::kPair) oarg[f][i] = __ldg(g.carry_arg + at + i);
          }
        }
#pragma unroll
        for (int f = 0; f < kFold; ++f) acc.merge(oval[f], oarg[f]);
      }
      for (; cc < w; cc += eps) {
        const int64_t at = ((b * g.chunks + cc) * 2 + 1) * p.K + c * VEC;
        A oval[VEC];
        int64_t oarg[Acc::kPair ? VEC : 1];
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          oval[i] = __ldg(carry + at + i);
          if (Acc::kPair) oarg[i] = __ldg(g.carry_arg + at + i);
        }
        acc.merge(oval, oarg);
      }
    }
    acc.butterfly(L, 32);
    if (sub == 0 && col_ok) {
      const int64_t at = (chunk_id * 2) * p.K + c * VEC;  // this chunk's HEAD partial
      A oval[VEC];
      int64_t oarg[Acc::kPair ? VEC : 1];
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        oval[i] = carry[at + i];
        if (Acc::kPair) oarg[i] = g.carry_arg[at + i];
      }
      acc.merge(oval, oarg);
      if (!store_wide_routed<T, REDUCE, VEC, EXTRAS, int64_t>(p, acc, grow, c * VEC))
        write_row<T, REDUCE, VEC, int64_t>(acc, row_address<T, REDUCE, EXTRAS>(p, grow, c * VEC),
                                           kArg ? p.arg_out + grow * p.K + c * VEC : nullptr, re - rs, p.mode, p.E,
                                           0, p.E);
    }
  }
  if (lane == 0 && p.count_out != nullptr) {
    static_cast<T *>(p.count_out)[grow] = from_acc<T>((A)(re - rs > 0 ? re - rs : 1));
  }
}

// CTAs of the fix-up kernel: a warp per chunk, and enough warps that none looks at more than 32 rows for rows without
// entries.
inline int64_t fixup_blocks(int64_t total_chunks, int64_t total_rows) {
  const int64_t row_warps = (total_rows + 31) / 32;
  const int64_t warps = total_chunks > row_warps ? total_chunks : row_warps;
  return (warps + (kThreads / 32) - 1) / (kThreads / 32);
}

size_t carry_bytes(int64_t total_chunks, int64_t K, size_t acc_size, bool with_arg, size_t *arg_off, size_t *row_off) {
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  size_t off = up((size_t)total_chunks * 2 * (size_t)K * acc_size);
  *arg_off = off;
  if (with_arg) off += up((size_t)total_chunks * 2 * (size_t)K * sizeof(int64_t));
  *row_off = off;
  off += up((size_t)total_chunks * sizeof(int64_t));
  return off;
}

// Which kernel reduces the chunks.  Both are bound by instruction issue, not by DRAM, whenever a 512-byte step holds
// many elements or rows are short; which one issues less depends on the shape.  Measured on the 1,048,576-row power-law
// workload (ms, streaming / walking): fp32 F=16 max 0.500 / 0.390, sum 0.261 / 0.277; fp32 F=64 max 0.870 / 0.884;
// bf16 F=64 sum 0.509 / 0.485, mean 0.617 / 0.649, max 0.882 / 0.840; log-sum-exp fp32 F=64 1.187 / 1.127; scatter of
// bf16 F=128 into 10 M rows of 2.5 entries 2.91 / 2.70.  With two packs per lane (32 bytes) the walking kernel also
// beats the streaming one on the contiguous fp32 sum it was not meant for (F=64: 0.733 -> 0.714 ms, 0.986 of the
// measured HBM peak) but spills for every reduction with a second word per value, so that form is built for fp32
// sum / mean over a contiguous source only.  TSB_CSR_KERNEL=walk|stream (test hook) dictates the choice where the
// shapes allow both.
enum WalkChoice { kStream = 0, kWalk = 1, kWalkWide = 2 };

template <typename T, int REDUCE, int MODE> constexpr bool walk_wide_built() {
  return std::is_same<T, float>::value && (REDUCE == kSum || REDUCE == kMean) && MODE == 0;
}

template <typename T, int REDUCE>
inline int choose_kernel(const CsrParams &p, int64_t packs_per_entry, bool wide_possible) {
  const bool can_walk = packs_per_entry >= 4;
  int forced = -1;
  if (const char *v = std::getenv("TSB_CSR_KERNEL")) forced = (*v == 'w') ? 1 : (*v == 's' ? 0 : -1);
  const int64_t entry_bytes = p.K * (int64_t)sizeof(T);
  const int64_t rows = p.N > 0 ? p.N : 1;
  const bool contiguous = p.perm == nullptr && !p.skip_outside && p.route_world == 0;
  if (wide_possible && forced != 0 && contiguous && entry_bytes >= 256 && entry_bytes <= 256 &&
      std::is_same<T, float>::value && (REDUCE == kSum || REDUCE == kMean))
    return kWalkWide;
  if (!can_walk || forced == 0) return kStream;
  if (forced == 1) return kWalk;
  if (REDUCE == kLse) return kWalk;
  if (REDUCE == kMin || REDUCE == kMax) return entry_bytes <= 128 ? kWalk : kStream;
  if (REDUCE == kMean) return kStream;
  if (sizeof(T) == 2 && entry_bytes <= 128) return kWalk;
  return p.E / rows < 6 ? kWalk : kStream;   // sums over rows of a few entries
}

// The row-parallel kernel (segment_csr_rows.cu) is chosen for rows of fewer than 4 entries on average AND entries of at
// most 64 bytes.  Measured (ms, row-parallel / walking / streaming): 4 M rows of ~2 entries, fp32 F=16: sum 0.291 / 0.496
// / 0.593, max 0.450 / 0.628 / 1.364.  With wider entries it loses, because a CTA then holds few rows and every row is
// a chain of three dependent loads (row pointers, permutation, source) with nothing else of that lane group in flight:
// fp32 F=64, ~2 entries: sum 1.088 / 0.701 / 0.616; bf16 F=128, 25 M entries into 10 M rows through a permutation (an
// edge shard of a power-law graph): sum 11.06 / 2.89 / 2.90.  TSB_CSR_KERNEL=rows (test hook) dictates it.
inline bool short_rows_preferred(const CsrParams &p, size_t elem) {
  if (const char *v = std::getenv("TSB_CSR_KERNEL")) return *v == 'r';
  const int64_t rows = p.B * p.N > 0 ? p.B * p.N : 1;
  return p.B * p.E < 4 * rows && p.K * (int64_t)elem <= 64;
}

template <typename T> constexpr int dtype_code() {
  if (std::is_same<T, float>::value) return TSB_F32;
  if (std::is_same<T, double>::value) return TSB_F64;
  if (std::is_same<T, __half>::value) return TSB_F16;
  if (std::is_same<T, __nv_bfloat16>::value) return TSB_BF16;
  if (std::is_same<T, int32_t>::value) return TSB_I32;
  if (std::is_same<T, uint8_t>::value) return TSB_U8;
  if (std::is_same<T, int8_t>::value) return TSB_I8;
  if (std::is_same<T, int16_t>::value) return TSB_I16;
  return TSB_I64;
}

template <typename T, int REDUCE, int VEC, int MODE>
void launch_chunks(const CsrParams &p, const CsrGeom &g, unsigned total_chunks, bool walk, cudaStream_t stream) {
  constexpr bool kWide = VEC > full_vec<T>();
  if constexpr (kWide) {
    launch_csr_walk(p, &g, total_chunks, dtype_code<T>(), REDUCE, true, MODE, stream);   // built: see choose_kernel
  } else {
    if constexpr (VEC > 1) {   // (scalar packs always stream)
      if (walk && launch_csr_walk(p, &g, total_chunks, dtype_code<T>(), REDUCE, false, MODE, stream)) return;
    }
    csr_stream_kernel<T, REDUCE, VEC, MODE><<<total_chunks, 32, 0, stream>>>(p, g);
  }
}

template <typename T, int REDUCE, int VEC>
int launch_vec(const CsrParams &p, CsrGeom g_in, cudaStream_t stream) {
  // VEC > full_vec: the walking kernel with two 16-byte packs per lane; the fix-up kernel keeps single packs (the
  // carries are plain arrays of K values, any pack width reads them) and therefore its own lane geometry
  constexpr int FIX = VEC > full_vec<T>() ? full_vec<T>() : VEC;
  CsrGeom g = g_in, gf = g_in;
  const int64_t Kv = p.K / VEC;
  g.l_log2 = (int)(Kv >= 32 ? 5 : ilog2_ceil(Kv));
  const int64_t Kf = p.K / FIX;
  gf.l_log2 = (int)(Kf >= 32 ? 5 : ilog2_ceil(Kf));
  const int64_t total_chunks = p.B * g.chunks;
  if (total_chunks > 2147483647LL) return TSB_ERR_TOO_LARGE;
  const bool extras = p.skip_outside || p.route_world > 0;
  g.fill_empty = gf.fill_empty = true;
  const int64_t blocks = fixup_blocks(total_chunks, p.B * p.N);
  if (blocks > 2147483647LL) return TSB_ERR_TOO_LARGE;
  const bool walk = VEC > full_vec<T>() || choose_kernel<T, REDUCE>(p, p.K / VEC, false) == kWalk;
  if constexpr (REDUCE == kMul) {  // the product exists for scatter only: through the permutation, whole problem
    if (p.perm == nullptr || extras) return TSB_ERR_REDUCE;
    launch_chunks<T, REDUCE, VEC, 1>(p, g, (unsigned)total_chunks, walk, stream);
    csr_fixup_kernel<T, REDUCE, FIX, false><<<(unsigned)blocks, kThreads, 0, stream>>>(p, gf);
    return launch_status();
  } else if (p.perm != nullptr || extras) {
    if constexpr (REDUCE == kLse) {
      return TSB_ERR_REDUCE;
    } else {
      if (p.perm == nullptr && p.E > 0) return TSB_ERR_ARG;  // the sharded-scatter features come with a permutation
      if (extras) launch_chunks<T, REDUCE, VEC, 2>(p, g, (unsigned)total_chunks, walk, stream);
      else launch_chunks<T, REDUCE, VEC, 1>(p, g, (unsigned)total_chunks, walk, stream);
      if (extras) csr_fixup_kernel<T, REDUCE, FIX, true><<<(unsigned)blocks, kThreads, 0, stream>>>(p, gf);
      else csr_fixup_kernel<T, REDUCE, FIX, false><<<(unsigned)blocks, kThreads, 0, stream>>>(p, gf);
    }
  } else {
    launch_chunks<T, REDUCE, VEC, 0>(p, g, (unsigned)total_chunks, walk, stream);
    csr_fixup_kernel<T, REDUCE, FIX, false><<<(unsigned)blocks, kThreads, 0, stream>>>(p, gf);
  }
  return launch_status();
}

template <typename T, int REDUCE>
int launch_typed(const CsrParams &p, cudaStream_t stream) {
  using A = acc_t<T>;
  constexpr int kFull = full_vec<T>();
  constexpr bool kArg = (REDUCE == kMin || REDUCE == kMax || REDUCE == kLse);  // a second word per value
  if (p.B * p.N == 0) return TSB_OK;
  CsrGeom g;
  g.l_log2 = 0;
  g.chunk_entries = chunk_entries_for(p.K, sizeof(T), p.E);
  g.chunks = (p.E + g.chunk_entries - 1) / g.chunk_entries;
  if (g.chunks < 1) g.chunks = 1;
  size_t arg_off = 0, row_off = 0;
  const size_t need = carry_bytes(p.B * g.chunks, p.K, sizeof(A), kArg, &arg_off, &row_off);
  if (p.workspace == nullptr || p.workspace_bytes < need || (reinterpret_cast<uintptr_t>(p.workspace) & 255u)) return TSB_ERR_WORKSPACE;
  unsigned char *ws = static_cast<unsigned char *>(p.workspace);
  g.carry_val = ws;
  g.carry_arg = reinterpret_cast<int64_t *>(ws + arg_off);
  g.head_row = reinterpret_cast<int64_t *>(ws + row_off);
  if constexpr (REDUCE != kMul) {
  if (flat_rows(p.K, sizeof(T)) && p.perm == nullptr && !p.skip_outside && p.route_world == 0 &&
      (size_t)g.chunk_entries * (size_t)p.K * sizeof(T) <= (size_t)kFlatTileBytes) {
    const int64_t total_chunks = p.B * g.chunks;
    if (total_chunks > 2147483647LL) return TSB_ERR_TOO_LARGE;
    const bool vec = (p.K % kFull == 0) && aligned16(p.src) && aligned16(p.out);
    const int64_t Kv = p.K / (vec ? kFull : 1);
    if (Kv <= 32) {
      g.l_log2 = ilog2_ceil(Kv);
      const size_t smem = (size_t)g.chunk_entries * (size_t)p.K * sizeof(T);
      const int64_t blocks = fixup_blocks(total_chunks, 0);   // the staged kernel writes its own rows without entries
      if (vec) {
        csr_flat_kernel<T, REDUCE, kFull><<<(unsigned)total_chunks, kFlatThreads, smem, stream>>>(p, g);
        if (g.chunks > 1) csr_fixup_kernel<T, REDUCE, kFull, false><<<(unsigned)blocks, kThreads, 0, stream>>>(p, g);
      } else {
        csr_flat_kernel<T, REDUCE, 1><<<(unsigned)total_chunks, kFlatThreads, smem, stream>>>(p, g);
        if (g.chunks > 1) csr_fixup_kernel<T, REDUCE, 1, false><<<(unsigned)blocks, kThreads, 0, stream>>>(p, g);
      }
      return launch_status();
    }
  }
  }
  bool vec_ok = (p.K % kFull == 0) && aligned16(p.src) && aligned16(p.out);
  for (int q = 0; q < p.route_world; ++q) vec_ok = vec_ok && aligned16(p.route_base[q]);
  if constexpr (REDUCE != kLse) {
    // rows of only a few entries: a lane group per row instead of chunks (segment_csr_rows.cu)
    const bool extras = p.skip_outside || p.route_world > 0;
    if (short_rows_preferred(p, sizeof(T)) && (!extras || p.perm != nullptr || p.E == 0)) {
      const int mode = extras ? 2 : (p.perm != nullptr ? 1 : 0);
      if (launch_csr_short_rows(p, dtype_code<T>(), REDUCE, vec_ok, mode, stream)) return launch_status();
    }
  }
  if (vec_ok) {
    // two packs (32 bytes) per lane: every row of src / out must start on a 32-byte boundary
    const bool wide = (p.K % (2 * kFull) == 0) && p.K / (2 * kFull) >= 4 && aligned32(p.src) && aligned32(p.out);
    if constexpr (walk_wide_built<T, REDUCE, 0>()) {
      if (choose_kernel<T, REDUCE>(p, p.K / kFull, wide) == kWalkWide) return launch_vec<T, REDUCE, 2 * kFull>(p, g, stream);
    }
    return launch_vec<T, REDUCE, kFull>(p, g, stream);
  }
  return launch_vec<T, REDUCE, 1>(p, g, stream);
}

}  // namespace

size_t csr_reduce_workspace_bytes(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce) {
  (void)N;
  if (B <= 0 || K <= 0 || E < 0) return 256;
  const size_t elem = dtype_elem_bytes(dtype), acc = dtype_acc_bytes(dtype);
  const int c = chunk_entries_for(K, elem, E);
  int64_t chunks = (E + c - 1) / c;
  if (chunks < 1) chunks = 1;
  size_t a = 0, r = 0;
  return carry_bytes(B * chunks, K, acc, reduce == TSB_MIN || reduce == TSB_MAX || reduce == TSB_LSE, &a, &r);
}

int launch_csr_reduce(const CsrParams &p, int dtype, int reduce, cudaStream_t stream) {
  if (p.B < 0 || p.E < 0 || p.K < 0 || p.N < 0) return TSB_ERR_ARG;
  if (p.B * p.N * p.K == 0) return TSB_OK;
  if (p.src == nullptr && p.E > 0) return TSB_ERR_ARG;
  if (p.indptr == nullptr || (p.out == nullptr && p.route_world == 0)) return TSB_ERR_ARG;
  if (p.route_world != 0) {
    if (p.route_world < 0 || p.route_world > CsrParams::kMaxRoute || p.route_rank < 0 || p.route_rank >= p.route_world ||
        p.route_rows < 1 || p.route_rows * p.route_world < p.N || p.B != 1 || p.mode == kCooSeeded || reduce != TSB_SUM)
      return TSB_ERR_ARG;
    for (int q = 0; q < p.route_world; ++q)
      if (p.route_base[q] == nullptr) return TSB_ERR_ARG;
  }
  if ((reduce == TSB_MIN || reduce == TSB_MAX) && p.arg_out == nullptr) return TSB_ERR_ARG;
  if (p.perm != nullptr && (p.E >= kRelInf || p.K >= (1ll << 31))) return TSB_ERR_TOO_LARGE;
  if (p.skip_outside && p.B != 1) return TSB_ERR_ARG;
  return TSB_DISPATCH_DTYPE(dtype, [&]() -> int {
    switch (reduce) {
      case TSB_SUM: return launch_typed<scalar_t, kSum>(p, stream);
      case TSB_MEAN: return launch_typed<scalar_t, kMean>(p, stream);
      case TSB_MIN: return launch_typed<scalar_t, kMin>(p, stream);
      case TSB_MAX: return launch_typed<scalar_t, kMax>(p, stream);
      case TSB_MUL: return launch_typed<scalar_t, kMul>(p, stream);
      case TSB_LSE:
        if constexpr (std::is_same<acc_t<scalar_t>, float>::value) return launch_typed<scalar_t, kLse>(p, stream);
        else return TSB_ERR_DTYPE;
      default: return TSB_ERR_REDUCE;
    }
  });
}

}  // namespace tsb

extern "C" size_t tsb_segment_csr_workspace_bytes(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce) {
  return tsb::csr_reduce_workspace_bytes(B, E, K, N, dtype, reduce);
}

extern "C" int tsb_segment_csr(const void *src, const int64_t *indptr, void *out, int64_t *arg_out,
                               int64_t B, int64_t E, int64_t K, int64_t N, int64_t indptr_batch_stride,
                               int dtype, int reduce, void *workspace, size_t workspace_bytes,
                               tsb_stream_t stream) {
  tsb::CsrParams p;
  p.src = src;
  p.indptr = indptr;
  p.out = out;
  p.arg_out = arg_out;
  p.count_out = nullptr;
  p.B = B; p.E = E; p.K = K; p.N = N;
  p.bstride = indptr_batch_stride;
  p.mode = tsb::kCsr;
  p.workspace = workspace;
  p.workspace_bytes = workspace_bytes;
  return tsb::launch_csr_reduce(p, dtype, reduce, reinterpret_cast<cudaStream_t>(stream));
}

// -------------------------------------------------------------------------------------------------
// segment_csr without a caller-provided workspace.
//
// Some hosts cannot hand this library a scratch buffer: they gave all device memory to their own
// pool at start-up, or they sit in a latency-critical loop where a cudaMalloc (an implicit device
// synchronisation that can also fail under fragmentation) is not acceptable, and they have no
// caching allocator to ask instead.  For them the partial-row scratch of the reduction lives in the
// fixed array below.  It is part of the library image: every GPU that loads the library holds these
// 8 MiB until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[TSB_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_scratch_mutex;
void *g_static_scratch_addr[64] = {nullptr};  // device address of the array, per device ordinal

// In host code `g_static_scratch` is only a handle for the symbol, not a device address: handing
// it to a kernel would fault (or, where the GPU can reach host memory, silently use the wrong
// bytes).  The real address is asked for once per device, with that device current.
int static_scratch_of_current_device(void **addr) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TSB_ERR_LAUNCH;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void *ptr = nullptr;
    if (cudaGetSymbolAddress((void **)&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return TSB_ERR_LAUNCH;
    g_static_scratch_addr[dev] = ptr;
  }
  *addr = g_static_scratch_addr[dev];
  return TSB_OK;
}
}  // namespace

extern "C" int tsb_segment_csr_noalloc(const void *src, const int64_t *indptr, void *out, int64_t *arg_out,
                                       int64_t B, int64_t E, int64_t K, int64_t N, int64_t indptr_batch_stride,
                                       int dtype, int reduce, tsb_stream_t stream) {
  if (B < 0 || E < 0 || K < 0 || N < 0) return TSB_ERR_ARG;
  if (B * N * K == 0) return TSB_OK;
  // Nothing in the scratch has to start at zero: every chunk stores its row id slot before the
  // fix-up kernel reads it, and a partial row is only read where this same call stored it.  So the
  // contents left behind by the previous call are simply overwritten.
  const size_t need = tsb::csr_reduce_workspace_bytes(B, E, K, N, dtype, reduce);
  if (need > (size_t)TSB_STATIC_SCRATCH_BYTES) return TSB_ERR_TOO_LARGE;
  void *scratch = nullptr;
  const int st = static_scratch_of_current_device(&scratch);
  if (st != TSB_OK) return st;
  return tsb_segment_csr(src, indptr, out, arg_out, B, E, K, N, indptr_batch_stride, dtype, reduce, scratch,
                         (size_t)TSB_STATIC_SCRATCH_BYTES, stream);
}
