// The walking chunk kernel of the row-pointer reduction (see segment_csr.cu for the chunking, the carries and the
// fix-up that it shares with the streaming kernel).  A translation unit of its own: it is instantiated for every dtype,
// reduction and source mode, and compiles side by side with the streaming kernels.
#include "csr_rows.cuh"

namespace tsb {
namespace {

// ---------------------------------------------------------------------------------------------------------------
// Walking kernel: the same chunks, carries and fix-up as the streaming kernel, another division of labour inside
// the warp.  The streaming kernel spreads every 512-byte step over all lane groups and closes rows with a shuffle
// butterfly over the groups: at fp32 with 256-byte entries that is hidden behind DRAM, but with 16-bit data, narrow
// entries or rows of two or three entries it is what bounds the kernel (86 to 169 warp instructions per step
// counted).  Here every lane group (the L lanes that hold one entry) owns a contiguous PIECE of the chunk,
// C / (32 / L) entries, and walks it entry by entry on its own: accumulate while the row lasts, write the row when
// it ends - no shuffle per step, no butterfly per row.  What the groups share is settled once per chunk:
//   * before the walk the warp scans the row pointers from the chunk's first row (32 per load) and counts, for each
//     group, the rows that end at or before the piece's start: that is the group's first row;
//   * a row that runs from one piece into the next is never written during the walk.  The group where it ends keeps
//     what it saw of it (its "head"), every group keeps the row still open at its piece's end (its "tail"), and after
//     the walk a scan over the groups hands every tail to the group where the row goes on, in a fixed order.  The
//     chunk's own HEAD / TAIL partials go to the workspace exactly as in the streaming kernel.
// Row pointers live in per-group register windows (lane j of a group holds pointer j of the window, L - 1 rows per
// reload, reloads hit L1 after the scan); all shuffles inside a group's divergent code name that group's lanes only.
// Entries of at least four 16-byte packs' worth of lanes are required (L >= 4).
// 16-bit MIN/MAX (eight values and eight arg indices per lane, twice with the head copy), CTAs per SM / registers /
// segment_coo max bf16 F=64: 12 / 161 / 0.830 ms, 16 / 128 / 0.751 ms, 20 / 96 with 292 bytes spilled / 1.048 ms.
template <typename T, int REDUCE, int VEC> constexpr int walk_ctas_per_sm() {
  return (sizeof(T) == 2 && VEC > 1 && (REDUCE == kMin || REDUCE == kMax)) ? 16 : 20;
}
constexpr int kWalkRing = 12;   // entries in flight per lane group

template <typename T, int REDUCE, int VEC, int MODE>
__global__ void __launch_bounds__(32, walk_ctas_per_sm<T, REDUCE, VEC>()) csr_walk_kernel(CsrParams p, CsrGeom g) {
  constexpr bool INDIRECT = MODE >= 1;
  constexpr bool EXTRAS = MODE == 2;
  using A = acc_t<T>;
  using Acc = RowAcc<T, REDUCE, VEC, int>;  // arg indices relative to the chunk start (source entries with a permutation)
  constexpr bool kArg = Acc::kArg;
  constexpr int kBefore = -1;               // a row pointer that lies before the chunk

  const T *__restrict__ src = static_cast<const T *>(p.src);
  const int L = 1 << g.l_log2;
  const int lane = threadIdx.x;
  const int col = lane & (L - 1);
  const int sub = lane >> g.l_log2;
  const int eps = 32 >> g.l_log2;
  const unsigned gmask = (L == 32 ? kFullMask : ((1u << L) - 1u)) << (sub << g.l_log2);  // this group's lanes
  const int gbase = sub << g.l_log2;
  const int64_t Kv = p.K / VEC;

  int64_t chunk_id = blockIdx.x;
  if (EXTRAS && p.route_world > 1) {  // start with the next owner's rows (see the streaming kernel)
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
  if (lane == 0) g.head_row[chunk_id] = -1;
  if (EXTRAS && p.skip_outside && (ce <= ip[0] || cs >= ip[p.N])) return;  // warp-uniform

  const int piece = g.chunk_entries >> (5 - g.l_log2);
  const int ps = (sub * piece < t) ? sub * piece : t;
  const int pe = ((sub + 1) * piece < t) ? (sub + 1) * piece : t;
  const int my_n = pe - ps;

  // ---- first row of the chunk, then of every piece ---------------------------------------------------------------
  const int64_t r_first = (w > 0) ? first_row_ending_after(ip, p.N, cs, lane) : 0;
  int64_t my_first = r_first;
  {
    // rows r >= r_first with ends[r] <= cs + ps belong to earlier pieces; count them 32 at a time
    int before = 0;
    bool counted = false;
    for (int it = 0; it < 4; ++it) {   // up to 128 rows by counting; chunks with more (runs of empty rows) search instead
      const int64_t r0 = r_first + 32 * it;
      if (r0 >= p.N) { counted = true; break; }
      const int64_t r = r0 + lane;
      const int64_t end = (r < p.N) ? __ldg(ip + r + 1) - cs : (int64_t)kRelInf;
      for (int q = 1; q < eps; ++q) {
        const int bound = (q * piece < t) ? q * piece : t;
        const int c = __popc(__ballot_sync(kFullMask, end <= (int64_t)bound));
        if (q == sub) before += c;
      }
      if (__any_sync(kFullMask, end > (int64_t)t)) { counted = true; break; }  // the rows that follow end after the chunk
    }
    if (counted) {
      my_first += before;
    } else {
      for (int q = 1; q < eps; ++q) {   // warp-uniform: one cooperative search per piece border
        const int bound = (q * piece < t) ? q * piece : t;
        const int64_t r = first_row_ending_after(ip, p.N, cs + bound, lane);
        if (q == sub) my_first = r > r_first ? r : r_first;
      }
    }
  }

  const T *bsrc = src + (b * p.E) * p.K;
  A *carry = static_cast<A *>(g.carry_val) + chunk_id * 2 * p.K;
  int64_t *carry_arg = Acc::kPair ? g.carry_arg + chunk_id * 2 * p.K : nullptr;
  extern __shared__ __align__(16) unsigned char s_walk_raw[];
  auto s_ring = reinterpret_cast<Pack<T, VEC>(*)[32]>(s_walk_raw);             // [kWalkRing][32]
  int(*s_id)[32] = reinterpret_cast<int(*)[32]>(s_walk_raw + sizeof(Pack<T, VEC>) * kWalkRing * 32);  // INDIRECT MIN/MAX

  for (int64_t cb = 0; cb < Kv; cb += L) {
    const int64_t c = cb + col;
    const bool col_ok = c < Kv;

    // ---- this group's window of row pointers: lane j holds pointer j of rows [win, win + L - 1] ------------------
    int64_t win = my_first;
    int rel = 0;
    auto load_window = [&]() {
      const int64_t r = win + col;
      int64_t v = (r <= p.N) ? __ldg(ip + r) - cs : (int64_t)kRelInf;
      rel = v < 0 ? kBefore : (v > kRelInf ? kRelInf : (int)v);
      for (int off = 1; off < L; off <<= 1) {  // monotone inside the window, so that bad pointers stay harmless
        const int o = __shfl_up_sync(gmask, rel, off, L);
        if (col >= off && o > rel) rel = o;
      }
    };
    load_window();
    int cur = 0;
    int cur_start = __shfl_sync(gmask, rel, gbase + 0);
    int cur_end = __shfl_sync(gmask, rel, gbase + 1);
    if (win >= p.N) { cur_start = kRelInf; cur_end = kRelInf; }

    Acc acc, head;
    acc.init(kRelInf);
    head.init(kRelInf);
    int empty_windows = 0;   // windows in a row without any entry
    int64_t head_row = -1;   // the row that began before this piece and ended inside it
    int head_len = 0;
    bool head_from_before_chunk = false;

    // closes the open row (it ends at or before the position the walk has reached)
    auto close_row = [&]() {
      const int64_t row = win + cur;
      if (cur_start < ps) {
        // began before this piece (in an earlier piece, or before the chunk): only the scan after the walk knows
        // what the earlier pieces hold of it
        head = acc;
        head_row = row;
        head_len = cur_end - cur_start;
        head_from_before_chunk = cur_start == kBefore;
      } else {
        const int64_t grow = b * p.N + row;
        if (col_ok && !store_wide_routed<T, REDUCE, VEC, EXTRAS, int>(p, acc, grow, c * VEC)) {
          write_row<T, REDUCE, VEC, int>(acc, row_address<T, REDUCE, EXTRAS>(p, grow, c * VEC),
                                         kArg ? p.arg_out + grow * p.K + c * VEC : nullptr,
                                         (int64_t)(cur_end - cur_start), p.mode, p.E, INDIRECT ? 0 : cs, kRelInf);
        }
        if (col == 0 && cb == 0 && p.count_out != nullptr) {
          const int len = cur_end - cur_start;
          static_cast<T *>(p.count_out)[grow] = from_acc<T>((A)(len > 0 ? len : 1));
        }
      }
      acc.init(kRelInf);
      ++cur;
      if (cur == L - 1) {
        win += L - 1;
        cur = 0;
        load_window();
        // a long run of rows without entries (see the streaming kernel): once enough windows in a row held no entry at
        // all, search for the run's end; the fix-up kernel writes the rows in between
        if (__all_sync(gmask, rel == cur_end)) {
          if (++empty_windows * (L - 1) > kEmptyRun + L - 2) {   // kEmptyRun or more such rows are closed already
            empty_windows = 0;
            const int64_t r_next = first_row_ending_after_group(ip, win, p.N, cs + cur_end, col, L, gmask, gbase);
            if (r_next > win) {
              win = r_next;
              load_window();
            }
          }
        } else {
          empty_windows = 0;
        }
      }
      cur_start = cur_end;
      cur_end = __shfl_sync(gmask, rel, gbase + cur + 1);
      if (win + cur >= p.N) { cur_start = kRelInf; cur_end = kRelInf; }  // past the last row: nothing more closes
    };

    // ---- the ring: every lane copies the packs of its own group's entries, kWalkRing entries ahead ----------------
    const int row_elems = (int)p.K;
    const T *next_ptr = bsrc + (cs + ps) * p.K + c * VEC;
    const T *perm_col = bsrc + c * VEC;
    // INDIRECT: lane j of the group holds the source entry of position (window start + j); two windows are kept
    int pw0 = 0, pw1 = 0;
    auto load_perm_window = [&](int first) -> int {
      const int q = first + col;
      int v = (q < my_n) ? p.perm[cs + ps + q] : 0;
      const int last = (int)p.E - 1;
      return v < 0 ? 0 : (v > last ? last : v);
    };
    if (INDIRECT) { pw0 = load_perm_window(0); pw1 = load_perm_window(L); }
    int next_step = 0;
    auto issue = [&](int into) {
      if (INDIRECT) {
        if (next_step > 0 && (next_step & (L - 1)) == 0) { pw0 = pw1; pw1 = load_perm_window(next_step + L); }
        const int id = __shfl_sync(kFullMask, pw0, gbase + (next_step & (L - 1)));
        if (col_ok && next_step < my_n) {
          async_copy_pack<T, VEC>(&s_ring[into][lane], perm_col + (int64_t)id * row_elems);
          if (kArg) s_id[into][lane] = id;
        }
      } else {
        if (col_ok && next_step < my_n) async_copy_pack<T, VEC>(&s_ring[into][lane], next_ptr);
        next_ptr += p.K;
      }
      async_commit();
      ++next_step;
    };
#pragma unroll
    for (int j = 0; j < kWalkRing; ++j) issue(j);

    int slot = 0;
    for (int step = 0; step < piece; ++step) {   // warp-uniform trip count
      async_wait_all_but<kWalkRing - 1>();
      const int e = ps + step;
      if (step < my_n) {
        while (cur_end <= e) close_row();
        const Pack<T, VEC> v = s_ring[slot][lane];
        const int id = (INDIRECT && kArg) ? s_id[slot][lane] : e;
        if (e >= cur_start) acc.template update<INDIRECT>(v, id, kRelInf);
      }
      issue(slot);
      slot = (slot + 1 == kWalkRing) ? 0 : slot + 1;
    }
    async_wait_all_but<0>();
    while (cur_end <= pe) close_row();   // rows that end exactly at the piece's end, empty ones included

    // ---- settle the rows that run over piece borders ---------------------------------------------------------------
    // tail: the row still open at the end of this piece (acc holds what this piece saw of it)
    const bool tail_open = (win + cur < p.N) && cur_start < pe;
    const bool tail_fresh = tail_open && cur_start >= ps;   // it began inside this piece
    Acc carry_in;
    carry_in.init(kRelInf);
    for (int q = 1; q < eps; ++q) {   // warp-uniform: group q takes over from group q - 1
      A oval[VEC];
      int oarg[Acc::kPair ? VEC : 1];
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        oval[i] = __shfl_up_sync(kFullMask, acc.val[i], L);
        if (Acc::kPair) oarg[i] = __shfl_up_sync(kFullMask, acc.arg[i], L);
      }
      const int prev_open = __shfl_up_sync(kFullMask, (int)tail_open, L);
      if (sub == q && prev_open) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          carry_in.val[i] = oval[i];
          if (Acc::kPair) carry_in.arg[i] = oarg[i];
        }
        if (tail_open && !tail_fresh) {   // the same row runs on through this whole piece: earlier pieces first
          Acc merged = carry_in;
          merged.merge(acc.val, acc.arg);
          acc = merged;
        }
      }
    }
    if (head_row >= 0) {
      Acc total = carry_in;   // the earlier pieces' share (identity if the row began before the chunk in piece 0)
      total.merge(head.val, head.arg);
      if (head_from_before_chunk) {
        // the row began in an earlier chunk: leave this chunk's share for the fix-up kernel
        if (col_ok) {
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            carry[c * VEC + i] = total.val[i];
            if (kArg) carry_arg[c * VEC + i] = total.arg[i] == kRelInf ? p.E : (INDIRECT ? 0 : cs) + total.arg[i];
            if (Acc::kLseAcc) carry_arg[c * VEC + i] = total.arg[i];
          }
        }
        if (col == 0 && cb == 0) g.head_row[chunk_id] = head_row;
      } else {
        const int64_t grow = b * p.N + head_row;
        if (col_ok && !store_wide_routed<T, REDUCE, VEC, EXTRAS, int>(p, total, grow, c * VEC)) {
          write_row<T, REDUCE, VEC, int>(total, row_address<T, REDUCE, EXTRAS>(p, grow, c * VEC),
                                         kArg ? p.arg_out + grow * p.K + c * VEC : nullptr, (int64_t)head_len, p.mode, p.E,
                                         INDIRECT ? 0 : cs, kRelInf);
        }
        if (col == 0 && cb == 0 && p.count_out != nullptr)
          static_cast<T *>(p.count_out)[grow] = from_acc<T>((A)(head_len > 0 ? head_len : 1));
      }
    }
    // the row still open at the chunk's end runs on into the next chunk: store what this chunk holds of it
    if (sub == eps - 1 && tail_open && col_ok) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        carry[p.K + c * VEC + i] = acc.val[i];
        if (kArg) carry_arg[p.K + c * VEC + i] = acc.arg[i] == kRelInf ? p.E : (INDIRECT ? 0 : cs) + acc.arg[i];
        if (Acc::kLseAcc) carry_arg[p.K + c * VEC + i] = acc.arg[i];
      }
    }
  }
}


template <typename T, int REDUCE, int VEC, int MODE>
void launch_one(const CsrParams &p, const CsrGeom &g, unsigned total_chunks, cudaStream_t stream) {
  constexpr bool kIds = MODE >= 1 && (REDUCE == kMin || REDUCE == kMax);
  const size_t smem = sizeof(Pack<T, VEC>) * kWalkRing * 32 + (kIds ? sizeof(int) * kWalkRing * 32 : 0);
  csr_walk_kernel<T, REDUCE, VEC, MODE><<<total_chunks, 32, smem, stream>>>(p, g);
}

template <typename T, int REDUCE>
bool launch_reduce(const CsrParams &p, const CsrGeom &g, unsigned total_chunks, bool wide, int mode, cudaStream_t stream) {
  constexpr int kFull = full_vec<T>();
  if constexpr (kFull == 1) return false;   // element-by-element types stream
  if (wide) {
    if constexpr (std::is_same<T, float>::value && (REDUCE == kSum || REDUCE == kMean)) {
      if (mode == 0) { launch_one<T, REDUCE, 2 * kFull, 0>(p, g, total_chunks, stream); return true; }
    }
    return false;
  }
  if constexpr (REDUCE == kMul) {          // products exist for scatter only: through the permutation, whole problem
    if (mode == 1) { launch_one<T, REDUCE, kFull, 1>(p, g, total_chunks, stream); return true; }
    return false;
  } else if constexpr (REDUCE == kLse) {   // contiguous source only
    if (mode == 0) { launch_one<T, REDUCE, kFull, 0>(p, g, total_chunks, stream); return true; }
    return false;
  } else {
    if (mode == 0) launch_one<T, REDUCE, kFull, 0>(p, g, total_chunks, stream);
    else if (mode == 1) launch_one<T, REDUCE, kFull, 1>(p, g, total_chunks, stream);
    else launch_one<T, REDUCE, kFull, 2>(p, g, total_chunks, stream);
    return true;
  }
}

}  // namespace

bool launch_csr_walk(const CsrParams &p, const void *geom, unsigned total_chunks, int dtype, int reduce, bool wide, int mode,
                     cudaStream_t stream) {
  const CsrGeom &g = *static_cast<const CsrGeom *>(geom);
  return TSB_DISPATCH_DTYPE(dtype, [&]() -> int {
    switch (reduce) {
      case TSB_SUM: return launch_reduce<scalar_t, kSum>(p, g, total_chunks, wide, mode, stream);
      case TSB_MEAN: return launch_reduce<scalar_t, kMean>(p, g, total_chunks, wide, mode, stream);
      case TSB_MIN: return launch_reduce<scalar_t, kMin>(p, g, total_chunks, wide, mode, stream);
      case TSB_MAX: return launch_reduce<scalar_t, kMax>(p, g, total_chunks, wide, mode, stream);
      case TSB_MUL: return launch_reduce<scalar_t, kMul>(p, g, total_chunks, wide, mode, stream);
      case TSB_LSE:
        if constexpr (std::is_same<acc_t<scalar_t>, float>::value) return launch_reduce<scalar_t, kLse>(p, g, total_chunks, wide, mode, stream);
        else return 0;
      default: return 0;
    }
  }) > 0;
}

}  // namespace tsb
