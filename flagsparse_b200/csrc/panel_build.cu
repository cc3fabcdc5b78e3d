// Device-side construction of the panel layout (the regrouping that fsb_spmv_csr_panel multiplies from).
//
// A few passes over the matrix, each one kernel, so that preparing a matrix costs tens of products instead of
// hundreds or thousands:
//   count   entries per (row block, column chunk), one CTA per row block, counted in shared memory
//   sort    every entry to its place in unit order -- units by (row block, chunk), inside a unit the entries keep
//           their CSR order (a stable counting sort: one CTA per row block walks its entries in tiles of 1024)
//   runs    statistics of the runs (consecutive entries of one row inside one unit): how many, the longest, how
//           many longer than 4 / 8 / 16 -- they decide the piece size and the kernel mode
//   core    (layouts with mostly one entry per row and unit) the single entries of every accumulator class fill
//           "core" pieces in which lane l only meets accumulators congruent to l modulo 32; the rest is copied out
//   cut     greedy cuts of every unit (or of its rest) into pieces of at most `slots` entries that never split a run
//   fill    one warp per piece: entries ordered by the shared-memory bank of their accumulator (stable), then
//           written to the interleaved slot positions the kernel loads from; unused slots get the spare accumulator
// The small tables in between (unit list, prefix sums, the final order of core and rest pieces) are made by the host
// code.  The result is bit-identical to the host-side reference builder (flagsparse_b200/panel.py: _build_slab,
// pack_pieces, pack_pieces_core).
#include <limits.h>

#include "fsb_common.cuh"

namespace fsb {

constexpr int kBuildThreads = 1024;
constexpr int kBuildWarps = kBuildThreads / 32;
constexpr int kBuildWindowSmall = 128; // distinct chunks a tile of 1024 consecutive entries may span: narrow bands
constexpr int kBuildWindowLarge = 640; // ... and wide ones (more table to clear and to scan per tile)
constexpr int kBuildMaxChunks = 32768; // the count pass keeps one counter per chunk in shared memory

__device__ __forceinline__ int warp_min_i(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <typename I>
__device__ __forceinline__ int chunk_of(I col, int chunk_cols) {
  return (int)((uint32_t)col / (uint32_t)chunk_cols);   // columns are below 2^31
}

// ---- count ---------------------------------------------------------------------------------------
template <typename I, typename P>
__global__ void __launch_bounds__(kBuildThreads, 1)
panel_count_kernel(const I* __restrict__ idx, const P* __restrict__ ptr, int64_t n_rows, int rb_rows, int chunk_cols,
                   int n_ch, int32_t* __restrict__ cnt) {
  extern __shared__ int32_t s_cnt[];
  const int tid = threadIdx.x, lane = tid & 31;
  const int64_t r0 = (int64_t)blockIdx.x * rb_rows;
  const int64_t r1 = (r0 + rb_rows) < n_rows ? (r0 + rb_rows) : n_rows;
  for (int i = tid; i < n_ch; i += kBuildThreads) s_cnt[i] = 0;
  __syncthreads();
  const int64_t e0 = (int64_t)ptr[r0], e1 = (int64_t)ptr[r1];
  constexpr int U = 4;                                  // tiles whose loads are in flight together
  for (int64_t base = e0; base < e1; base += U * kBuildThreads) {
    int c[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int64_t e = base + k * kBuildThreads + tid;
      c[k] = e < e1 ? chunk_of(idx[e], chunk_cols) : -1;
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const unsigned peers = __match_any_sync(0xffffffffu, c[k]);
      if (c[k] >= 0 && lane == __ffs(peers) - 1) atomicAdd(&s_cnt[c[k]], __popc(peers));
    }
  }
  __syncthreads();
  int32_t* out = cnt + (int64_t)blockIdx.x * n_ch;
  for (int i = tid; i < n_ch; i += kBuildThreads) out[i] = s_cnt[i];
}

// ---- sort ----------------------------------------------------------------------------------------
// unit_base[rb * n_ch + c] = position of the first entry of unit (rb, c) in the sorted arrays
template <typename V, typename I, typename P, int kBuildWindow>
__global__ void __launch_bounds__(kBuildThreads, 1)
panel_sort_kernel(const V* __restrict__ data, const I* __restrict__ idx, const P* __restrict__ ptr, int64_t n_rows,
                  int rb_rows, int chunk_cols, int n_ch, const int32_t* __restrict__ unit_base,
                  V* __restrict__ o_val, int32_t* __restrict__ o_row, int32_t* __restrict__ o_col,
                  int32_t* __restrict__ status) {
  extern __shared__ int32_t s_run[];                      // next free position of every unit of this row block
  // entries of (warp, chunk) in the tile, then their prefix over the warps; rows padded by one 32-bit word so that
  // a column (one chunk, all warps) falls into 32 different banks
  __shared__ uint16_t s_cntw[kBuildWarps][kBuildWindow + 2];
  __shared__ int32_t s_tile_base[kBuildWindow];
  __shared__ int s_min[kBuildWarps], s_max[kBuildWarps];
  __shared__ int s_tmin, s_tmax, s_fail;
  __shared__ long long s_tile_row;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t r0 = (int64_t)blockIdx.x * rb_rows;
  const int64_t r1 = (r0 + rb_rows) < n_rows ? (r0 + rb_rows) : n_rows;
  const int32_t* base_row = unit_base + (int64_t)blockIdx.x * n_ch;
  for (int i = tid; i < n_ch; i += kBuildThreads) s_run[i] = base_row[i];
  for (int i = tid; i < kBuildWarps * (kBuildWindow + 2); i += kBuildThreads) (&s_cntw[0][0])[i] = 0;
  if (tid == 0) {
    s_fail = 0;
    s_tile_row = r0;
  }
  __syncthreads();
  const int64_t e0 = (int64_t)ptr[r0], e1 = (int64_t)ptr[r1];
  // the next tile's column and value are requested while this tile is placed
  I col_next = (e0 + tid) < e1 ? idx[e0 + tid] : (I)0;
  V val_next = (e0 + tid) < e1 ? data[e0 + tid] : (V)0;
  for (int64_t base = e0; base < e1; base += kBuildThreads) {
    const int64_t e = base + tid;
    const bool live = e < e1;
    const I col = col_next;
    const V val_here = val_next;
    if (e + kBuildThreads < e1) {
      col_next = idx[e + kBuildThreads];
      val_next = data[e + kBuildThreads];
    }
    const int c = live ? chunk_of(col, chunk_cols) : INT_MAX;
    const int wm = warp_min_i(c);
    const int wx = -warp_min_i(live ? -c : 0);           // chunks are >= 0: a dead lane does not raise the maximum
    if (lane == 0) {
      s_min[warp] = wm;
      s_max[warp] = wx;
    }
    __syncthreads();
    if (warp == 0) {
      const int m = warp_min_i(s_min[lane]);
      const int x = -warp_min_i(-s_max[lane]);
      if (lane == 0) {
        s_tmin = m;
        s_tmax = x;
      }
    }
    __syncthreads();
    const int tmin = s_tmin;
    // chunks of the window this tile uses; only they are scanned below and cleared for the next tile
    const int span = (s_tmax - tmin + 1) < kBuildWindow ? (s_tmax - tmin + 1) : kBuildWindow;
    const int64_t tile_row = s_tile_row;
    const int b = live ? (c - tmin) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, b);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (live) {
      if (b >= kBuildWindow) s_fail = 1;
      else if (rank == 0) s_cntw[warp][b] = (uint16_t)__popc(peers);
    }
    __syncthreads();
    if (s_fail) break;                                   // the same answer for every thread
    // per chunk of the window: exclusive prefix of the 32 warps' counts (lane = source warp), then the unit's
    // running offset moves on by the total; warp w looks after chunks w, w + 32, ...
    for (int bin = warp; bin < span; bin += kBuildWarps) {
      const int mine = s_cntw[lane][bin];
      int incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int other = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += other;
      }
      s_cntw[lane][bin] = (uint16_t)(incl - mine);
      if (lane == 31 && incl > 0) {
        s_tile_base[bin] = s_run[tmin + bin];
        s_run[tmin + bin] += incl;
      }
    }
    __syncthreads();
    if (live) {
      const int64_t pos = (int64_t)s_tile_base[b] + s_cntw[warp][b] + rank;
      // the row that holds entry e: the last row r of the block with ptr[r] <= e.  It is not in front of the row
      // of the tile's first entry, and seldom far behind it: gallop from there, then bisect
      int64_t lo = tile_row, hi = r1 - 1;
      for (int64_t step = 32; lo + step < hi; step <<= 1) {
        if ((int64_t)ptr[lo + step] > e) {
          hi = lo + step - 1;
          break;
        }
        lo += step;
      }
      while (lo < hi) {
        const int64_t mid = (lo + hi + 1) >> 1;
        if ((int64_t)ptr[mid] <= e) lo = mid;
        else hi = mid - 1;
      }
      o_val[pos] = val_here;
      o_row[pos] = (int32_t)lo;
      o_col[pos] = (int32_t)col;
      if (tid == kBuildThreads - 1) s_tile_row = lo;   // the next tile's entries are in this row or behind it
    }
    __syncthreads();   // every read of the tables is done
    for (int bin = lane; bin < span; bin += 32) s_cntw[warp][bin] = 0;   // two barriers ahead of the next writes
  }
  if (s_fail && tid == 0) *status = 1;
}

// ---- runs ----------------------------------------------------------------------------------------
__device__ __forceinline__ bool run_starts_at(const int32_t* __restrict__ row, const int32_t* __restrict__ col,
                                              int64_t e, int chunk_cols) {
  if (e == 0) return true;
  return row[e] != row[e - 1] || chunk_of(col[e], chunk_cols) != chunk_of(col[e - 1], chunk_cols);
}

constexpr int kRunsScanLimit = 1 << 16;   // a run longer than this is longer than any piece anyway

// stats[0] = runs, [1] = longest run, [2..4] = runs longer than 4 / 8 / 16 entries.  Positions are kept relative
// to the CTA's first entry (32-bit: a CTA covers tiles_per_cta * 1024 entries, the look-back at most kRunsScanLimit).
__global__ void __launch_bounds__(kBuildThreads)
panel_runs_kernel(const int32_t* __restrict__ row, const int32_t* __restrict__ col, int64_t nnz, int chunk_cols,
                  int tiles_per_cta, unsigned long long* __restrict__ stats) {
  __shared__ int s_warp_last[kBuildWarps];
  __shared__ int s_before[kBuildWarps];
  __shared__ int s_carry;
  __shared__ unsigned long long s_acc[5];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t first = (int64_t)blockIdx.x * tiles_per_cta * kBuildThreads;
  if (first >= nnz) return;
  if (tid == 0) {
    int64_t p = first;
    int steps = 0;
    while (p > 0 && steps < kRunsScanLimit && !run_starts_at(row, col, p, chunk_cols)) { --p; ++steps; }
    s_carry = (int)(p - first);                         // <= 0: the start of the run that holds the first entry
  }
  if (tid < 5) s_acc[tid] = 0;
  __syncthreads();
  constexpr int kNone = INT_MIN;
  unsigned long long n_start = 0, g4 = 0, g8 = 0, g16 = 0;
  int mx = 0;
  for (int t = 0; t < tiles_per_cta; ++t) {
    const int rel = t * kBuildThreads + tid;
    const int64_t e = first + rel;
    const bool live = e < nnz;
    const bool st = live && run_starts_at(row, col, e, chunk_cols);
    int last = st ? rel : kNone;                        // the last start at or in front of this entry, within the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int other = __shfl_up_sync(0xffffffffu, last, o);
      if (lane >= o && other > last) last = other;
    }
    if (lane == 31) s_warp_last[warp] = last;
    __syncthreads();
    if (warp == 0) {                                    // s_before[w] = the last start in front of warp w
      int v = s_warp_last[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int other = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o && other > v) v = other;
      }
      const int carry = s_carry;
      int excl = __shfl_up_sync(0xffffffffu, v, 1);
      if (lane == 0 || excl < carry) excl = carry;
      s_before[lane] = excl;
    }
    __syncthreads();
    const int before = s_before[warp];
    if (last < before) last = before;
    if (live) {
      const int d = rel - last;                         // entries of the run in front of this one
      n_start += st ? 1 : 0;
      mx = d + 1 > mx ? d + 1 : mx;
      g4 += d == 4;
      g8 += d == 8;
      g16 += d == 16;
    }
    __syncthreads();   // every thread has read the carry and the warps' last starts
    if (tid == kBuildThreads - 1 && live) s_carry = last;   // read again only after the next tile's barrier
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    n_start += __shfl_xor_sync(0xffffffffu, n_start, o);
    g4 += __shfl_xor_sync(0xffffffffu, g4, o);
    g8 += __shfl_xor_sync(0xffffffffu, g8, o);
    g16 += __shfl_xor_sync(0xffffffffu, g16, o);
    const int om = __shfl_xor_sync(0xffffffffu, mx, o);
    mx = om > mx ? om : mx;
  }
  if (lane == 0) {
    atomicAdd(&s_acc[0], n_start);
    atomicMax(&s_acc[1], (unsigned long long)mx);
    atomicAdd(&s_acc[2], g4);
    atomicAdd(&s_acc[3], g8);
    atomicAdd(&s_acc[4], g16);
  }
  __syncthreads();
  if (tid == 0) {
    atomicAdd(&stats[0], s_acc[0]);
    atomicMax(&stats[1], s_acc[1]);
    atomicAdd(&stats[2], s_acc[2]);
    atomicAdd(&stats[3], s_acc[3]);
    atomicAdd(&stats[4], s_acc[4]);
  }
}

// ---- cut -----------------------------------------------------------------------------------------
// One thread per unit.  First call (piece_start == nullptr): piece_count[u] = pieces of unit u.  Second call:
// piece_start[unit_piece_ptr[u] + k] = first entry of the unit's k-th piece.  status: a run longer than a piece.
__global__ void __launch_bounds__(256)
panel_cut_kernel(const int32_t* __restrict__ row, const int32_t* __restrict__ unit_start, int n_units, int slots,
                 const int32_t* __restrict__ unit_piece_ptr, int32_t* __restrict__ piece_count,
                 int32_t* __restrict__ piece_start, int32_t* __restrict__ status) {
  const int u = blockIdx.x * 256 + threadIdx.x;
  if (u >= n_units) return;
  int64_t cur = unit_start[u];
  const int64_t end = unit_start[u + 1];
  int n = 0;
  while (cur < end) {
    if (piece_start != nullptr) piece_start[unit_piece_ptr[u] + n] = (int32_t)cur;
    ++n;
    const int64_t t = cur + slots;
    if (t >= end) break;
    int64_t p = t;                                       // back to the first entry of the run that holds entry t
    while (p > cur && row[p] == row[p - 1]) --p;
    if (p <= cur) {                                      // one run fills more than a piece
      *status = 2;
      break;
    }
    cur = p;
  }
  if (piece_count != nullptr) piece_count[u] = n;
}

// ---- fill ----------------------------------------------------------------------------------------
constexpr int kFillWarps = 8;

template <typename V>
__global__ void __launch_bounds__(kFillWarps * 32)
panel_fill_kernel(const V* __restrict__ s_val, const int32_t* __restrict__ s_row, const int32_t* __restrict__ s_col,
                  const int32_t* __restrict__ piece_start, const int32_t* __restrict__ unit_piece_ptr, int n_units,
                  const int32_t* __restrict__ unit_rb, const int32_t* __restrict__ unit_ord, int n_pieces,
                  int rb_rows, int chunk_cols, int n_buffers, int rounds, int banks, uint32_t pad_row,
                  V* __restrict__ val, uint32_t* __restrict__ rc) {
  __shared__ int s_bank[kFillWarps][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int p = blockIdx.x * kFillWarps + warp;
  if (p >= n_pieces) return;
  const int slots = 32 * rounds;
  const int64_t ps = piece_start[p];
  const int n = (int)(piece_start[p + 1] - ps);
  // the unit of this piece: the last u with unit_piece_ptr[u] <= p
  int lo = 0, hi = n_units - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (unit_piece_ptr[mid] <= p) lo = mid;
    else hi = mid - 1;
  }
  const int u = lo;
  const int rb = unit_rb[u];
  const int x_base = (unit_ord[u] % n_buffers) * chunk_cols;
  const int64_t row0 = (int64_t)rb * rb_rows;
  constexpr int E = 16 / (int)sizeof(V);
  int* bank_pos = s_bank[warp];
  bank_pos[lane] = 0;
  __syncwarp();
  // entries per bank, then the first slot of every bank
  for (int i0 = 0; i0 < n; i0 += 32) {
    const int i = i0 + lane;
    const bool live = i < n;
    const int bk = live ? (int)((s_row[ps + i] - row0) % banks) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, bk);
    if (live && lane == __ffs(peers) - 1) bank_pos[bk] += __popc(peers);
    __syncwarp();
  }
  {
    const int mine = bank_pos[lane];
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int other = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += other;
    }
    __syncwarp();
    bank_pos[lane] = incl - mine;
    __syncwarp();
  }
  const size_t piece_base = (size_t)p * slots;
  for (int i0 = 0; i0 < n; i0 += 32) {
    const int i = i0 + lane;
    const bool live = i < n;
    int acc = 0, col = 0;
    V v = (V)0;
    if (live) {
      acc = (int)(s_row[ps + i] - row0);
      col = s_col[ps + i];
      v = s_val[ps + i];
    }
    const int bk = live ? acc % banks : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, bk);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    const int s = live ? bank_pos[bk] + rank : 0;
    __syncwarp();
    if (live && rank == 0) bank_pos[bk] += __popc(peers);
    __syncwarp();
    if (live) {
      const int ln = s / rounds, k = s % rounds;
      val[piece_base + (size_t)(k / E) * (32 * E) + ln * E + k % E] = v;
      rc[piece_base + (size_t)(k >> 2) * 128 + ln * 4 + (k & 3)] =
          ((uint32_t)acc << 16) | (uint32_t)(x_base + (int)((uint32_t)col % (uint32_t)chunk_cols));
    }
  }
  for (int s = n + lane; s < slots; s += 32) {
    const int ln = s / rounds, k = s % rounds;
    val[piece_base + (size_t)(k / E) * (32 * E) + ln * E + k % E] = (V)0;
    rc[piece_base + (size_t)(k >> 2) * 128 + ln * 4 + (k & 3)] = pad_row << 16;
  }
}

// ---- core pieces ---------------------------------------------------------------------------------
// For layouts in which most rows have one entry per unit: the entries that are alone in their run ("singles") are
// listed per class (local row mod 32) in unit order; with J = (shortest list) / rounds, the first J * rounds singles of
// every class fill J core pieces of the unit completely (piece j takes entries j * rounds .. of every list, lane =
// class), so that the 32 accumulators of a round lie in 32 different banks.  Everything else (the "rest") keeps its
// order and is cut and filled like an ordinary unit.  One warp per unit, entries taken 32 at a time in unit order.
constexpr int kCoreWarps = 8;

__device__ __forceinline__ bool single_at(const int32_t* __restrict__ row, int64_t e, int64_t u0, int64_t u1) {
  const int32_t r = row[e];
  return (e == u0 || row[e - 1] != r) && (e + 1 == u1 || row[e + 1] != r);
}

__global__ void __launch_bounds__(kCoreWarps * 32)
panel_core_count_kernel(const int32_t* __restrict__ s_row, const int32_t* __restrict__ unit_start,
                        const int32_t* __restrict__ unit_rb, int n_units, int rb_rows, int rounds,
                        int32_t* __restrict__ core_pieces, int32_t* __restrict__ rest_count) {
  __shared__ int s_cls[kCoreWarps][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int u = blockIdx.x * kCoreWarps + warp;
  if (u >= n_units) return;
  const int64_t u0 = unit_start[u], u1 = unit_start[u + 1];
  const int64_t row0 = (int64_t)unit_rb[u] * rb_rows;
  int* cls_n = s_cls[warp];
  cls_n[lane] = 0;
  __syncwarp();
  for (int64_t e0 = u0; e0 < u1; e0 += 32) {
    const int64_t e = e0 + lane;
    int key = -1;
    if (e < u1 && single_at(s_row, e, u0, u1)) key = (int)((s_row[e] - row0) & 31);
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    if (key >= 0 && lane == __ffs(peers) - 1) cls_n[key] += __popc(peers);
    __syncwarp();
  }
  int m = cls_n[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = min(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) {
    const int j = m / rounds;
    core_pieces[u] = j;
    rest_count[u] = (int)(u1 - u0) - j * rounds * 32;
  }
}

template <typename V>
__global__ void __launch_bounds__(kCoreWarps * 32)
panel_core_place_kernel(const V* __restrict__ s_val, const int32_t* __restrict__ s_row,
                        const int32_t* __restrict__ s_col, const int32_t* __restrict__ unit_start,
                        const int32_t* __restrict__ unit_rb, const int32_t* __restrict__ unit_ord, int n_units,
                        int rb_rows, int chunk_cols, int n_buffers, int rounds,
                        const int32_t* __restrict__ core_pieces, const int32_t* __restrict__ core_base,
                        const int32_t* __restrict__ rest_start, V* __restrict__ core_val,
                        uint32_t* __restrict__ core_rc, V* __restrict__ rest_val, int32_t* __restrict__ rest_row,
                        int32_t* __restrict__ rest_col) {
  __shared__ int s_cls[kCoreWarps][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int u = blockIdx.x * kCoreWarps + warp;
  if (u >= n_units) return;
  const int64_t u0 = unit_start[u], u1 = unit_start[u + 1];
  const int64_t row0 = (int64_t)unit_rb[u] * rb_rows;
  const int x_base = (unit_ord[u] % n_buffers) * chunk_cols;
  const int core_entries = core_pieces[u] * rounds;          // per class
  const size_t piece0 = (size_t)core_base[u];
  const int slots = 32 * rounds;
  constexpr int E = 16 / (int)sizeof(V);
  int64_t rest_pos = rest_start[u];
  int* cls_pos = s_cls[warp];
  cls_pos[lane] = 0;
  __syncwarp();
  for (int64_t e0 = u0; e0 < u1; e0 += 32) {
    const int64_t e = e0 + lane;
    const bool live = e < u1;
    int key = -1, acc = 0, col = 0;
    V v = (V)0;
    if (live) {
      acc = (int)(s_row[e] - row0);
      col = s_col[e];
      v = s_val[e];
      if (single_at(s_row, e, u0, u1)) key = acc & 31;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    const int rank = key >= 0 ? cls_pos[key] + __popc(peers & ((1u << lane) - 1u)) : 0;
    __syncwarp();
    if (key >= 0 && lane == __ffs(peers) - 1) cls_pos[key] += __popc(peers);
    __syncwarp();
    const bool core = key >= 0 && rank < core_entries;
    const unsigned rest_mask = __ballot_sync(0xffffffffu, live && !core);
    if (core) {
      const int k = rank % rounds;
      const size_t base = (piece0 + (size_t)(rank / rounds)) * slots;
      core_val[base + (size_t)(k / E) * (32 * E) + key * E + k % E] = v;
      core_rc[base + (size_t)(k >> 2) * 128 + key * 4 + (k & 3)] =
          ((uint32_t)acc << 16) | (uint32_t)(x_base + (int)((uint32_t)col % (uint32_t)chunk_cols));
    } else if (live) {
      const int64_t at = rest_pos + __popc(rest_mask & ((1u << lane) - 1u));
      rest_val[at] = v;
      rest_row[at] = s_row[e];
      rest_col[at] = col;
    }
    rest_pos += __popc(rest_mask);
  }
}

static bool build_types_ok(int vtype, int itype, int ptype) {
  return (vtype == FSB_F32 || vtype == FSB_F64) && (itype == FSB_I32 || itype == FSB_I64) &&
         (ptype == FSB_I32 || ptype == FSB_I64);
}

}  // namespace fsb

using namespace fsb;

extern "C" int fsb_panel_build_max_chunks(void) { return kBuildMaxChunks; }

extern "C" int fsb_panel_build_count(int itype, int ptype, const void* indices, const void* indptr, int64_t n_rows,
                                     int64_t n_cols, int32_t rb_rows, int32_t chunk_cols, int32_t* cnt, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (!build_types_ok(FSB_F32, itype, ptype) || n_rows < 0 || n_cols < 0 || rb_rows <= 0 || chunk_cols <= 0)
    return FSB_EINVAL;
  if (n_rows == 0) return FSB_OK;
  if (!indices || !indptr || !cnt) return FSB_EINVAL;
  const int64_t n_ch = (n_cols + chunk_cols - 1) / chunk_cols;
  const int64_t n_rb = (n_rows + rb_rows - 1) / rb_rows;
  if (n_ch > kBuildMaxChunks || n_rb >= INT32_MAX || n_cols >= INT32_MAX) return FSB_ERANGE;
  const size_t smem = (size_t)n_ch * sizeof(int32_t);
#define FSB_COUNT_(I_, P_)                                                                                        \
  do {                                                                                                            \
    cudaError_t e = cudaFuncSetAttribute(panel_count_kernel<I_, P_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int)smem);                                                              \
    if (e != cudaSuccess) return cuda_rc(e);                                                                      \
    panel_count_kernel<I_, P_><<<(unsigned)n_rb, kBuildThreads, smem, st>>>(                                      \
        (const I_*)indices, (const P_*)indptr, n_rows, rb_rows, chunk_cols, (int)n_ch, cnt);                      \
  } while (0)
  if (itype == FSB_I32 && ptype == FSB_I32) FSB_COUNT_(int32_t, int32_t);
  else if (itype == FSB_I32) FSB_COUNT_(int32_t, int64_t);
  else if (ptype == FSB_I32) FSB_COUNT_(int64_t, int32_t);
  else FSB_COUNT_(int64_t, int64_t);
#undef FSB_COUNT_
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}

extern "C" int fsb_panel_build_sort(int vtype, int itype, int ptype, const void* data, const void* indices,
                                    const void* indptr, int64_t n_rows, int64_t n_cols, int32_t rb_rows,
                                    int32_t chunk_cols, int32_t wide_window, const int32_t* unit_base, void* sorted_val,
                                    int32_t* sorted_row, int32_t* sorted_col, int32_t* status, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (!build_types_ok(vtype, itype, ptype) || n_rows < 0 || n_cols < 0 || rb_rows <= 0 || chunk_cols <= 0)
    return FSB_EINVAL;
  if (n_rows == 0) return FSB_OK;
  if (!data || !indices || !indptr || !unit_base || !sorted_val || !sorted_row || !sorted_col || !status)
    return FSB_EINVAL;
  const int64_t n_ch = (n_cols + chunk_cols - 1) / chunk_cols;
  const int64_t n_rb = (n_rows + rb_rows - 1) / rb_rows;
  if (n_ch > kBuildMaxChunks || n_rb >= INT32_MAX || n_cols >= INT32_MAX) return FSB_ERANGE;
  const size_t smem = (size_t)n_ch * sizeof(int32_t);
#define FSB_SORT_W_(V_, I_, P_, W_)                                                                                  \
  do {                                                                                                               \
    cudaError_t e = cudaFuncSetAttribute(panel_sort_kernel<V_, I_, P_, W_>,                                          \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                    \
    if (e != cudaSuccess) return cuda_rc(e);                                                                         \
    panel_sort_kernel<V_, I_, P_, W_><<<(unsigned)n_rb, kBuildThreads, smem, st>>>(                                  \
        (const V_*)data, (const I_*)indices, (const P_*)indptr, n_rows, rb_rows, chunk_cols, (int)n_ch, unit_base,   \
        (V_*)sorted_val, sorted_row, sorted_col, status);                                                            \
  } while (0)
#define FSB_SORT_(V_, I_, P_)                                      \
  do {                                                             \
    if (wide_window) FSB_SORT_W_(V_, I_, P_, kBuildWindowLarge);   \
    else FSB_SORT_W_(V_, I_, P_, kBuildWindowSmall);               \
  } while (0)
#define FSB_SORT_V_(V_)                                              \
  do {                                                               \
    if (itype == FSB_I32 && ptype == FSB_I32) FSB_SORT_(V_, int32_t, int32_t); \
    else if (itype == FSB_I32) FSB_SORT_(V_, int32_t, int64_t);      \
    else if (ptype == FSB_I32) FSB_SORT_(V_, int64_t, int32_t);      \
    else FSB_SORT_(V_, int64_t, int64_t);                            \
  } while (0)
  if (vtype == FSB_F32) FSB_SORT_V_(float);
  else FSB_SORT_V_(double);
#undef FSB_SORT_V_
#undef FSB_SORT_
#undef FSB_SORT_W_
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}

extern "C" int fsb_panel_build_runs(const int32_t* sorted_row, const int32_t* sorted_col, int64_t nnz,
                                    int32_t chunk_cols, int64_t* stats, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (nnz < 0 || chunk_cols <= 0 || !stats) return FSB_EINVAL;
  cudaError_t e = cudaMemsetAsync(stats, 0, 5 * sizeof(int64_t), st);
  if (e != cudaSuccess) return cuda_rc(e);
  if (nnz == 0) return FSB_OK;
  if (!sorted_row || !sorted_col) return FSB_EINVAL;
  const int tiles_per_cta = 16;
  const int64_t per_cta = (int64_t)tiles_per_cta * kBuildThreads;
  const int64_t g = (nnz + per_cta - 1) / per_cta;
  if (g >= INT32_MAX) return FSB_ERANGE;
  panel_runs_kernel<<<(unsigned)g, kBuildThreads, 0, st>>>(sorted_row, sorted_col, nnz, chunk_cols, tiles_per_cta,
                                                           reinterpret_cast<unsigned long long*>(stats));
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}

extern "C" int fsb_panel_build_cut(const int32_t* sorted_row, const int32_t* unit_start, int32_t n_units, int32_t slots,
                                   const int32_t* unit_piece_ptr, int32_t* piece_count, int32_t* piece_start,
                                   int32_t* status, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (n_units < 0 || slots <= 0 || !status) return FSB_EINVAL;
  if (n_units == 0) return FSB_OK;
  if (!sorted_row || !unit_start || (piece_start != nullptr && unit_piece_ptr == nullptr) ||
      (piece_start == nullptr && piece_count == nullptr))
    return FSB_EINVAL;
  panel_cut_kernel<<<(unsigned)((n_units + 255) / 256), 256, 0, st>>>(sorted_row, unit_start, n_units, slots,
                                                                      unit_piece_ptr, piece_count, piece_start, status);
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}

extern "C" int fsb_panel_build_fill(int vtype, const void* sorted_val, const int32_t* sorted_row,
                                    const int32_t* sorted_col, const int32_t* piece_start,
                                    const int32_t* unit_piece_ptr, int32_t n_units, const int32_t* unit_rb,
                                    const int32_t* unit_ord, int32_t n_pieces, int32_t rb_rows, int32_t chunk_cols,
                                    int32_t n_buffers, int32_t rounds, void* val, uint32_t* rc, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (vtype != FSB_F32 && vtype != FSB_F64) return FSB_EINVAL;
  if (n_units < 0 || n_pieces < 0 || rb_rows <= 0 || rb_rows >= 65535 || chunk_cols <= 0 || n_buffers < 1) return FSB_EINVAL;
  if (rounds != 4 && rounds != 8 && rounds != 16) return FSB_EINVAL;
  if ((int64_t)n_buffers * chunk_cols > 65536) return FSB_EINVAL;
  if (n_pieces == 0) return FSB_OK;
  if (!sorted_val || !sorted_row || !sorted_col || !piece_start || !unit_piece_ptr || !unit_rb || !unit_ord ||
      !val || !rc)
    return FSB_EINVAL;
  const unsigned g = (unsigned)((n_pieces + kFillWarps - 1) / kFillWarps);
  if (vtype == FSB_F32)
    panel_fill_kernel<float><<<g, kFillWarps * 32, 0, st>>>(
        (const float*)sorted_val, sorted_row, sorted_col, piece_start, unit_piece_ptr, n_units, unit_rb, unit_ord,
        n_pieces, rb_rows, chunk_cols, n_buffers, rounds, 32, (uint32_t)rb_rows, (float*)val, rc);
  else
    panel_fill_kernel<double><<<g, kFillWarps * 32, 0, st>>>(
        (const double*)sorted_val, sorted_row, sorted_col, piece_start, unit_piece_ptr, n_units, unit_rb, unit_ord,
        n_pieces, rb_rows, chunk_cols, n_buffers, rounds, 16, (uint32_t)rb_rows, (double*)val, rc);
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}

extern "C" int fsb_panel_build_window(int wide) { return wide ? kBuildWindowLarge : kBuildWindowSmall; }

extern "C" int fsb_panel_build_core_count(const int32_t* sorted_row, const int32_t* unit_start, const int32_t* unit_rb,
                                          int32_t n_units, int32_t rb_rows, int32_t rounds, int32_t* core_pieces,
                                          int32_t* rest_count, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (n_units < 0 || rb_rows <= 0 || (rounds != 4 && rounds != 8 && rounds != 16)) return FSB_EINVAL;
  if (n_units == 0) return FSB_OK;
  if (!sorted_row || !unit_start || !unit_rb || !core_pieces || !rest_count) return FSB_EINVAL;
  panel_core_count_kernel<<<(unsigned)((n_units + kCoreWarps - 1) / kCoreWarps), kCoreWarps * 32, 0, st>>>(
      sorted_row, unit_start, unit_rb, n_units, rb_rows, rounds, core_pieces, rest_count);
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}

extern "C" int fsb_panel_build_core_place(int vtype, const void* sorted_val, const int32_t* sorted_row,
                                          const int32_t* sorted_col, const int32_t* unit_start, const int32_t* unit_rb,
                                          const int32_t* unit_ord, int32_t n_units, int32_t rb_rows, int32_t chunk_cols,
                                          int32_t n_buffers, int32_t rounds, const int32_t* core_pieces,
                                          const int32_t* core_base, const int32_t* rest_start, void* core_val,
                                          uint32_t* core_rc, void* rest_val, int32_t* rest_row, int32_t* rest_col,
                                          void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (vtype != FSB_F32 && vtype != FSB_F64) return FSB_EINVAL;
  if (n_units < 0 || rb_rows <= 0 || rb_rows >= 65535 || chunk_cols <= 0 || n_buffers < 1) return FSB_EINVAL;
  if ((rounds != 4 && rounds != 8 && rounds != 16) || (int64_t)n_buffers * chunk_cols > 65536) return FSB_EINVAL;
  if (n_units == 0) return FSB_OK;
  if (!sorted_val || !sorted_row || !sorted_col || !unit_start || !unit_rb || !unit_ord || !core_pieces || !core_base ||
      !rest_start || !core_val || !core_rc || !rest_val || !rest_row || !rest_col)
    return FSB_EINVAL;
  const unsigned g = (unsigned)((n_units + kCoreWarps - 1) / kCoreWarps);
  if (vtype == FSB_F32)
    panel_core_place_kernel<float><<<g, kCoreWarps * 32, 0, st>>>(
        (const float*)sorted_val, sorted_row, sorted_col, unit_start, unit_rb, unit_ord, n_units, rb_rows, chunk_cols,
        n_buffers, rounds, core_pieces, core_base, rest_start, (float*)core_val, core_rc, (float*)rest_val, rest_row,
        rest_col);
  else
    panel_core_place_kernel<double><<<g, kCoreWarps * 32, 0, st>>>(
        (const double*)sorted_val, sorted_row, sorted_col, unit_start, unit_rb, unit_ord, n_units, rb_rows, chunk_cols,
        n_buffers, rounds, core_pieces, core_base, rest_start, (double*)core_val, core_rc, (double*)rest_val, rest_row,
        rest_col);
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}
