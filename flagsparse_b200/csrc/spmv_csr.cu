// CSR SpMV for sm_100a: a lanes-per-row "vector" kernel and an nnz-tiled "stream" kernel.
//
// Stream kernel (the load-balanced one).  The nnz range is cut into tiles of T = 256*IPT entries, so
// every tile starts on a 16-byte boundary of `data` and `indices` whatever the row structure is and is
// read with fully coalesced 128-bit streaming loads.  A CTA owns one tile:
//   A  load IPT values + IPT column indices per thread, gather x through the read-only path, multiply,
//      park the products in shared memory;
//   B  load indptr[ra .. rb] (ra, rb from the tile plan) as tile-relative offsets into shared memory;
//   C  segmented reduction: groups of L lanes (L = power of two picked per tile from its mean row
//      length) each sum one row's slice of the products and finish with a shuffle tree; rows that are
//      much longer than the tile's mean are deferred to a second pass that gives them a full warp and
//      a double-precision accumulator.
// Rows that end in the tile are written to y.  The one row that may continue into the next tile leaves
// its partial sum in carry[t]; the one row that may have started before the tile leaves its partial sum
// in head[t] instead of y.  A second tiny kernel (one thread per tile) adds head[t] and the carries of
// the tiles the row crossed, in a fixed order, and writes y -- no floating-point atomics anywhere, so
// the result is bit-reproducible.
#include <mutex>

#include "fsb_common.cuh"

namespace fsb {

constexpr int kThreads = 256;

// ---------------------------------------------------------------------------------------------------
// output policies: plain local y, or the same value stored to every peer's y (row-sharded driver)
// ---------------------------------------------------------------------------------------------------
template <typename V>
struct LocalOut {
  static constexpr bool kStaged = false;  // local stores of scattered rows are cheap enough
  V* y;
  __device__ __forceinline__ void store(int64_t i, V v) const { y[i] = v; }
  // rows row0+first .. row0+last-1 from a shared-memory staging array, thread-strided
  __device__ __forceinline__ void store_block(int64_t row0, const V* src, int first, int last, int tid) const {
    for (int i = first + tid; i < last; i += kThreads) y[row0 + i] = src[i];
  }
};
template <typename V>
struct PeerOut {
  static constexpr bool kStaged = true;   // every row goes to n_peers destinations: make the stores coalesced
  V* const* peers;
  int n_peers;
  int64_t row_offset;
  int first_peer;                          // this GPU's index: destinations are taken in an order rotated by it
  // Destination visited k-th by this CTA.  Rotating by the GPU's own index and by the CTA keeps the GPUs (and the
  // CTAs of one GPU) from all writing to the same destination at the same moment.
  __device__ __forceinline__ int dest(int k) const {
    return (int)(((unsigned)first_peer + 1u + blockIdx.x + (unsigned)k) % (unsigned)n_peers);
  }
  __device__ __forceinline__ void store(int64_t i, V v) const {
    for (int k = 0; k < n_peers; ++k) peers[dest(k)][row_offset + i] = v;
  }
  __device__ __forceinline__ void store_block(int64_t row0, const V* src, int first, int last, int tid) const {
    for (int k = 0; k < n_peers; ++k) {
      V* dst = peers[dest(k)] + row_offset + row0;
      for (int i = first + tid; i < last; i += kThreads) dst[i] = src[i];
    }
  }
};

// ---------------------------------------------------------------------------------------------------
// vector kernel: L lanes per row.
//   ALIGNED: every lane reads whole 4-element groups of `data` / `indices` (one or two 128-bit loads
//            each) starting at the group that contains the row's first entry; entries of neighbouring rows
//            that share the first or last group are masked off.  A row of 32 entries then costs two or three
//            requests per array instead of one per eight entries.
//   otherwise: scalar loads, used when the arrays are not 16-byte aligned.
// ---------------------------------------------------------------------------------------------------
template <typename V, typename I, typename P, int L, bool ALIGNED, typename Out>
__global__ void __launch_bounds__(kThreads) spmv_vector_kernel(const V* __restrict__ data,
                                                              const I* __restrict__ idx,
                                                              const P* __restrict__ ptr,
                                                              const V* __restrict__ x, Out out,
                                                              int64_t n_rows, int64_t nnz) {
  const int64_t gtid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  const int64_t row = gtid / L;
  const int lane = (int)(gtid % L);
  int64_t s = 0, e = 0;
  if (row < n_rows) {
    s = (int64_t)ptr[row];
    e = (int64_t)ptr[row + 1];
  }
  V acc0 = 0, acc1 = 0;
  if (ALIGNED) {
    const int64_t full = nnz & ~(int64_t)3;  // groups below this index lie wholly inside the arrays
    for (int64_t q = (s & ~(int64_t)3) + 4 * lane; q < e; q += 4 * L) {
      V a[4];
      I c[4];
      if (q + 4 <= full) {
        ld_stream4(data + q, a);
        ld_stream4(idx + q, c);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          a[j] = (q + j < nnz) ? data[q + j] : (V)0;
          c[j] = (q + j < nnz) ? idx[q + j] : (I)0;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int64_t pp = q + j;
        if (pp >= s && pp < e) {
          if (j & 1) acc1 += a[j] * __ldg(x + (int64_t)c[j]);
          else acc0 += a[j] * __ldg(x + (int64_t)c[j]);
        }
      }
    }
  } else {
    int64_t p = s + lane;
    for (; p + L < e; p += 2 * L) {
      const V a0 = ld_stream(data + p), a1 = ld_stream(data + p + L);
      const int64_t c0 = (int64_t)ld_stream(idx + p), c1 = (int64_t)ld_stream(idx + p + L);
      acc0 += a0 * __ldg(x + c0);
      acc1 += a1 * __ldg(x + c1);
    }
    if (p < e) acc0 += ld_stream(data + p) * __ldg(x + (int64_t)ld_stream(idx + p));
  }
  V acc = acc0 + acc1;
#pragma unroll
  for (int o = L >> 1; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
  if (lane == 0 && row < n_rows) out.store(row, acc);
}

// ---------------------------------------------------------------------------------------------------
// stream kernel
// ---------------------------------------------------------------------------------------------------
template <typename V>
struct Wide { typedef double type; };  // accumulator of the long-row pass and of the fix-up

template <typename V, typename I, typename P, int IPT, bool VEC, typename Out>
__global__ void __launch_bounds__(kThreads)
spmv_stream_kernel(const V* __restrict__ data, const I* __restrict__ idx, const P* __restrict__ ptr,
                   const V* __restrict__ x, Out out, const int32_t* __restrict__ tile_row,
                   V* __restrict__ carry, V* __restrict__ head, int64_t nnz, int lane_shift) {
  constexpr int T = kThreads * IPT;
  // segments handled per pass (offsets kept in shared memory: RC + 1); smaller where 48 KB would not hold it
  constexpr int RC = (T >= 4096 && sizeof(V) == 8) ? 1024 : (T < 2048 ? T : 2048);
  constexpr bool STAGED = Out::kStaged;  // collect finished rows in shared memory and write them out coalesced
  constexpr int LONG_CAP = T / 32 + 2;
  constexpr int HUGE_LEN = 512;               // segments longer than this are summed by the whole CTA
  constexpr int HUGE_CAP = T / HUGE_LEN + 2;
  constexpr int NW = kThreads / 32;
  typedef typename Wide<V>::type W;
  __shared__ __align__(16) V s_prod[T];
  __shared__ int32_t s_off[RC + 1];
  __shared__ V s_y[STAGED ? RC : 1];  // results of the rows that end in this tile (staged write-out only)
  __shared__ int32_t s_long[LONG_CAP];
  __shared__ int32_t s_huge[HUGE_CAP];
  __shared__ W s_part[HUGE_CAP][NW];
  __shared__ int s_nlong;
  __shared__ int s_nhuge;
  __shared__ int s_head_partial;

  const int tid = threadIdx.x;
  const int64_t t = blockIdx.x;
  const int64_t lo = t * (int64_t)T;
  const int cnt = (int)((nnz - lo) < (int64_t)T ? (nnz - lo) : (int64_t)T);
  const int32_t ra = tile_row[t];
  const int32_t rb = tile_row[t + 1];

  // segments = rows ending here (ra..rb-1) + the row that continues (tail)
  const int nrf = rb - ra;
  const int nseg = nrf + 1;
  // offsets of the segments [base, base + m] of this tile, relative to the tile, into shared memory
  auto load_offsets = [&](int base, int m) {
    for (int k = tid; k <= m; k += kThreads) {
      const int g = base + k;  // offset entry g: start of segment g
      int32_t o = cnt;         // g == nseg: end of the tail segment
      if (g <= nrf) {
        const int64_t d = (int64_t)ptr[(int64_t)ra + g] - lo;
        o = d < 0 ? 0 : (d > cnt ? cnt : (int32_t)d);
        if (g == 0) s_head_partial = (d < 0 && nrf > 0) ? 1 : 0;
      }
      s_off[k] = o;
    }
    if (tid == 0) {
      s_nlong = 0;
      s_nhuge = 0;
    }
  };
  const int m0 = nseg < RC ? nseg : RC;

  // ---- A: products into shared memory (the first pass of offsets is fetched while the gathers fly) -----
  if (VEC && cnt == T) {
    V v[IPT];
    I c[IPT];
#pragma unroll
    for (int j = 0; j < IPT / 4; ++j) {
      const int64_t e = lo + (int64_t)(j * kThreads + tid) * 4;
      ld_stream4(data + e, *reinterpret_cast<V(*)[4]>(&v[4 * j]));
      ld_stream4(idx + e, *reinterpret_cast<I(*)[4]>(&c[4 * j]));
    }
    if (rb != ra) load_offsets(0, m0);
#pragma unroll
    for (int k = 0; k < IPT; ++k) v[k] *= __ldg(x + (int64_t)c[k]);
    if (rb == ra) {
      // The whole tile lies inside one row (no row ends here): its sum is the carry.  Reduce straight from
      // registers -- lane, then warp, then the eight warp sums in order -- and skip the staging altogether.
      W acc = 0;
#pragma unroll
      for (int k = 0; k < IPT; ++k) acc += (W)v[k];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
      if ((tid & 31) == 0) s_part[0][tid >> 5] = acc;
      __syncthreads();
      if (tid == 0) {
        W tot = 0;
#pragma unroll
        for (int q = 0; q < NW; ++q) tot += s_part[0][q];
        carry[t] = (V)tot;
      }
      return;
    }
#pragma unroll
    for (int j = 0; j < IPT / 4; ++j)
      st_shared4(&s_prod[(j * kThreads + tid) * 4], *reinterpret_cast<V(*)[4]>(&v[4 * j]));
  } else {
    load_offsets(0, m0);
    for (int e = tid; e < cnt; e += kThreads)
      s_prod[e] = ld_stream(data + lo + e) * __ldg(x + (int64_t)ld_stream(idx + lo + e));
  }

  // ---- C: segmented reduction ------------------------------------------------------------------------
  int L;
  {
    const int mean = cnt / nseg;
    L = pow2_floor(mean >> lane_shift);
    L = L > 32 ? 32 : L;
  }
  const int lane = tid & (L - 1);
  const int grp = tid / L;
  const int ngrp = kThreads / L;
  const int long_len = 32 * L;

  for (int base = 0; base < nseg; base += RC) {
    const int m = (nseg - base) < RC ? (nseg - base) : RC;  // segments in this pass
    if (base > 0) {
      __syncthreads();  // previous pass done with s_off / s_long / s_huge
      load_offsets(base, m);
    }
    __syncthreads();  // products and offsets visible

    // pass 1: L lanes per segment
    const int iters = (m + ngrp - 1) / ngrp;
    for (int it = 0; it < iters; ++it) {
      const int k = it * ngrp + grp;
      const bool valid = k < m;
      int s = 0, e = 0;
      if (valid) {
        s = s_off[k];
        e = s_off[k + 1];
      }
      const bool is_huge = e - s > HUGE_LEN;
      const bool is_long = is_huge || ((L < 32) && (e - s > long_len));
      V acc = 0;
      if (!is_long) {
        // four independent partial sums: four shared-memory loads in flight instead of a chain of single ones
        V a1 = 0, a2 = 0, a3 = 0;
        for (int p = s + lane; p < e; p += 4 * L) {
          acc += s_prod[p];
          if (p + L < e) a1 += s_prod[p + L];
          if (p + 2 * L < e) a2 += s_prod[p + 2 * L];
          if (p + 3 * L < e) a3 += s_prod[p + 3 * L];
        }
        acc = (acc + a1) + (a2 + a3);
      }
      for (int o = L >> 1; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
      if (valid && lane == 0) {
        if (is_huge) {
          s_huge[atomicAdd(&s_nhuge, 1)] = k;
        } else if (is_long) {
          s_long[atomicAdd(&s_nlong, 1)] = k;
        } else {
          const int g = base + k;
          if (g == nrf) carry[t] = acc;
          else if (g == 0 && s_head_partial) head[t] = acc;
          else if (STAGED) s_y[k] = acc;
          else out.store((int64_t)ra + g, acc);
        }
      }
    }
    __syncthreads();

    // pass 2: one warp per long segment, wide accumulators
    const int nlong = s_nlong;
    const int w = tid >> 5, l32 = tid & 31;
    for (int q = w; q < nlong; q += NW) {
      const int k = s_long[q];
      const int s = s_off[k], e = s_off[k + 1];
      W a0 = 0, a1 = 0;
      int p = s + l32;
      for (; p + 32 < e; p += 64) {
        a0 += (W)s_prod[p];
        a1 += (W)s_prod[p + 32];
      }
      if (p < e) a0 += (W)s_prod[p];
      W acc = a0 + a1;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
      if (l32 == 0) {
        const int g = base + k;
        if (g == nrf) carry[t] = (V)acc;
        else if (g == 0 && s_head_partial) head[t] = (V)acc;
        else if (STAGED) s_y[k] = (V)acc;
        else out.store((int64_t)ra + g, (V)acc);
      }
    }

    // pass 3: segments of more than HUGE_LEN entries (at most a handful per tile): every warp sums one
    // slice of each, then one thread per segment adds the warp sums in order
    const int nhuge = s_nhuge;
    if (nhuge > 0) {
      for (int q = 0; q < nhuge; ++q) {
        const int k = s_huge[q];
        const int s = s_off[k], e = s_off[k + 1];
        const int slice = (((e - s) + NW - 1) / NW + 31) & ~31;
        const int b0 = s + w * slice;
        const int b1 = (b0 + slice) < e ? (b0 + slice) : e;
        W acc = 0;
        for (int p = b0 + l32; p < b1; p += 32) acc += (W)s_prod[p];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
        if (l32 == 0) s_part[q][w] = acc;
      }
      __syncthreads();
      if (tid < nhuge) {
        W tot = 0;
#pragma unroll
        for (int q = 0; q < NW; ++q) tot += s_part[tid][q];
        const int g = base + s_huge[tid];
        if (g == nrf) carry[t] = (V)tot;
        else if (g == 0 && s_head_partial) head[t] = (V)tot;
        else if (STAGED) s_y[s_huge[tid]] = (V)tot;
        else out.store((int64_t)ra + g, (V)tot);
      }
    }

    // write-out: consecutive threads store consecutive rows (one request per 32 rows and destination)
    if (STAGED) {
      __syncthreads();
      const int first = (base == 0 && s_head_partial) ? 1 : 0;   // row 0 of the tile is finished by the fix-up
      const int last = (base + m) < nrf ? m : (nrf - base);       // the tail segment is not a row of this tile
      out.store_block((int64_t)ra + base, s_y, first, last, tid);
    }
  }
}

// Neumaier-compensated running sum in double: exact enough for either value type whatever the row length
__device__ __forceinline__ void comp_add(double& sum, double& comp, double v) {
  const double s2 = sum + v;
  comp += (fabs(sum) >= fabs(v)) ? ((sum - s2) + v) : ((v - s2) + sum);
  sum = s2;
}

constexpr int kFixupSerial = 32;   // a row that crossed more tiles than this is summed by its whole warp

// one thread per tile t >= 1: if the first row written by tile t started in an earlier tile, finish it.
// The carries of a row that crossed many tiles (a single row of 2^30 entries leaves half a million of them) are
// summed by the 32 lanes of the thread's warp, lane-strided, and combined in a fixed order.
template <typename V, typename P, typename Out>
__global__ void __launch_bounds__(kThreads)
spmv_fixup_kernel(const P* __restrict__ ptr, const int32_t* __restrict__ tile_row,
                  const V* __restrict__ carry, const V* __restrict__ head, Out out, int64_t n_tiles,
                  int log2_tile) {
  const int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x + 1;
  const int lane = threadIdx.x & 31;
  int32_t ra = 0;
  long long t0 = 0;
  bool need = false;
  if (t < n_tiles) {
    ra = tile_row[t];
    if (ra < tile_row[t + 1]) {                 // some row ends in this tile
      const int64_t p = (int64_t)ptr[ra];
      if (p < (t << log2_tile)) {               // and its first row started in an earlier one
        need = true;
        t0 = p >> log2_tile;
      }
    }
  }
  const bool wide = need && ((long long)t - t0) > kFixupSerial;
  if (need && !wide) {
    double sum = (double)head[t], comp = 0.0;
    for (int64_t u = t0; u < t; ++u) comp_add(sum, comp, (double)carry[u]);
    out.store((int64_t)ra, (V)(sum + comp));
  }
  unsigned todo = __ballot_sync(0xffffffffu, wide);
  while (todo) {
    const int src = __ffs(todo) - 1;
    todo &= todo - 1;
    const long long a = __shfl_sync(0xffffffffu, t0, src);
    const long long b = __shfl_sync(0xffffffffu, (long long)t, src);
    double sum = 0.0, comp = 0.0;
    for (long long u = a + lane; u < b; u += 32) comp_add(sum, comp, (double)carry[u]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const double os = __shfl_down_sync(0xffffffffu, sum, o);
      const double oc = __shfl_down_sync(0xffffffffu, comp, o);
      comp_add(sum, comp, os);
      comp += oc;
    }
    sum = __shfl_sync(0xffffffffu, sum, 0);
    comp = __shfl_sync(0xffffffffu, comp, 0);
    if (lane == src) {
      comp_add(sum, comp, (double)head[t]);
      out.store((int64_t)ra, (V)(sum + comp));
    }
  }
}

template <typename V, typename Out>
__global__ void __launch_bounds__(kThreads) fill_zero_kernel(Out out, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i < n) out.store(i, (V)0);
}

// ---------------------------------------------------------------------------------------------------
// host-side dispatch
// ---------------------------------------------------------------------------------------------------
static int ipt_of(int tuning) {
  switch ((tuning >> 8) & 3) {
    case 1: return 4;
    case 3: return 16;
    default: return 8;
  }
}

template <typename V, typename I, typename P, int L, typename Out>
static void launch_vector(const void* data, const void* idx, const void* ptr, const void* x, Out out,
                          int64_t n_rows, int64_t nnz, cudaStream_t st) {
  const int64_t threads = n_rows * L;
  const unsigned g = (unsigned)((threads + kThreads - 1) / kThreads);
  if (aligned_to(data, 16) && aligned_to(idx, 16))
    spmv_vector_kernel<V, I, P, L, true, Out><<<g, kThreads, 0, st>>>((const V*)data, (const I*)idx, (const P*)ptr,
                                                                      (const V*)x, out, n_rows, nnz);
  else
    spmv_vector_kernel<V, I, P, L, false, Out><<<g, kThreads, 0, st>>>((const V*)data, (const I*)idx, (const P*)ptr,
                                                                       (const V*)x, out, n_rows, nnz);
}

template <typename V, typename I, typename P, typename Out>
static int run_vector(const void* data, const void* idx, const void* ptr, const void* x, Out out,
                      int64_t n_rows, int64_t nnz, int tuning, cudaStream_t st) {
  int L = tuning & 0xff;
  if (L == 0) {
    // eight to sixteen entries (two to four 4-element groups) per lane: measured best on 32-entry rows
    const int64_t mean = n_rows > 0 ? nnz / n_rows : 0;
    L = 2;
    while (L < 32 && 16 * L < mean + 3) L <<= 1;
  }
  if (n_rows * (int64_t)L / kThreads >= INT32_MAX) return FSB_ERANGE;
  switch (L) {
    case 2: launch_vector<V, I, P, 2, Out>(data, idx, ptr, x, out, n_rows, nnz, st); break;
    case 4: launch_vector<V, I, P, 4, Out>(data, idx, ptr, x, out, n_rows, nnz, st); break;
    case 8: launch_vector<V, I, P, 8, Out>(data, idx, ptr, x, out, n_rows, nnz, st); break;
    case 16: launch_vector<V, I, P, 16, Out>(data, idx, ptr, x, out, n_rows, nnz, st); break;
    case 32: launch_vector<V, I, P, 32, Out>(data, idx, ptr, x, out, n_rows, nnz, st); break;
    default: return FSB_EINVAL;
  }
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}

template <typename V, typename I, typename P, int IPT, typename Out>
static int launch_stream(const void* data, const void* idx, const void* ptr, const void* x, Out out,
                         const int32_t* tile_row, void* scratch, int64_t nnz, int tuning, cudaStream_t st) {
  constexpr int T = kThreads * IPT;
  const int64_t n_tiles = (nnz + T - 1) / T;
  V* carry = (V*)scratch;
  V* head = carry + n_tiles;
  int shift = (tuning & 0xff) ? (tuning & 0xff) - 1 : 3;
  if (shift > 16) shift = 16;
  const bool vec = aligned_to(data, 16) && aligned_to(idx, 16);
  if (vec)
    spmv_stream_kernel<V, I, P, IPT, true, Out><<<(unsigned)n_tiles, kThreads, 0, st>>>(
        (const V*)data, (const I*)idx, (const P*)ptr, (const V*)x, out, tile_row, carry, head, nnz, shift);
  else
    spmv_stream_kernel<V, I, P, IPT, false, Out><<<(unsigned)n_tiles, kThreads, 0, st>>>(
        (const V*)data, (const I*)idx, (const P*)ptr, (const V*)x, out, tile_row, carry, head, nnz, shift);
  FSB_RETURN_IF_LAUNCH_FAILED();
  if (n_tiles > 1) {
    int log2_tile = 0;
    while ((1 << log2_tile) < T) ++log2_tile;
    const int64_t g = (n_tiles - 1 + kThreads - 1) / kThreads;
    spmv_fixup_kernel<V, P, Out><<<(unsigned)g, kThreads, 0, st>>>((const P*)ptr, tile_row, carry, head, out,
                                                                  n_tiles, log2_tile);
    FSB_RETURN_IF_LAUNCH_FAILED();
  }
  return FSB_OK;
}

template <typename V, typename I, typename P, typename Out>
static int run_stream(const void* data, const void* idx, const void* ptr, const void* x, Out out,
                      const int32_t* tile_row, void* scratch, int64_t nnz, int tuning, cudaStream_t st) {
  switch (ipt_of(tuning)) {
    case 4: return launch_stream<V, I, P, 4, Out>(data, idx, ptr, x, out, tile_row, scratch, nnz, tuning, st);
    case 16: return launch_stream<V, I, P, 16, Out>(data, idx, ptr, x, out, tile_row, scratch, nnz, tuning, st);
    default: return launch_stream<V, I, P, 8, Out>(data, idx, ptr, x, out, tile_row, scratch, nnz, tuning, st);
  }
}

struct SpmvArgs {
  const void *data, *idx, *ptr, *x;
  void* y;
  void* const* y_peers;
  int n_peers, first_peer;
  int64_t row_offset, n_rows, nnz;
  int algo, tuning;
  const int32_t* tile_row;
  void* scratch;
  cudaStream_t st;
};

template <typename V, typename I, typename P>
static int spmv_typed(const SpmvArgs& a) {
  if (a.algo == FSB_SPMV_VECTOR) {
    if (a.y_peers) {
      PeerOut<V> out{(V* const*)a.y_peers, a.n_peers, a.row_offset, a.first_peer};
      return run_vector<V, I, P, PeerOut<V>>(a.data, a.idx, a.ptr, a.x, out, a.n_rows, a.nnz, a.tuning & 0xff, a.st);
    }
    LocalOut<V> out{(V*)a.y};
    return run_vector<V, I, P, LocalOut<V>>(a.data, a.idx, a.ptr, a.x, out, a.n_rows, a.nnz, a.tuning, a.st);
  }
  if (a.y_peers) {
    PeerOut<V> out{(V* const*)a.y_peers, a.n_peers, a.row_offset, a.first_peer};
    return run_stream<V, I, P, PeerOut<V>>(a.data, a.idx, a.ptr, a.x, out, a.tile_row, a.scratch, a.nnz,
                                           a.tuning, a.st);
  }
  LocalOut<V> out{(V*)a.y};
  return run_stream<V, I, P, LocalOut<V>>(a.data, a.idx, a.ptr, a.x, out, a.tile_row, a.scratch, a.nnz,
                                          a.tuning, a.st);
}

static int spmv_dispatch(int vtype, int itype, int ptype, const SpmvArgs& a) {
#define FSB_CASE(VT, V, IT, I, PT, P) \
  if (vtype == VT && itype == IT && ptype == PT) return spmv_typed<V, I, P>(a);
  FSB_CASE(FSB_F32, float, FSB_I32, int32_t, FSB_I32, int32_t)
  FSB_CASE(FSB_F32, float, FSB_I32, int32_t, FSB_I64, int64_t)
  FSB_CASE(FSB_F32, float, FSB_I64, int64_t, FSB_I32, int32_t)
  FSB_CASE(FSB_F32, float, FSB_I64, int64_t, FSB_I64, int64_t)
  FSB_CASE(FSB_F64, double, FSB_I32, int32_t, FSB_I32, int32_t)
  FSB_CASE(FSB_F64, double, FSB_I32, int32_t, FSB_I64, int64_t)
  FSB_CASE(FSB_F64, double, FSB_I64, int64_t, FSB_I32, int32_t)
  FSB_CASE(FSB_F64, double, FSB_I64, int64_t, FSB_I64, int64_t)
#undef FSB_CASE
  return FSB_EINVAL;
}

static int check_common(int vtype, int itype, int ptype, const void* data, const void* indices,
                        const void* indptr, const void* x, int64_t n_rows, int64_t n_cols, int64_t nnz) {
  if ((vtype != FSB_F32 && vtype != FSB_F64) || (itype != FSB_I32 && itype != FSB_I64) ||
      (ptype != FSB_I32 && ptype != FSB_I64))
    return FSB_EINVAL;
  if (n_rows < 0 || n_cols < 0 || nnz < 0) return FSB_EINVAL;
  if (n_rows >= INT32_MAX || n_cols >= INT32_MAX) return FSB_ERANGE;
  if (ptype == FSB_I32 && nnz > INT32_MAX) return FSB_ERANGE;
  if (indptr == nullptr) return FSB_EINVAL;
  if (nnz > 0 && (data == nullptr || indices == nullptr || x == nullptr)) return FSB_EINVAL;
  const size_t sv = vtype == FSB_F32 ? 4 : 8, si = itype == FSB_I32 ? 4 : 8, sp = ptype == FSB_I32 ? 4 : 8;
  if (!aligned_to(data, sv) || !aligned_to(x, sv) || !aligned_to(indices, si) || !aligned_to(indptr, sp))
    return FSB_EALIGN;
  return FSB_OK;
}

}  // namespace fsb

using namespace fsb;

extern "C" int fsb_spmv_tile_nnz(int vtype, int tuning) {
  (void)vtype;
  return kThreads * ipt_of(tuning);
}

extern "C" size_t fsb_spmv_csr_scratch_bytes(int vtype, int64_t nnz, int tuning) {
  const int T = fsb_spmv_tile_nnz(vtype, tuning);
  const int64_t n_tiles = fsb_csr_num_tiles(nnz, T);
  const size_t sv = vtype == FSB_F32 ? 4 : 8;
  size_t b = (size_t)n_tiles * 2 * sv;
  return (b + 255) & ~(size_t)255;
}

extern "C" int fsb_spmv_csr(int vtype, int itype, int ptype, const void* data, const void* indices,
                            const void* indptr, const void* x, void* y, int64_t n_rows, int64_t n_cols,
                            int64_t nnz, int algo, int tuning, const int32_t* tile_row, void* scratch,
                            size_t scratch_bytes, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  int rc = check_common(vtype, itype, ptype, data, indices, indptr, x, n_rows, n_cols, nnz);
  if (rc != FSB_OK) return rc;
  FSB_WALK_FIRST(check_csr(itype, ptype, indices, indptr, n_rows, n_cols, nnz, st));
  if (n_rows == 0) return FSB_OK;
  if (y == nullptr) return FSB_EINVAL;
  const size_t sv = vtype == FSB_F32 ? 4 : 8;
  if (!aligned_to(y, sv)) return FSB_EALIGN;
  if (nnz == 0) return cuda_rc(cudaMemsetAsync(y, 0, (size_t)n_rows * sv, st));
  if (algo == FSB_SPMV_AUTO)
    algo = (tile_row != nullptr && scratch != nullptr && nnz >= (1 << 20)) ? FSB_SPMV_STREAM : FSB_SPMV_VECTOR;
  if (algo != FSB_SPMV_VECTOR && algo != FSB_SPMV_STREAM) return FSB_EINVAL;
  if (algo == FSB_SPMV_STREAM) {
    if (tile_row == nullptr || scratch == nullptr) return FSB_EINVAL;
    if (scratch_bytes < fsb_spmv_csr_scratch_bytes(vtype, nnz, tuning)) return FSB_ESCRATCH;
    if (!aligned_to(scratch, 16)) return FSB_EALIGN;
  }
  SpmvArgs a{data, indices, indptr, x, y, nullptr, 0, 0, 0, n_rows, nnz, algo, tuning, tile_row, scratch, st};
  return spmv_dispatch(vtype, itype, ptype, a);
}

extern "C" int fsb_spmv_csr_scatter(int vtype, int itype, int ptype, const void* data, const void* indices,
                                    const void* indptr, const void* x, void* const* y_peers, int n_peers,
                                    int first_peer, int64_t row_offset, int64_t n_rows, int64_t n_cols, int64_t nnz,
                                    int algo,
                                    int tuning, const int32_t* tile_row, void* scratch, size_t scratch_bytes,
                                    void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  int rc = check_common(vtype, itype, ptype, data, indices, indptr, x, n_rows, n_cols, nnz);
  if (rc != FSB_OK) return rc;
  FSB_WALK_FIRST(check_csr(itype, ptype, indices, indptr, n_rows, n_cols, nnz, st));
  if (y_peers == nullptr || n_peers < 1 || n_peers > 64 || row_offset < 0) return FSB_EINVAL;
  if (first_peer < 0 || first_peer >= n_peers) return FSB_EINVAL;
  if (n_rows == 0) return FSB_OK;
  if (nnz == 0) {
    const unsigned g = (unsigned)((n_rows + kThreads - 1) / kThreads);
    if (vtype == FSB_F32)
      fill_zero_kernel<float, PeerOut<float>><<<g, kThreads, 0, st>>>(
          PeerOut<float>{(float* const*)y_peers, n_peers, row_offset, first_peer}, n_rows);
    else
      fill_zero_kernel<double, PeerOut<double>><<<g, kThreads, 0, st>>>(
          PeerOut<double>{(double* const*)y_peers, n_peers, row_offset, first_peer}, n_rows);
    FSB_RETURN_IF_LAUNCH_FAILED();
    return FSB_OK;
  }
  if (algo == FSB_SPMV_AUTO) algo = (tile_row != nullptr && scratch != nullptr) ? FSB_SPMV_STREAM : FSB_SPMV_VECTOR;
  if (algo != FSB_SPMV_VECTOR && algo != FSB_SPMV_STREAM) return FSB_EINVAL;
  if (algo == FSB_SPMV_STREAM) {
    if (tile_row == nullptr || scratch == nullptr) return FSB_EINVAL;
    if (scratch_bytes < fsb_spmv_csr_scratch_bytes(vtype, nnz, tuning)) return FSB_ESCRATCH;
    if (!aligned_to(scratch, 16)) return FSB_EALIGN;
  }
  SpmvArgs a{data, indices, indptr, x, nullptr, y_peers, n_peers, first_peer, row_offset, n_rows, nnz,
             algo, tuning, tile_row, scratch, st};
  return spmv_dispatch(vtype, itype, ptype, a);
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant of the stream SpMV.
//
// Some hosts of this library may not create device memory at the moment they need a product: code running
// while a memory pool is frozen or under a fixed-footprint policy, plugins that are handed tensors by a
// framework but have no allocator of their own, and callers bound to a real-time loop where a cudaMalloc
// (which can synchronise the whole device) is off limits.  For them the per-tile partial sums live in the
// array below, which is part of the library image: it exists on every GPU that loads libfsb.so, from load
// until the process exits, and is never resized.
// ---------------------------------------------------------------------------------------------------
namespace fsb {

static __device__ __align__(256) unsigned char g_noalloc_scratch[(size_t)FSB_NOALLOC_MAX_TILES * 2 * sizeof(double)];

constexpr int kMaxDevices = 64;
static void* g_noalloc_ptr[kMaxDevices];  // device address of the array above, per device ordinal
static std::mutex g_noalloc_mutex;

// The array's name is only a stand-in on the host; the address the kernels need comes from the runtime,
// once per device, with that device current.
static int noalloc_scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_rc(e);
  if (dev < 0 || dev >= kMaxDevices) return FSB_ERANGE;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return cuda_rc(e);
    if (p == nullptr) return FSB_EINVAL;
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return FSB_OK;
}

}  // namespace fsb

extern "C" int fsb_spmv_csr_noalloc(int vtype, int itype, int ptype, const void* data, const void* indices,
                                    const void* indptr, const void* x, void* y, int64_t n_rows, int64_t n_cols,
                                    int64_t nnz, int tuning, const int32_t* tile_row, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  int rc = check_common(vtype, itype, ptype, data, indices, indptr, x, n_rows, n_cols, nnz);
  if (rc != FSB_OK) return rc;
  FSB_WALK_FIRST(check_csr(itype, ptype, indices, indptr, n_rows, n_cols, nnz, st));
  if (n_rows == 0) return FSB_OK;
  if (y == nullptr) return FSB_EINVAL;
  const size_t sv = vtype == FSB_F32 ? 4 : 8;
  if (!aligned_to(y, sv)) return FSB_EALIGN;
  if (nnz == 0) return cuda_rc(cudaMemsetAsync(y, 0, (size_t)n_rows * sv, st));
  if (tile_row == nullptr) return FSB_EINVAL;
  // the built-in array holds two partial sums per tile for at most FSB_NOALLOC_MAX_TILES tiles
  const int64_t n_tiles = fsb_csr_num_tiles(nnz, fsb_spmv_tile_nnz(vtype, tuning));
  if (n_tiles > FSB_NOALLOC_MAX_TILES) return FSB_ENOSPACE;
  void* scratch = nullptr;
  rc = noalloc_scratch_address(&scratch);
  if (rc != FSB_OK) return rc;
  SpmvArgs a{data, indices, indptr, x, y, nullptr, 0, 0, 0, n_rows, nnz, FSB_SPMV_STREAM, tuning, tile_row, scratch, st};
  return spmv_dispatch(vtype, itype, ptype, a);
}
