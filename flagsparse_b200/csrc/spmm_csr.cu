// CSR SpMM (C = A B, B and C dense row-major) for sm_100a.
//
// Same tiling as the SpMV stream kernel: the nnz range is cut into tiles of T entries, so a tile of
// `data` and of `indices` is one contiguous, 16-byte aligned block.  A CTA stages its tile in shared
// memory -- with one cp.async.bulk (TMA 1-D bulk copy) per array completing on an mbarrier, or with
// ordinary coalesced loads -- and loads indptr[ra .. rb] as tile-relative offsets.  Then groups of LR
// lanes (LR = columns / VW rounded up to a power of two, VW = elements per 128-bit access) each take one
// row segment: the (value, column) pairs come from shared memory as broadcasts, each lane gathers VW
// consecutive elements of B's row through the read-only path, and the accumulators stay in registers.
// This is CUDA-core work on purpose: the operand is an irregular gather with at most 0.5 flop per byte.
// Rows ending in the tile are written to C with streaming stores; a row continuing into the next tile
// leaves its partial row in carry[t, :], a row that began in an earlier tile leaves it in head[t, :],
// and a second kernel adds them up in a fixed order (deterministic, no atomics).
#include "fsb_common.cuh"

namespace fsb {

constexpr int kMmThreads = 256;
constexpr int kMmTile = 1024;  // nnz per tile
constexpr int kWaitSpins = 1 << 22;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}
// 1-D bulk copy global -> this CTA's shared memory; src, dst and bytes are multiples of 16
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t phase) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(phase)
      : "memory");
  return ok != 0;
}
// bounded: gives up after kWaitSpins polls and reports it
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t phase) {
  for (int i = 0; i < kWaitSpins; ++i)
    if (mbar_try_wait(bar, phase)) return true;
  return false;
}

// ACCUM: add to what C holds instead of overwriting it (rows without entries are then left alone) -- the later
// passes of a product that the host code splits into column panels of A.
template <typename V, typename I, typename P, int VW, bool BULK, bool ACCUM>
__global__ void __launch_bounds__(kMmThreads)
spmm_tile_kernel(const V* __restrict__ data, const I* __restrict__ idx, const P* __restrict__ ptr,
                 const V* __restrict__ B, int64_t ldb, V* __restrict__ C, int64_t ldc,
                 const int32_t* __restrict__ tile_row, V* __restrict__ carry, V* __restrict__ head,
                 int64_t nnz, int n_dense, int LR, int32_t* __restrict__ status) {
  constexpr int T = kMmTile;
  constexpr int RC = T;
  __shared__ __align__(128) V s_val[T];
  __shared__ __align__(128) I s_idx[T];
  __shared__ int32_t s_off[RC + 1];
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ int s_head_partial;
  __shared__ int s_failed;

  const int tid = threadIdx.x;
  const int64_t t = blockIdx.x;
  const int64_t lo = t * (int64_t)T;
  const int cnt = (int)((nnz - lo) < (int64_t)T ? (nnz - lo) : (int64_t)T);
  const int32_t ra = tile_row[t];
  const int32_t rb = tile_row[t + 1];

  // ---- stage the tile -------------------------------------------------------------------------
  bool bulk = BULK && cnt == T;
  if (bulk) {
    if (tid == 0) {
      s_failed = 0;
      mbar_init(&s_bar, 1);
      fence_barrier_init();
    }
    __syncthreads();
    if (tid == 0) {
      mbar_expect_tx(&s_bar, (uint32_t)(T * (sizeof(V) + sizeof(I))));
      bulk_g2s(s_val, data + lo, (uint32_t)(T * sizeof(V)), &s_bar);
      bulk_g2s(s_idx, idx + lo, (uint32_t)(T * sizeof(I)), &s_bar);
    }
  } else {
    for (int e = tid; e < cnt; e += kMmThreads) {
      s_val[e] = ld_stream(data + lo + e);
      s_idx[e] = ld_stream(idx + lo + e);
    }
  }

  const int nrf = rb - ra;
  const int nseg = nrf + 1;
  const int lane = tid & (LR - 1);
  const int grp = tid / LR;
  const int ngrp = kMmThreads / LR;
  const int col0 = (blockIdx.y * LR + lane) * VW;
  const bool col_ok = col0 < n_dense;

  for (int base = 0; base < nseg; base += RC) {
    const int m = (nseg - base) < RC ? (nseg - base) : RC;
    __syncthreads();
    for (int k = tid; k <= m; k += kMmThreads) {
      const int g = base + k;
      int32_t o = cnt;
      if (g <= nrf) {
        const int64_t d = (int64_t)ptr[(int64_t)ra + g] - lo;
        o = d < 0 ? 0 : (d > cnt ? cnt : (int32_t)d);
        if (g == 0) s_head_partial = (d < 0 && nrf > 0) ? 1 : 0;
      }
      s_off[k] = o;
    }
    if (bulk && base == 0) {
      // every thread polls the barrier itself: completion makes the copied bytes visible to it
      if (!mbar_wait_bounded(&s_bar, 0)) s_failed = 1;
    }
    __syncthreads();
    if (bulk && s_failed) {
      // the copy did not land within the bound: report it and leave this tile unwritten
      if (tid == 0 && status != nullptr) *reinterpret_cast<volatile int32_t*>(status) = 1;  // may be host memory
      mbar_wait_bounded(&s_bar, 0);  // one more bounded wait so that no copy is in flight at exit
      return;
    }

    for (int k = grp; k < m; k += ngrp) {
      const int s = s_off[k], e = s_off[k + 1];
      V acc[VW];
#pragma unroll
      for (int i = 0; i < VW; ++i) acc[i] = 0;
      if (col_ok) {
        int p = s;
        for (; p + 4 <= e; p += 4) {
          V a[4];
          int64_t c[4];
          V b[4][VW];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            a[u] = s_val[p + u];
            c[u] = (int64_t)s_idx[p + u];
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) ld_dense<V, VW>(B + c[u] * ldb + col0, b[u]);
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int i = 0; i < VW; ++i) acc[i] += a[u] * b[u][i];
        }
        for (; p < e; ++p) {
          const V a = s_val[p];
          V b[VW];
          ld_dense<V, VW>(B + (int64_t)s_idx[p] * ldb + col0, b);
#pragma unroll
          for (int i = 0; i < VW; ++i) acc[i] += a * b[i];
        }
        const int g = base + k;
        if (g == nrf) {
#pragma unroll
          for (int i = 0; i < VW; ++i) carry[t * n_dense + col0 + i] = acc[i];
        } else if (g == 0 && s_head_partial) {
#pragma unroll
          for (int i = 0; i < VW; ++i) head[t * n_dense + col0 + i] = acc[i];
        } else if (!ACCUM) {
          st_dense_stream<V, VW>(C + ((int64_t)ra + g) * ldc + col0, acc);
        } else if (e > s) {
          V* dst = C + ((int64_t)ra + g) * ldc + col0;
          V old[VW];
          ld_dense_stream<V, VW>(dst, old);
#pragma unroll
          for (int i = 0; i < VW; ++i) acc[i] += old[i];
          st_dense_stream<V, VW>(dst, acc);
        }
      }
    }
  }
}

// one thread per (tile t >= 1, column): finish the row that started before tile t and ends in it
template <typename V, typename P, bool ACCUM>
__global__ void __launch_bounds__(kMmThreads)
spmm_fixup_kernel(const P* __restrict__ ptr, const int32_t* __restrict__ tile_row,
                  const V* __restrict__ carry, const V* __restrict__ head, V* __restrict__ C, int64_t ldc,
                  int64_t n_tiles, int n_dense, int log2_tile) {
  const int64_t gid = (int64_t)blockIdx.x * kMmThreads + threadIdx.x;
  const int64_t t = gid / n_dense + 1;
  const int j = (int)(gid % n_dense);
  if (t >= n_tiles) return;
  const int32_t ra = tile_row[t];
  const int32_t rb = tile_row[t + 1];
  if (ra >= rb) return;
  const int64_t p = (int64_t)ptr[ra];
  if (p >= (t << log2_tile)) return;
  const int64_t t0 = p >> log2_tile;
  double sum = (double)head[t * n_dense + j], comp = 0.0;
  for (int64_t u = t0; u < t; ++u) {
    const double v = (double)carry[u * n_dense + j];
    const double s2 = sum + v;
    comp += (fabs(sum) >= fabs(v)) ? ((sum - s2) + v) : ((v - s2) + sum);
    sum = s2;
  }
  V* dst = C + (int64_t)ra * ldc + j;
  *dst = ACCUM ? (V)(((double)*dst + sum) + comp) : (V)(sum + comp);
}

template <typename V>
__global__ void __launch_bounds__(kMmThreads) zero_rows_kernel(V* __restrict__ C, int64_t ldc, int64_t n_rows,
                                                              int n_dense) {
  const int64_t gid = (int64_t)blockIdx.x * kMmThreads + threadIdx.x;
  const int64_t r = gid / n_dense;
  const int j = (int)(gid % n_dense);
  if (r < n_rows) C[r * ldc + j] = (V)0;
}

struct SpmmArgs {
  const void *data, *idx, *ptr, *B;
  int64_t ldb;
  void* C;
  int64_t ldc, n_rows, n_dense, nnz;
  int algo;
  bool accumulate;
  const int32_t* tile_row;
  void* scratch;
  int32_t* status;
  cudaStream_t st;
};

template <typename V, typename I, typename P, int VW>
static int launch_spmm(const SpmmArgs& a) {
  constexpr int T = kMmTile;
  const int64_t n_tiles = (a.nnz + T - 1) / T;
  const int n_dense = (int)a.n_dense;
  int need = (n_dense + VW - 1) / VW;  // lanes needed to cover a row of B
  int LR = 1;
  while (LR < 32 && LR < need) LR <<= 1;
  const int col_tiles = (need + LR - 1) / LR;
  V* carry = (V*)a.scratch;
  V* head = carry + n_tiles * n_dense;
  bool bulk = a.algo != FSB_SPMM_PLAIN && aligned_to(a.data, 16) && aligned_to(a.idx, 16);
  dim3 grid((unsigned)n_tiles, (unsigned)col_tiles);
#define FSB_SPMM_LAUNCH(BULK_, ACC_)                                                                          \
  spmm_tile_kernel<V, I, P, VW, BULK_, ACC_><<<grid, kMmThreads, 0, a.st>>>(                                  \
      (const V*)a.data, (const I*)a.idx, (const P*)a.ptr, (const V*)a.B, a.ldb, (V*)a.C, a.ldc, a.tile_row,   \
      carry, head, a.nnz, n_dense, LR, a.status)
  if (bulk) {
    if (a.accumulate) FSB_SPMM_LAUNCH(true, true); else FSB_SPMM_LAUNCH(true, false);
  } else {
    if (a.accumulate) FSB_SPMM_LAUNCH(false, true); else FSB_SPMM_LAUNCH(false, false);
  }
#undef FSB_SPMM_LAUNCH
  FSB_RETURN_IF_LAUNCH_FAILED();
  if (n_tiles > 1) {
    int log2_tile = 0;
    while ((1 << log2_tile) < T) ++log2_tile;
    const int64_t n = (n_tiles - 1) * n_dense;
    const int64_t g = (n + kMmThreads - 1) / kMmThreads;
    if (g >= INT32_MAX) return FSB_ERANGE;
    if (a.accumulate)
      spmm_fixup_kernel<V, P, true><<<(unsigned)g, kMmThreads, 0, a.st>>>((const P*)a.ptr, a.tile_row, carry, head,
                                                                         (V*)a.C, a.ldc, n_tiles, n_dense, log2_tile);
    else
      spmm_fixup_kernel<V, P, false><<<(unsigned)g, kMmThreads, 0, a.st>>>((const P*)a.ptr, a.tile_row, carry, head,
                                                                          (V*)a.C, a.ldc, n_tiles, n_dense, log2_tile);
    FSB_RETURN_IF_LAUNCH_FAILED();
  }
  return FSB_OK;
}

template <typename V, typename I, typename P>
static int spmm_typed(const SpmmArgs& a) {
  // widest access that divides the row length and keeps every row of B and C aligned
  constexpr int VMAX = 16 / sizeof(V);
  int vw = VMAX;
  while (vw > 1 && !(a.n_dense % vw == 0 && a.ldb % vw == 0 && a.ldc % vw == 0 &&
                     aligned_to(a.B, vw * sizeof(V)) && aligned_to(a.C, vw * sizeof(V)) &&
                     aligned_to(a.scratch, vw * sizeof(V))))
    vw >>= 1;
  if constexpr (VMAX == 4) {
    if (vw == 4) return launch_spmm<V, I, P, 4>(a);
  }
  if (vw == 2) return launch_spmm<V, I, P, 2>(a);
  return launch_spmm<V, I, P, 1>(a);
}

}  // namespace fsb

using namespace fsb;

extern "C" int fsb_spmm_tile_nnz(int vtype) {
  (void)vtype;
  return kMmTile;
}

extern "C" size_t fsb_spmm_csr_scratch_bytes(int vtype, int64_t nnz, int64_t n_dense) {
  const int64_t n_tiles = fsb_csr_num_tiles(nnz, kMmTile);
  const size_t sv = vtype == FSB_F32 ? 4 : 8;
  size_t b = (size_t)n_tiles * 2 * (size_t)(n_dense > 0 ? n_dense : 0) * sv;
  return (b + 255) & ~(size_t)255;
}

extern "C" int fsb_spmm_csr(int vtype, int itype, int ptype, const void* data, const void* indices,
                            const void* indptr, const void* B, int64_t ldb, void* C, int64_t ldc,
                            int64_t n_rows, int64_t n_cols, int64_t n_dense, int64_t nnz, int algo,
                            const int32_t* tile_row, void* scratch, size_t scratch_bytes, int32_t* status,
                            void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if ((vtype != FSB_F32 && vtype != FSB_F64) || (itype != FSB_I32 && itype != FSB_I64) ||
      (ptype != FSB_I32 && ptype != FSB_I64))
    return FSB_EINVAL;
  const bool accumulate = (algo & FSB_SPMM_ACCUMULATE) != 0;
  algo &= ~FSB_SPMM_ACCUMULATE;
  if (algo != FSB_SPMM_AUTO && algo != FSB_SPMM_PLAIN && algo != FSB_SPMM_BULK) return FSB_EINVAL;
  if (n_rows < 0 || n_cols < 0 || n_dense < 0 || nnz < 0) return FSB_EINVAL;
  if (n_rows >= INT32_MAX || n_cols >= INT32_MAX || n_dense >= (1 << 24)) return FSB_ERANGE;
  if (ptype == FSB_I32 && nnz > INT32_MAX) return FSB_ERANGE;
  if (n_rows == 0 || n_dense == 0) return FSB_OK;
  if (C == nullptr || indptr == nullptr || ldc < n_dense) return FSB_EINVAL;
  const size_t sv = vtype == FSB_F32 ? 4 : 8, si = itype == FSB_I32 ? 4 : 8, sp = ptype == FSB_I32 ? 4 : 8;
  if (!aligned_to(C, sv) || !aligned_to(indptr, sp)) return FSB_EALIGN;
  FSB_WALK_FIRST(check_csr(itype, ptype, indices, indptr, n_rows, n_cols, nnz, st));
  if (nnz == 0 && accumulate) return FSB_OK;   // nothing to add
  if (nnz == 0) {
    const int64_t n = n_rows * n_dense;
    const int64_t g = (n + kMmThreads - 1) / kMmThreads;
    if (g >= INT32_MAX) return FSB_ERANGE;
    if (vtype == FSB_F32)
      zero_rows_kernel<float><<<(unsigned)g, kMmThreads, 0, st>>>((float*)C, ldc, n_rows, (int)n_dense);
    else
      zero_rows_kernel<double><<<(unsigned)g, kMmThreads, 0, st>>>((double*)C, ldc, n_rows, (int)n_dense);
    FSB_RETURN_IF_LAUNCH_FAILED();
    return FSB_OK;
  }
  if (data == nullptr || indices == nullptr || B == nullptr || ldb < n_dense) return FSB_EINVAL;
  if (!aligned_to(data, sv) || !aligned_to(B, sv) || !aligned_to(indices, si)) return FSB_EALIGN;
  if (tile_row == nullptr || scratch == nullptr) return FSB_EINVAL;
  if (scratch_bytes < fsb_spmm_csr_scratch_bytes(vtype, nnz, n_dense)) return FSB_ESCRATCH;
  if (!aligned_to(scratch, 16)) return FSB_EALIGN;
  if (fsb_csr_num_tiles(nnz, kMmTile) >= 65535LL * 32768LL) return FSB_ERANGE;

  SpmmArgs a{data, indices, indptr, B, ldb, C, ldc, n_rows, n_dense, nnz, algo, accumulate, tile_row, scratch,
             status, st};
#define FSB_CASE(VT, V, IT, I, PT, P) \
  if (vtype == VT && itype == IT && ptype == PT) return spmm_typed<V, I, P>(a);
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
