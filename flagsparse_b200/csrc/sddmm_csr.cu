// CSR SDDMM for sm_100a: out[p] = alpha * dot(X[row(p), :], Y[col(p), :]) + beta * data[p] for every entry p of a
// CSR pattern (X is n_rows x K, Y is n_cols x K, both row-major with a row stride).
//
// A group of LG lanes (LG = K / VW rounded up to a power of two, at most 32; VW = elements per 128-bit access)
// owns batches of 8 consecutive entries.  A CTA first copies the column and row ids of its tile (up to 2048
// entries; the row of an entry comes from the row-id array built at prepare time, 4 bytes per entry) into shared
// memory, so that the only trip to global memory inside the loop over batches is the gather; every lane then
// requests its slice of all eight rows of Y through the read-only path before it uses any of them, so a group has
// eight gathers in flight; a batch that lies inside one row (the common case) needs one slice of X's row, a batch
// that crosses rows loads a slice of X per entry.  Each lane ends with eight partial sums (one per entry);
// they are reduced across the group by a transposed exchange (halve the entries a lane is responsible for at every
// step: 7 shuffles for 8 entries x 8 lanes instead of 24), after which the results of consecutive entries sit in
// consecutive lanes and leave as one contiguous streaming store.  Rows of X longer than LG * VW elements are
// walked in several steps.  The summation order is fixed, so results are bit-reproducible.
// CUDA-core work on purpose: one dot product per entry over gathered rows is about 0.5 flop per byte.
#include "fsb_common.cuh"

namespace fsb {

#ifndef FSB_SDDMM_MIN_CTAS
#define FSB_SDDMM_MIN_CTAS 3   // resident CTAs per SM the register budget is set for (80 registers: no spills)
#endif
constexpr int kSdThreads = 256;
constexpr int kSdBatch = 8;   // consecutive entries one group handles

// entries one CTA handles: J passes of (threads / LG) groups x 8 entries, at most 2048
__host__ __device__ constexpr int sddmm_passes(int LG) {
  const int per_pass = (kSdThreads / LG) * kSdBatch;
  return per_pass >= 2048 ? 1 : (2048 / per_pass < 8 ? 2048 / per_pass : 8);
}
__host__ __device__ constexpr int sddmm_tile(int LG) { return (kSdThreads / LG) * kSdBatch * sddmm_passes(LG); }

template <typename V, int VW, int LG>
__global__ void __launch_bounds__(kSdThreads, FSB_SDDMM_MIN_CTAS)
sddmm_kernel(const int32_t* __restrict__ indices, const int32_t* __restrict__ row_ids, const V* __restrict__ X,
             int64_t ldx, const V* __restrict__ Y, int64_t ldy, const V* __restrict__ data, V* __restrict__ out,
             int64_t nnz, int k_dim, V alpha, V beta, int ids_aligned) {
  constexpr int E = kSdBatch;
  constexpr int step = LG * VW;
  constexpr int kGroups = kSdThreads / LG;
  constexpr int J = sddmm_passes(LG);
  constexpr int T = sddmm_tile(LG);
  constexpr int kHeld = (LG >= E) ? 1 : E / LG;   // results a lane ends up with
  constexpr int kDup = (LG > E) ? LG / E : 1;     // lanes that end up with the same result
  __shared__ __align__(16) int32_t s_cols[T];
  __shared__ __align__(16) int32_t s_rows[T];

  // the tile's column and row ids go to shared memory once (entries past the end repeat the last one; they are
  // never stored), so that the loop below has one trip to global memory per batch: the gathers
  const int64_t tile0 = (int64_t)blockIdx.x * T;
  const int64_t left = nnz - tile0;
  if (left >= T && ids_aligned) {
    for (int i = threadIdx.x; i < T / 4; i += kSdThreads) {
      reinterpret_cast<int4*>(s_cols)[i] = __ldcs(reinterpret_cast<const int4*>(indices + tile0) + i);
      reinterpret_cast<int4*>(s_rows)[i] = __ldcs(reinterpret_cast<const int4*>(row_ids + tile0) + i);
    }
  } else {
    for (int i = threadIdx.x; i < T; i += kSdThreads) {
      const int64_t p = tile0 + (i < left ? i : left - 1);
      s_cols[i] = __ldg(indices + p);
      s_rows[i] = __ldg(row_ids + p);
    }
  }
  __syncthreads();

  const int lane = threadIdx.x & (LG - 1);
  const int group = threadIdx.x / LG;
  const unsigned gmask = LG == 32 ? 0xffffffffu : (((1u << LG) - 1u) << ((threadIdx.x & 31) & ~(LG - 1)));
#pragma unroll 1
  for (int j = 0; j < J; ++j) {
    const int local = (j * kGroups + group) * E;
    if (local >= left) break;   // whole groups leave together: the shuffles below stay inside a group
    const int64_t p0 = tile0 + local;
    const int n = (int)((left - local) < E ? (left - local) : E);
    int32_t rows[E], cols[E];
    {
      const int4 c0 = *reinterpret_cast<const int4*>(s_cols + local);
      const int4 c1 = *reinterpret_cast<const int4*>(s_cols + local + 4);
      const int4 r0 = *reinterpret_cast<const int4*>(s_rows + local);
      const int4 r1 = *reinterpret_cast<const int4*>(s_rows + local + 4);
      cols[0] = c0.x; cols[1] = c0.y; cols[2] = c0.z; cols[3] = c0.w;
      cols[4] = c1.x; cols[5] = c1.y; cols[6] = c1.z; cols[7] = c1.w;
      rows[0] = r0.x; rows[1] = r0.y; rows[2] = r0.z; rows[3] = r0.w;
      rows[4] = r1.x; rows[5] = r1.y; rows[6] = r1.z; rows[7] = r1.w;
    }

    // the values of `data` this lane will need at the end are requested before the gathers, not after them
    const bool writer = (lane % kDup) == 0;
    const int first = (lane / kDup) * kHeld;
    V din[kHeld];
#pragma unroll
    for (int i = 0; i < kHeld; ++i)
      din[i] = (data != nullptr && writer && first + i < n) ? __ldcs(data + p0 + first + i) : (V)0;

    V acc[E];
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = (V)0;
    // Row ids never decrease along a CSR pattern, so the batch lies in one row of X iff its first and last ids
    // agree.  Then one slice of X serves all eight gathers, which leave together.  Otherwise every entry gets its
    // own slice of X, four entries at a time (reloading X only where the row changes would make each gather wait
    // for the previous entry's arithmetic).
    if (rows[0] == rows[E - 1]) {
      for (int k = lane * VW; k < k_dim; k += step) {
        V xr[VW], yv[E][VW];
        ld_dense<V, VW>(X + (int64_t)rows[0] * ldx + k, xr);
#pragma unroll
        for (int e = 0; e < E; ++e) ld_dense<V, VW>(Y + (int64_t)cols[e] * ldy + k, yv[e]);
#pragma unroll
        for (int e = 0; e < E; ++e)
#pragma unroll
          for (int i = 0; i < VW; ++i) acc[e] += xr[i] * yv[e][i];
      }
    } else {
      for (int k = lane * VW; k < k_dim; k += step) {
#pragma unroll
        for (int h = 0; h < E; h += E / 2) {
          V xv[E / 2][VW], yv[E / 2][VW];
#pragma unroll
          for (int e = 0; e < E / 2; ++e) {
            ld_dense<V, VW>(X + (int64_t)rows[h + e] * ldx + k, xv[e]);
            ld_dense<V, VW>(Y + (int64_t)cols[h + e] * ldy + k, yv[e]);
          }
#pragma unroll
          for (int e = 0; e < E / 2; ++e)
#pragma unroll
            for (int i = 0; i < VW; ++i) acc[h + e] += xv[e][i] * yv[e][i];
        }
      }
    }

    // transposed reduction: at each step a lane hands half of its entries to its partner and takes the partner's
    // partial sums of the half it keeps; once one entry is left the remaining steps are plain butterfly adds
    int held = E;
#pragma unroll
    for (int off = LG >> 1; off >= 1; off >>= 1) {
      if (held > 1) {
        held >>= 1;
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < E / 2; ++i) {
          if (i < held) {
            const V send = upper ? acc[i] : acc[i + held];
            const V keep = upper ? acc[i + held] : acc[i];
            acc[i] = keep + __shfl_xor_sync(gmask, send, off, LG);
          }
        }
      } else {
        acc[0] += __shfl_xor_sync(gmask, acc[0], off, LG);
      }
    }
    // a lane now holds kHeld consecutive entries starting at `first`; where LG > E, kDup lanes hold the same sum
    if (writer) {
#pragma unroll
      for (int i = 0; i < kHeld; ++i) {
        const int e = first + i;
        if (e < n) {
          V v = acc[i] * alpha;
          if (data != nullptr) v += din[i] * beta;
          __stcs(out + p0 + e, v);
        }
      }
    }
  }
}

template <typename V, int VW>
static int sddmm_launch(int LG, unsigned blocks, cudaStream_t st, const int32_t* indices, const int32_t* row_ids,
                        const V* X, int64_t ldx, const V* Y, int64_t ldy, const V* data, V* out, int64_t nnz,
                        int k_dim, V alpha, V beta, int ids_aligned) {
#define FSB_SDDMM_CASE(LG_)                                                                                      \
  case LG_:                                                                                                      \
    sddmm_kernel<V, VW, LG_><<<blocks, kSdThreads, 0, st>>>(indices, row_ids, X, ldx, Y, ldy, data, out, nnz,    \
                                                            k_dim, alpha, beta, ids_aligned);                   \
    break
  switch (LG) {
    FSB_SDDMM_CASE(1);
    FSB_SDDMM_CASE(2);
    FSB_SDDMM_CASE(4);
    FSB_SDDMM_CASE(8);
    FSB_SDDMM_CASE(16);
    FSB_SDDMM_CASE(32);
    default: return FSB_EINVAL;
  }
#undef FSB_SDDMM_CASE
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}

template <typename V>
static int sddmm_typed(const int32_t* indices, const int32_t* row_ids, const void* X, int64_t ldx, const void* Y,
                       int64_t ldy, const void* data, void* out, int64_t nnz, int k_dim, double alpha, double beta,
                       cudaStream_t st) {
  constexpr int VMAX = 16 / sizeof(V);
  int vw = VMAX;
  while (vw > 1 && !(k_dim % vw == 0 && ldx % vw == 0 && ldy % vw == 0 && aligned_to(X, vw * sizeof(V)) &&
                     aligned_to(Y, vw * sizeof(V))))
    vw >>= 1;
  const int need = (k_dim + vw - 1) / vw;
  int LG = 1;
  while (LG < 32 && LG < need) LG <<= 1;
  const int tile = LG == 1 ? sddmm_tile(1) : LG == 2 ? sddmm_tile(2) : LG == 4 ? sddmm_tile(4) : LG == 8 ? sddmm_tile(8)
                   : LG == 16 ? sddmm_tile(16) : sddmm_tile(32);
  const int64_t blocks = (nnz + tile - 1) / tile;
  if (blocks >= INT32_MAX) return FSB_ERANGE;
  const int ids_aligned = aligned_to(indices, 16) && aligned_to(row_ids, 16);
  const V* Xv = (const V*)X;
  const V* Yv = (const V*)Y;
  const V* dv = (const V*)data;
  V* ov = (V*)out;
  if constexpr (VMAX == 4) {
    if (vw == 4)
      return sddmm_launch<V, 4>(LG, (unsigned)blocks, st, indices, row_ids, Xv, ldx, Yv, ldy, dv, ov, nnz, k_dim,
                                (V)alpha, (V)beta, ids_aligned);
  }
  if (vw == 2)
    return sddmm_launch<V, 2>(LG, (unsigned)blocks, st, indices, row_ids, Xv, ldx, Yv, ldy, dv, ov, nnz, k_dim,
                              (V)alpha, (V)beta, ids_aligned);
  return sddmm_launch<V, 1>(LG, (unsigned)blocks, st, indices, row_ids, Xv, ldx, Yv, ldy, dv, ov, nnz, k_dim,
                            (V)alpha, (V)beta, ids_aligned);
}

}  // namespace fsb

using namespace fsb;

extern "C" int fsb_sddmm_csr(int vtype, const int32_t* indices, const int32_t* row_ids, const void* X, int64_t ldx,
                             const void* Y, int64_t ldy, const void* data, void* out, int64_t n_rows, int64_t n_cols,
                             int64_t nnz, int64_t k_dim, double alpha, double beta, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (vtype != FSB_F32 && vtype != FSB_F64) return FSB_EINVAL;
  if (n_rows < 0 || n_cols < 0 || nnz < 0 || k_dim < 0) return FSB_EINVAL;
  if (n_rows >= INT32_MAX || n_cols >= INT32_MAX || k_dim >= (1 << 24)) return FSB_ERANGE;
  if (nnz == 0) return FSB_OK;
  if (indices == nullptr || row_ids == nullptr || out == nullptr) return FSB_EINVAL;
  if (k_dim > 0 && (X == nullptr || Y == nullptr || ldx < k_dim || ldy < k_dim)) return FSB_EINVAL;
  const size_t sv = vtype == FSB_F32 ? 4 : 8;
  if (!aligned_to(X, sv) || !aligned_to(Y, sv) || !aligned_to(out, sv) || !aligned_to(data, sv) ||
      !aligned_to(indices, 4) || !aligned_to(row_ids, 4))
    return FSB_EALIGN;
  FSB_WALK_FIRST(check_entry_ids(indices, row_ids, n_rows, n_cols, nnz, st));
  if (vtype == FSB_F32)
    return sddmm_typed<float>(indices, row_ids, X, ldx, Y, ldy, data, out, nnz, (int)k_dim, alpha, beta, st);
  return sddmm_typed<double>(indices, row_ids, X, ldx, Y, ldy, data, out, nnz, (int)k_dim, alpha, beta, st);
}
