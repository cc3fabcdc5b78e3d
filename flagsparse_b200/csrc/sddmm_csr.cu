// CSR SDDMM for sm_100a: out[p] = alpha * dot(X[row(p), :], Y[col(p), :]) + beta * data[p] for every entry p of a
// CSR pattern (X is n_rows x K, Y is n_cols x K, both row-major with a row stride).
//
// A group of LG lanes (LG = K / VW rounded up to a power of two, at most 32; VW = elements per 128-bit access)
// owns a run of consecutive entries.  Consecutive entries mostly share their row, so the lanes keep their slice
// of X's row in registers and reload it only when the row changes (the row of an entry comes from the row-id
// array built at prepare time, 4 bytes per entry); the slice of Y's row is gathered through the read-only path,
// two entries in flight per group (rows that fit one step); products are summed per lane, then across the group with a shuffle tree, and
// lane 0 writes the result with a streaming store.  Rows of X longer than LG * VW elements are walked in several
// steps.  CUDA-core work on purpose: one dot product per entry over gathered rows is about 0.5 flop per byte.
#include "fsb_common.cuh"

namespace fsb {

constexpr int kSdThreads = 256;
constexpr int kSdEntriesPerGroup = 8;   // consecutive entries one group walks

template <typename V, int VW>
__global__ void __launch_bounds__(kSdThreads)
sddmm_kernel(const int32_t* __restrict__ indices, const int32_t* __restrict__ row_ids, const V* __restrict__ X,
             int64_t ldx, const V* __restrict__ Y, int64_t ldy, const V* __restrict__ data, V* __restrict__ out,
             int64_t nnz, int k_dim, int LG, V alpha, V beta) {
  const int lane = threadIdx.x & (LG - 1);
  const int64_t group = ((int64_t)blockIdx.x * kSdThreads + threadIdx.x) / LG;
  const int64_t p0 = group * kSdEntriesPerGroup;
  if (p0 >= nnz) return;   // whole groups leave together: the shuffles below stay inside a group
  const int n = (int)((nnz - p0) < kSdEntriesPerGroup ? (nnz - p0) : kSdEntriesPerGroup);
  const unsigned gmask = LG == 32 ? 0xffffffffu : (((1u << LG) - 1u) << ((threadIdx.x & 31) & ~(LG - 1)));
  const int step = LG * VW;
  const bool one_step = k_dim <= step;
  int32_t cur_row = -1;
  V xr[VW];
#pragma unroll
  for (int i = 0; i < VW; ++i) xr[i] = (V)0;
  auto finish = [&](int64_t p, V acc) {
    for (int o = LG >> 1; o > 0; o >>= 1) acc += __shfl_down_sync(gmask, acc, o, LG);
    if (lane == 0) {
      V v = acc * alpha;
      if (data != nullptr) v += __ldcs(data + p) * beta;
      __stcs(out + p, v);
    }
  };
  if (one_step) {
    const int k = lane * VW;
    const bool mine = k < k_dim;
    for (int e = 0; e < n; e += 2) {
      // two entries at a time: both slices of Y are requested before either is used
      const int64_t p = p0 + e;
      const bool two = e + 1 < n;
      const int32_t ra = __ldg(row_ids + p), rb = two ? __ldg(row_ids + p + 1) : ra;
      const int64_t ca = (int64_t)__ldg(indices + p), cb = two ? (int64_t)__ldg(indices + p + 1) : ca;
      V ya[VW], yb[VW], xb[VW];
#pragma unroll
      for (int i = 0; i < VW; ++i) ya[i] = yb[i] = xb[i] = (V)0;
      if (mine) {
        ld_dense<V, VW>(Y + ca * ldy + k, ya);
        if (two) ld_dense<V, VW>(Y + cb * ldy + k, yb);
        if (ra != cur_row) ld_dense<V, VW>(X + (int64_t)ra * ldx + k, xr);
        if (rb != ra) ld_dense<V, VW>(X + (int64_t)rb * ldx + k, xb);
      }
      cur_row = ra;
      V acc_a = (V)0, acc_b = (V)0;
#pragma unroll
      for (int i = 0; i < VW; ++i) acc_a += xr[i] * ya[i];
      if (rb != ra) {
#pragma unroll
        for (int i = 0; i < VW; ++i) xr[i] = xb[i];
        cur_row = rb;
      }
#pragma unroll
      for (int i = 0; i < VW; ++i) acc_b += xr[i] * yb[i];
      finish(p, acc_a);
      if (two) finish(p + 1, acc_b);
    }
  } else {
    for (int e = 0; e < n; ++e) {
      const int64_t p = p0 + e;
      const int32_t r = __ldg(row_ids + p);
      const int64_t c = (int64_t)__ldg(indices + p);
      V acc = (V)0;
      for (int k = lane * VW; k < k_dim; k += step) {
        V xs[VW], yr[VW];
        ld_dense<V, VW>(X + (int64_t)r * ldx + k, xs);
        ld_dense<V, VW>(Y + c * ldy + k, yr);
#pragma unroll
        for (int i = 0; i < VW; ++i) acc += xs[i] * yr[i];
      }
      finish(p, acc);
    }
  }
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
  const int64_t groups = (nnz + kSdEntriesPerGroup - 1) / kSdEntriesPerGroup;
  const int64_t blocks = (groups * LG + kSdThreads - 1) / kSdThreads;
  if (blocks >= INT32_MAX) return FSB_ERANGE;
#define FSB_SDDMM_LAUNCH(VW_)                                                                                  \
  sddmm_kernel<V, VW_><<<(unsigned)blocks, kSdThreads, 0, st>>>(indices, row_ids, (const V*)X, ldx, (const V*)Y, \
                                                                ldy, (const V*)data, (V*)out, nnz, k_dim, LG,   \
                                                                (V)alpha, (V)beta)
  if constexpr (VMAX == 4) {
    if (vw == 4) { FSB_SDDMM_LAUNCH(4); FSB_RETURN_IF_LAUNCH_FAILED(); return FSB_OK; }
  }
  if (vw == 2) FSB_SDDMM_LAUNCH(2); else FSB_SDDMM_LAUNCH(1);
#undef FSB_SDDMM_LAUNCH
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
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
  if (vtype == FSB_F32)
    return sddmm_typed<float>(indices, row_ids, X, ldx, Y, ldy, data, out, nnz, (int)k_dim, alpha, beta, st);
  return sddmm_typed<double>(indices, row_ids, X, ldx, Y, ldy, data, out, nnz, (int)k_dim, alpha, beta, st);
}
