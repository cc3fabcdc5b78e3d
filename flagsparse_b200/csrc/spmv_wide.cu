// CSR SpMV and SpMM for the value types the float32 / float64 kernels do not stream themselves: float16 and bfloat16
// values (2 bytes per entry in memory, products and sums in float32, the dense operand and the result in float32: the
// caller widens x / B once per call and rounds y / C once, as the reference's base path does) and complex64 /
// complex128 values (interleaved real and imaginary parts, one pass over the matrix, complex multiply-add in the
// component precision).  The values are read as they are stored -- no widened or split copy of the matrix exists
// anywhere.  Rows are summed in a fixed order: bit-reproducible.
//
// SpMV: L lanes per row (L = 2 .. 32 from the mean row length), every lane walks the row with stride L, two partial
// sums, a shuffle tree, lane 0 stores.  SpMM: a group of LN lanes per row (LN = dense width rounded up to a power of
// two, at most 32; wider B in column tiles of 32 along gridDim.y), every lane owns one column of C, walks the row's
// entries (value and column index are the same address for the whole group: one broadcast load) and gathers its
// element of B's row, two entries in flight.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fsb_common.cuh"

namespace fsb {

constexpr int kWideThreads = 256;

// How one stored value type is computed with: accumulator type, element type of x and y, multiply-add, shuffle.
template <typename S>
struct WideOps;

template <>
struct WideOps<__half> {
  typedef float Acc;
  typedef float Dense;
  static __device__ __forceinline__ void fma(Acc& acc, __half a, Dense b) { acc = fmaf(__half2float(a), b, acc); }
};
template <>
struct WideOps<__nv_bfloat16> {
  typedef float Acc;
  typedef float Dense;
  static __device__ __forceinline__ void fma(Acc& acc, __nv_bfloat16 a, Dense b) {
    acc = fmaf(__bfloat162float(a), b, acc);
  }
};
template <>
struct WideOps<float2> {
  typedef float2 Acc;
  typedef float2 Dense;
  static __device__ __forceinline__ void fma(Acc& acc, float2 a, Dense b) {
    acc.x += a.x * b.x - a.y * b.y;
    acc.y += a.x * b.y + a.y * b.x;
  }
};
template <>
struct WideOps<double2> {
  typedef double2 Acc;
  typedef double2 Dense;
  static __device__ __forceinline__ void fma(Acc& acc, double2 a, Dense b) {
    acc.x += a.x * b.x - a.y * b.y;
    acc.y += a.x * b.y + a.y * b.x;
  }
};

__device__ __forceinline__ float w_zero(float*) { return 0.f; }
__device__ __forceinline__ float2 w_zero(float2*) { return make_float2(0.f, 0.f); }
__device__ __forceinline__ double2 w_zero(double2*) { return make_double2(0.0, 0.0); }
__device__ __forceinline__ float w_add(float a, float b) { return a + b; }
__device__ __forceinline__ float2 w_add(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ double2 w_add(double2 a, double2 b) { return make_double2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ float w_down(float v, int o) { return __shfl_down_sync(0xffffffffu, v, o); }
__device__ __forceinline__ float2 w_down(float2 v, int o) {
  return make_float2(__shfl_down_sync(0xffffffffu, v.x, o), __shfl_down_sync(0xffffffffu, v.y, o));
}
__device__ __forceinline__ double2 w_down(double2 v, int o) {
  return make_double2(__shfl_down_sync(0xffffffffu, v.x, o), __shfl_down_sync(0xffffffffu, v.y, o));
}

template <typename S, typename P, int L>
__global__ void __launch_bounds__(kWideThreads)
spmv_wide_kernel(const S* __restrict__ data, const int32_t* __restrict__ idx, const P* __restrict__ ptr,
                 const typename WideOps<S>::Dense* __restrict__ x, typename WideOps<S>::Dense* __restrict__ y,
                 int64_t n_rows) {
  typedef typename WideOps<S>::Acc A;
  const int64_t gtid = (int64_t)blockIdx.x * kWideThreads + threadIdx.x;
  const int64_t row = gtid / L;
  const int lane = (int)(gtid % L);
  int64_t s = 0, e = 0;
  if (row < n_rows) {
    s = (int64_t)ptr[row];
    e = (int64_t)ptr[row + 1];
  }
  A acc0 = w_zero((A*)nullptr), acc1 = w_zero((A*)nullptr);
  int64_t p = s + lane;
  for (; p + L < e; p += 2 * L) {
    const S a0 = __ldcs(data + p), a1 = __ldcs(data + p + L);
    const int64_t c0 = (int64_t)__ldcs(idx + p), c1 = (int64_t)__ldcs(idx + p + L);
    WideOps<S>::fma(acc0, a0, __ldg(x + c0));
    WideOps<S>::fma(acc1, a1, __ldg(x + c1));
  }
  if (p < e) WideOps<S>::fma(acc0, __ldcs(data + p), __ldg(x + (int64_t)__ldcs(idx + p)));
  A acc = w_add(acc0, acc1);
#pragma unroll
  for (int o = L >> 1; o > 0; o >>= 1) acc = w_add(acc, w_down(acc, o));
  if (lane == 0 && row < n_rows) y[row] = acc;
}

template <typename S, typename P>
__global__ void __launch_bounds__(kWideThreads)
spmm_wide_kernel(const S* __restrict__ data, const int32_t* __restrict__ idx, const P* __restrict__ ptr,
                 const typename WideOps<S>::Dense* __restrict__ B, int64_t ldb,
                 typename WideOps<S>::Dense* __restrict__ C, int64_t ldc, int64_t n_rows, int n_dense, int LN) {
  typedef typename WideOps<S>::Acc A;
  const int lane = threadIdx.x % LN;
  const int64_t row = (int64_t)blockIdx.x * (kWideThreads / LN) + threadIdx.x / LN;
  const int col = (int)blockIdx.y * LN + lane;
  if (row >= n_rows || col >= n_dense) return;   // no shuffles below: threads may leave on their own
  const int64_t s = (int64_t)ptr[row], e = (int64_t)ptr[row + 1];
  A acc0 = w_zero((A*)nullptr), acc1 = w_zero((A*)nullptr);
  int64_t p = s;
  for (; p + 1 < e; p += 2) {
    const S a0 = __ldg(data + p), a1 = __ldg(data + p + 1);
    const int64_t c0 = (int64_t)__ldg(idx + p), c1 = (int64_t)__ldg(idx + p + 1);
    WideOps<S>::fma(acc0, a0, __ldg(B + c0 * ldb + col));
    WideOps<S>::fma(acc1, a1, __ldg(B + c1 * ldb + col));
  }
  if (p < e) WideOps<S>::fma(acc0, __ldg(data + p), __ldg(B + (int64_t)__ldg(idx + p) * ldb + col));
  C[row * ldc + col] = w_add(acc0, acc1);
}

template <typename S, typename P>
static int wide_launch(const void* data, const int32_t* idx, const void* ptr, const void* x, void* y, int64_t n_rows,
                       int64_t nnz, cudaStream_t st) {
  typedef typename WideOps<S>::Dense D;
  const int64_t mean = n_rows > 0 ? nnz / n_rows : 0;
  int L = 2;
  while (L < 32 && 8 * L < mean + 3) L <<= 1;
  const int64_t blocks = (n_rows * L + kWideThreads - 1) / kWideThreads;
  if (blocks >= INT32_MAX) return FSB_ERANGE;
#define FSB_WIDE_CASE(L_)                                                                                         \
  case L_:                                                                                                        \
    spmv_wide_kernel<S, P, L_><<<(unsigned)blocks, kWideThreads, 0, st>>>((const S*)data, idx, (const P*)ptr,     \
                                                                          (const D*)x, (D*)y, n_rows);           \
    break
  switch (L) {
    FSB_WIDE_CASE(2);
    FSB_WIDE_CASE(4);
    FSB_WIDE_CASE(8);
    FSB_WIDE_CASE(16);
    default:
      FSB_WIDE_CASE(32);
  }
#undef FSB_WIDE_CASE
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}

}  // namespace fsb

using namespace fsb;

extern "C" int fsb_spmv_csr_wide(int vtype, int ptype, const void* data, const int32_t* indices, const void* indptr,
                                 const void* x, void* y, int64_t n_rows, int64_t n_cols, int64_t nnz, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (vtype != FSB_F16 && vtype != FSB_BF16 && vtype != FSB_C64 && vtype != FSB_C128) return FSB_EINVAL;
  if (ptype != FSB_I32 && ptype != FSB_I64) return FSB_EINVAL;
  if (n_rows < 0 || n_cols < 0 || nnz < 0) return FSB_EINVAL;
  if (n_rows >= INT32_MAX || n_cols >= INT32_MAX) return FSB_ERANGE;
  if (n_rows == 0) return FSB_OK;
  if (indptr == nullptr || y == nullptr || (nnz > 0 && (data == nullptr || indices == nullptr || x == nullptr)))
    return FSB_EINVAL;
  const size_t sv = vtype == FSB_C128 ? 16 : (vtype == FSB_C64 ? 8 : 2);    // stored value
  const size_t sd = vtype == FSB_C128 ? 16 : (vtype == FSB_C64 ? 8 : 4);    // element of x and y
  if (!aligned_to(data, sv) || !aligned_to(x, sd) || !aligned_to(y, sd) || !aligned_to(indices, 4) ||
      !aligned_to(indptr, ptype == FSB_I32 ? 4 : 8))
    return FSB_EALIGN;
  FSB_WALK_FIRST(check_csr(FSB_I32, ptype, indices, indptr, n_rows, n_cols, nnz, st));
#define FSB_WIDE_TYPE(S_)                                                                                     \
  return ptype == FSB_I32 ? wide_launch<S_, int32_t>(data, indices, indptr, x, y, n_rows, nnz, st)            \
                          : wide_launch<S_, int64_t>(data, indices, indptr, x, y, n_rows, nnz, st)
  switch (vtype) {
    case FSB_F16: FSB_WIDE_TYPE(__half);
    case FSB_BF16: FSB_WIDE_TYPE(__nv_bfloat16);
    case FSB_C64: FSB_WIDE_TYPE(float2);
    default: FSB_WIDE_TYPE(double2);
  }
#undef FSB_WIDE_TYPE
}

template <typename S, typename P>
static int wide_spmm_launch(const void* data, const int32_t* idx, const void* ptr, const void* B, int64_t ldb, void* C,
                            int64_t ldc, int64_t n_rows, int n_dense, cudaStream_t st) {
  typedef typename WideOps<S>::Dense D;
  int LN = 1;
  while (LN < 32 && LN < n_dense) LN <<= 1;
  const int64_t gx = (n_rows + kWideThreads / LN - 1) / (kWideThreads / LN);
  const int64_t gy = (n_dense + LN - 1) / LN;
  if (gx >= INT32_MAX || gy > 65535) return FSB_ERANGE;
  spmm_wide_kernel<S, P><<<dim3((unsigned)gx, (unsigned)gy), kWideThreads, 0, st>>>(
      (const S*)data, idx, (const P*)ptr, (const D*)B, ldb, (D*)C, ldc, n_rows, n_dense, LN);
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}

extern "C" int fsb_spmm_csr_wide(int vtype, int ptype, const void* data, const int32_t* indices, const void* indptr,
                                 const void* B, int64_t ldb, void* C, int64_t ldc, int64_t n_rows, int64_t n_cols,
                                 int64_t n_dense, int64_t nnz, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (vtype != FSB_F16 && vtype != FSB_BF16 && vtype != FSB_C64 && vtype != FSB_C128) return FSB_EINVAL;
  if (ptype != FSB_I32 && ptype != FSB_I64) return FSB_EINVAL;
  if (n_rows < 0 || n_cols < 0 || nnz < 0 || n_dense < 0 || ldb < n_dense || ldc < n_dense) return FSB_EINVAL;
  if (n_rows >= INT32_MAX || n_cols >= INT32_MAX || n_dense >= (1 << 21)) return FSB_ERANGE;
  if (n_rows == 0 || n_dense == 0) return FSB_OK;
  if (indptr == nullptr || C == nullptr || (nnz > 0 && (data == nullptr || indices == nullptr || B == nullptr)))
    return FSB_EINVAL;
  const size_t sv = vtype == FSB_C128 ? 16 : (vtype == FSB_C64 ? 8 : 2);
  const size_t sd = vtype == FSB_C128 ? 16 : (vtype == FSB_C64 ? 8 : 4);
  if (!aligned_to(data, sv) || !aligned_to(B, sd) || !aligned_to(C, sd) || !aligned_to(indices, 4) ||
      !aligned_to(indptr, ptype == FSB_I32 ? 4 : 8))
    return FSB_EALIGN;
  FSB_WALK_FIRST(check_csr(FSB_I32, ptype, indices, indptr, n_rows, n_cols, nnz, st));
#define FSB_WIDE_TYPE(S_)                                                                                         \
  return ptype == FSB_I32                                                                                         \
             ? wide_spmm_launch<S_, int32_t>(data, indices, indptr, B, ldb, C, ldc, n_rows, (int)n_dense, st)      \
             : wide_spmm_launch<S_, int64_t>(data, indices, indptr, B, ldb, C, ldc, n_rows, (int)n_dense, st)
  switch (vtype) {
    case FSB_F16: FSB_WIDE_TYPE(__half);
    case FSB_BF16: FSB_WIDE_TYPE(__nv_bfloat16);
    case FSB_C64: FSB_WIDE_TYPE(float2);
    default: FSB_WIDE_TYPE(double2);
  }
#undef FSB_WIDE_TYPE
}
