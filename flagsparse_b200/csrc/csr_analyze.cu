// CSR structure analysis (one pass over indptr, one over indices) and the nnz-tile plan.
#include "fsb_common.cuh"

namespace fsb {

enum { S_PTR_FIRST = 0, S_PTR_LAST, S_DECREASING, S_MIN_IDX, S_MAX_IDX, S_MAX_ROW, S_EMPTY, S_LONG };

__global__ void stats_init_kernel(int64_t* s) {
  s[S_PTR_FIRST] = 0;
  s[S_PTR_LAST] = 0;
  s[S_DECREASING] = 0;
  s[S_MIN_IDX] = INT64_MAX;
  s[S_MAX_IDX] = INT64_MIN;
  s[S_MAX_ROW] = 0;
  s[S_EMPTY] = 0;
  s[S_LONG] = 0;
}

__device__ __forceinline__ long long warp_max(long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    long long u = __shfl_xor_sync(0xffffffffu, v, o);
    v = u > v ? u : v;
  }
  return v;
}
__device__ __forceinline__ long long warp_min(long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    long long u = __shfl_xor_sync(0xffffffffu, v, o);
    v = u < v ? u : v;
  }
  return v;
}
__device__ __forceinline__ long long warp_sum(long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// grid-stride over rows; one atomic per warp per statistic that changed
template <typename P>
__global__ void __launch_bounds__(256) indptr_stats_kernel(const P* __restrict__ ptr, int64_t n_rows,
                                                          int64_t long_len, int64_t* __restrict__ s) {
  long long mx = 0, dec = 0, empty = 0, lng = 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_rows; i += stride) {
    long long len = (long long)ptr[i + 1] - (long long)ptr[i];
    mx = len > mx ? len : mx;
    dec += len < 0;
    empty += len == 0;
    lng += len > long_len;
  }
  mx = warp_max(mx);
  dec = warp_sum(dec);
  empty = warp_sum(empty);
  lng = warp_sum(lng);
  if ((threadIdx.x & 31) == 0) {
    if (mx > 0) atomicMax(reinterpret_cast<long long*>(s + S_MAX_ROW), mx);
    if (dec) atomicAdd(reinterpret_cast<unsigned long long*>(s + S_DECREASING), (unsigned long long)dec);
    if (empty) atomicAdd(reinterpret_cast<unsigned long long*>(s + S_EMPTY), (unsigned long long)empty);
    if (lng) atomicAdd(reinterpret_cast<unsigned long long*>(s + S_LONG), (unsigned long long)lng);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    s[S_PTR_FIRST] = (int64_t)ptr[0];
    s[S_PTR_LAST] = (int64_t)ptr[n_rows];
  }
}

template <typename I>
__global__ void __launch_bounds__(256) index_range_kernel(const I* __restrict__ idx, int64_t nnz,
                                                         int64_t* __restrict__ s) {
  long long mn = INT64_MAX, mx = INT64_MIN;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nnz; i += stride) {
    long long c = (long long)idx[i];
    mn = c < mn ? c : mn;
    mx = c > mx ? c : mx;
  }
  mn = warp_min(mn);
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) {
    if (mn != INT64_MAX) atomicMin(reinterpret_cast<long long*>(s + S_MIN_IDX), mn);
    if (mx != INT64_MIN) atomicMax(reinterpret_cast<long long*>(s + S_MAX_IDX), mx);
  }
}

// tile_row[t] = (first j with ptr[j] > t*T) - 1, i.e. the row that holds nnz number t*T
template <typename P>
__global__ void __launch_bounds__(256) tile_plan_kernel(const P* __restrict__ ptr, int64_t n_rows,
                                                       int64_t n_tiles, int64_t tile_nnz,
                                                       int32_t* __restrict__ tile_row) {
  int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t > n_tiles) return;
  if (t == 0) { tile_row[0] = 0; return; }
  if (t == n_tiles) { tile_row[t] = (int32_t)n_rows; return; }
  const long long v = (long long)t * tile_nnz;
  int64_t lo = 0, hi = n_rows + 1;  // search over ptr[0..n_rows]; ptr[0] = 0 <= v, ptr[n_rows] = nnz > v
  while (lo < hi) {
    int64_t mid = (lo + hi) >> 1;
    if ((long long)ptr[mid] > v) hi = mid; else lo = mid + 1;
  }
  tile_row[t] = (int32_t)(lo - 1);
}

static int grid_for(int64_t n, int threads, int cap) {
  int64_t g = (n + threads - 1) / threads;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return (int)g;
}

}  // namespace fsb

using namespace fsb;

extern "C" int fsb_version(void) { return FSB_VERSION; }

extern "C" int fsb_csr_analyze(int itype, int ptype, const void* indices, const void* indptr,
                               int64_t n_rows, int64_t nnz, int64_t* stats, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if ((itype != FSB_I32 && itype != FSB_I64) || (ptype != FSB_I32 && ptype != FSB_I64)) return FSB_EINVAL;
  if (n_rows < 0 || nnz < 0 || stats == nullptr || indptr == nullptr) return FSB_EINVAL;
  if (nnz > 0 && indices == nullptr) return FSB_EINVAL;
  if (n_rows >= INT32_MAX) return FSB_ERANGE;
  stats_init_kernel<<<1, 1, 0, stream>>>(stats);
  FSB_RETURN_IF_LAUNCH_FAILED();
  // "long" = more than 32x the mean row length (at least 64)
  int64_t mean_up = n_rows > 0 ? (nnz + n_rows - 1) / n_rows : 0;
  int64_t long_len = mean_up * 32 < 64 ? 64 : mean_up * 32;
  const int cap = 148 * 16;  // a few resident CTAs per SM, grid-stride over the rest
  {
    int g = grid_for(n_rows, 256, cap);
    if (ptype == FSB_I32)
      indptr_stats_kernel<int32_t><<<g, 256, 0, stream>>>((const int32_t*)indptr, n_rows, long_len, stats);
    else
      indptr_stats_kernel<int64_t><<<g, 256, 0, stream>>>((const int64_t*)indptr, n_rows, long_len, stats);
    FSB_RETURN_IF_LAUNCH_FAILED();
  }
  if (nnz > 0) {
    int g = grid_for(nnz, 256, cap);
    if (itype == FSB_I32)
      index_range_kernel<int32_t><<<g, 256, 0, stream>>>((const int32_t*)indices, nnz, stats);
    else
      index_range_kernel<int64_t><<<g, 256, 0, stream>>>((const int64_t*)indices, nnz, stats);
    FSB_RETURN_IF_LAUNCH_FAILED();
  }
  return FSB_OK;
}

extern "C" int64_t fsb_csr_num_tiles(int64_t nnz, int tile_nnz) {
  if (nnz <= 0 || tile_nnz <= 0) return 0;
  return (nnz + tile_nnz - 1) / tile_nnz;
}

extern "C" int fsb_csr_tile_plan(int ptype, const void* indptr, int64_t n_rows, int64_t nnz, int tile_nnz,
                                 int32_t* tile_row, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (ptype != FSB_I32 && ptype != FSB_I64) return FSB_EINVAL;
  if (n_rows < 0 || nnz < 0 || tile_nnz <= 0 || (tile_nnz & (tile_nnz - 1)) != 0) return FSB_EINVAL;
  if (indptr == nullptr || tile_row == nullptr) return FSB_EINVAL;
  if (n_rows >= INT32_MAX) return FSB_ERANGE;
  const int64_t n_tiles = fsb_csr_num_tiles(nnz, tile_nnz);
  if (n_tiles >= INT32_MAX) return FSB_ERANGE;
  const int64_t n = n_tiles + 1;
  const int g = (int)((n + 255) / 256);
  if (ptype == FSB_I32)
    tile_plan_kernel<int32_t><<<g, 256, 0, stream>>>((const int32_t*)indptr, n_rows, n_tiles, tile_nnz, tile_row);
  else
    tile_plan_kernel<int64_t><<<g, 256, 0, stream>>>((const int64_t*)indptr, n_rows, n_tiles, tile_nnz, tile_row);
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}
