// Shared device helpers for libfsb (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "fsb.h"

namespace fsb {

inline int cuda_rc(cudaError_t e) { return e == cudaSuccess ? FSB_OK : FSB_CUDA_ERROR_BASE + (int)e; }

#define FSB_RETURN_IF_LAUNCH_FAILED()                      \
  do {                                                     \
    cudaError_t e__ = cudaGetLastError();                  \
    if (e__ != cudaSuccess) return ::fsb::cuda_rc(e__);    \
  } while (0)

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
__device__ __forceinline__ bool aligned_to_dev(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- the checking build: entry points walk their index arrays first (bounds_check.cu) ----------------
#ifdef FSB_BOUNDS_CHECK
int check_csr(int itype, int ptype, const void* indices, const void* indptr, int64_t n_rows, int64_t n_cols,
              int64_t nnz, cudaStream_t st);
int check_entry_ids(const int32_t* indices, const int32_t* row_ids, int64_t n_rows, int64_t n_cols, int64_t nnz,
                    cudaStream_t st);
int check_panel(const uint32_t* rc_words, const int32_t* unit_piece_ptr, const int32_t* unit_chunk,
                const int32_t* owner_unit_ptr, int n_owners, int slots, int max_row, int chunk_cols, int n_buffers,
                int64_t n_cols, cudaStream_t st);
#define FSB_WALK_FIRST(call)                       \
  do {                                             \
    const int rc__ = ::fsb::call;                  \
    if (rc__ != FSB_OK) return rc__;               \
  } while (0)
#else
#define FSB_WALK_FIRST(call) \
  do {                       \
  } while (0)
#endif

// ---- streaming (read-once) loads: evict-first so that A does not push x / B out of L2 -------------
template <typename T>
__device__ __forceinline__ T ld_stream(const T* p) {
  return __ldcs(p);
}

// four consecutive elements, 16-byte (f32/i32) or 2x16-byte (f64/i64) vector loads
__device__ __forceinline__ void ld_stream4(const float* p, float (&v)[4]) {
  float4 t = __ldcs(reinterpret_cast<const float4*>(p));
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void ld_stream4(const double* p, double (&v)[4]) {
  double2 a = __ldcs(reinterpret_cast<const double2*>(p));
  double2 b = __ldcs(reinterpret_cast<const double2*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void ld_stream4(const int32_t* p, int32_t (&v)[4]) {
  int4 t = __ldcs(reinterpret_cast<const int4*>(p));
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void ld_stream4(const int64_t* p, int64_t (&v)[4]) {
  longlong2 a = __ldcs(reinterpret_cast<const longlong2*>(p));
  longlong2 b = __ldcs(reinterpret_cast<const longlong2*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

__device__ __forceinline__ void st_shared4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void st_shared4(double* p, const double (&v)[4]) {
  *reinterpret_cast<double2*>(p) = make_double2(v[0], v[1]);
  *(reinterpret_cast<double2*>(p) + 1) = make_double2(v[2], v[3]);
}

// ---- dense-row vector access for SpMM (VW elements, VW*sizeof(V) <= 16 bytes) ---------------------
template <typename V, int VW>
struct Vec;
template <> struct Vec<float, 1> { typedef float type; };
template <> struct Vec<float, 2> { typedef float2 type; };
template <> struct Vec<float, 4> { typedef float4 type; };
template <> struct Vec<double, 1> { typedef double type; };
template <> struct Vec<double, 2> { typedef double2 type; };

template <typename V, int VW>
__device__ __forceinline__ void ld_dense(const V* p, V (&v)[VW]) {
  typedef typename Vec<V, VW>::type VT;
  VT t = __ldg(reinterpret_cast<const VT*>(p));
  const V* e = reinterpret_cast<const V*>(&t);
#pragma unroll
  for (int i = 0; i < VW; ++i) v[i] = e[i];
}
template <typename V, int VW>
__device__ __forceinline__ void ld_dense_stream(const V* p, V (&v)[VW]) {
  typedef typename Vec<V, VW>::type VT;
  VT t = __ldcs(reinterpret_cast<const VT*>(p));
  const V* e = reinterpret_cast<const V*>(&t);
#pragma unroll
  for (int i = 0; i < VW; ++i) v[i] = e[i];
}
template <typename V, int VW>
__device__ __forceinline__ void st_dense_stream(V* p, const V (&v)[VW]) {
  typedef typename Vec<V, VW>::type VT;
  VT t;
  V* e = reinterpret_cast<V*>(&t);
#pragma unroll
  for (int i = 0; i < VW; ++i) e[i] = v[i];
  __stcs(reinterpret_cast<VT*>(p), t);
}

__device__ __forceinline__ int pow2_floor(int v) { return v <= 1 ? 1 : (1 << (31 - __clz(v))); }

}  // namespace fsb
