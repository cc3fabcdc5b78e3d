// The checking build of libfsb (compiled with -DFSB_BOUNDS_CHECK into libfsb_check.so).
//
// Every product entry point of the checking build first walks the index arrays it was given -- column
// indices, row pointers, row ids, the packed words and tables of a panel layout -- with the kernels of this
// file.  An index that would take a later load or store out of its array is recorded (what, where, value, limit),
// the entry point returns FSB_EBOUNDS and launches nothing else: no trap, no fault, the context stays usable.
// fsb_bounds_check_report() hands the record of the last refused call to the host.  The ordinary build compiles
// the same entry points without the walk; there the two functions below report "not a checking build".
#include "fsb_common.cuh"

namespace fsb {

#ifdef FSB_BOUNDS_CHECK

// {violations seen, kind of the first one recorded, its position in the array, the value found, the limit}
__device__ unsigned long long g_bad[5];
static long long g_last_report[5] = {0, 0, 0, 0, 0};

__device__ __forceinline__ void note(int kind, long long where, long long value, long long limit) {
  if (atomicAdd(&g_bad[0], 1ull) == 0ull) {
    g_bad[1] = (unsigned long long)kind;
    g_bad[2] = (unsigned long long)where;
    g_bad[3] = (unsigned long long)value;
    g_bad[4] = (unsigned long long)limit;
  }
}

constexpr int kCheckThreads = 256;
constexpr int kCheckBlocks = 148 * 8;

template <typename I, typename P>
__global__ void __launch_bounds__(kCheckThreads)
check_csr_kernel(const I* __restrict__ idx, const P* __restrict__ ptr, int64_t n_rows, int64_t n_cols, int64_t nnz) {
  const int64_t stride = (int64_t)gridDim.x * kCheckThreads;
  const int64_t first = (int64_t)blockIdx.x * kCheckThreads + threadIdx.x;
  if (idx != nullptr) {
    for (int64_t i = first; i < nnz; i += stride) {
      const long long c = (long long)idx[i];
      if (c < 0 || c >= n_cols) note(FSB_BAD_COLUMN, i, c, n_cols);
    }
  }
  if (ptr != nullptr) {
    for (int64_t r = first; r <= n_rows; r += stride) {
      const long long p = (long long)ptr[r];
      if (p < 0 || p > nnz) {
        note(FSB_BAD_ROW_POINTER, r, p, nnz);
      } else if (r < n_rows) {
        const long long q = (long long)ptr[r + 1];
        if (q < p) note(FSB_ROW_POINTER_DECREASES, r + 1, q, p);
      }
    }
  }
}

__global__ void __launch_bounds__(kCheckThreads)
check_row_ids_kernel(const int32_t* __restrict__ row_ids, int64_t n_rows, int64_t nnz) {
  const int64_t stride = (int64_t)gridDim.x * kCheckThreads;
  for (int64_t i = (int64_t)blockIdx.x * kCheckThreads + threadIdx.x; i < nnz; i += stride) {
    const long long r = row_ids[i];
    if (r < 0 || r >= n_rows) note(FSB_BAD_ROW_ID, i, r, n_rows);
  }
}

// A panel layout: `owner_unit_ptr` (n_owners + 1 entries) is rb_unit_ptr or cta_unit_ptr.  The tables are walked
// only as far as the entries before them allow (a bad count ends the walk).
__global__ void __launch_bounds__(kCheckThreads)
check_panel_kernel(const uint32_t* __restrict__ rc, const int32_t* __restrict__ unit_piece_ptr,
                   const int32_t* __restrict__ unit_chunk, const int32_t* __restrict__ owner_unit_ptr, int n_owners,
                   int slots, uint32_t max_row, uint32_t n_x_slots, int64_t n_chunks) {
  const int64_t stride = (int64_t)gridDim.x * kCheckThreads;
  const int64_t first = (int64_t)blockIdx.x * kCheckThreads + threadIdx.x;
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  for (int64_t b = threadIdx.x; b < n_owners; b += kCheckThreads) {   // every CTA looks at the whole (short) table
    const int u0 = owner_unit_ptr[b], u1 = owner_unit_ptr[b + 1];
    if (u0 < 0 || u1 < u0) {
      if (blockIdx.x == 0) note(FSB_BAD_UNIT_TABLE, b, u1, u0);
      ok = 0;
    }
  }
  __syncthreads();
  if (!ok) return;
  const int64_t n_units = owner_unit_ptr[n_owners];
  __syncthreads();
  for (int64_t u = threadIdx.x; u < n_units; u += kCheckThreads) {
    const int p0 = unit_piece_ptr[u], p1 = unit_piece_ptr[u + 1];
    if (p0 < 0 || p1 < p0) {
      if (blockIdx.x == 0) note(FSB_BAD_UNIT_TABLE, u, p1, p0);
      ok = 0;
    }
    const long long c = unit_chunk[u];
    if ((c < 0 || c >= n_chunks) && blockIdx.x == 0) note(FSB_BAD_CHUNK, u, c, n_chunks);
  }
  __syncthreads();
  if (!ok) return;
  const int64_t n_slots = (int64_t)unit_piece_ptr[n_units] * slots;
  for (int64_t s = first; s < n_slots; s += stride) {
    const uint32_t w = rc[s];
    if ((w >> 16) > max_row) note(FSB_BAD_SLOT_ROW, s, (long long)(w >> 16), (long long)max_row);
    if ((w & 0xffffu) >= n_x_slots) note(FSB_BAD_SLOT_COLUMN, s, (long long)(w & 0xffffu), (long long)n_x_slots);
  }
}

static int begin_check(cudaStream_t st, void** rec) {
  cudaError_t e = cudaGetSymbolAddress(rec, g_bad);
  if (e != cudaSuccess) return cuda_rc(e);
  return cuda_rc(cudaMemsetAsync(*rec, 0, sizeof(unsigned long long) * 5, st));
}

// Waits for the walk and reads its record; FSB_EBOUNDS when something was recorded.
static int end_check(cudaStream_t st, void* rec) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_rc(e);
  unsigned long long host[5];
  e = cudaMemcpyAsync(host, rec, sizeof(host), cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) return cuda_rc(e);
  e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_rc(e);
  if (host[0] == 0) return FSB_OK;
  for (int i = 0; i < 5; ++i) g_last_report[i] = (long long)host[i];
  return FSB_EBOUNDS;
}

static unsigned grid_for(int64_t n) {
  const int64_t g = (n + kCheckThreads - 1) / kCheckThreads;
  return (unsigned)(g < 1 ? 1 : (g > kCheckBlocks ? kCheckBlocks : g));
}

int check_csr(int itype, int ptype, const void* indices, const void* indptr, int64_t n_rows, int64_t n_cols,
              int64_t nnz, cudaStream_t st) {
  if (n_rows < 0 || nnz < 0 || (indices == nullptr && indptr == nullptr)) return FSB_OK;  // the entry point refuses these
  void* rec = nullptr;
  int rc = begin_check(st, &rec);
  if (rc != FSB_OK) return rc;
  const unsigned g = grid_for(nnz > n_rows + 1 ? nnz : n_rows + 1);
  if (itype == FSB_I32 && ptype == FSB_I32)
    check_csr_kernel<int32_t, int32_t><<<g, kCheckThreads, 0, st>>>((const int32_t*)indices, (const int32_t*)indptr,
                                                                    n_rows, n_cols, nnz);
  else if (itype == FSB_I32)
    check_csr_kernel<int32_t, int64_t><<<g, kCheckThreads, 0, st>>>((const int32_t*)indices, (const int64_t*)indptr,
                                                                    n_rows, n_cols, nnz);
  else if (ptype == FSB_I32)
    check_csr_kernel<int64_t, int32_t><<<g, kCheckThreads, 0, st>>>((const int64_t*)indices, (const int32_t*)indptr,
                                                                    n_rows, n_cols, nnz);
  else
    check_csr_kernel<int64_t, int64_t><<<g, kCheckThreads, 0, st>>>((const int64_t*)indices, (const int64_t*)indptr,
                                                                    n_rows, n_cols, nnz);
  return end_check(st, rec);
}

int check_entry_ids(const int32_t* indices, const int32_t* row_ids, int64_t n_rows, int64_t n_cols, int64_t nnz,
                    cudaStream_t st) {
  if (nnz <= 0 || indices == nullptr || row_ids == nullptr) return FSB_OK;
  void* rec = nullptr;
  int rc = begin_check(st, &rec);
  if (rc != FSB_OK) return rc;
  check_csr_kernel<int32_t, int32_t><<<grid_for(nnz), kCheckThreads, 0, st>>>(indices, nullptr, 0, n_cols, nnz);
  check_row_ids_kernel<<<grid_for(nnz), kCheckThreads, 0, st>>>(row_ids, n_rows, nnz);
  return end_check(st, rec);
}

int check_panel(const uint32_t* rc_words, const int32_t* unit_piece_ptr, const int32_t* unit_chunk,
                const int32_t* owner_unit_ptr, int n_owners, int slots, int max_row, int chunk_cols, int n_buffers,
                int64_t n_cols, cudaStream_t st) {
  if (!rc_words || !unit_piece_ptr || !unit_chunk || !owner_unit_ptr || n_owners <= 0 || chunk_cols <= 0) return FSB_OK;
  void* rec = nullptr;
  int rc = begin_check(st, &rec);
  if (rc != FSB_OK) return rc;
  const int64_t n_chunks = (n_cols + chunk_cols - 1) / chunk_cols;
  check_panel_kernel<<<kCheckBlocks, kCheckThreads, 0, st>>>(rc_words, unit_piece_ptr, unit_chunk, owner_unit_ptr,
                                                            n_owners, slots, (uint32_t)max_row,
                                                            (uint32_t)(chunk_cols * n_buffers), n_chunks);
  return end_check(st, rec);
}

#endif  // FSB_BOUNDS_CHECK

}  // namespace fsb

extern "C" int fsb_bounds_check_enabled(void) {
#ifdef FSB_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

extern "C" int fsb_bounds_check_report(int64_t* out) {
  if (out == nullptr) return FSB_EINVAL;
#ifdef FSB_BOUNDS_CHECK
  for (int i = 0; i < 5; ++i) {
    out[i] = fsb::g_last_report[i];
    fsb::g_last_report[i] = 0;
  }
  return FSB_OK;
#else
  for (int i = 0; i < 5; ++i) out[i] = 0;
  return FSB_EINVAL;
#endif
}
