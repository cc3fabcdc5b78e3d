/*
 * Plain-C restatement of the reference's CSR SpMV / SpMM arithmetic -- TEST INFRASTRUCTURE ONLY (the
 * checker and the timed CPU baseline; never linked into libfsb.so or imported by the package).
 *
 * Follows the reference's base path: one output element per (row[, column]), the products of the row
 * accumulated in double precision and rounded once to the value type
 *   SpMV  src/flagsparse/sparse_operations/spmv_csr.py:94-120 (kernel), :516-535 (float64 compute dtype)
 *   SpMM  src/flagsparse/sparse_operations/spmm_csr.py:92-134 (kernel), :548-573
 * and, with native = 1, the opt path's native-precision accumulation (spmv_csr.py:161-279,
 * spmm_csr.py:602-775).  Rows are independent, so contiguous row ranges holding about the same number
 * of nnz each are handed to POSIX threads.
 * Index type: int32 or int64 for `indices`, int64 for `indptr` (the caller widens a 32-bit indptr).
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <unistd.h>

int csr_ref_max_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n < 1 ? 1 : (int)n;
}

typedef struct {
  const void* data;
  const int32_t* idx32;
  const int64_t* idx64;
  const int64_t* ptr;
  const void* dense; /* x or B */
  int64_t ldb;
  void* out; /* y or C */
  int64_t ldc, n_dense;
  int is64, native, spmm;
  int64_t r0, r1;
} job_t;

#define COL(j, p) ((j)->idx64 ? (j)->idx64[p] : (int64_t)(j)->idx32[p])

#define DEFINE_ROWS(NAME, V)                                                                        \
  static void NAME(const job_t* j) {                                                                \
    const V* data = (const V*)j->data;                                                              \
    const V* dense = (const V*)j->dense;                                                            \
    V* out = (V*)j->out;                                                                            \
    if (!j->spmm) {                                                                                 \
      for (int64_t i = j->r0; i < j->r1; ++i) {                                                     \
        if (j->native) {                                                                            \
          V acc = 0;                                                                                \
          for (int64_t p = j->ptr[i]; p < j->ptr[i + 1]; ++p) acc += data[p] * dense[COL(j, p)];    \
          out[i] = acc;                                                                             \
        } else {                                                                                    \
          double acc = 0.0;                                                                         \
          for (int64_t p = j->ptr[i]; p < j->ptr[i + 1]; ++p)                                       \
            acc += (double)data[p] * (double)dense[COL(j, p)];                                      \
          out[i] = (V)acc;                                                                          \
        }                                                                                           \
      }                                                                                             \
      return;                                                                                       \
    }                                                                                               \
    const int64_t n = j->n_dense;                                                                   \
    double* acc = (double*)malloc(sizeof(double) * (size_t)(n > 0 ? n : 1));                        \
    for (int64_t i = j->r0; i < j->r1; ++i) {                                                       \
      for (int64_t c = 0; c < n; ++c) acc[c] = 0.0;                                                 \
      for (int64_t p = j->ptr[i]; p < j->ptr[i + 1]; ++p) {                                         \
        const V a = data[p];                                                                        \
        const V* brow = dense + COL(j, p) * j->ldb;                                                 \
        if (j->native)                                                                              \
          for (int64_t c = 0; c < n; ++c) acc[c] = (double)((V)acc[c] + a * brow[c]);               \
        else                                                                                        \
          for (int64_t c = 0; c < n; ++c) acc[c] += (double)a * (double)brow[c];                    \
      }                                                                                             \
      for (int64_t c = 0; c < n; ++c) out[i * j->ldc + c] = (V)acc[c];                              \
    }                                                                                               \
    free(acc);                                                                                      \
  }

DEFINE_ROWS(rows_f32, float)
DEFINE_ROWS(rows_f64, double)

static void* worker(void* arg) {
  const job_t* j = (const job_t*)arg;
  if (j->is64) rows_f64(j); else rows_f32(j);
  return NULL;
}

/* first row whose indptr value is >= target */
static int64_t lower_row(const int64_t* ptr, int64_t n_rows, int64_t target) {
  int64_t lo = 0, hi = n_rows;
  while (lo < hi) {
    int64_t mid = (lo + hi) / 2;
    if (ptr[mid] < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}

static void run(job_t base, int64_t n_rows, int threads) {
  if (threads < 1) threads = 1;
  if (threads > 256) threads = 256;
  if (threads == 1 || n_rows < 2 * threads) {
    base.r0 = 0;
    base.r1 = n_rows;
    worker(&base);
    return;
  }
  pthread_t tid[256];
  job_t jobs[256];
  const int64_t nnz = base.ptr[n_rows];
  int64_t prev = 0;
  for (int t = 0; t < threads; ++t) {
    int64_t end = (t == threads - 1) ? n_rows : lower_row(base.ptr, n_rows, nnz / threads * (t + 1));
    if (end < prev) end = prev;
    jobs[t] = base;
    jobs[t].r0 = prev;
    jobs[t].r1 = end;
    prev = end;
    pthread_create(&tid[t], NULL, worker, &jobs[t]);
  }
  for (int t = 0; t < threads; ++t) pthread_join(tid[t], NULL);
}

void csr_ref_spmv(int is64, const void* data, const int32_t* idx32, const int64_t* idx64, const int64_t* ptr,
                  const void* x, void* y, int64_t n_rows, int native, int threads) {
  job_t j = {data, idx32, idx64, ptr, x, 0, y, 0, 0, is64, native, 0, 0, 0};
  run(j, n_rows, threads);
}

void csr_ref_spmm(int is64, const void* data, const int32_t* idx32, const int64_t* idx64, const int64_t* ptr,
                  const void* b, int64_t ldb, void* c, int64_t ldc, int64_t n_rows, int64_t n_dense, int native,
                  int threads) {
  job_t j = {data, idx32, idx64, ptr, b, ldb, c, ldc, n_dense, is64, native, 1, 0, 0};
  run(j, n_rows, threads);
}
