// CSR SpMV, "panel" kernel for matrices whose rows reach a limited range of columns (banded, stencil,
// finite-element matrices): the x operand is kept in shared memory.
//
// Why: in a CSR SpMV every entry gathers one element of x.  When consecutive entries of a row are far
// apart each gather touches its own 32-byte sector, and an SM issues only about one request per clock
// towards L2, so the product runs at the speed of the gathers, not of HBM.  Shared memory serves 32
// scattered 4-byte reads per clock.  The prepare step therefore regroups the entries (once per matrix)
// into units = (block of RB consecutive rows) x (chunk of CW consecutive columns); inside a unit the
// entries keep their row-major order and are cut into pieces of 64 slots such that the entries of one row
// never straddle two pieces (unused slots hold a sentinel).  An entry is a value plus one packed word
// (local row << 16 | buffer parity * CW + local column): 8 bytes for float32, the same as CSR with 32-bit
// indices.  One CTA owns one row block:
//   - the CW elements of x a unit needs arrive in shared memory by a cp.async.bulk copy (mbarrier
//     completion), double-buffered so that the next unit's chunk is in flight while this one is used;
//   - each warp takes whole pieces (fully coalesced 128-byte loads, several pieces in flight), multiplies
//     with x from shared memory and adds the products to the row accumulators of the block, which also
//     live in shared memory.  Entries of one row inside a 32-entry round are added in the order of their
//     position (one pass per position in the run), rounds and pieces in program order, units in sequence
//     with a CTA barrier in between: every sum is formed in one fixed order, so the result is
//     bit-reproducible, and because a row occurs in one piece per unit no two warps update the same
//     accumulator at the same time;
//   - after the last unit the accumulators are written to y, each row exactly once.
#include "fsb_common.cuh"

namespace fsb {

constexpr int kPanelWarps = 16;
constexpr int kPanelThreads = kPanelWarps * 32;
constexpr int kPieceSlots = 64;
constexpr int kPanelWaitSpins = 1 << 22;
constexpr uint32_t kNoRow = 0xFFFFu;

__device__ __forceinline__ uint32_t p_smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void p_mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(p_smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void p_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void p_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(p_smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void p_bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   p_smem_addr(dst)), "l"(src), "r"(bytes), "r"(p_smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool p_try_wait(uint64_t* bar, uint32_t phase) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(p_smem_addr(bar)), "r"(phase) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool p_wait_bounded(uint64_t* bar, uint32_t phase) {
  for (int i = 0; i < kPanelWaitSpins; ++i)
    if (p_try_wait(bar, phase)) return true;
  return false;
}

// one round: 32 consecutive slots of a piece, one per lane
template <typename V>
__device__ __forceinline__ void panel_round(V v, uint32_t w, const V* __restrict__ xs, V* __restrict__ y_part,
                                            uint32_t col_mask, int lane) {
  const uint32_t row = w >> 16;
  const bool live = row != kNoRow;
  const V p = live ? v * xs[w & col_mask] : (V)0;
  const uint32_t prev = __shfl_up_sync(0xffffffffu, row, 1);
  const bool head = (lane == 0) || (prev != row);
  const uint32_t heads = __ballot_sync(0xffffffffu, head);
  const int start = 31 - __clz(heads & (0xffffffffu >> (31 - lane)));  // first lane of this lane's run
  const unsigned rank = (unsigned)(lane - start);
  const unsigned max_rank = __reduce_max_sync(0xffffffffu, live ? rank : 0u);
  for (unsigned j = 0; j <= max_rank; ++j) {
    if (live && rank == j) y_part[row] += p;
    __syncwarp();
  }
}

template <typename V>
__global__ void __launch_bounds__(kPanelThreads, 2)
spmv_panel_kernel(const V* __restrict__ val, const uint32_t* __restrict__ rc, const int32_t* __restrict__ unit_piece_ptr,
                  const int32_t* __restrict__ unit_chunk, const int32_t* __restrict__ rb_unit_ptr,
                  const V* __restrict__ x, V* __restrict__ y, int64_t n_rows, int64_t n_cols, int rb_rows,
                  int chunk_cols, int32_t* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char p_smem[];
  V* xs = reinterpret_cast<V*>(p_smem);  // 2 * chunk_cols
  V* y_part = xs + 2 * chunk_cols;       // rb_rows
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ int s_failed;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rb = blockIdx.x;
  const int64_t r0 = (int64_t)rb * rb_rows;
  const int nr = (int)((n_rows - r0) < (int64_t)rb_rows ? (n_rows - r0) : (int64_t)rb_rows);
  const int u0 = rb_unit_ptr[rb], u1 = rb_unit_ptr[rb + 1];
  const uint32_t col_mask = (uint32_t)(2 * chunk_cols - 1);

  for (int i = tid; i < nr; i += kPanelThreads) y_part[i] = (V)0;
  if (tid == 0) {
    s_failed = 0;
    p_mbar_init(&bars[0], 1);
    p_mbar_init(&bars[1], 1);
    p_fence_init();
  }
  __syncthreads();

  // chunk `c` of x into buffer `b`: bulk copy when the byte count is a multiple of 16, else plain loads
  auto load_chunk = [&](int c, int b) {
    const int64_t c0 = (int64_t)c * chunk_cols;
    const int n = (int)((n_cols - c0) < (int64_t)chunk_cols ? (n_cols - c0) : (int64_t)chunk_cols);
    const uint32_t bytes = (uint32_t)(n * sizeof(V));
    if ((bytes & 15u) == 0 && aligned_to_dev(x + c0)) {
      if (tid == 0) {
        p_expect_tx(&bars[b], bytes);
        p_bulk_g2s(xs + (size_t)b * chunk_cols, x + c0, bytes, &bars[b]);
      }
      return false;
    }
    for (int i = tid; i < n; i += kPanelThreads) xs[(size_t)b * chunk_cols + i] = __ldg(x + c0 + i);
    if (tid == 0) p_expect_tx(&bars[b], 0);  // the phase completes as soon as this arrival lands
    return true;
  };

  bool plain = false;  // some chunk of this unit was written with ordinary stores: needs a CTA barrier
  if (u0 < u1) plain = load_chunk(unit_chunk[u0], 0);
  for (int u = u0; u < u1; ++u) {
    const int ord = u - u0, b = ord & 1;
    // the other buffer was last read before the barrier that closed the previous unit: free to refill
    bool plain_next = false;
    if (u + 1 < u1) plain_next = load_chunk(unit_chunk[u + 1], b ^ 1);
    if (!p_wait_bounded(&bars[b], (uint32_t)((ord >> 1) & 1))) s_failed = 1;
    if (plain) __syncthreads();
    const V* xb = xs;  // both buffers: the packed word carries the parity
    const int p_end = unit_piece_ptr[u + 1];
    int pc = unit_piece_ptr[u] + warp;
    // four pieces per trip: sixteen 128-byte loads in flight per warp
    for (; pc + 3 * kPanelWarps < p_end; pc += 4 * kPanelWarps) {
      V v[8];
      uint32_t w[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int64_t base = (int64_t)(pc + q * kPanelWarps) * kPieceSlots + lane;
        v[2 * q] = ld_stream(val + base);
        v[2 * q + 1] = ld_stream(val + base + 32);
        w[2 * q] = ld_stream(rc + base);
        w[2 * q + 1] = ld_stream(rc + base + 32);
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) panel_round<V>(v[q], w[q], xb, y_part, col_mask, lane);
    }
    for (; pc < p_end; pc += kPanelWarps) {
      const int64_t base = (int64_t)pc * kPieceSlots + lane;
      const V v0 = ld_stream(val + base), v1 = ld_stream(val + base + 32);
      const uint32_t w0 = ld_stream(rc + base), w1 = ld_stream(rc + base + 32);
      panel_round<V>(v0, w0, xb, y_part, col_mask, lane);
      panel_round<V>(v1, w1, xb, y_part, col_mask, lane);
    }
    __syncthreads();  // every add of this unit is done; its x buffer may be refilled
    if (s_failed) {
      if (tid == 0 && status != nullptr) atomicExch(status, 2);
      return;
    }
    plain = plain_next;
  }
  for (int i = tid; i < nr; i += kPanelThreads) y[r0 + i] = y_part[i];
}

}  // namespace fsb

using namespace fsb;

extern "C" int fsb_spmv_panel_piece_slots(void) { return kPieceSlots; }

extern "C" size_t fsb_spmv_panel_smem_bytes(int vtype, int rb_rows, int chunk_cols) {
  const size_t sv = vtype == FSB_F32 ? 4 : 8;
  return 2 * (size_t)chunk_cols * sv + (((size_t)rb_rows + 3) & ~(size_t)3) * sv;
}

extern "C" int fsb_spmv_csr_panel(int vtype, const void* val, const uint32_t* rc, const int32_t* unit_piece_ptr,
                                  const int32_t* unit_chunk, const int32_t* rb_unit_ptr, int32_t n_row_blocks,
                                  int32_t rb_rows, int32_t chunk_cols, const void* x, void* y, int64_t n_rows,
                                  int64_t n_cols, int32_t* status, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (vtype != FSB_F32 && vtype != FSB_F64) return FSB_EINVAL;
  if (n_rows < 0 || n_cols < 0 || n_row_blocks < 0 || rb_rows <= 0 || rb_rows >= 65535) return FSB_EINVAL;
  if (chunk_cols <= 0 || (chunk_cols & (chunk_cols - 1)) != 0 || chunk_cols > 16384) return FSB_EINVAL;
  if (n_rows == 0) return FSB_OK;
  if ((int64_t)n_row_blocks * rb_rows < n_rows) return FSB_EINVAL;
  if (!val || !rc || !unit_piece_ptr || !unit_chunk || !rb_unit_ptr || !x || !y) return FSB_EINVAL;
  const size_t smem = fsb_spmv_panel_smem_bytes(vtype, rb_rows, chunk_cols);
  if (smem > 227 * 1024) return FSB_ERANGE;
  cudaError_t e;
  if (vtype == FSB_F32) {
    e = cudaFuncSetAttribute(spmv_panel_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_rc(e);
    spmv_panel_kernel<float><<<(unsigned)n_row_blocks, kPanelThreads, smem, st>>>(
        (const float*)val, rc, unit_piece_ptr, unit_chunk, rb_unit_ptr, (const float*)x, (float*)y, n_rows, n_cols,
        rb_rows, chunk_cols, status);
  } else {
    e = cudaFuncSetAttribute(spmv_panel_kernel<double>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_rc(e);
    spmv_panel_kernel<double><<<(unsigned)n_row_blocks, kPanelThreads, smem, st>>>(
        (const double*)val, rc, unit_piece_ptr, unit_chunk, rb_unit_ptr, (const double*)x, (double*)y, n_rows, n_cols,
        rb_rows, chunk_cols, status);
  }
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}
