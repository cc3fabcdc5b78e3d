// CSR SpMV, "panel" kernel for matrices whose rows reach a limited range of columns (banded, stencil,
// finite-element matrices): the x operand is kept in shared memory.
//
// Why: in a CSR SpMV every entry gathers one element of x.  When consecutive entries of a row are far
// apart each gather touches its own 32-byte sector, and an SM issues only about one request per clock
// towards L2, so the product runs at the speed of the gathers, not of HBM.  Shared memory serves 32
// scattered 4-byte reads per clock.  The prepare step therefore regroups the entries (once per matrix)
// into units = (block of RB consecutive rows) x (chunk of CW consecutive columns); inside a unit the
// entries keep their row-major order and are cut into pieces of 512 slots such that the entries of one
// row never straddle two pieces (unused slots hold a sentinel).  An entry is a value plus one packed word
// (local row << 16 | buffer parity * CW + local column): 8 bytes for float32, the same as CSR with 32-bit
// indices.  One CTA owns one row block:
//   - the CW elements of x a unit needs arrive in shared memory by a cp.async.bulk copy (mbarrier
//     completion), double-buffered so that the next unit's chunk is in flight while this one is used;
//   - a warp takes a whole piece: lane l owns slots 16l .. 16l+15 (stored interleaved so that each 128-bit
//     load of the warp is contiguous).  In round k every lane handles its k-th slot.  Two slots of one round are at least 16 positions apart,
//     and a row has at most 16 entries in a unit (the prepare step refuses the matrix otherwise), so the
//     32 lanes of a round always touch 32 different rows: each lane simply adds value * x[column] to its
//     row's accumulator in shared memory, with no shuffles and no atomics.  Rounds follow each other in
//     program order, a row lives in one piece per unit, and units are separated by a CTA barrier, so
//     every accumulator receives its terms in one fixed order: the result is bit-reproducible;
//   - after the last unit the accumulators are written to y, each row exactly once.
#include "fsb_common.cuh"

namespace fsb {

constexpr int kPanelWarps = 32;
constexpr int kPanelThreads = kPanelWarps * 32;
constexpr int kPieceSlots = 512;   // 32 lanes x 16 rounds
constexpr int kPieceRounds = 16;
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

// G consecutive slots of one lane (rounds k0 .. k0+G-1 of the piece).  Products of one row are summed in a
// register and added to the row's accumulator when the row ends (next_row is the row of the lane's next slot,
// or kNoRow after its last one).  Within one round the 32 lanes are on 32 different rows; a row that spans two
// lanes ends in the first of them at its last slot and in the second one earlier, i.e. in different rounds.
template <typename V, int G>
__device__ __forceinline__ void panel_rounds(const V (&v)[G], const uint32_t (&w)[G], uint32_t next_word, V& acc,
                                             const V* __restrict__ xs, V* __restrict__ y_part, uint32_t col_mask) {
  // x does not change during a unit: all G gathers go out first, so that their latencies overlap instead of
  // queueing behind the per-round ordering points below
  V p[G];
#pragma unroll
  for (int k = 0; k < G; ++k) p[k] = v[k] * xs[w[k] & col_mask];   // padding slots: value 0, column 0
#pragma unroll
  for (int k = 0; k < G; ++k) {
    const uint32_t row = w[k] >> 16;
    const uint32_t next_row = (k + 1 < G ? w[k + 1] : next_word) >> 16;
    const bool live = row != kNoRow;
    if (live) acc += p[k];
    if (live && next_row != row) {
      y_part[row] += acc;
      acc = (V)0;
    }
    __syncwarp();  // orders this round's accumulator updates before the next round's
  }
}

// Storage inside a piece: slot (lane, k), k = 0..15, of the value array sits at (k / E) * 32 * E + lane * E + k % E
// with E = elements per 16 bytes, and of the packed-word array at (k / 4) * 128 + lane * 4 + k % 4, so that every
// 128-bit load of a warp reads 512 contiguous bytes.
template <int G>
__device__ __forceinline__ void ld_group(const float* piece, int lane, int g, float (&v)[G]) {
  static_assert(G == 8, "float32 groups hold eight slots");
  ld_stream4(piece + (2 * g) * 128 + lane * 4, *reinterpret_cast<float(*)[4]>(&v[0]));
  ld_stream4(piece + (2 * g + 1) * 128 + lane * 4, *reinterpret_cast<float(*)[4]>(&v[4]));
}
template <int G>
__device__ __forceinline__ void ld_group(const double* piece, int lane, int g, double (&v)[G]) {
  static_assert(G == 4, "float64 groups hold four slots");
  const double2 a = __ldcs(reinterpret_cast<const double2*>(piece + (2 * g) * 64 + lane * 2));
  const double2 b = __ldcs(reinterpret_cast<const double2*>(piece + (2 * g + 1) * 64 + lane * 2));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <int G>
__device__ __forceinline__ void ld_words(const uint32_t* piece, int lane, int g, uint32_t (&w)[G]) {
#pragma unroll
  for (int q = 0; q < G / 4; ++q) {
    const uint4 t = __ldcs(reinterpret_cast<const uint4*>(piece + (g * (G / 4) + q) * 128 + lane * 4));
    w[4 * q] = t.x; w[4 * q + 1] = t.y; w[4 * q + 2] = t.z; w[4 * q + 3] = t.w;
  }
}

constexpr int kMaxXBuffers = 8;
constexpr int kUnitWindow = 512;   // units whose tables are kept in shared memory at a time
constexpr int kUnitLookahead = kMaxXBuffers;

// The shared-memory state of one CTA: the x buffers, the row accumulators, the copy barriers, the unit tables.
template <typename V>
struct PanelShared {
  V* xs;      // n_buf * chunk_cols
  V* y_part;  // one accumulator per (virtual) row of the CTA
  uint64_t* bars;
  int* failed;
  int32_t* upp;   // unit_piece_ptr of the current window of units (kUnitWindow + 1 entries)
  int32_t* uch;   // unit_chunk of the window and of the next few units (kUnitWindow + kUnitLookahead)
};

// Units u0 .. u1-1 of one CTA, in order: chunk of x in, pieces added into y_part.  Returns false when a bounded
// wait ran out (every thread of the CTA gets the same answer).
//   - x chunks are fetched n_buf - 1 units ahead into n_buf buffers (unit number `ord` of the CTA uses buffer
//     ord % n_buf; the packed word of a slot already holds buffer * chunk_cols + local column);
//   - the pieces of the CTA are dealt to its warps round-robin ACROSS units (piece p goes to warp
//     (p - first piece of the CTA) % 32), and a warp fetches the first entries of its next piece while it works
//     on the current one, whichever unit that piece belongs to: a unit with only a few pieces costs neither a
//     trip to DRAM for its entries nor one for its tables.
template <typename V>
__device__ __forceinline__ bool panel_run_units(const V* __restrict__ val, const uint32_t* __restrict__ rc,
                                                const int32_t* __restrict__ unit_piece_ptr,
                                                const int32_t* __restrict__ unit_chunk, int u0, int u1,
                                                const V* __restrict__ x, int64_t n_cols, int chunk_cols, int n_buf,
                                                const PanelShared<V>& sh) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  V* xs = sh.xs;
  V* y_part = sh.y_part;
  uint64_t* bars = sh.bars;
  const uint32_t col_mask = (uint32_t)(n_buf * chunk_cols - 1);
  const int buf_mask = n_buf - 1;
  if (u0 >= u1) return true;

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

  constexpr int G = sizeof(V) == 4 ? 8 : 4;   // slots per load group
  constexpr int NG = kPieceRounds / G;        // groups per piece
  const int p_cta_end = unit_piece_ptr[u1];
  int pc = unit_piece_ptr[u0] + warp;         // this warp's next piece
  // the entries do not depend on x: the first group of the warp's first piece is fetched before anything else
  V v[G];
  uint32_t w[G];
  if (pc < p_cta_end) {
    ld_group<G>(val + (size_t)pc * kPieceSlots, lane, 0, v);
    ld_words<G>(rc + (size_t)pc * kPieceSlots, lane, 0, w);
  }
  // chunks of the first n_buf - 1 units
  bool plain = false;  // some chunk was written with ordinary stores: needs a CTA barrier before its first use
  for (int a = 0; a < n_buf - 1 && u0 + a < u1; ++a) plain |= load_chunk(unit_chunk[u0 + a], a);

  for (int w0 = u0; w0 < u1; w0 += kUnitWindow) {
    const int nwin = (u1 - w0) < kUnitWindow ? (u1 - w0) : kUnitWindow;
    const int nch = (u1 - w0) < (kUnitWindow + kUnitLookahead) ? (u1 - w0) : (kUnitWindow + kUnitLookahead);
    if (w0 > u0) __syncthreads();  // the previous window's tables are no longer read
    for (int i = tid; i <= nwin; i += kPanelThreads) sh.upp[i] = unit_piece_ptr[w0 + i];
    for (int i = tid; i < nch; i += kPanelThreads) sh.uch[i] = unit_chunk[w0 + i];
    __syncthreads();
    for (int u = w0; u < w0 + nwin; ++u) {
      const int ord = u - u0, b = ord & buf_mask;
      // the buffer of the previous unit was last read before the barrier that closed it: free to refill
      if (u + n_buf - 1 < u1) plain |= load_chunk(sh.uch[u + n_buf - 1 - w0], (ord + n_buf - 1) & buf_mask);
      const int p_end = sh.upp[u - w0 + 1];
      if (!p_wait_bounded(&bars[b], (uint32_t)((ord / n_buf) & 1))) *sh.failed = 1;
      if (plain && ord == 0) __syncthreads();  // later plain chunks are written at least one unit (barrier) ahead
      while (pc < p_end) {
        V acc = (V)0;
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          // next group (of this piece, or the first one of this warp's next piece) in flight while this one is used
          V v2[G];
          uint32_t w2[G];
          const bool more = g + 1 < NG;
          const int np = more ? pc : pc + kPanelWarps;
          const bool have = np < p_cta_end;
          if (have) {
            ld_group<G>(val + (size_t)np * kPieceSlots, lane, more ? g + 1 : 0, v2);
            ld_words<G>(rc + (size_t)np * kPieceSlots, lane, more ? g + 1 : 0, w2);
          }
          const uint32_t next_word = more ? w2[0] : (kNoRow << 16);  // a lane's run ends with its last slot
          panel_rounds<V, G>(v, w, next_word, acc, xs, y_part, col_mask);
          if (have) {
#pragma unroll
            for (int k = 0; k < G; ++k) { v[k] = v2[k]; w[k] = w2[k]; }
          }
        }
        pc += kPanelWarps;
      }
      __syncthreads();  // every add of this unit is done; its x buffer may be refilled
      if (*sh.failed) return false;
    }
  }
  return true;
}

struct PanelStatic {
  uint64_t bars[kMaxXBuffers];
  int32_t upp[kUnitWindow + 1];
  int32_t uch[kUnitWindow + kUnitLookahead];
  int failed;
};

template <typename V>
__device__ __forceinline__ void panel_setup(PanelShared<V>& sh, unsigned char* smem, PanelStatic* st, int chunk_cols,
                                            int n_buf, int n_acc) {
  sh.xs = reinterpret_cast<V*>(smem);
  sh.y_part = sh.xs + (size_t)n_buf * chunk_cols;
  sh.bars = st->bars;
  sh.failed = &st->failed;
  sh.upp = st->upp;
  sh.uch = st->uch;
  const int tid = threadIdx.x;
  for (int i = tid; i < n_acc; i += kPanelThreads) sh.y_part[i] = (V)0;
  if (tid == 0) {
    st->failed = 0;
    for (int b = 0; b < n_buf; ++b) p_mbar_init(&st->bars[b], 1);
    p_fence_init();
  }
  __syncthreads();
}

// One CTA per block of rb_rows consecutive rows; every row of y is written exactly once (to y, or, when y_peers
// is given, to y_peers[p][row_offset + row] for every p).
template <typename V>
__global__ void __launch_bounds__(kPanelThreads, 1)
spmv_panel_kernel(const V* __restrict__ val, const uint32_t* __restrict__ rc, const int32_t* __restrict__ unit_piece_ptr,
                  const int32_t* __restrict__ unit_chunk, const int32_t* __restrict__ rb_unit_ptr,
                  const V* __restrict__ x, V* __restrict__ y, V* const* __restrict__ y_peers, int n_peers,
                  int64_t row_offset, int64_t n_rows, int64_t n_cols, int rb_rows, int chunk_cols, int n_buf,
                  int32_t* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char p_smem[];
  __shared__ __align__(8) PanelStatic p_static;
  const int tid = threadIdx.x;
  const int rb = blockIdx.x;
  const int64_t r0 = (int64_t)rb * rb_rows;
  const int nr = (int)((n_rows - r0) < (int64_t)rb_rows ? (n_rows - r0) : (int64_t)rb_rows);
  PanelShared<V> sh;
  panel_setup<V>(sh, p_smem, &p_static, chunk_cols, n_buf, nr);
  if (!panel_run_units<V>(val, rc, unit_piece_ptr, unit_chunk, rb_unit_ptr[rb], rb_unit_ptr[rb + 1], x, n_cols,
                          chunk_cols, n_buf, sh)) {
    if (tid == 0 && status != nullptr) atomicExch(status, 2);
    return;
  }
  if (y_peers == nullptr) {
    for (int i = tid; i < nr; i += kPanelThreads) y[r0 + i] = sh.y_part[i];
  } else {
    // sharded product: this GPU's rows go straight into every GPU's copy of y (coalesced stores over NVLink)
    for (int p = 0; p < n_peers; ++p) {
      V* dst = y_peers[p] + row_offset + r0;
      for (int i = tid; i < nr; i += kPanelThreads) dst[i] = sh.y_part[i];
    }
  }
}

// Row-group form, for a set of long rows picked out of a matrix (the rest of the matrix goes through the CSR
// kernels).  The picked rows are numbered q = 0 .. n_long-1 and cut into groups; row q owns the accumulators
// vbase[q] .. vbase[q+1]-1 of its group ("virtual rows": a row with more than 16 entries in one chunk spreads
// them over several accumulators, 16 to each, so that the rule "at most 16 entries of an accumulator per
// unit" still holds).  The units of a group are dealt to several CTAs by column range, so a CTA ends with
// partial sums of its group's rows: it writes them to part[cta_part_ptr[cta] + (q - first q of the group)],
// and panel_group_reduce_kernel adds the partial sums of each row in CTA order.
template <typename V>
__global__ void __launch_bounds__(kPanelThreads, 1)
spmv_panel_groups_kernel(const V* __restrict__ val, const uint32_t* __restrict__ rc,
                         const int32_t* __restrict__ unit_piece_ptr, const int32_t* __restrict__ unit_chunk,
                         const int32_t* __restrict__ cta_unit_ptr, const int32_t* __restrict__ cta_group,
                         const int32_t* __restrict__ group_q_ptr, const int32_t* __restrict__ vbase,
                         const int64_t* __restrict__ cta_part_ptr, V* __restrict__ part, const V* __restrict__ x,
                         int64_t n_cols, int chunk_cols, int n_buf, int32_t* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char p_smem[];
  __shared__ __align__(8) PanelStatic p_static;
  const int tid = threadIdx.x;
  const int cta = blockIdx.x;
  const int g = cta_group[cta];
  const int q0 = group_q_ptr[g], q1 = group_q_ptr[g + 1];
  const int vb0 = vbase[q0];
  const int n_acc = vbase[q1] - vb0;
  PanelShared<V> sh;
  panel_setup<V>(sh, p_smem, &p_static, chunk_cols, n_buf, n_acc);
  if (!panel_run_units<V>(val, rc, unit_piece_ptr, unit_chunk, cta_unit_ptr[cta], cta_unit_ptr[cta + 1], x, n_cols,
                          chunk_cols, n_buf, sh)) {
    if (tid == 0 && status != nullptr) atomicExch(status, 2);
    return;
  }
  V* out = part + cta_part_ptr[cta];
  for (int i = tid; i < q1 - q0; i += kPanelThreads) {
    const int a = vbase[q0 + i] - vb0, b = vbase[q0 + i + 1] - vb0;
    V s = (V)0;
    for (int v = a; v < b; ++v) s += sh.y_part[v];
    out[i] = s;
  }
}

// y[long_rows[q]] = sum over the CTAs of q's group, in CTA order, of their partial sums (in double).
template <typename V>
__global__ void __launch_bounds__(256)
panel_group_reduce_kernel(const V* __restrict__ part, const int32_t* __restrict__ q_group,
                          const int32_t* __restrict__ group_q_ptr, const int32_t* __restrict__ group_cta_ptr,
                          const int64_t* __restrict__ cta_part_ptr, const int32_t* __restrict__ long_rows,
                          V* __restrict__ y, int n_long) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= n_long) return;
  const int g = q_group[q];
  const int i = q - group_q_ptr[g];
  double s = 0.0;
  for (int c = group_cta_ptr[g]; c < group_cta_ptr[g + 1]; ++c) s += (double)part[cta_part_ptr[c] + i];
  y[long_rows[q]] = (V)s;
}

}  // namespace fsb

using namespace fsb;

extern "C" int fsb_spmv_panel_piece_slots(void) { return kPieceSlots; }

extern "C" size_t fsb_spmv_panel_smem_bytes(int vtype, int rb_rows, int chunk_cols, int n_buffers) {
  const size_t sv = vtype == FSB_F32 ? 4 : 8;
  return (size_t)n_buffers * (size_t)chunk_cols * sv + (((size_t)rb_rows + 3) & ~(size_t)3) * sv;
}

extern "C" size_t fsb_spmv_panel_static_smem_bytes(void) { return sizeof(PanelStatic); }

static bool panel_buffers_ok(int n_buffers, int chunk_cols) {
  return (n_buffers == 2 || n_buffers == 4 || n_buffers == 8) && (int64_t)n_buffers * chunk_cols <= 65536;
}

static int panel_launch(int vtype, const void* val, const uint32_t* rc, const int32_t* unit_piece_ptr,
                        const int32_t* unit_chunk, const int32_t* rb_unit_ptr, int32_t n_row_blocks, int32_t rb_rows,
                        int32_t chunk_cols, int32_t n_buffers, const void* x, void* y, void* const* y_peers,
                        int n_peers, int64_t row_offset, int64_t n_rows, int64_t n_cols, int32_t* status,
                        void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (vtype != FSB_F32 && vtype != FSB_F64) return FSB_EINVAL;
  if (n_rows < 0 || n_cols < 0 || n_row_blocks < 0 || rb_rows <= 0 || rb_rows >= 65535) return FSB_EINVAL;
  if (chunk_cols <= 0 || (chunk_cols & (chunk_cols - 1)) != 0 || chunk_cols > 16384) return FSB_EINVAL;
  if (!panel_buffers_ok(n_buffers, chunk_cols)) return FSB_EINVAL;
  if (n_rows == 0) return FSB_OK;
  if ((int64_t)n_row_blocks * rb_rows < n_rows) return FSB_EINVAL;
  if (!val || !rc || !unit_piece_ptr || !unit_chunk || !rb_unit_ptr || !x || (!y && !y_peers)) return FSB_EINVAL;
  const size_t smem = fsb_spmv_panel_smem_bytes(vtype, rb_rows, chunk_cols, n_buffers);
  if (smem + sizeof(PanelStatic) > 227 * 1024) return FSB_ERANGE;
  if (!aligned_to(val, 16) || !aligned_to(rc, 16)) return FSB_EALIGN;
#define FSB_PANEL_LAUNCH(V)                                                                                   \
  do {                                                                                                        \
    cudaError_t e = cudaFuncSetAttribute(spmv_panel_kernel<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int)smem);                                                          \
    if (e != cudaSuccess) return cuda_rc(e);                                                                  \
    spmv_panel_kernel<V><<<(unsigned)n_row_blocks, kPanelThreads, smem, st>>>(                                \
        (const V*)val, rc, unit_piece_ptr, unit_chunk, rb_unit_ptr, (const V*)x, (V*)y, (V* const*)y_peers,   \
        n_peers, row_offset, n_rows, n_cols, rb_rows, chunk_cols, n_buffers, status);                         \
  } while (0)
  if (vtype == FSB_F32) FSB_PANEL_LAUNCH(float); else FSB_PANEL_LAUNCH(double);
#undef FSB_PANEL_LAUNCH
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}

extern "C" int fsb_spmv_csr_panel(int vtype, const void* val, const uint32_t* rc, const int32_t* unit_piece_ptr,
                                  const int32_t* unit_chunk, const int32_t* rb_unit_ptr, int32_t n_row_blocks,
                                  int32_t rb_rows, int32_t chunk_cols, int32_t n_buffers, const void* x, void* y,
                                  int64_t n_rows, int64_t n_cols, int32_t* status, void* stream_) {
  if (y == nullptr && n_rows > 0) return FSB_EINVAL;
  return panel_launch(vtype, val, rc, unit_piece_ptr, unit_chunk, rb_unit_ptr, n_row_blocks, rb_rows, chunk_cols,
                      n_buffers, x, y, nullptr, 0, 0, n_rows, n_cols, status, stream_);
}

extern "C" int fsb_spmv_csr_panel_scatter(int vtype, const void* val, const uint32_t* rc,
                                          const int32_t* unit_piece_ptr, const int32_t* unit_chunk,
                                          const int32_t* rb_unit_ptr, int32_t n_row_blocks, int32_t rb_rows,
                                          int32_t chunk_cols, int32_t n_buffers, const void* x, void* const* y_peers,
                                          int n_peers, int64_t row_offset, int64_t n_rows, int64_t n_cols,
                                          int32_t* status, void* stream_) {
  if (y_peers == nullptr || n_peers < 1 || n_peers > 64 || row_offset < 0) return FSB_EINVAL;
  return panel_launch(vtype, val, rc, unit_piece_ptr, unit_chunk, rb_unit_ptr, n_row_blocks, rb_rows, chunk_cols,
                      n_buffers, x, nullptr, y_peers, n_peers, row_offset, n_rows, n_cols, status, stream_);
}

extern "C" int fsb_spmv_csr_panel_groups(int vtype, const void* val, const uint32_t* rc, const int32_t* unit_piece_ptr,
                                         const int32_t* unit_chunk, const int32_t* cta_unit_ptr, int32_t n_ctas,
                                         int32_t chunk_cols, int32_t n_buffers, int32_t max_group_acc,
                                         const int32_t* cta_group,
                                         const int32_t* group_q_ptr, const int32_t* group_cta_ptr, const int32_t* vbase,
                                         const int32_t* q_group, const int32_t* long_rows, int32_t n_long,
                                         const int64_t* cta_part_ptr, void* part, const void* x, void* y,
                                         int64_t n_cols, int32_t* status, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (vtype != FSB_F32 && vtype != FSB_F64) return FSB_EINVAL;
  if (n_cols < 0 || n_ctas < 0 || n_long < 0 || max_group_acc < 0 || max_group_acc >= 65535) return FSB_EINVAL;
  if (chunk_cols <= 0 || (chunk_cols & (chunk_cols - 1)) != 0 || chunk_cols > 16384) return FSB_EINVAL;
  if (!panel_buffers_ok(n_buffers, chunk_cols)) return FSB_EINVAL;
  if (n_long == 0 || n_ctas == 0) return FSB_OK;
  if (!val || !rc || !unit_piece_ptr || !unit_chunk || !cta_unit_ptr || !cta_group || !group_q_ptr ||
      !group_cta_ptr || !vbase || !q_group || !long_rows || !cta_part_ptr || !part || !x || !y)
    return FSB_EINVAL;
  const size_t smem = fsb_spmv_panel_smem_bytes(vtype, max_group_acc, chunk_cols, n_buffers);
  if (smem + sizeof(PanelStatic) > 227 * 1024) return FSB_ERANGE;
  if (!aligned_to(val, 16) || !aligned_to(rc, 16)) return FSB_EALIGN;
  const unsigned rgrid = (unsigned)((n_long + 255) / 256);
#define FSB_GROUPS_LAUNCH(V)                                                                                       \
  do {                                                                                                             \
    cudaError_t e = cudaFuncSetAttribute(spmv_panel_groups_kernel<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int)smem);                                                               \
    if (e != cudaSuccess) return cuda_rc(e);                                                                       \
    spmv_panel_groups_kernel<V><<<(unsigned)n_ctas, kPanelThreads, smem, st>>>(                                    \
        (const V*)val, rc, unit_piece_ptr, unit_chunk, cta_unit_ptr, cta_group, group_q_ptr, vbase, cta_part_ptr,  \
        (V*)part, (const V*)x, n_cols, chunk_cols, n_buffers, status);                                             \
    FSB_RETURN_IF_LAUNCH_FAILED();                                                                                 \
    panel_group_reduce_kernel<V><<<rgrid, 256, 0, st>>>((const V*)part, q_group, group_q_ptr, group_cta_ptr,       \
                                                        cta_part_ptr, long_rows, (V*)y, n_long);                   \
  } while (0)
  if (vtype == FSB_F32) FSB_GROUPS_LAUNCH(float); else FSB_GROUPS_LAUNCH(double);
#undef FSB_GROUPS_LAUNCH
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}
