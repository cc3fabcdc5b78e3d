// CSR SpMV, "panel" kernel for matrices whose rows reach a limited range of columns (banded, stencil,
// finite-element matrices): the x operand is kept in shared memory.
//
// Why: in a CSR SpMV every entry gathers one element of x.  When consecutive entries of a row are far
// apart each gather touches its own 32-byte sector, and an SM issues only about one request per clock
// towards L2, so the product runs at the speed of the gathers, not of HBM.  Shared memory serves 32
// scattered 4-byte reads per clock.  The prepare step therefore regroups the entries (once per matrix)
// into units = (block of RB consecutive rows) x (chunk of CW consecutive columns); inside a unit the
// entries keep their row-major order and are cut into pieces of 32 * R slots (R = 4, 8 or 16, fixed per
// layout) such that the entries of one row never straddle two pieces (unused slots hold a sentinel).
// An entry is a value plus one packed word (local row << 16 | x buffer * CW + local column): 8 bytes for
// float32, the same as CSR with 32-bit indices.  One CTA owns one row block:
//   - the CW elements of x a unit needs arrive in shared memory by a cp.async.bulk copy (mbarrier
//     completion), n_buffers - 1 units ahead of their use;
//   - a warp takes a whole piece: lane l owns slots R*l .. R*l+R-1 (stored interleaved so that each 128-bit
//     load of the warp is contiguous).  In round k every lane handles its k-th slot: value * x[column] is added
//     to the row's accumulator in shared memory.  Two slots of one round are R positions apart and a row has at
//     most R entries in the unit, so the 32 lanes of a round always add into 32 different accumulators: no
//     shuffles, no atomics, no predicates.  Where rows have several entries per unit (FSB_PANEL_RUNS) a lane
//     instead sums a row's products in a register and adds the sum when the row ends; layouts that hold runs
//     longer than R say so (FSB_PANEL_LONG_RUNS), and a lane's last slot then goes through a segmented warp
//     reduction whenever two neighbouring lanes end on the same row;
//   - the pieces of the CTA are dealt to its warps round-robin across unit boundaries, and every warp keeps
//     the next group of slots of its own pieces in flight, whichever unit it belongs to: a unit with only a
//     few pieces costs no trip to DRAM of its own;
//   - rounds follow each other in program order, a row lives in one piece per unit, and units are separated
//     by a CTA barrier, so every accumulator receives its terms in one fixed order: bit-reproducible;
//   - after the last unit the accumulators are written to y, each row exactly once.
#include "fsb_common.cuh"

namespace fsb {

constexpr int kPanelWarps = 32;
constexpr int kPanelThreads = kPanelWarps * 32;
constexpr int kPanelWaitSpins = 1 << 22;
constexpr int kPanelWaitSpinsDebug = 1 << 10;   // FSB_PANEL_DEBUG_TIMEOUT: give up quickly

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
__device__ __forceinline__ bool p_wait_bounded(uint64_t* bar, uint32_t phase, int spins) {
  for (int i = 0; i < spins; ++i)
    if (p_try_wait(bar, phase)) return true;
  return false;
}

// G consecutive slots of one lane (G = 4 or 8): rounds G*g .. G*g+G-1 of a piece.
template <typename V, int G>
struct Group {
  V v[G];
  uint32_t w[G];
};

// Storage inside a piece of 32 * R slots: slot (lane, k), k = 0..R-1, of the value array sits at
// (k / E) * 32 * E + lane * E + k % E with E = elements per 16 bytes, and of the packed-word array at
// (k / 4) * 128 + lane * 4 + k % 4, so that every 128-bit load of a warp reads 512 contiguous bytes.
// slots 4q .. 4q+3 of a lane (q-th 128-bit quad of the piece)
__device__ __forceinline__ void ld_quad(const float* piece_val, int lane, int q, float* v) {
  const float4 t = __ldcs(reinterpret_cast<const float4*>(piece_val + q * 128 + lane * 4));
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void ld_quad(const double* piece_val, int lane, int q, double* v) {
  const double2 a = __ldcs(reinterpret_cast<const double2*>(piece_val + (2 * q) * 64 + lane * 2));
  const double2 b = __ldcs(reinterpret_cast<const double2*>(piece_val + (2 * q + 1) * 64 + lane * 2));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void ld_quad(const uint32_t* piece_rc, int lane, int q, uint32_t* w) {
  const uint4 t = __ldcs(reinterpret_cast<const uint4*>(piece_rc + q * 128 + lane * 4));
  w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
}
template <typename V, int G>
__device__ __forceinline__ void ld_group(const V* piece_val, const uint32_t* piece_rc, int lane, int g,
                                         Group<V, G>& out) {
#pragma unroll
  for (int j = 0; j < G / 4; ++j) {
    ld_quad(piece_val, lane, g * (G / 4) + j, &out.v[4 * j]);
    ld_quad(piece_rc, lane, g * (G / 4) + j, &out.w[4 * j]);
  }
}

// The G rounds of one group, for layouts in which no row has more entries in a unit than a lane has rounds
// (every round then finds its 32 lanes on 32 different accumulators): each slot adds its product straight into
// its row's accumulator.  Unused slots carry value 0 and the index of a spare accumulator, so nothing is
// predicated and the warp stays converged; rounds follow each other in program order.
template <typename V, int GS>
__device__ __forceinline__ void panel_rounds_direct(const Group<V, GS>& G, const V* __restrict__ xs,
                                                    V* __restrict__ y_part) {
  // x does not change during a unit: the gathers go out first, so that their latencies overlap instead of
  // queueing behind the per-round ordering points below
  V xv[GS];
#pragma unroll
  for (int k = 0; k < GS; ++k) xv[k] = xs[G.w[k] & 0xFFFFu];
#pragma unroll
  for (int k = 0; k < GS; ++k) {
    const uint32_t row = G.w[k] >> 16;
    y_part[row] = fma(G.v[k], xv[k], y_part[row]);
    __syncwarp();  // orders this round's accumulator updates before the next round's
  }
}

// The G rounds of one group, for layouts whose rows mostly have several entries per unit (FSB_PANEL_RUNS).
// Products of one row are summed in a register and added to the row's accumulator when the row ends (next_word
// is the lane's next slot, or a word of the spare accumulator after its last one): one trip to shared memory
// per run instead of one per entry.  CLASH (layouts flagged FSB_PANEL_LONG_RUNS): a row with more than R
// entries in the unit covers whole lanes, which all close it with their last slot, i.e. in the same round;
// those sums are combined by a segmented scan over the lanes (fixed order) and added once.
//   LAST   this is the lane's last group of the piece (a constant once the caller's loops are unrolled)
template <typename V, int GS, bool CLASH>
__device__ __forceinline__ void panel_rounds_runs(const Group<V, GS>& G, uint32_t next_word, const bool LAST, V& acc,
                                                  const V* __restrict__ xs, V* __restrict__ y_part, int lane,
                                                  uint32_t pad_row) {
  V p[GS];
#pragma unroll
  for (int k = 0; k < GS; ++k) p[k] = G.v[k] * xs[G.w[k] & 0xFFFFu];   // unused slots: value 0, column 0
#pragma unroll
  for (int k = 0; k < GS; ++k) {
    const uint32_t row = G.w[k] >> 16;
    const uint32_t next_row = (k < GS - 1 ? G.w[k + 1] : next_word) >> 16;
    const bool live = row != pad_row;
    if (live) acc += p[k];
    const bool flush = live && next_row != row;
    if (CLASH && LAST && k == GS - 1) {
      const uint32_t row_up = __shfl_down_sync(0xffffffffu, row, 1);
      const bool clash = flush && lane < 31 && row_up == row;
      if (__any_sync(0xffffffffu, clash)) {
        // inclusive segmented sum over the lanes that close the same row, then the last of them adds it
        V s = flush ? acc : (V)0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const V t = __shfl_up_sync(0xffffffffu, s, o);
          const uint32_t r = __shfl_up_sync(0xffffffffu, row, o);
          if (lane >= o && r == row) s += t;
        }
        if (flush && (lane == 31 || row_up != row)) y_part[row] += s;
        acc = (V)0;
      } else if (flush) {
        y_part[row] += acc;
        acc = (V)0;
      }
    } else if (flush) {
      y_part[row] += acc;
      acc = (V)0;
    }
    __syncwarp();  // orders this round's accumulator updates before the next round's
  }
}

constexpr int kModeDirect = 0, kModeRuns = 1, kModeRunsClash = 2;
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

struct PanelGeom {
  int64_t n_cols;
  int chunk_cols;
  int n_buf;
  int debug;      // FSB_PANEL_DEBUG_TIMEOUT: the first chunk's barrier expects bytes that never come
  uint32_t pad_row;  // accumulator index carried by unused slots (one past the CTA's real accumulators)
};

// Units u0 .. u1-1 of one CTA, in order: chunk of x in, pieces added into y_part.  Returns false when a bounded
// wait ran out (every thread of the CTA gets the same answer).
//   - x chunks are fetched n_buf - 1 units ahead into n_buf buffers (unit number `ord` of the CTA uses buffer
//     ord % n_buf; the packed word of a slot already holds buffer * chunk_cols + local column);
//   - piece p goes to warp (p - first piece of the CTA) % 32; a warp walks its pieces in groups of G slots per
//     lane (group q % (R/G) of its piece number q / (R/G)) and always has the next group on its way.
template <typename V, int R, int G, int MODE>
__device__ __forceinline__ bool panel_run_units(const V* __restrict__ val, const uint32_t* __restrict__ rc,
                                                const int32_t* __restrict__ unit_piece_ptr,
                                                const int32_t* __restrict__ unit_chunk, int u0, int u1,
                                                const V* __restrict__ x, const PanelGeom& gm,
                                                const PanelShared<V>& sh) {
  constexpr int GPP = R / G;          // groups per piece
  constexpr int SLOTS = 32 * R;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunk_cols = gm.chunk_cols, n_buf = gm.n_buf;
  const int spins = gm.debug ? kPanelWaitSpinsDebug : kPanelWaitSpins;
  V* xs = sh.xs;
  V* y_part = sh.y_part;
  uint64_t* bars = sh.bars;
  if (u0 >= u1) return true;

  // chunk `c` of x into buffer `b`: bulk copy when the byte count is a multiple of 16, else plain loads
  auto load_chunk = [&](int c, int b, bool first) {
    const int64_t c0 = (int64_t)c * chunk_cols;
    const int n = (int)((gm.n_cols - c0) < (int64_t)chunk_cols ? (gm.n_cols - c0) : (int64_t)chunk_cols);
    const uint32_t bytes = (uint32_t)(n * sizeof(V));
    if ((bytes & 15u) == 0 && aligned_to_dev(x + c0)) {
      if (tid == 0) {
        p_expect_tx(&bars[b], bytes + ((first && gm.debug) ? 16u : 0u));
        p_bulk_g2s(xs + (size_t)b * chunk_cols, x + c0, bytes, &bars[b]);
      }
      return false;
    }
    for (int i = tid; i < n; i += kPanelThreads) xs[(size_t)b * chunk_cols + i] = __ldg(x + c0 + i);
    if (tid == 0) p_expect_tx(&bars[b], (first && gm.debug) ? 16u : 0u);  // completes as soon as this arrival lands
    return true;
  };

  const int p_first = unit_piece_ptr[u0];
  const int p_cta_end = unit_piece_ptr[u1];
  int pc = p_first + warp;            // this warp's next piece
  // The entries do not depend on x: the warp's first group(s) are requested before anything else.
  //   RING   two groups in a register ring, refilled as soon as a group has been consumed (the request for
  //          group q + 2 leaves after group q); measured best where every slot costs a trip to an accumulator
  //   else   the next group is requested right before the current one is used, into registers that are dead
  //          otherwise; measured best for the run-summing rounds, which need the registers themselves
  constexpr bool RING = MODE == kModeDirect;
  const int n_my = (p_cta_end - p_first - warp + kPanelWarps - 1) / kPanelWarps;   // pieces of this warp (may be <= 0)
  const int n_groups = n_my > 0 ? n_my * GPP : 0;
  Group<V, G> ring[2];
  auto request = [&](int q, Group<V, G>& slot) {
    if (q < n_groups) {
      const size_t piece = (size_t)(p_first + warp + kPanelWarps * (q / GPP));
      ld_group(val + piece * SLOTS, rc + piece * SLOTS, lane, q % GPP, slot);
    }
  };
  int q = 0, phase = 0;
  if (RING) {
    request(0, ring[0]);
    request(1, ring[1]);
  } else if (pc < p_cta_end) {
    ld_group(val + (size_t)pc * SLOTS, rc + (size_t)pc * SLOTS, lane, 0, ring[0]);
  }

  // chunks of the first n_buf - 1 units (a chunk written with ordinary stores is also at least one CTA barrier
  // ahead of its first use)
  for (int a = 0; a < n_buf - 1 && u0 + a < u1; ++a) load_chunk(unit_chunk[u0 + a], a, a == 0);

  int b = 0, par = 0;                  // buffer and barrier parity of the current unit
  // One thread waits for a chunk of x; the CTA barrier that follows hands what it has seen on to everybody
  // (1023 threads polling the same mbarrier cost more issue slots than the products themselves).
  if (tid == 0 && !p_wait_bounded(&bars[0], 0u, spins)) *sh.failed = 1;
  for (int w0 = u0; w0 < u1; w0 += kUnitWindow) {
    const int nwin = (u1 - w0) < kUnitWindow ? (u1 - w0) : kUnitWindow;
    const int nch = (u1 - w0) < (kUnitWindow + kUnitLookahead) ? (u1 - w0) : (kUnitWindow + kUnitLookahead);
    if (w0 > u0) __syncthreads();  // the previous window's tables are no longer read
    for (int i = tid; i <= nwin; i += kPanelThreads) sh.upp[i] = unit_piece_ptr[w0 + i];
    for (int i = tid; i < nch; i += kPanelThreads) sh.uch[i] = unit_chunk[w0 + i];
    __syncthreads();               // also: the first chunk has landed (or the wait for it was given up)
    for (int u = w0; u < w0 + nwin; ++u) {
      if (*sh.failed) {
        // leave no copy in flight into this CTA's shared memory: one more bounded wait per chunk requested ahead
        int bb = b, pp = par;
        for (int a = 1; a < n_buf - 1 && u + a < u1; ++a) {
          if (++bb == n_buf) { bb = 0; pp ^= 1; }
          p_wait_bounded(&bars[bb], (uint32_t)pp, spins);
        }
        return false;
      }
      // the buffer of the previous unit was last read before the barrier that closed it: free to refill
      if (u + n_buf - 1 < u1) {
        int bn = b + n_buf - 1;
        bn = bn >= n_buf ? bn - n_buf : bn;
        load_chunk(sh.uch[u + n_buf - 1 - w0], bn, false);
      }
      const int p_end = sh.upp[u - w0 + 1];
      while (pc < p_end) {
        V acc = (V)0;
#pragma unroll
        for (int g = 0; g < GPP; ++g) {
          if (RING) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              if (phase == i) {
                panel_rounds_direct<V, G>(ring[i], xs, y_part);
                request(q + 2, ring[i]);
              }
            }
            phase ^= 1;
            ++q;
          } else {
            // the next group (of this piece, or the first one of this warp's next piece, whichever unit that
            // piece belongs to) is in flight while this one is used
            Group<V, G> nxt;
            const bool more = g + 1 < GPP;
            const int np = more ? pc : pc + kPanelWarps;
            const bool have = np < p_cta_end;
            if (have) ld_group(val + (size_t)np * SLOTS, rc + (size_t)np * SLOTS, lane, more ? g + 1 : 0, nxt);
            // a lane's run ends with its last slot of the piece; inside the piece the next group tells
            const uint32_t next_word = more ? nxt.w[0] : (gm.pad_row << 16);
            panel_rounds_runs<V, G, MODE == kModeRunsClash>(ring[0], next_word, !more, acc, xs, y_part, lane,
                                                             gm.pad_row);
            if (have) ring[0] = nxt;
          }
        }
        pc += kPanelWarps;
      }
      if (++b == n_buf) { b = 0; par ^= 1; }
      // the next unit's chunk must have landed before anybody gathers from it
      if (tid == 0 && u + 1 < u1 && !p_wait_bounded(&bars[b], (uint32_t)par, spins)) *sh.failed = 1;
      __syncthreads();  // every add of this unit is done (its x buffer may be refilled); the next chunk is in
    }
  }
  if (*sh.failed) return false;
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
                                            int n_buf, int n_acc, uint32_t pad_row) {
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
    sh.y_part[pad_row] = (V)0;
    for (int b = 0; b < n_buf; ++b) p_mbar_init(&st->bars[b], 1);
    p_fence_init();
  }
  __syncthreads();
}

// One CTA per block of rb_rows consecutive rows (block block_begin + blockIdx.x); every row of y the launch
// covers is written exactly once.
template <typename V, int R, int G, int MODE>
__global__ void __launch_bounds__(kPanelThreads, 1)
spmv_panel_kernel(const V* __restrict__ val, const uint32_t* __restrict__ rc, const int32_t* __restrict__ unit_piece_ptr,
                  const int32_t* __restrict__ unit_chunk, const int32_t* __restrict__ rb_unit_ptr,
                  const V* __restrict__ x, V* __restrict__ y, int block_begin, int64_t n_rows, int rb_rows,
                  PanelGeom gm, int32_t* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char p_smem[];
  __shared__ __align__(8) PanelStatic p_static;
  const int tid = threadIdx.x;
  const int rb = block_begin + (int)blockIdx.x;
  const int64_t r0 = (int64_t)rb * rb_rows;
  const int nr = (int)((n_rows - r0) < (int64_t)rb_rows ? (n_rows - r0) : (int64_t)rb_rows);
  PanelShared<V> sh;
  panel_setup<V>(sh, p_smem, &p_static, gm.chunk_cols, gm.n_buf, nr, gm.pad_row);
  if (!panel_run_units<V, R, G, MODE>(val, rc, unit_piece_ptr, unit_chunk, rb_unit_ptr[rb], rb_unit_ptr[rb + 1], x,
                                       gm, sh)) {
    if (tid == 0 && status != nullptr) *reinterpret_cast<volatile int32_t*>(status) = 2;  // may be host memory
    return;
  }
  // the accumulators start on a 16-byte boundary of shared memory; so does y + r0 when rb_rows is a multiple of 4
  V* dst = y + r0;
  constexpr int E = 16 / (int)sizeof(V);
  if (aligned_to_dev(dst)) {
    const int nv = nr / E;
    const float4* src4 = reinterpret_cast<const float4*>(sh.y_part);
    float4* dst4 = reinterpret_cast<float4*>(dst);
    for (int i = tid; i < nv; i += kPanelThreads) dst4[i] = src4[i];
    for (int i = nv * E + tid; i < nr; i += kPanelThreads) dst[i] = sh.y_part[i];
  } else {
    for (int i = tid; i < nr; i += kPanelThreads) dst[i] = sh.y_part[i];
  }
}

// Row-group form, for a set of long rows picked out of a matrix (the rest of the matrix goes through the CSR
// kernels).  The picked rows are numbered q = 0 .. n_long-1 and cut into groups; row q owns the accumulators
// vbase[q] .. vbase[q+1]-1 of its group ("virtual rows": a row with more than 16 entries in one chunk spreads
// them over several accumulators, 16 to each, so that the rule "at most 16 entries of an accumulator per
// unit" still holds).  The units of a group are dealt to several CTAs by column range, so a CTA ends with
// partial sums of its group's rows: it writes them to part[cta_part_ptr[cta] + (q - first q of the group)],
// and panel_group_reduce_kernel adds the partial sums of each row in CTA order.
template <typename V, int R, int G, int MODE>
__global__ void __launch_bounds__(kPanelThreads, 1)
spmv_panel_groups_kernel(const V* __restrict__ val, const uint32_t* __restrict__ rc,
                         const int32_t* __restrict__ unit_piece_ptr, const int32_t* __restrict__ unit_chunk,
                         const int32_t* __restrict__ cta_unit_ptr, const int32_t* __restrict__ cta_group,
                         const int32_t* __restrict__ group_q_ptr, const int32_t* __restrict__ vbase,
                         const int64_t* __restrict__ cta_part_ptr, V* __restrict__ part, const V* __restrict__ x,
                         PanelGeom gm, int32_t* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char p_smem[];
  __shared__ __align__(8) PanelStatic p_static;
  const int tid = threadIdx.x;
  const int cta = blockIdx.x;
  const int g = cta_group[cta];
  const int q0 = group_q_ptr[g], q1 = group_q_ptr[g + 1];
  const int vb0 = vbase[q0];
  const int n_acc = vbase[q1] - vb0;
  PanelShared<V> sh;
  panel_setup<V>(sh, p_smem, &p_static, gm.chunk_cols, gm.n_buf, n_acc, gm.pad_row);
  if (!panel_run_units<V, R, G, MODE>(val, rc, unit_piece_ptr, unit_chunk, cta_unit_ptr[cta], cta_unit_ptr[cta + 1],
                                       x, gm, sh)) {
    if (tid == 0 && status != nullptr) *reinterpret_cast<volatile int32_t*>(status) = 2;  // may be host memory
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

// Slots per group by value type and piece size.  float32: 8-slot groups (eight gathers of x leave together)
// except for the 4-round pieces; float64: 4-slot groups.  Two groups live in registers (the one being consumed and
// the next); with 1024 threads per CTA and 64 registers per thread, deeper prefetch measured slower.
template <typename V, int R> struct Shape { static constexpr int G = R >= 8 ? 8 : 4; };
template <int R> struct Shape<double, R> { static constexpr int G = 4; };

}  // namespace fsb

using namespace fsb;

extern "C" int fsb_spmv_panel_piece_slots(int rounds) {
  return (rounds == 4 || rounds == 8 || rounds == 16) ? 32 * rounds : 0;
}

extern "C" size_t fsb_spmv_panel_smem_bytes(int vtype, int rb_rows, int chunk_cols, int n_buffers) {
  const size_t sv = vtype == FSB_F32 ? 4 : 8;
  // the accumulators of the CTA plus the spare one that unused slots add their zeros to
  return (size_t)n_buffers * (size_t)chunk_cols * sv + (((size_t)rb_rows + 1 + 3) & ~(size_t)3) * sv;
}

extern "C" size_t fsb_spmv_panel_static_smem_bytes(void) { return sizeof(PanelStatic); }

static bool panel_buffers_ok(int n_buffers, int chunk_cols) {
  return n_buffers >= 2 && n_buffers <= kMaxXBuffers && (int64_t)n_buffers * chunk_cols <= 65536;
}

// FN<V, R, G, MODE> for the runtime (vtype, rounds, mode)
#define FSB_PANEL_CASE(FN, V, R_, LAUNCH)                                                        \
  do {                                                                                           \
    if (mode == kModeRunsClash) LAUNCH((FN<V, R_, Shape<V, R_>::G, kModeRunsClash>));            \
    else if (mode == kModeRuns) LAUNCH((FN<V, R_, Shape<V, R_>::G, kModeRuns>));                 \
    else LAUNCH((FN<V, R_, Shape<V, R_>::G, kModeDirect>));                                      \
  } while (0)
#define FSB_PANEL_DISPATCH(FN, V, LAUNCH)                                                        \
  do {                                                                                           \
    if (rounds == 4) FSB_PANEL_CASE(FN, V, 4, LAUNCH);                                           \
    else if (rounds == 8) FSB_PANEL_CASE(FN, V, 8, LAUNCH);                                      \
    else FSB_PANEL_CASE(FN, V, 16, LAUNCH);                                                      \
  } while (0)

extern "C" int fsb_spmv_csr_panel(int vtype, const void* val, const uint32_t* rc, const int32_t* unit_piece_ptr,
                                  const int32_t* unit_chunk, const int32_t* rb_unit_ptr, int32_t n_row_blocks,
                                  int32_t rb_rows, int32_t chunk_cols, int32_t n_buffers, int32_t rounds,
                                  int32_t flags, int32_t block_begin, int32_t block_end, const void* x, void* y,
                                  int64_t n_rows, int64_t n_cols, int32_t* status, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (vtype != FSB_F32 && vtype != FSB_F64) return FSB_EINVAL;
  if (n_rows < 0 || n_cols < 0 || n_row_blocks < 0 || rb_rows <= 0 || rb_rows >= 65535) return FSB_EINVAL;
  if (chunk_cols <= 0 || (chunk_cols % 4) != 0 || chunk_cols > 16384) return FSB_EINVAL;
  if (!panel_buffers_ok(n_buffers, chunk_cols)) return FSB_EINVAL;
  if (fsb_spmv_panel_piece_slots(rounds) == 0) return FSB_EINVAL;
  if (block_begin < 0 || block_end > n_row_blocks || block_begin > block_end) return FSB_EINVAL;
  if (n_rows == 0 || block_begin == block_end) return FSB_OK;
  if ((int64_t)n_row_blocks * rb_rows < n_rows) return FSB_EINVAL;
  if (!val || !rc || !unit_piece_ptr || !unit_chunk || !rb_unit_ptr || !x || !y) return FSB_EINVAL;
  const size_t smem = fsb_spmv_panel_smem_bytes(vtype, rb_rows, chunk_cols, n_buffers);
  if (smem + sizeof(PanelStatic) > 227 * 1024) return FSB_ERANGE;
  if (!aligned_to(val, 16) || !aligned_to(rc, 16)) return FSB_EALIGN;
  FSB_WALK_FIRST(check_panel(rc, unit_piece_ptr, unit_chunk, rb_unit_ptr, n_row_blocks,
                             fsb_spmv_panel_piece_slots(rounds), rb_rows, chunk_cols, n_buffers, n_cols, st));
  const int mode = (flags & FSB_PANEL_LONG_RUNS) ? kModeRunsClash : ((flags & FSB_PANEL_RUNS) ? kModeRuns : kModeDirect);
  const PanelGeom gm{n_cols, chunk_cols, n_buffers, (flags & FSB_PANEL_DEBUG_TIMEOUT) ? 1 : 0, (uint32_t)rb_rows};
  const unsigned grid = (unsigned)(block_end - block_begin);
#define FSB_PANEL_LAUNCH_(K)                                                                                    \
  do {                                                                                                          \
    cudaError_t e = cudaFuncSetAttribute(K, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
    if (e != cudaSuccess) return cuda_rc(e);                                                                    \
    K<<<grid, kPanelThreads, smem, st>>>((const VT_*)val, rc, unit_piece_ptr, unit_chunk, rb_unit_ptr,          \
                                         (const VT_*)x, (VT_*)y, block_begin, n_rows, rb_rows, gm, status);     \
  } while (0)
  if (vtype == FSB_F32) {
    typedef float VT_;
    FSB_PANEL_DISPATCH(spmv_panel_kernel, float, FSB_PANEL_LAUNCH_);
  } else {
    typedef double VT_;
    FSB_PANEL_DISPATCH(spmv_panel_kernel, double, FSB_PANEL_LAUNCH_);
  }
#undef FSB_PANEL_LAUNCH_
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}

extern "C" int fsb_spmv_csr_panel_groups(int vtype, const void* val, const uint32_t* rc, const int32_t* unit_piece_ptr,
                                         const int32_t* unit_chunk, const int32_t* cta_unit_ptr, int32_t n_ctas,
                                         int32_t chunk_cols, int32_t n_buffers, int32_t rounds, int32_t flags,
                                         int32_t max_group_acc, const int32_t* cta_group,
                                         const int32_t* group_q_ptr, const int32_t* group_cta_ptr, const int32_t* vbase,
                                         const int32_t* q_group, const int32_t* long_rows, int32_t n_long,
                                         const int64_t* cta_part_ptr, void* part, const void* x, void* y,
                                         int64_t n_cols, int32_t* status, void* stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (vtype != FSB_F32 && vtype != FSB_F64) return FSB_EINVAL;
  if (n_cols < 0 || n_ctas < 0 || n_long < 0 || max_group_acc < 0 || max_group_acc >= 65535) return FSB_EINVAL;
  if (chunk_cols <= 0 || (chunk_cols % 4) != 0 || chunk_cols > 16384) return FSB_EINVAL;
  if (!panel_buffers_ok(n_buffers, chunk_cols)) return FSB_EINVAL;
  if (fsb_spmv_panel_piece_slots(rounds) == 0) return FSB_EINVAL;
  if (n_long == 0 || n_ctas == 0) return FSB_OK;
  if (!val || !rc || !unit_piece_ptr || !unit_chunk || !cta_unit_ptr || !cta_group || !group_q_ptr ||
      !group_cta_ptr || !vbase || !q_group || !long_rows || !cta_part_ptr || !part || !x || !y)
    return FSB_EINVAL;
  const size_t smem = fsb_spmv_panel_smem_bytes(vtype, max_group_acc, chunk_cols, n_buffers);
  if (smem + sizeof(PanelStatic) > 227 * 1024) return FSB_ERANGE;
  if (!aligned_to(val, 16) || !aligned_to(rc, 16)) return FSB_EALIGN;
  FSB_WALK_FIRST(check_panel(rc, unit_piece_ptr, unit_chunk, cta_unit_ptr, n_ctas, fsb_spmv_panel_piece_slots(rounds),
                             max_group_acc, chunk_cols, n_buffers, n_cols, st));
  const int mode = (flags & FSB_PANEL_LONG_RUNS) ? kModeRunsClash : ((flags & FSB_PANEL_RUNS) ? kModeRuns : kModeDirect);
  const PanelGeom gm{n_cols, chunk_cols, n_buffers, (flags & FSB_PANEL_DEBUG_TIMEOUT) ? 1 : 0,
                     (uint32_t)max_group_acc};
  const unsigned rgrid = (unsigned)((n_long + 255) / 256);
#define FSB_GROUPS_LAUNCH_(K)                                                                                    \
  do {                                                                                                           \
    cudaError_t e = cudaFuncSetAttribute(K, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
    if (e != cudaSuccess) return cuda_rc(e);                                                                     \
    K<<<(unsigned)n_ctas, kPanelThreads, smem, st>>>((const VT_*)val, rc, unit_piece_ptr, unit_chunk,            \
                                                     cta_unit_ptr, cta_group, group_q_ptr, vbase, cta_part_ptr,  \
                                                     (VT_*)part, (const VT_*)x, gm, status);                     \
  } while (0)
  if (vtype == FSB_F32) {
    typedef float VT_;
    FSB_PANEL_DISPATCH(spmv_panel_groups_kernel, float, FSB_GROUPS_LAUNCH_);
    FSB_RETURN_IF_LAUNCH_FAILED();
    panel_group_reduce_kernel<float><<<rgrid, 256, 0, st>>>((const float*)part, q_group, group_q_ptr, group_cta_ptr,
                                                             cta_part_ptr, long_rows, (float*)y, n_long);
  } else {
    typedef double VT_;
    FSB_PANEL_DISPATCH(spmv_panel_groups_kernel, double, FSB_GROUPS_LAUNCH_);
    FSB_RETURN_IF_LAUNCH_FAILED();
    panel_group_reduce_kernel<double><<<rgrid, 256, 0, st>>>((const double*)part, q_group, group_q_ptr,
                                                              group_cta_ptr, cta_part_ptr, long_rows, (double*)y,
                                                              n_long);
  }
#undef FSB_GROUPS_LAUNCH_
  FSB_RETURN_IF_LAUNCH_FAILED();
  return FSB_OK;
}
