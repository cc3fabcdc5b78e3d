/*
 * fsb.h -- C ABI of libfsb.so, the sm_100a CUDA library behind flagsparse_b200.
 *
 * The reference package (zyq1105331849/flagsparse) has no C/FFI layer: its CSR SpMV and CSR SpMM are
 * Python functions that launch Triton kernels.  Each entry point below replaces one of those launch sites;
 * the comment on each names the reference function it stands in for (paths are relative to the reference
 * project root).  The Python host code in flagsparse_b200/ validates arguments exactly where the reference
 * does and then calls these functions through ctypes with raw device pointers.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless the comment says "host".
 *   - vtype: value dtype of data / x / B / y / C.  itype: dtype of `indices`.  ptype: dtype of `indptr`.
 *   - All work is enqueued on `stream` (a cudaStream_t passed as void*); no call synchronises the host
 *     and no call allocates or frees device memory -- the caller owns every buffer, scratch included (the one
 *     exception is fsb_spmv_csr_noalloc, whose scratch is an array built into the library).
 *   - Return value: 0 on success, a negative FSB_E* code for an argument error detected on the host, or
 *     FSB_CUDA_ERROR_BASE + cudaError_t when a launch failed.
 *   - Inputs are assumed validated (indptr non-decreasing, indptr[0]==0, indptr[n_rows]==nnz,
 *     0 <= indices < n_cols).  fsb_csr_analyze gathers what the host needs to check that in one pass.
 *   - n_rows and n_cols must be < 2^31; nnz may exceed 2^31 when ptype is FSB_I64.
 */
#ifndef FSB_H_
#define FSB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FSB_VERSION 100

/* dtype tags */
#define FSB_F32 0
#define FSB_F64 1
#define FSB_F16 2             /* fsb_spmv_csr_wide / fsb_spmm_csr_wide only */
#define FSB_BF16 3
#define FSB_C64 4             /* interleaved (re, im) float32 pairs */
#define FSB_C128 5            /* interleaved (re, im) float64 pairs */
#define FSB_I32 0
#define FSB_I64 1

/* error codes (negative) */
#define FSB_OK 0
#define FSB_EINVAL (-1)      /* bad enum / negative size / null pointer where one is required */
#define FSB_ERANGE (-2)      /* n_rows, n_cols or a tile count outside the supported range   */
#define FSB_EALIGN (-3)      /* pointer not aligned to its element size                      */
#define FSB_ESCRATCH (-4)    /* scratch buffer smaller than fsb_*_scratch_bytes() asks for   */
#define FSB_ENOSPACE (-5)    /* problem too large for the library's built-in scratch array   */
#define FSB_EBOUNDS (-6)     /* checking build only: an index array would take a kernel out of bounds; nothing ran */
#define FSB_CUDA_ERROR_BASE 1000

/* SpMV algorithm selector */
#define FSB_SPMV_AUTO 0
#define FSB_SPMV_VECTOR 1    /* a group of 2..32 lanes per row; one launch, no scratch       */
#define FSB_SPMV_STREAM 2    /* fixed-size nnz tiles (load-balanced); needs plan + scratch   */

/* SpMM staging selector */
#define FSB_SPMM_AUTO 0
#define FSB_SPMM_PLAIN 1     /* tile of data/indices staged in shared memory by ordinary loads   */
#define FSB_SPMM_BULK 2      /* tile staged by cp.async.bulk (TMA 1-D bulk copy) + mbarrier       */
#define FSB_SPMM_ACCUMULATE 16 /* or-ed into the selector: C += A B instead of C = A B            */

int fsb_version(void);

/* nnz per tile of the tiled kernels (a power of two).  `tuning` is the value later passed to
 * fsb_spmv_csr: bits 8-9 pick the SpMV tile (0 = default 2048, 1 = 1024, 3 = 4096). */
int fsb_spmv_tile_nnz(int vtype, int tuning);
int fsb_spmm_tile_nnz(int vtype);

/*
 * Statistics of a CSR structure, written to 8 consecutive int64 on the DEVICE (`stats`):
 *   [0] indptr[0]            [1] indptr[n_rows]      [2] number of i with indptr[i+1] < indptr[i]
 *   [3] min(indices)         [4] max(indices)        [5] max row length
 *   [6] number of empty rows [7] number of rows longer than 32x the mean row length (rounded up)
 * ([3] = INT64_MAX and [4] = INT64_MIN when nnz == 0; [5] = 0 when n_rows == 0.)
 * Replaces the six separate device reductions + host syncs of the reference's
 * _prepare_spmv_csr_matrix (src/flagsparse/sparse_operations/spmv_csr.py:404-427) and
 * _prepare_spmm_csr_matrix (src/flagsparse/sparse_operations/spmm_csr.py:226-254): the host reads the
 * eight numbers back with one copy.  `indices` may be NULL when nnz == 0.
 */
int fsb_csr_analyze(int itype, int ptype, const void* indices, const void* indptr, int64_t n_rows,
                    int64_t nnz, int64_t* stats, void* stream);

/*
 * Tile plan: tile_row[t] for t = 0..n_tiles, n_tiles = ceil(nnz / tile_nnz), int32 on the device.
 *   tile_row[0] = 0, tile_row[n_tiles] = n_rows, otherwise the row that holds nnz number t*tile_nnz.
 * Rows [tile_row[t], tile_row[t+1]) are the rows whose last nnz lies in tile t (empty rows go to the
 * tile in which their indptr value falls), i.e. the rows tile t writes.  Plays the part of the
 * reference's row buckets (_build_spmv_opt_buckets, spmv_csr.py:281-327; _build_spmm_opt_buckets and
 * _build_spmm_opt_split_metadata, spmm_csr.py:417-477): it is built once per matrix at prepare time.
 */
int64_t fsb_csr_num_tiles(int64_t nnz, int tile_nnz);
int fsb_csr_tile_plan(int ptype, const void* indptr, int64_t n_rows, int64_t nnz, int tile_nnz,
                      int32_t* tile_row, void* stream);

/*
 * y = A x for CSR A.  Replaces the launches in _triton_spmv_csr_impl_opt_prepared
 * (spmv_csr.py:329-376, kernels :161-279) and _triton_spmv_csr_impl_prepared (:510-554, kernel :94-120).
 * Every y[i] is written exactly once per call (empty rows get an exact 0), nothing else is written.
 *   algo      FSB_SPMV_VECTOR needs neither tile_row nor scratch.
 *             FSB_SPMV_STREAM needs tile_row from fsb_csr_tile_plan(tile_nnz = fsb_spmv_tile_nnz(vtype, tuning))
 *             and `scratch` of at least fsb_spmv_csr_scratch_bytes() bytes, 16-byte aligned.
 *             FSB_SPMV_AUTO picks STREAM when tile_row and scratch are given and nnz is large, else VECTOR.
 *   tuning    0 = default; otherwise kernel-specific knob (VECTOR: lanes per row, a power of two 2..32;
 *             STREAM: bits 0-7 = 1 + the right-shift applied to a tile's mean row length to get the
 *             lanes per row; bits 8-9 = tile size, see fsb_spmv_tile_nnz).  Results stay within tolerance for any value; only speed changes.
 * The result is deterministic: the same inputs give the same bits on every call (no floating atomics).
 */
size_t fsb_spmv_csr_scratch_bytes(int vtype, int64_t nnz, int tuning);
int fsb_spmv_csr(int vtype, int itype, int ptype, const void* data, const void* indices,
                 const void* indptr, const void* x, void* y, int64_t n_rows, int64_t n_cols, int64_t nnz,
                 int algo, int tuning, const int32_t* tile_row, void* scratch, size_t scratch_bytes,
                 void* stream);

/*
 * Same product, but every finished y value is stored into n_peers output vectors (one per GPU of the
 * box, the local one included) through peer-mapped pointers, at element offset row_offset + i: the
 * SpMV epilogue doubles as the all-gather of the row-sharded driver.  y_peers is a DEVICE array of
 * n_peers pointers.  algo: FSB_SPMV_VECTOR (no plan, no scratch) or FSB_SPMV_STREAM, as for fsb_spmv_csr;
 * FSB_SPMV_AUTO takes STREAM when tile_row and scratch are given.  first_peer = this GPU's index in y_peers: the
 * destinations are visited in an order rotated by it (and by the CTA), so that the GPUs of a box do not all write
 * to the same destination at once.  The reference has no multi-GPU path; this
 * stands in for "each rank runs spmv_csr.py:329-376 on its row shard, then y is all-gathered".
 */
int fsb_spmv_csr_scatter(int vtype, int itype, int ptype, const void* data, const void* indices,
                         const void* indptr, const void* x, void* const* y_peers, int n_peers, int first_peer,
                         int64_t row_offset, int64_t n_rows, int64_t n_cols, int64_t nnz, int algo, int tuning,
                         const int32_t* tile_row, void* scratch, size_t scratch_bytes, void* stream);

/*
 * y = A x from the "panel" regrouping of a CSR matrix (built once per matrix by the host code,
 * flagsparse_b200/panel.py): entries grouped into units = (block of rb_rows rows) x (chunk of chunk_cols
 * columns), row-major inside a unit, each unit cut into pieces of fsb_spmv_panel_piece_slots(rounds) =
 * 32 * rounds slots so that no row's entries straddle two pieces.
 *   val[s], rc[s]        per slot: value and packed word (local row << 16 | buffer * chunk_cols + local
 *                        column), buffer = ordinal of the unit inside its row block modulo n_buffers; unused
 *                        slots carry value 0, column 0 and local row = rb_rows (a spare accumulator)
 *   chunk_cols           columns of x per unit: a multiple of 4, at most 16384 (a chunk is one bulk copy into
 *                        shared memory; the host code uses 10240 for float32 and 4096 for float64)
 *   rounds               4, 8 or 16: slots per lane and piece.  Small pieces suit units with few entries
 *                        (every warp of the CTA gets work in every unit)
 *   flags                FSB_PANEL_RUNS: rows have several entries per unit on average; the kernel then sums a
 *                        row's products in a register and visits the accumulator once per run (otherwise once
 *                        per entry, with no predicates).  Only speed depends on this flag.
 *                        FSB_PANEL_LONG_RUNS: some row has more than `rounds` entries inside one unit (never
 *                        more than a piece holds); the kernel then also combines the lanes that finish on the
 *                        same row.  Must be set for such layouts.  FSB_PANEL_DEBUG_TIMEOUT (tests only): the first copy of x of every CTA is made to
 *                        look incomplete and the wait limit is lowered, so that the kernel takes its time-out
 *                        path -- it reports through `status` and returns without touching y
 *   n_buffers            2..8 chunks of x in shared memory (n_buffers * chunk_cols <= 65536): chunks are
 *                        fetched n_buffers - 1 units ahead of their use
 *   unit_piece_ptr       pieces [unit_piece_ptr[u], unit_piece_ptr[u+1]) belong to unit u
 *   unit_chunk           column chunk of unit u
 *   rb_unit_ptr          units [rb_unit_ptr[b], rb_unit_ptr[b+1]) belong to row block b, in chunk order
 *   block_begin/_end     the launch covers row blocks [block_begin, block_end) only (rows block_begin * rb_rows
 *                        onward); the row-sharded driver issues one launch per slice of its shard and ships a
 *                        finished slice to the other GPUs while the next one is computed
 * One CTA per row block keeps the block's y accumulators and n_buffers chunks of x in shared memory
 * (fsb_spmv_panel_smem_bytes() + fsb_spmv_panel_static_smem_bytes() must fit in 227 KiB; rb_rows < 65535).  Another stand-in for the launches of
 * _triton_spmv_csr_impl_opt_prepared (spmv_csr.py:329-376), for matrices whose rows span few column chunks.
 * status: optional int32 in device memory or in page-locked host memory, set non-zero (a plain store) if a bounded
 * wait on a bulk copy of x ran out.
 */
#define FSB_PANEL_LONG_RUNS 1
#define FSB_PANEL_RUNS 2
#define FSB_PANEL_DEBUG_TIMEOUT 256
int fsb_spmv_panel_piece_slots(int rounds);
size_t fsb_spmv_panel_smem_bytes(int vtype, int rb_rows, int chunk_cols, int n_buffers);
size_t fsb_spmv_panel_static_smem_bytes(void);
int fsb_spmv_csr_panel(int vtype, const void* val, const uint32_t* rc, const int32_t* unit_piece_ptr,
                       const int32_t* unit_chunk, const int32_t* rb_unit_ptr, int32_t n_row_blocks,
                       int32_t rb_rows, int32_t chunk_cols, int32_t n_buffers, int32_t rounds, int32_t flags,
                       int32_t block_begin, int32_t block_end, const void* x, void* y, int64_t n_rows,
                       int64_t n_cols, int32_t* status, void* stream);

/*
 * Row-group form of the panel product, for the LONG rows of a skewed matrix: y[long_rows[q]] = (A x)[long_rows[q]]
 * for q = 0 .. n_long-1; the other rows of y are not touched (the host code runs fsb_spmv_csr on the remaining
 * short rows first).  Replaces, for those rows, the long-row buckets of _triton_spmv_csr_impl_opt_prepared
 * (spmv_csr.py:329-376 with the bucket tables :64-89: one Triton program per long row).
 * The picked rows are cut into groups; row q owns accumulators vbase[q] .. vbase[q+1]-1 ("virtual rows": at most
 * `rounds` entries of a virtual row in one column chunk) and the packed word of a slot holds the virtual row relative
 * to its group (unused slots: max_group_acc).  The units (group x column chunk) are ordered by group, then chunk, and dealt to n_ctas CTAs:
 *   cta_unit_ptr         units [cta_unit_ptr[c], cta_unit_ptr[c+1]) belong to CTA c (buffer of a slot's packed
 *                        word = ordinal of the unit inside its CTA modulo n_buffers)
 *   cta_group            group of CTA c;  group_cta_ptr: CTAs [group_cta_ptr[g], group_cta_ptr[g+1]) work on group g
 *   group_q_ptr          rows q in [group_q_ptr[g], group_q_ptr[g+1]) form group g;  q_group[q]: group of row q
 *   max_group_acc        largest number of accumulators of a group (shared memory: fsb_spmv_panel_smem_bytes)
 *   cta_part_ptr, part   CTA c writes one partial sum per row of its group to part[cta_part_ptr[c] + ...]; a
 *                        second kernel adds the partial sums of a row in CTA order (in double) and stores y.
 *                        part must hold sum over CTAs of the row count of their group, in elements of vtype.
 * Everything else (rounds and flags included) as for fsb_spmv_csr_panel.  Results are bit-reproducible.
 */
int fsb_spmv_csr_panel_groups(int vtype, const void* val, const uint32_t* rc, const int32_t* unit_piece_ptr,
                              const int32_t* unit_chunk, const int32_t* cta_unit_ptr, int32_t n_ctas,
                              int32_t chunk_cols, int32_t n_buffers, int32_t rounds, int32_t flags,
                              int32_t max_group_acc, const int32_t* cta_group,
                              const int32_t* group_q_ptr, const int32_t* group_cta_ptr, const int32_t* vbase,
                              const int32_t* q_group, const int32_t* long_rows, int32_t n_long,
                              const int64_t* cta_part_ptr, void* part, const void* x, void* y, int64_t n_cols,
                              int32_t* status, void* stream);

/*
 * y = A x with the STREAM algorithm for callers that must not (or cannot) allocate device memory: code
 * running inside a frozen or fixed-size memory pool, plugins that only ever receive buffers from their
 * host framework, latency-critical loops where cudaMalloc's device-wide synchronisation is unacceptable.
 * This entry point has no counterpart in the reference (its Triton launches allocate through torch).
 * The per-tile partial sums that fsb_spmv_csr keeps in caller scratch live here in an array that is part
 * of the library image -- FSB_NOALLOC_MAX_TILES tiles, 4 MiB, resident on every GPU that loads the
 * library until the process exits.  The call itself allocates and frees nothing; inputs, y and tile_row
 * (fsb_csr_tile_plan with tile_nnz = fsb_spmv_tile_nnz(vtype, tuning)) still come from the caller.
 *   - Limit: ceil(nnz / tile_nnz) <= FSB_NOALLOC_MAX_TILES (about 5.3e8 nnz at the default tile of 2048);
 *     a larger matrix is refused with FSB_ENOSPACE before anything is launched.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current).  Make that first call outside any stream capture.
 *   - All calls on a device share the one array, which keeps whatever the previous call left in it.
 *     Nothing in it needs clearing -- each launch writes every slot it later reads -- but two calls that
 *     overlap on the GPU (different streams, or different host threads) would overwrite each other's
 *     partial sums: serialise them.
 * Results are bit-identical to fsb_spmv_csr(FSB_SPMV_STREAM) with the same tuning.
 */
/*
 * Construction of the panel layout on the device (the reference has no counterpart: its prepare step builds row
 * buckets, spmv_csr.py:281-327).  Passes called in this order by flagsparse_b200/panel.py, every array caller-owned:
 *   count  cnt[rb * n_ch + c] = entries of row block rb (rb_rows rows) in column chunk c (chunk_cols columns);
 *          n_ch = ceil(n_cols / chunk_cols) <= fsb_panel_build_max_chunks()
 *   sort   the entries in unit order (units = non-empty (rb, c) cells in row-major cell order; inside a unit the CSR
 *          order is kept): sorted_val / sorted_row (global row) / sorted_col (global column), nnz < 2^31 elements each;
 *          unit_base[rb * n_ch + c] = position of the unit's first entry.  *status (device int32) is set to 1 when 1024
 *          consecutive entries of the matrix span more than fsb_panel_build_window(wide_window) chunks -- the caller
 *          then falls back to another builder (the wide window costs more per tile: for wide bands only)
 *   runs   stats[0..4] (device int64) = runs (consecutive sorted entries of one row in one unit), longest run, runs
 *          longer than 4 / 8 / 16 entries
 *   cut    greedy cuts of every unit into pieces of at most `slots` entries that split no run.  With piece_start ==
 *          NULL: piece_count[u] = pieces of unit u.  With piece_start: piece_start[unit_piece_ptr[u] + k] = first sorted
 *          entry of the k-th piece of unit u (the caller sets piece_start[n_pieces] = nnz).  *status = 2 when a run is
 *          longer than a piece
 *   fill   val / rc of fsb_spmv_csr_panel (n_pieces * 32 * rounds slots): per piece, entries in stable order of
 *          (local row mod 32 for float32, mod 16 for float64), slot s of that order in lane s / rounds, round s % rounds;
 *          unit_rb[u] = row block of unit u, unit_ord[u] = its ordinal inside that row block (picks the x buffer);
 *          unused slots carry value 0 and the spare accumulator rb_rows
 *   core_count / core_place (float32 layouts whose rows mostly have one entry per unit): the entries alone in their run,
 *          listed per class (local row mod 32) in unit order, fill core_pieces[u] = (shortest list) / rounds pieces of
 *          unit u completely, lane = class, so that a round's 32 accumulators lie in 32 banks; core_place writes those
 *          pieces (core_base[u] = first of them in core_val / core_rc) and copies every other entry, in order, to
 *          rest_val / rest_row / rest_col from rest_start[u] on, for cut and fill to treat like an ordinary unit
 */
int fsb_panel_build_max_chunks(void);
int fsb_panel_build_count(int itype, int ptype, const void* indices, const void* indptr, int64_t n_rows,
                          int64_t n_cols, int32_t rb_rows, int32_t chunk_cols, int32_t* cnt, void* stream);
int fsb_panel_build_sort(int vtype, int itype, int ptype, const void* data, const void* indices, const void* indptr,
                         int64_t n_rows, int64_t n_cols, int32_t rb_rows, int32_t chunk_cols, int32_t wide_window,
                         const int32_t* unit_base, void* sorted_val, int32_t* sorted_row, int32_t* sorted_col,
                         int32_t* status, void* stream);
int fsb_panel_build_window(int wide);
int fsb_panel_build_runs(const int32_t* sorted_row, const int32_t* sorted_col, int64_t nnz, int32_t chunk_cols,
                         int64_t* stats, void* stream);
int fsb_panel_build_cut(const int32_t* sorted_row, const int32_t* unit_start, int32_t n_units, int32_t slots,
                        const int32_t* unit_piece_ptr, int32_t* piece_count, int32_t* piece_start, int32_t* status,
                        void* stream);
int fsb_panel_build_fill(int vtype, const void* sorted_val, const int32_t* sorted_row, const int32_t* sorted_col,
                         const int32_t* piece_start, const int32_t* unit_piece_ptr, int32_t n_units,
                         const int32_t* unit_rb, const int32_t* unit_ord, int32_t n_pieces, int32_t rb_rows,
                         int32_t chunk_cols, int32_t n_buffers, int32_t rounds, void* val, uint32_t* rc, void* stream);
int fsb_panel_build_core_count(const int32_t* sorted_row, const int32_t* unit_start, const int32_t* unit_rb,
                               int32_t n_units, int32_t rb_rows, int32_t rounds, int32_t* core_pieces,
                               int32_t* rest_count, void* stream);
int fsb_panel_build_core_place(int vtype, const void* sorted_val, const int32_t* sorted_row, const int32_t* sorted_col,
                               const int32_t* unit_start, const int32_t* unit_rb, const int32_t* unit_ord,
                               int32_t n_units, int32_t rb_rows, int32_t chunk_cols, int32_t n_buffers, int32_t rounds,
                               const int32_t* core_pieces, const int32_t* core_base, const int32_t* rest_start,
                               void* core_val, uint32_t* core_rc, void* rest_val, int32_t* rest_row, int32_t* rest_col,
                               void* stream);

#define FSB_NOALLOC_MAX_TILES 262144
int fsb_spmv_csr_noalloc(int vtype, int itype, int ptype, const void* data, const void* indices,
                         const void* indptr, const void* x, void* y, int64_t n_rows, int64_t n_cols,
                         int64_t nnz, int tuning, const int32_t* tile_row, void* stream);

/*
 * C = A B for CSR A and dense row-major B (n_cols x n_dense, leading dimension ldb elements);
 * C is n_rows x n_dense with leading dimension ldc.  Replaces _triton_spmm_csr_impl
 * (spmm_csr.py:525-599, kernel :92-134) and _triton_spmm_csr_impl_opt_prepared (:1033-1055, kernels
 * :602-919, split workspace :976-1030).  Every C[i, j] is written exactly once per call.
 *   algo      staging selector, optionally or-ed with FSB_SPMM_ACCUMULATE: the product is then added to what C
 *             holds (rows of A without entries leave their row of C untouched).  The host code uses it to
 *             multiply by column panels of A one after the other, each panel's slice of B small enough to stay
 *             in L2 while it is gathered from, and by column tiles of B / C (pass the tile's first element and the
 *             full leading dimensions).
 *   tile_row  from fsb_csr_tile_plan(tile_nnz = fsb_spmm_tile_nnz(vtype)).
 *   scratch   at least fsb_spmm_csr_scratch_bytes() bytes, 16-byte aligned (per-tile partial rows of
 *             rows that cross a tile boundary -- the counterpart of the reference's split workspace).
 *   status    optional int32 (device or page-locked host memory); set to a non-zero code if a bounded wait on a bulk copy ran out
 *             (the affected tiles are then left unwritten).  May be NULL.
 */
size_t fsb_spmm_csr_scratch_bytes(int vtype, int64_t nnz, int64_t n_dense);
int fsb_spmm_csr(int vtype, int itype, int ptype, const void* data, const void* indices,
                 const void* indptr, const void* B, int64_t ldb, void* C, int64_t ldc, int64_t n_rows,
                 int64_t n_cols, int64_t n_dense, int64_t nnz, int algo, const int32_t* tile_row,
                 void* scratch, size_t scratch_bytes, int32_t* status, void* stream);

/*
 * y = A x for float16, bfloat16, complex64 and complex128 values, read as they are stored (no widened or split copy of
 * the matrix).  vtype FSB_F16 / FSB_BF16: data holds 2-byte values, x and y are float32 (the caller widens x and rounds
 * y once per call, which is what the reference's base path computes: spmv_csr.py:496-535 with the kernel :94-120 on
 * float32 copies); products and sums in float32.  vtype FSB_C64 / FSB_C128: data, x and y hold interleaved (re, im)
 * pairs of float32 / float64; replaces the launch of _spmv_csr_complex_kernel (spmv_csr.py:123-155, 536-554).
 * indices are int32, indptr int32 or int64 (ptype).  One launch, no scratch, bit-reproducible.
 */
int fsb_spmv_csr_wide(int vtype, int ptype, const void* data, const int32_t* indices, const void* indptr,
                      const void* x, void* y, int64_t n_rows, int64_t n_cols, int64_t nnz, void* stream);

/*
 * C = A B for the same four value types, with the same conventions (B and C float32 for the half precisions, of the
 * matrix's own interleaved type for complex values; row-major with leading dimensions ldb / ldc in elements of that
 * type).  Replaces the launch in _triton_spmm_csr_impl for these types (spmm_csr.py:525-599, complex kernel :138-195).
 */
int fsb_spmm_csr_wide(int vtype, int ptype, const void* data, const int32_t* indices, const void* indptr,
                      const void* B, int64_t ldb, void* C, int64_t ldc, int64_t n_rows, int64_t n_cols,
                      int64_t n_dense, int64_t nnz, void* stream);

/*
 * Sampled dense-dense product on a CSR pattern: out[p] = alpha * dot(X[row(p), :], Y[indices[p], :]) + beta * data[p]
 * for every entry p.  X is n_rows x k_dim and Y is n_cols x k_dim, row-major with leading dimensions ldx / ldy
 * (elements); row_ids[p] is the row of entry p (int32, built once per pattern from indptr); data may be NULL (then
 * beta is ignored); out has nnz elements and may alias data.  Dot products are accumulated in the value type.
 * Replaces the launch in _run_sddmm_prepared (src/flagsparse/sparse_operations/sddmm_csr.py:265-347, kernel
 * :107-152); the row-id array is the reference's too (:83-91).
 */
int fsb_sddmm_csr(int vtype, const int32_t* indices, const int32_t* row_ids, const void* X, int64_t ldx,
                  const void* Y, int64_t ldy, const void* data, void* out, int64_t n_rows, int64_t n_cols,
                  int64_t nnz, int64_t k_dim, double alpha, double beta, void* stream);

/*
 * The checking build (the same sources compiled with -DFSB_BOUNDS_CHECK into libfsb_check.so; the stand-in for a
 * memory checker on hosts where none can be run).  There every product entry point above first walks the index arrays
 * it was handed -- column indices against n_cols, row pointers against nnz and against each other, SDDMM row ids
 * against n_rows, the packed words and unit tables of a panel layout against the shared-memory arrays they index --
 * waits for the walk, and if anything is out of range returns FSB_EBOUNDS without launching the product: no trap, no
 * fault, the context stays usable.  (The walk synchronises the stream, so the checking build cannot be captured into
 * a CUDA graph.)  fsb_bounds_check_report() then gives out[0..4] = {violations seen, FSB_BAD_* kind of the first one
 * recorded, its position in its array, the value found, the limit it broke} of the last refused call and clears the
 * record.  In the ordinary build fsb_bounds_check_enabled() is 0 and the report returns FSB_EINVAL.
 */
#define FSB_BAD_COLUMN 1              /* indices[position] outside [0, n_cols)                       */
#define FSB_BAD_ROW_POINTER 2         /* indptr[position] outside [0, nnz]                           */
#define FSB_ROW_POINTER_DECREASES 3   /* indptr[position] < indptr[position - 1] (the limit)         */
#define FSB_BAD_ROW_ID 4              /* row_ids[position] outside [0, n_rows)                       */
#define FSB_BAD_SLOT_ROW 5            /* accumulator of slot `position` beyond the spare accumulator */
#define FSB_BAD_SLOT_COLUMN 6         /* x slot of slot `position` >= n_buffers * chunk_cols         */
#define FSB_BAD_CHUNK 7               /* unit_chunk[position] * chunk_cols >= n_cols                 */
#define FSB_BAD_UNIT_TABLE 8          /* a unit / piece pointer table that is negative or decreases  */
int fsb_bounds_check_enabled(void);
int fsb_bounds_check_report(int64_t* out);

#ifdef __cplusplus
}
#endif
#endif /* FSB_H_ */
