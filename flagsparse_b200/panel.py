"""Prepare-time regrouping of a CSR matrix for the panel SpMV kernel (csrc/spmv_panel.cu).

The reference's prepare step builds row-length buckets (src/flagsparse/sparse_operations/spmv_csr.py:281-327);
this one builds, for matrices whose rows reach a limited range of columns, a second copy of the entries
grouped into units = (block of RB rows) x (chunk of CW columns), so that the kernel can keep the part of x a
unit needs in shared memory.  It runs once per matrix, off the timed path: by the kernels of
csrc/panel_build.cu (_build_fused) where they apply, else by torch operations on the device (_build_slab,
pack_pieces, pack_pieces_core -- also the reference the kernels are tested against, bit for bit); the product
itself is one launch of fsb_spmv_csr_panel.
"""

import os

import torch

from . import _lib
from ._common import StatusWord, _VTYPE

SM_COUNT_FALLBACK = 148
CTAS_PER_SM = 1              # one 1024-thread CTA (row block) per SM
# the kernel is worth its second copy of the matrix only when the extra reads of x and the padding stay small
# bytes of x chunks loaded / bytes of entries streamed.  float32: measured on a band of +-2^20 columns (0.89: 319 G
# entries/s against 231 G/s of the vector kernel; the SM's intake of about 37 GB/s is what bounds it, which puts the
# break-even near 1.9).  float64 entries are 12 bytes and their chunks hold half the columns: estimate, not measured.
MAX_X_OVERHEAD = 1.3
MAX_X_OVERHEAD_F64 = 0.8
MAX_SLOT_OVERHEAD = 1.25    # slots stored / entries
N_BUFFERS = 2               # chunks of x in shared memory (fetched N_BUFFERS - 1 units ahead)
ROUNDS = (4, 8, 16)         # slots per lane and piece the kernel is built for (see csrc/spmv_panel.cu)
FLAG_LONG_RUNS = 1          # FSB_PANEL_LONG_RUNS
FLAG_RUNS = 2               # FSB_PANEL_RUNS
# mean entries of a row inside one unit from which summing a run in a register beats one accumulator update per entry
RUNS_MIN_MEAN = 1.5
FLAG_DEBUG_TIMEOUT = 256    # FSB_PANEL_DEBUG_TIMEOUT
MAX_ROW_NNZ = 512
MIN_NNZ = 1 << 22
ACC_BANKS = {4: 32, 8: 16}   # accumulators that sit in different shared-memory banks (32 banks of 4 bytes), by value size


class PanelLayout:
    """Device arrays of the regrouped matrix plus the launch geometry."""

    __slots__ = ("val", "rc", "unit_piece_ptr", "unit_chunk", "rb_unit_ptr", "n_row_blocks", "rb_rows", "chunk_cols",
                 "n_buffers", "rounds", "flags", "max_run", "pad_row", "n_units", "n_pieces", "x_overhead",
                 "slot_overhead", "status")

    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in (self.val, self.rc, self.unit_piece_ptr, self.unit_chunk,
                                                           self.rb_unit_ptr))


def smem_budget():
    """Dynamic shared memory one CTA of the panel kernels may use (227 KiB per CTA less the kernel's own tables)."""
    return 227 * 1024 - int(_lib.lib().fsb_spmv_panel_static_smem_bytes()) - 1024


def default_buffers():
    return int(os.environ.get("FSB_PANEL_BUFFERS", "0")) or N_BUFFERS


def default_rounds():
    """FSB_PANEL_ROUNDS=4|8|16 fixes the piece size; unset, build_panel_layout picks it from the run lengths."""
    r = int(os.environ.get("FSB_PANEL_ROUNDS", "0"))
    return r if r in ROUNDS else None


def _geometry(dtype, n_rows, device, n_buffers):
    L = _lib.lib()
    vt = _VTYPE[dtype]
    sv = 4 if dtype == torch.float32 else 8
    # columns per chunk of x (any multiple of 4; two buffers of it sit beside the accumulators).  Measured on the two
    # banded benchmark matrices: 10240 beats 8192 by 2-4 % (fewer, fuller units), 12288 and more lose on the narrow
    # band (less room for accumulators)
    chunk_cols = int(os.environ.get("FSB_PANEL_CHUNK", "0")) or (10240 if sv == 4 else 4096)
    try:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
    except Exception:
        sms = SM_COUNT_FALLBACK
    budget = smem_budget() // CTAS_PER_SM
    fixed = int(L.fsb_spmv_panel_smem_bytes(vt, 0, chunk_cols, n_buffers))
    rb_cap = min(49152, (budget - fixed) // sv // 64 * 64)
    if rb_cap < 1024:
        return None              # the x buffers alone (nearly) fill the shared memory
    # whole waves of CTAs: the number of row blocks is a multiple of the CTAs the GPU runs at once
    slots_gpu = sms * CTAS_PER_SM
    n_blocks = max(1, -(-n_rows // rb_cap))
    n_blocks = -(-n_blocks // slots_gpu) * slots_gpu
    rb_rows = min(rb_cap, max(1024, -(-n_rows // n_blocks)))
    rb_rows = -(-rb_rows // 4) * 4
    return vt, sv, chunk_cols, rb_rows


SLAB_NNZ = 1 << 27           # the regrouping works on this many entries at a time (bounds its temporaries)


def _slabs(indptr, n_rows, rb_rows, slab_nnz=None):
    """Row ranges (r0, r1) made of whole row blocks, each holding about slab_nnz entries (at least one block)."""
    slab_nnz = slab_nnz or SLAB_NNZ
    n_rb = -(-n_rows // rb_rows)
    marks = torch.arange(0, n_rb + 1, device=indptr.device) * rb_rows
    marks[-1] = n_rows
    at = indptr[marks].to(torch.int64).tolist()        # entries in front of every row block
    out, b0 = [], 0
    for b in range(1, n_rb + 1):
        # close the slab in front of block b when b is the end, or when block b would take it over the limit
        if b == n_rb or at[b + 1] - at[b0] > slab_nnz:
            out.append((b0 * rb_rows, min(b * rb_rows, n_rows)))
            b0 = b
    return out


def scan_structure(indices, indptr, n_rows, n_cols, rb_rows, chunk_cols):
    """(number of non-empty (row block, column chunk) units, [runs longer than 4, 8, 16 entries]) without sorting
    anything; a run = consecutive entries of one row inside one column chunk (rows with sorted columns: all of the
    row's entries in that chunk).  None when the unit grid is too large to mark."""
    n_rb = -(-n_rows // rb_rows)
    n_ch = -(-n_cols // chunk_cols)
    if n_rb * n_ch > (1 << 31):
        return None
    total = 0
    long_runs = [0, 0, 0]
    dev = indices.device
    for r0, r1 in _slabs(indptr, n_rows, rb_rows):
        e0, e1 = int(indptr[r0]), int(indptr[r1])
        if e1 == e0:
            continue
        lens = (indptr[r0 + 1:r1 + 1] - indptr[r0:r1]).to(torch.int64)
        rows = torch.repeat_interleave(torch.arange(r0, r1, device=dev), lens)
        b0 = r0 // rb_rows
        chunk = indices[e0:e1].to(torch.int64) // chunk_cols
        key = (rows // rb_rows - b0) * n_ch + chunk
        mark = torch.zeros((-(-(r1 - r0) // rb_rows)) * n_ch, dtype=torch.bool, device=dev)
        mark[key] = True
        total += int(mark.sum().item())
        del key, mark
        run_key = rows * n_ch + chunk
        del rows, chunk, lens
        start = torch.ones(e1 - e0, dtype=torch.bool, device=dev)
        start[1:] = run_key[1:] != run_key[:-1]
        del run_key
        first = torch.nonzero(start, as_tuple=False).flatten()
        del start
        length = torch.diff(first, append=torch.tensor([e1 - e0], device=dev))
        for k, bound in enumerate(ROUNDS):
            long_runs[k] += int((length > bound).sum().item())
        del first, length
    return total, long_runs


def estimate_units(indices, indptr, n_rows, n_cols, rb_rows, chunk_cols):
    """Number of non-empty (row block, column chunk) units, without sorting anything."""
    scan = scan_structure(indices, indptr, n_rows, n_cols, rb_rows, chunk_cols)
    return None if scan is None else scan[0]


def choose_rounds(long_runs):
    """Smallest piece (rounds per lane) that holds every run of the matrix in one lane's rounds, so that the kernel
    can add every product straight into its accumulator; the largest piece when some run is longer than that."""
    for k, rounds in enumerate(ROUNDS):
        if long_runs[k] == 0:
            return rounds
    return ROUNDS[-1]


def _cumsum0(counts):
    out = torch.zeros(counts.numel() + 1, dtype=torch.int64, device=counts.device)
    torch.cumsum(counts, 0, out=out[1:])
    return out


def pack_pieces(data_p, acc_p, cols_p, run_key_p, unit_of_entry, ustart, u_ord, CW, rounds, max_slot_overhead,
                n_buffers=2, pad_row=0xFFFF, bank_sort=True):
    """Cut the entries of every unit (already in unit order, row-major inside a unit) into pieces of 32 * rounds
    slots and lay them out for the kernel.  acc_p: accumulator (local row) of each entry; run_key_p: entries that
    follow each other with the same key inside one unit form a run, which must not straddle two pieces; pad_row:
    the (spare) accumulator unused slots point at, with value 0 and column 0.  Returns
    (val, rc, first piece of each unit [n_units + 1], n_pieces, longest run, number of runs), or None when a run does not fit in
    a piece or the padding exceeds max_slot_overhead."""
    dev = data_p.device
    nnz = data_p.numel()
    sv = data_p.element_size()
    SLOTS = 32 * rounds
    ar = torch.arange(nnz, device=dev)
    new_run = torch.ones(nnz, dtype=torch.bool, device=dev)
    new_run[1:] = (run_key_p[1:] != run_key_p[:-1]) | (unit_of_entry[1:] != unit_of_entry[:-1])
    run_id = torch.cumsum(new_run.to(torch.int64), 0) - 1
    n_runs = int(run_id[-1].item()) + 1
    run_first = ar[new_run]                            # global index of each run's first entry
    run_end = torch.empty(n_runs, dtype=torch.int64, device=dev)
    run_end[:-1] = run_first[1:]
    run_end[-1] = nnz
    max_run = int((run_end - run_first).max().item())
    del run_end, new_run
    if max_run > SLOTS:
        return None
    # Pieces: greedy packing of whole runs into pieces of at most SLOTS entries, all units advancing one
    # piece per step (the cut after a piece that starts at s is the last run boundary at or before s + SLOTS).
    n_units = ustart.numel() - 1
    uend = ustart[1:]
    cur = ustart[:-1].clone()
    active = torch.arange(n_units, device=dev)
    cuts = [cur.clone()]
    while True:
        t = cur[active] + SLOTS
        end_a = uend[active]
        inside = t < end_a
        nxt = torch.where(inside, run_first[run_id[torch.clamp(t, max=nnz - 1)]], end_a)
        cur[active] = nxt
        keep = nxt < end_a
        if not bool(keep.any()):
            break
        active = active[keep]
        cuts.append(nxt[keep])
    piece_start = torch.sort(torch.cat(cuts)).values          # global index of each piece's first entry
    n_pieces = piece_start.numel()
    del run_id, run_first, cuts
    if max_slot_overhead is not None and n_pieces * SLOTS > max_slot_overhead * nnz + 4096:
        return None
    piece = torch.searchsorted(piece_start, ar, right=True) - 1
    if bank_sort:
        # Inside a piece, order the entries by the shared-memory bank of their accumulator (a stable sort: the rows
        # of one bank stay in row order and the entries of a row stay together, so every rule above still holds).
        # A round takes every `rounds`-th entry of that order, so the 32 accumulators of a round spread over the
        # banks instead of falling on them at random (about two instead of 3.5 passes per shared-memory access).
        order = torch.sort(piece * 32 + (acc_p % ACC_BANKS[sv]), stable=True).indices
        data_p, acc_p, cols_p, unit_of_entry = data_p[order], acc_p[order], cols_p[order], unit_of_entry[order]
        del order
    slot = ar - piece_start[piece]
    # inside a piece, slot = rounds * lane + k; both arrays are interleaved so that each 128-bit load of a warp is
    # contiguous: values at (k // E) * 32 * E + lane * E + k % E (E = values per 16 bytes), words with E = 4
    lane_, k_ = slot // rounds, slot % rounds
    E = 16 // sv
    pos_val = piece * SLOTS + (k_ // E) * (32 * E) + lane_ * E + k_ % E
    pos = piece * SLOTS + (k_ >> 2) * 128 + lane_ * 4 + (k_ & 3)
    del lane_, k_, slot, piece, ar
    upiece = torch.searchsorted(piece_start, ustart)            # first piece of each unit (and the total)
    del piece_start
    field = (u_ord[unit_of_entry] % n_buffers) * CW + (cols_p - (cols_p // CW) * CW)
    val = torch.zeros(n_pieces * SLOTS, dtype=data_p.dtype, device=dev)
    val[pos_val] = data_p
    del pos_val
    word = (acc_p << 16) | field                         # fits 32 bits: accumulator index < 65535
    word = torch.where(word >= 2**31, word - 2**32, word).to(torch.int32)
    rc = torch.full((n_pieces * SLOTS,), pad_row << 16, dtype=torch.int64, device=dev)
    rc = torch.where(rc >= 2**31, rc - 2**32, rc).to(torch.int32)
    rc[pos] = word
    return val, rc, upiece, n_pieces, max_run, n_runs


def pack_pieces_core(data_p, acc_p, cols_p, run_key_p, unit_of_entry, ustart, u_ord, CW, rounds, max_slot_overhead,
                     n_buffers=2, pad_row=0xFFFF):
    """pack_pieces for layouts in which most rows have ONE entry per unit (wide bands).  Such entries can sit in any
    slot of any piece of their unit, so the bulk of a unit is laid out with lane l holding only entries whose
    accumulator index is l modulo 32: the 32 accumulators of a round then lie in 32 different shared-memory banks
    and their load and store take one pass each.  Per unit, the single entries of every class l are listed in row
    order; with J = (shortest list) // rounds, the first J * rounds entries of every list fill J "core" pieces
    completely (piece j takes entries j * rounds .. of every list, lane l from list l) -- no padding.  What is left
    (the tails of the longer lists, and every row with several entries in the unit) is packed by pack_pieces as
    before, into pieces that follow the core pieces of their unit.  Same return value as pack_pieces."""
    dev = data_p.device
    nnz = data_p.numel()
    sv = data_p.element_size()
    SLOTS = 32 * rounds
    n_units = ustart.numel() - 1
    fallback = lambda: pack_pieces(data_p, acc_p, cols_p, run_key_p, unit_of_entry, ustart, u_ord, CW, rounds,  # noqa: E731
                                   max_slot_overhead, n_buffers=n_buffers, pad_row=pad_row)
    ar = torch.arange(nnz, device=dev)
    new_run = torch.ones(nnz, dtype=torch.bool, device=dev)
    new_run[1:] = (run_key_p[1:] != run_key_p[:-1]) | (unit_of_entry[1:] != unit_of_entry[:-1])
    run_id = torch.cumsum(new_run.to(torch.int64), 0) - 1
    n_runs = int(run_id[-1].item()) + 1
    if nnz >= RUNS_MIN_MEAN * n_runs or sv != 4:
        # rows with several entries per unit keep the run-summing layout; 8-byte accumulators span two banks each,
        # so 32 lanes cannot all have a bank of their own
        return fallback()
    run_first = ar[new_run]
    run_len = torch.diff(run_first, append=torch.tensor([nnz], device=dev))
    single = run_len[run_id] == 1
    del new_run, run_id, run_first, run_len
    idx_s = torch.nonzero(single, as_tuple=False).flatten()
    del single
    key_s = unit_of_entry[idx_s] * 32 + acc_p[idx_s] % 32
    key_sorted, order = torch.sort(key_s, stable=True)          # row order survives inside a (unit, class) list
    idx_sorted = idx_s[order]
    del key_s, order, idx_s
    cnt = torch.bincount(key_sorted, minlength=n_units * 32)
    J = cnt.view(n_units, 32).min(dim=1).values // rounds       # core pieces of each unit
    if int(J.sum().item()) * SLOTS * 4 < nnz:
        return fallback()                       # too few entries would profit
    rank = torch.arange(key_sorted.numel(), device=dev) - _cumsum0(cnt)[:-1][key_sorted]
    unit_s = key_sorted // 32
    in_core = rank < J[unit_s] * rounds
    core_idx, core_rank = idx_sorted[in_core], rank[in_core]
    core_unit, core_lane = unit_s[in_core], key_sorted[in_core] % 32
    del rank, unit_s, in_core, idx_sorted, key_sorted, cnt
    # the rest, unit by unit in the old order, through the ordinary packer (units without a rest are left out of it)
    rest = torch.ones(nnz, dtype=torch.bool, device=dev)
    rest[core_idx] = False
    rest_idx = torch.nonzero(rest, as_tuple=False).flatten()
    del rest
    L = torch.zeros(n_units, dtype=torch.int64, device=dev)     # pieces of the rest, per unit
    max_run, rest_pieces = 1, 0
    if rest_idx.numel() > 0:
        rcnt = torch.bincount(unit_of_entry[rest_idx], minlength=n_units)
        has = rcnt > 0
        compact = torch.cumsum(has.to(torch.int64), 0) - 1
        packed = pack_pieces(data_p[rest_idx], acc_p[rest_idx], cols_p[rest_idx], run_key_p[rest_idx],
                             compact[unit_of_entry[rest_idx]], _cumsum0(rcnt[has]), u_ord[has], CW, rounds, None,
                             n_buffers=n_buffers, pad_row=pad_row)
        if packed is None:
            return None
        r_val, r_rc, r_upiece, rest_pieces, max_run, _ = packed
        L[has] = r_upiece[1:] - r_upiece[:-1]
        has_units = torch.nonzero(has, as_tuple=False).flatten()
    upiece = _cumsum0(J + L)
    n_pieces = int(upiece[-1].item())
    if max_slot_overhead is not None and n_pieces * SLOTS > max_slot_overhead * nnz + 4096:
        return None
    val = torch.zeros(n_pieces * SLOTS, dtype=data_p.dtype, device=dev)
    rc = torch.full((n_pieces * SLOTS,), pad_row << 16, dtype=torch.int64, device=dev)
    rc = torch.where(rc >= 2**31, rc - 2**32, rc).to(torch.int32)
    # core entries: piece = j-th core piece of the unit, lane = class, round = position in the slice of the list
    piece = upiece[core_unit] + core_rank // rounds
    k_ = core_rank % rounds
    E = 16 // sv
    pos_val = piece * SLOTS + (k_ // E) * (32 * E) + core_lane * E + k_ % E
    pos = piece * SLOTS + (k_ >> 2) * 128 + core_lane * 4 + (k_ & 3)
    val[pos_val] = data_p[core_idx]
    c = cols_p[core_idx]
    word = (acc_p[core_idx] << 16) | ((u_ord[core_unit] % n_buffers) * CW + (c - (c // CW) * CW))
    rc[pos] = torch.where(word >= 2**31, word - 2**32, word).to(torch.int32)
    del piece, k_, pos_val, pos, word, c
    if rest_pieces > 0:
        q = torch.arange(rest_pieces, device=dev)
        cu = torch.searchsorted(r_upiece, q, right=True) - 1           # (compacted) unit of each piece of the rest
        ru = has_units[cu]
        newp = upiece[ru] + J[ru] + (q - r_upiece[cu])
        val.view(n_pieces, SLOTS)[newp] = r_val.view(rest_pieces, SLOTS)
        rc.view(n_pieces, SLOTS)[newp] = r_rc.view(rest_pieces, SLOTS)
    return val, rc, upiece, n_pieces, max_run, n_runs


def _build_slab(data, indices, indptr, r0, r1, RB, CW, n_ch, rounds, NB, max_slot_overhead):
    """The units and pieces of rows r0 .. r1-1 (whole row blocks).  Returns (val, rc, first piece of each unit + total,
    chunk of each unit, row block of each unit, number of pieces, longest run); () when the rows hold no entry;
    None when the rows cannot be laid out."""
    dev = data.device
    e0, e1 = int(indptr[r0]), int(indptr[r1])
    if e1 == e0:
        return ()
    lens = (indptr[r0 + 1:r1 + 1] - indptr[r0:r1]).to(torch.int64)
    rows = torch.repeat_interleave(torch.arange(r0, r1, device=dev), lens)
    cols = indices[e0:e1].to(torch.int64)
    b0 = r0 // RB
    key = (rows // RB) * n_ch + cols // CW
    key_sorted, perm = torch.sort(key, stable=True)   # entries keep their row-major order inside a unit
    del key, lens
    ukey, ucnt = torch.unique_consecutive(key_sorted, return_counts=True)
    del key_sorted
    n_units = ukey.numel()
    u_rb = ukey // n_ch
    u_ch = ukey % n_ch
    ustart = _cumsum0(ucnt)
    unit_of_entry = torch.repeat_interleave(torch.arange(n_units, device=dev), ucnt)
    rows_p = rows[perm]
    cols_p = cols[perm]
    del rows, cols
    # ordinal of a unit inside its row block decides which of the x buffers it uses
    n_b = -(-(r1 - r0) // RB)
    first_unit = torch.searchsorted(u_rb.contiguous(), torch.arange(b0, b0 + n_b, device=dev))
    u_ord = torch.arange(n_units, device=dev) - first_unit[u_rb - b0]
    packer = pack_pieces if os.environ.get("FSB_PANEL_NO_CORE") else pack_pieces_core
    packed = packer(data[e0:e1][perm], rows_p - (rows_p // RB) * RB, cols_p, rows_p, unit_of_entry, ustart, u_ord,
                    CW, rounds, max_slot_overhead, n_buffers=NB, pad_row=RB)
    if packed is None:
        return None
    val, rc, upiece, n_pieces, max_run, n_runs = packed
    return val, rc, upiece, u_ch, u_rb, n_pieces, max_run, n_runs


FUSED_MAX_TABLE = 1 << 26    # (row blocks x column chunks) cells the device-side builder keeps a dense table of
_ITYPE = {torch.int32: _lib.FSB_I32, torch.int64: _lib.FSB_I64}


def _fused_applicable(data, indices, indptr, n_rows, n_cols, RB, CW):
    # FSB_PANEL_BUILDER=torch keeps the host-side builder (what the tests compare the device-side one with)
    if os.environ.get("FSB_PANEL_BUILDER", "") == "torch" or data.device.type != "cuda":
        return False
    if indices.dtype not in _ITYPE or indptr.dtype not in _ITYPE or data.numel() >= 2**31 - 1:
        return False
    n_rb, n_ch = -(-n_rows // RB), -(-n_cols // CW)
    return n_ch <= int(_lib.lib().fsb_panel_build_max_chunks()) and n_rb * n_ch <= FUSED_MAX_TABLE


def _fused_pieces(L, vt, st, s_val, s_row, s_col, ustart, u_rb, u_ord, n_units, nnz, RB, CW, NB, rounds, max_pieces):
    """Cut and fill of units given as ranges of sorted entries.  Returns (val, rc, pieces per unit as int64) or None
    when there would be more than max_pieces pieces."""
    dev = s_row.device
    SLOTS = 32 * rounds
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    pcount = torch.empty(n_units, dtype=torch.int32, device=dev)
    _lib.check(L.fsb_panel_build_cut(s_row.data_ptr(), ustart.data_ptr(), n_units, SLOTS, None, pcount.data_ptr(), None,
                                     flag.data_ptr(), st), "fsb_panel_build_cut")
    upiece = _cumsum0(pcount.to(torch.int64))
    n_pieces = int(upiece[-1].item())                                 # a sync
    if n_pieces >= 2**31 - 1 or (max_pieces is not None and n_pieces > max_pieces):
        return None
    upiece = upiece.to(torch.int32)
    pstart = torch.empty(n_pieces + 1, dtype=torch.int32, device=dev)
    pstart[-1] = nnz
    _lib.check(L.fsb_panel_build_cut(s_row.data_ptr(), ustart.data_ptr(), n_units, SLOTS, upiece.data_ptr(), None,
                                     pstart.data_ptr(), flag.data_ptr(), st), "fsb_panel_build_cut")
    val = torch.empty(n_pieces * SLOTS, dtype=s_val.dtype, device=dev)
    rc = torch.empty(n_pieces * SLOTS, dtype=torch.int32, device=dev)
    _lib.check(L.fsb_panel_build_fill(vt, s_val.data_ptr(), s_row.data_ptr(), s_col.data_ptr(), pstart.data_ptr(),
                                      upiece.data_ptr(), n_units, u_rb.data_ptr(), u_ord.data_ptr(), n_pieces, RB, CW, NB,
                                      rounds, val.data_ptr(), rc.data_ptr(), st), "fsb_panel_build_fill")
    return val, rc, pcount.to(torch.int64)


def _fused_core(L, vt, st, s_val, s_row, s_col, ustart, u_rb, u_ord, n_units, nnz, RB, CW, NB, rounds, max_slots):
    """The device-side form of pack_pieces_core.  Returns (val, rc, pieces per unit), None (too much padding), or
    "plain" when the core pieces would hold less than a quarter of the entries."""
    dev = s_row.device
    SLOTS = 32 * rounds
    J = torch.empty(n_units, dtype=torch.int32, device=dev)
    n_rest = torch.empty(n_units, dtype=torch.int32, device=dev)
    _lib.check(L.fsb_panel_build_core_count(s_row.data_ptr(), ustart.data_ptr(), u_rb.data_ptr(), n_units, RB, rounds,
                                            J.data_ptr(), n_rest.data_ptr(), st), "fsb_panel_build_core_count")
    J64 = J.to(torch.int64)
    core_total = int(J64.sum().item())                                # a sync
    if core_total * SLOTS * 4 < nnz:
        return "plain"
    rest_total = nnz - core_total * SLOTS
    core_base = _cumsum0(J64).to(torch.int32)
    rest_start = _cumsum0(n_rest.to(torch.int64)).to(torch.int32)
    core_val = torch.empty(core_total * SLOTS, dtype=s_val.dtype, device=dev)
    core_rc = torch.empty(core_total * SLOTS, dtype=torch.int32, device=dev)
    r_val = torch.empty(max(rest_total, 1), dtype=s_val.dtype, device=dev)
    r_row = torch.empty(max(rest_total, 1), dtype=torch.int32, device=dev)
    r_col = torch.empty(max(rest_total, 1), dtype=torch.int32, device=dev)
    _lib.check(L.fsb_panel_build_core_place(vt, s_val.data_ptr(), s_row.data_ptr(), s_col.data_ptr(), ustart.data_ptr(),
                                            u_rb.data_ptr(), u_ord.data_ptr(), n_units, RB, CW, NB, rounds, J.data_ptr(),
                                            core_base.data_ptr(), rest_start.data_ptr(), core_val.data_ptr(),
                                            core_rc.data_ptr(), r_val.data_ptr(), r_row.data_ptr(), r_col.data_ptr(), st),
               "fsb_panel_build_core_place")
    Lp = torch.zeros(n_units, dtype=torch.int64, device=dev)          # pieces of the rest, per unit
    rest_pieces = 0
    if rest_total > 0:
        has = n_rest > 0
        has_units = torch.nonzero(has, as_tuple=False).flatten()
        r_ustart = _cumsum0(n_rest[has].to(torch.int64)).to(torch.int32)
        packed = _fused_pieces(L, vt, st, r_val, r_row, r_col, r_ustart, u_rb[has].contiguous(), u_ord[has].contiguous(),
                               has_units.numel(), rest_total, RB, CW, NB, rounds, None)
        if packed is None:
            return None
        p_val, p_rc, p_cnt = packed
        Lp[has_units] = p_cnt
        r_upiece = _cumsum0(p_cnt)
        rest_pieces = int(p_val.numel() // SLOTS)
    upiece = _cumsum0(J64 + Lp)
    n_pieces = core_total + rest_pieces
    if max_slots is not None and n_pieces * SLOTS > max_slots:
        return None
    val = torch.empty(n_pieces * SLOTS, dtype=s_val.dtype, device=dev)
    rc = torch.empty(n_pieces * SLOTS, dtype=torch.int32, device=dev)
    q = torch.arange(core_total, device=dev)
    cu = torch.searchsorted(core_base.to(torch.int64), q, right=True) - 1     # unit of every core piece
    dst = upiece[cu] + (q - core_base.to(torch.int64)[cu])
    val.view(n_pieces, SLOTS)[dst] = core_val.view(core_total, SLOTS)
    rc.view(n_pieces, SLOTS)[dst] = core_rc.view(core_total, SLOTS)
    del core_val, core_rc, q, cu, dst
    if rest_pieces > 0:
        q = torch.arange(rest_pieces, device=dev)
        cu = torch.searchsorted(r_upiece, q, right=True) - 1                  # (compacted) unit of every rest piece
        ru = has_units[cu]
        dst = upiece[ru] + J64[ru] + (q - r_upiece[cu])
        val.view(n_pieces, SLOTS)[dst] = p_val.view(rest_pieces, SLOTS)
        rc.view(n_pieces, SLOTS)[dst] = p_rc.view(rest_pieces, SLOTS)
    return val, rc, J64 + Lp


def _build_fused(data, indices, indptr, n_rows, n_cols, geometry, NB, rounds, force):
    """The layout built by the kernels of csrc/panel_build.cu (count, sort, runs, core pieces, cut, fill) with a few
    host synchronisations, bit-identical to what _build_slab + pack_pieces_core give.  Returns a PanelLayout; None when
    the matrix should not (or cannot) take the panel kernel; or the string "host" when the host-side builder has to do
    it (1024 consecutive entries spread over more chunks than the sort pass has room for)."""
    L = _lib.lib()
    vt, sv, CW, RB = geometry
    dev = data.device
    nnz = data.numel()
    n_rb, n_ch = -(-n_rows // RB), -(-n_cols // CW)
    st = torch.cuda.current_stream(dev).cuda_stream
    it, pt = _ITYPE[indices.dtype], _ITYPE[indptr.dtype]
    data, indices, indptr = data.contiguous(), indices.contiguous(), indptr.contiguous()
    with torch.cuda.device(dev):
        cnt = torch.empty(n_rb * n_ch, dtype=torch.int32, device=dev)
        _lib.check(L.fsb_panel_build_count(it, pt, indices.data_ptr(), indptr.data_ptr(), n_rows, n_cols, RB, CW,
                                           cnt.data_ptr(), st), "fsb_panel_build_count")
        cell = torch.nonzero(cnt, as_tuple=False).flatten()          # units in (row block, chunk) order; a sync
        n_units = cell.numel()
        limit = MAX_X_OVERHEAD if sv == 4 else MAX_X_OVERHEAD_F64
        if not force and n_units * CW * sv > limit * nnz * (sv + 4):
            return None
        ustart = _cumsum0(cnt[cell].to(torch.int64)).to(torch.int32)
        unit_base = torch.zeros(n_rb * n_ch, dtype=torch.int32, device=dev)
        unit_base[cell] = ustart[:-1]
        del cnt
        rb_of_unit = cell // n_ch
        u_rb = rb_of_unit.to(torch.int32)
        u_ch = (cell % n_ch).to(torch.int32)
        rb_unit_ptr64 = _cumsum0(torch.bincount(rb_of_unit, minlength=n_rb))
        rb_unit_ptr = rb_unit_ptr64.to(torch.int32)
        u_ord = (torch.arange(n_units, device=dev) - rb_unit_ptr64[rb_of_unit]).to(torch.int32)
        del cell, rb_of_unit, rb_unit_ptr64
        s_val = torch.empty(nnz, dtype=data.dtype, device=dev)
        s_row = torch.empty(nnz, dtype=torch.int32, device=dev)
        s_col = torch.empty(nnz, dtype=torch.int32, device=dev)
        stats = torch.empty(5, dtype=torch.int64, device=dev)
        # the narrow window where a row block has few units (a tile's chunks are among them), else the wide one
        wide = n_units > (int(L.fsb_panel_build_window(0)) * 3 // 4) * n_rb
        while True:
            flag = torch.zeros(1, dtype=torch.int32, device=dev)
            _lib.check(L.fsb_panel_build_sort(vt, it, pt, data.data_ptr(), indices.data_ptr(), indptr.data_ptr(), n_rows,
                                              n_cols, RB, CW, int(wide), unit_base.data_ptr(), s_val.data_ptr(),
                                              s_row.data_ptr(), s_col.data_ptr(), flag.data_ptr(), st),
                       "fsb_panel_build_sort")
            _lib.check(L.fsb_panel_build_runs(s_row.data_ptr(), s_col.data_ptr(), nnz, CW, stats.data_ptr(), st),
                       "fsb_panel_build_runs")
            if not int(flag.item()):                                   # a sync
                break
            if wide:
                return "host"
            wide = True
        del unit_base
        n_runs, max_run, *long_runs = (int(v) for v in stats.tolist())
        rounds = rounds or choose_rounds(long_runs)
        core = sv == 4 and nnz < RUNS_MIN_MEAN * n_runs and not os.environ.get("FSB_PANEL_NO_CORE")
        while True:
            SLOTS = 32 * rounds
            packed = None
            if max_run <= SLOTS:
                max_slots = None if force else int(MAX_SLOT_OVERHEAD * nnz + 4096)
                if core:
                    packed = _fused_core(L, vt, st, s_val, s_row, s_col, ustart, u_rb, u_ord, n_units, nnz, RB, CW, NB,
                                         rounds, max_slots)
                    if isinstance(packed, str):
                        core, packed = False, None
                        continue
                else:
                    packed = _fused_pieces(L, vt, st, s_val, s_row, s_col, ustart, u_rb, u_ord, n_units, nnz, RB, CW, NB,
                                           rounds, None if max_slots is None else max_slots // SLOTS)
            if packed is not None:
                break
            if rounds == ROUNDS[-1]:
                return None
            rounds = ROUNDS[-1]      # a run that does not fit a small piece, or too much padding
        val, rc, per_unit = packed
        upiece = _cumsum0(per_unit).to(torch.int32)
        n_pieces = val.numel() // SLOTS
    lay = PanelLayout()
    lay.val, lay.rc = val, rc
    lay.unit_piece_ptr, lay.unit_chunk, lay.rb_unit_ptr = upiece, u_ch, rb_unit_ptr
    lay.n_row_blocks, lay.rb_rows, lay.chunk_cols, lay.n_buffers = n_rb, RB, CW, NB
    lay.rounds, lay.max_run, lay.pad_row = rounds, max_run, RB
    lay.flags = (FLAG_LONG_RUNS if max_run > rounds else 0) | (FLAG_RUNS if nnz >= RUNS_MIN_MEAN * n_runs else 0)
    lay.n_units, lay.n_pieces = n_units, n_pieces
    lay.x_overhead = n_units * CW * sv / float(nnz * (sv + 4))
    lay.slot_overhead = n_pieces * SLOTS / float(nnz)
    lay.status = StatusWord(dev)
    return lay


def build_panel_layout(data, indices, indptr, n_rows, n_cols, max_row_nnz, force=False, rounds=None):
    """PanelLayout for the matrix, or None when the panel kernel would not pay (or cannot be used)."""
    nnz = data.numel()
    if nnz == 0 or n_rows == 0 or n_cols == 0:
        return None
    if not force and (nnz < MIN_NNZ or max_row_nnz > MAX_ROW_NNZ):
        return None
    dev = data.device
    NB = default_buffers()
    geometry = _geometry(data.dtype, n_rows, dev, NB)
    if geometry is None:
        return None
    vt, sv, CW, RB = geometry
    n_rb = -(-n_rows // RB)
    n_ch = -(-n_cols // CW)
    rounds = rounds or default_rounds()
    if _fused_applicable(data, indices, indptr, n_rows, n_cols, RB, CW):
        lay = _build_fused(data, indices, indptr, n_rows, n_cols, geometry, NB, rounds, force)
        if not isinstance(lay, str):
            return lay
    if not force or rounds is None:
        scan = scan_structure(indices, indptr, n_rows, n_cols, RB, CW)
        if scan is None:
            if not force:
                return None
            rounds = rounds or ROUNDS[-1]
        else:
            n_units, long_runs = scan
            limit = MAX_X_OVERHEAD if sv == 4 else MAX_X_OVERHEAD_F64
            if not force and n_units * CW * sv > limit * nnz * (sv + 4):
                return None
            rounds = rounds or choose_rounds(long_runs)
    SLOTS = 32 * rounds
    vals, rcs, upieces, chunks, blocks = [], [], [], [], []
    piece_base = 0
    max_run = n_runs = 0
    for r0, r1 in _slabs(indptr, n_rows, RB):
        part = _build_slab(data, indices, indptr, r0, r1, RB, CW, n_ch, rounds, NB,
                           None if force else MAX_SLOT_OVERHEAD)
        if part is None:
            if rounds < ROUNDS[-1]:
                # a run that does not fit in a small piece (or too much padding): the largest piece may still do
                del vals, rcs
                return build_panel_layout(data, indices, indptr, n_rows, n_cols, max_row_nnz, force, ROUNDS[-1])
            return None
        if part == ():
            continue                 # no entries in these rows
        val_s, rc_s, upiece_s, u_ch_s, u_rb_s, n_pieces_s, max_run_s, n_runs_s = part
        n_runs += n_runs_s
        vals.append(val_s)
        rcs.append(rc_s)
        upieces.append(upiece_s[:-1] + piece_base)
        chunks.append(u_ch_s)
        blocks.append(u_rb_s)
        piece_base += n_pieces_s
        max_run = max(max_run, max_run_s)
    n_pieces = piece_base
    if n_pieces >= 2**31 - 1:
        return None
    val, rc = (t[0] if len(t) == 1 else torch.cat(t) for t in (vals, rcs))
    del vals, rcs
    upiece = torch.cat(upieces + [torch.tensor([n_pieces], dtype=torch.int64, device=dev)])
    u_ch = torch.cat(chunks)
    u_rb = torch.cat(blocks)
    n_units = u_ch.numel()
    rb_unit_ptr = torch.searchsorted(u_rb.contiguous(), torch.arange(n_rb + 1, device=dev))
    if not force and n_pieces * SLOTS > MAX_SLOT_OVERHEAD * nnz + 4096 * len(upieces):
        return None

    lay = PanelLayout()
    lay.val, lay.rc = val, rc
    lay.unit_piece_ptr = upiece.to(torch.int32)
    lay.unit_chunk = u_ch.to(torch.int32)
    lay.rb_unit_ptr = rb_unit_ptr.to(torch.int32)
    lay.n_row_blocks, lay.rb_rows, lay.chunk_cols, lay.n_buffers = n_rb, RB, CW, NB
    lay.rounds, lay.max_run, lay.pad_row = rounds, max_run, RB
    lay.flags = (FLAG_LONG_RUNS if max_run > rounds else 0) | (FLAG_RUNS if nnz >= RUNS_MIN_MEAN * n_runs else 0)
    lay.n_units, lay.n_pieces = n_units, n_pieces
    lay.x_overhead = n_units * CW * sv / float(nnz * (sv + 4))
    lay.slot_overhead = n_pieces * SLOTS / float(nnz)
    lay.status = StatusWord(dev)
    return lay


def launch_panel(layout, x, y, n_rows, n_cols, stream_ptr, block_begin=0, block_end=None, flags=0, record_on=None):
    """Enqueue the product (or the row blocks [block_begin, block_end) of it) on the stream behind stream_ptr;
    record_on: the torch stream object of that stream when it is not the current one."""
    L = _lib.lib()
    layout.status.poll()
    rc = L.fsb_spmv_csr_panel(
        _VTYPE[layout.val.dtype], layout.val.data_ptr(), layout.rc.data_ptr(), layout.unit_piece_ptr.data_ptr(),
        layout.unit_chunk.data_ptr(), layout.rb_unit_ptr.data_ptr(), layout.n_row_blocks, layout.rb_rows,
        layout.chunk_cols, layout.n_buffers, layout.rounds, layout.flags | flags, block_begin,
        layout.n_row_blocks if block_end is None else block_end, x.data_ptr(), y.data_ptr(), n_rows, n_cols,
        layout.status.data_ptr(), stream_ptr,
    )
    _lib.check(rc, "fsb_spmv_csr_panel")
    layout.status.posted("fsb_spmv_csr_panel", record_on)
