"""Prepare-time split of a skewed CSR matrix into its long rows (panel kernel, x in shared memory) and the rest.

The reference sends long rows to buckets of their own, one Triton program per row
(src/flagsparse/sparse_operations/spmv_csr.py:64-89 bucket tables, :281-327 bucket builder, :329-376 launches).
Here the longest rows are taken out of the matrix: together they hold a large share of the entries of a power-law
matrix, and a group of some ten thousand of them has tens of thousands of entries in every chunk of 8192 columns,
enough to pay for loading that chunk of x into shared memory once per group instead of gathering it entry by
entry through L2.  What remains (short rows only) goes through the CSR kernels.

Layout of the long part (csrc/spmv_panel.cu, spmv_panel_groups_kernel):
  * the long rows, longest first, are numbered q = 0 .. n_long-1;
  * a row with more entries in some chunk than a lane of the kernel has rounds (16) gets several accumulators
    ("virtual rows"), that many entries of a chunk to each, so that no two lanes finish on one accumulator;
  * consecutive rows form groups whose accumulators fit in shared memory; units = (group, chunk), ordered by
    group then chunk, are dealt to about one CTA per SM in proportion to their cost (entries streamed plus the
    chunk of x), never mixing groups in a CTA;
  * each CTA writes one partial sum per row of its group; a small second kernel adds them in CTA order.
"""

import os

import torch

from . import _lib
from ._common import _VTYPE
from . import panel as _panel

MIN_CANDIDATE_LEN = 64      # rows shorter than this are never taken out
# A unit costs the kernel about 2 us whatever it holds (the bulk copy of its x chunk is only one unit ahead) plus
# 0.2 ns per entry; the CSR kernels need about 0.9 ns per entry and SM.  Groups whose units hold fewer entries
# than this are left to the CSR kernels.
MIN_UNIT_ENTRIES = 4096
UNIT_FIXED_BYTES = 48 * 1024  # added to the x chunk: cost of a unit in streamed-byte equivalents (CTA balancing)
MIN_LONG_SHARE = 0.15       # of all entries: below this the split does not pay
MIN_LONG_NNZ = 1 << 22
MAX_CANDIDATE_NNZ = 1 << 29  # the regrouping sorts all candidate entries at once: beyond this it is not attempted
ACC_CAP = None              # accumulators per group; None = what fits in shared memory (tests lower it)


class LongRowLayout:
    __slots__ = ("val", "rc", "unit_piece_ptr", "unit_chunk", "cta_unit_ptr", "cta_group", "group_q_ptr",
                 "group_cta_ptr", "vbase", "q_group", "long_rows", "cta_part_ptr", "part", "n_ctas", "n_groups",
                 "n_long", "chunk_cols", "n_buffers", "rounds", "flags", "max_group_acc", "pad_row", "n_units", "n_pieces", "nnz",
                 "x_overhead", "slot_overhead", "status")

    def nbytes(self):
        names = ("val", "rc", "unit_piece_ptr", "unit_chunk", "cta_unit_ptr", "cta_group", "group_q_ptr",
                 "group_cta_ptr", "vbase", "q_group", "long_rows", "cta_part_ptr", "part")
        return sum(getattr(self, n).numel() * getattr(self, n).element_size() for n in names)


def _accumulator_cap(dtype, chunk_cols, n_buffers):
    L = _lib.lib()
    sv = 4 if dtype == torch.float32 else 8
    fixed = int(L.fsb_spmv_panel_smem_bytes(_VTYPE[dtype], 0, chunk_cols, n_buffers))
    return min(49152, (_panel.smem_budget() - fixed) // sv // 64 * 64)


def long_row_threshold():
    """FSB_SPMV_LONG_ROW=n takes out every row with at least n entries; unset, the choice is automatic: the longest
    rows, as many groups of them as have MIN_UNIT_ENTRIES entries per unit."""
    return int(os.environ.get("FSB_SPMV_LONG_ROW", "0")) or None


def split_rows(indptr, n_rows, threshold):
    """(row lengths, mask of the rows with at least `threshold` entries, entries in those rows)."""
    lens = (indptr[1:] - indptr[:-1]).to(torch.int64)
    is_long = lens >= threshold
    return lens, is_long, int((lens * is_long).sum().item())


def short_part(data, indices, indptr, lens, is_long):
    """CSR arrays of the matrix with its long rows emptied (same shape, same row numbering)."""
    n_rows = lens.numel()
    keep = ~torch.repeat_interleave(is_long, lens)
    ptr = torch.zeros(n_rows + 1, dtype=indptr.dtype, device=indptr.device)
    ptr[1:] = torch.cumsum(lens * (~is_long), 0).to(indptr.dtype)
    return data[keep].contiguous(), indices[keep].contiguous(), ptr


def build_long_row_layout(data, indices, indptr, lens, is_long, n_cols, n_ctas_target=None, chunk_cols=None,
                          acc_cap=None, min_unit_entries=0):
    """(LongRowLayout, mask of the rows it holds) for the candidate rows marked in is_long, or None when it cannot
    be built.  With min_unit_entries > 0 only the leading groups (longest rows) whose units hold at least that
    many entries on average are kept; the returned mask then marks fewer rows than is_long."""
    dev = data.device
    sv = data.element_size()
    CW = chunk_cols or int(os.environ.get("FSB_PANEL_CHUNK", "0")) or (8192 if sv == 4 else 4096)
    # a (row, chunk) run is cut into virtual rows of at most `rounds` entries, so no piece needs the kernel's
    # segmented path
    rounds = _panel.default_rounds() or _panel.ROUNDS[-1]
    SLOTS = int(_lib.lib().fsb_spmv_panel_piece_slots(rounds))
    NB = _panel.default_buffers()
    cap = acc_cap or ACC_CAP or _accumulator_cap(data.dtype, CW, NB)
    if n_ctas_target is None:
        try:
            n_ctas_target = torch.cuda.get_device_properties(dev).multi_processor_count
        except Exception:
            n_ctas_target = _panel.SM_COUNT_FALLBACK
    n_ch = -(-n_cols // CW)
    # long rows, longest first (ties in row order)
    cand = torch.nonzero(is_long, as_tuple=False).flatten()
    n_long = cand.numel()
    if n_long == 0 or n_long >= 2**31 - 1:
        return None
    order = torch.sort(lens[cand], descending=True, stable=True).indices
    long_rows = cand[order]
    lens_l = lens[long_rows]
    nnz = int(lens_l.sum().item())
    if nnz == 0 or nnz >= 2**31 - 64:
        return None
    # entries of the long rows, row q after row q-1, in their CSR order
    qstart = _panel._cumsum0(lens_l)
    q_of = torch.repeat_interleave(torch.arange(n_long, device=dev), lens_l)
    src = torch.arange(nnz, device=dev) - qstart[q_of] + indptr[long_rows].to(torch.int64)[q_of]
    cols = indices[src].to(torch.int64)
    chunk = cols // CW
    # (1) per (row, chunk): position of each entry in its run -> virtual rows needed per row
    k1, perm1 = torch.sort(q_of * n_ch + chunk, stable=True)
    first = torch.ones(nnz, dtype=torch.bool, device=dev)
    first[1:] = k1[1:] != k1[:-1]
    ar = torch.arange(nnz, device=dev)
    run_first = ar[first]
    j = ar - run_first[torch.cumsum(first.to(torch.int64), 0) - 1]      # position inside the (row, chunk) run
    sub_sorted = j // rounds
    del first, run_first, j, k1
    q_sorted = q_of[perm1]
    nv = torch.zeros(n_long, dtype=torch.int64, device=dev)
    nv.scatter_reduce_(0, q_sorted, sub_sorted + 1, reduce="amax", include_self=True)
    max_nv = int(nv.max().item())
    if max_nv >= cap // 2:
        return None
    vbase = _panel._cumsum0(nv)
    # (2) groups of consecutive rows whose accumulators fit: a row never straddles two groups because a group
    #     is closed max_nv accumulators early
    q_group = vbase[:-1] // (cap - max_nv)
    n_groups = int(q_group[-1].item()) + 1
    group_q_ptr = torch.searchsorted(q_group.contiguous(), torch.arange(n_groups + 1, device=dev))
    group_vb = vbase[group_q_ptr]                                        # first accumulator of each group
    max_group_acc = int((group_vb[1:] - group_vb[:-1]).max().item())
    if min_unit_entries > 0:
        group_nnz = torch.zeros(n_groups, dtype=torch.int64, device=dev).index_add_(0, q_group, lens_l)
        dense = (group_nnz >= min_unit_entries * n_ch).to(torch.int64)
        n_keep = int(torch.cumprod(dense, 0).sum().item())               # leading groups that are dense enough
        if n_keep == 0:
            return None
        if n_keep < n_groups:
            n_long = int(group_q_ptr[n_keep].item())
            keep = q_sorted < n_long
            q_sorted, sub_sorted, perm1 = q_sorted[keep], sub_sorted[keep], perm1[keep]
            del keep
            long_rows, lens_l, nv = long_rows[:n_long], lens_l[:n_long], nv[:n_long]
            vbase, q_group = vbase[:n_long + 1], q_group[:n_long]
            n_groups, group_q_ptr, group_vb = n_keep, group_q_ptr[:n_keep + 1], group_vb[:n_keep + 1]
            nnz = int(lens_l.sum().item())
            max_group_acc = int((group_vb[1:] - group_vb[:-1]).max().item())
    # (3) units = (group, chunk); a stable sort of the (row, chunk)-ordered entries keeps rows together in a unit
    g_sorted = q_group[q_sorted]
    chunk_sorted = chunk[perm1]
    src, cols = src[perm1], cols[perm1]                                  # entries in (row, chunk) order from here on
    k2, perm2 = torch.sort(g_sorted * n_ch + chunk_sorted, stable=True)
    del g_sorted, chunk_sorted, chunk
    del perm1
    perm = perm2
    q_p = q_sorted[perm2]
    sub_p = sub_sorted[perm2]
    del q_sorted, sub_sorted, perm2
    ukey, ucnt = torch.unique_consecutive(k2, return_counts=True)
    del k2
    n_units = ukey.numel()
    u_g = ukey // n_ch
    u_ch = ukey % n_ch
    ustart = _panel._cumsum0(ucnt)
    unit_of_entry = torch.repeat_interleave(torch.arange(n_units, device=dev), ucnt)
    # (4) CTAs: every group gets a share of the CTAs in proportion to its cost, its units are cut by column range
    cost = (ucnt * (sv + 4) + CW * sv + UNIT_FIXED_BYTES).to(torch.float64)
    gcost = torch.zeros(n_groups, dtype=torch.float64, device=dev).index_add_(0, u_g, cost)
    n_g = torch.clamp(torch.round(gcost * (n_ctas_target / float(gcost.sum().item()))), min=1).to(torch.int64)
    group_cta_ptr = _panel._cumsum0(n_g)
    n_ctas = int(group_cta_ptr[-1].item())
    before = torch.cumsum(cost, 0) - cost                                # cost of the units in front, all groups
    gbefore = torch.cumsum(gcost, 0) - gcost
    within = torch.clamp(before - gbefore[u_g], min=0.0)
    local = torch.minimum((within * n_g[u_g].to(torch.float64) / gcost[u_g]).floor().to(torch.int64), n_g[u_g] - 1)
    cta_of_unit = group_cta_ptr[u_g] + local
    cta_unit_ptr = torch.searchsorted(cta_of_unit.contiguous(), torch.arange(n_ctas + 1, device=dev))
    u_ord = torch.arange(n_units, device=dev) - cta_unit_ptr[cta_of_unit]
    cta_group = torch.repeat_interleave(torch.arange(n_groups, device=dev), n_g)
    rows_in_group = group_q_ptr[1:] - group_q_ptr[:-1]
    cta_part_ptr = _panel._cumsum0(rows_in_group[cta_group])
    # (5) pieces
    vrow_p = vbase[q_p] + sub_p                                          # global accumulator number = run key
    acc_p = vrow_p - group_vb[q_group[q_p]]
    del q_p, sub_p
    packed = _panel.pack_pieces(data[src[perm]], acc_p, cols[perm], vrow_p, unit_of_entry, ustart, u_ord, CW, rounds,
                                None, n_buffers=NB, pad_row=max_group_acc)
    del acc_p, vrow_p, unit_of_entry, src, cols, perm
    if packed is None:
        return None
    val, rc, upiece, n_pieces, max_run, n_runs = packed

    lay = LongRowLayout()
    lay.val, lay.rc = val, rc
    i32 = torch.int32
    lay.unit_piece_ptr, lay.unit_chunk = upiece.to(i32), u_ch.to(i32)
    lay.cta_unit_ptr, lay.cta_group = cta_unit_ptr.to(i32), cta_group.to(i32)
    lay.group_q_ptr, lay.group_cta_ptr = group_q_ptr.to(i32), group_cta_ptr.to(i32)
    lay.vbase, lay.q_group, lay.long_rows = vbase.to(i32), q_group.to(i32), long_rows.to(i32)
    lay.cta_part_ptr = cta_part_ptr[:-1].contiguous()
    lay.part = torch.zeros(max(1, int(cta_part_ptr[-1].item())), dtype=data.dtype, device=dev)
    lay.n_ctas, lay.n_groups, lay.n_long = n_ctas, n_groups, n_long
    lay.chunk_cols, lay.n_buffers, lay.max_group_acc = CW, NB, max_group_acc
    lay.pad_row = max_group_acc
    lay.rounds = rounds
    lay.flags = (_panel.FLAG_LONG_RUNS if max_run > rounds else 0) | (
        _panel.FLAG_RUNS if nnz >= _panel.RUNS_MIN_MEAN * n_runs else 0)
    lay.n_units, lay.n_pieces, lay.nnz = n_units, n_pieces, nnz
    lay.x_overhead = n_units * CW * sv / float(nnz * (sv + 4))
    lay.slot_overhead = n_pieces * SLOTS / float(nnz)
    lay.status = _panel.StatusWord(dev)
    mask = torch.zeros_like(is_long)
    mask[long_rows] = True
    return lay, mask


def launch_long_rows(layout, x, y, n_cols, stream_ptr, flags=0):
    """y[long rows] = (A x)[long rows]; the other elements of y are left alone."""
    la = layout
    la.status.poll()
    rc = _lib.lib().fsb_spmv_csr_panel_groups(
        _VTYPE[la.val.dtype], la.val.data_ptr(), la.rc.data_ptr(), la.unit_piece_ptr.data_ptr(),
        la.unit_chunk.data_ptr(), la.cta_unit_ptr.data_ptr(), la.n_ctas, la.chunk_cols, la.n_buffers, la.rounds,
        la.flags | flags, la.max_group_acc,
        la.cta_group.data_ptr(), la.group_q_ptr.data_ptr(), la.group_cta_ptr.data_ptr(), la.vbase.data_ptr(),
        la.q_group.data_ptr(), la.long_rows.data_ptr(), la.n_long, la.cta_part_ptr.data_ptr(), la.part.data_ptr(),
        x.data_ptr(), y.data_ptr(), n_cols, la.status.data_ptr(), stream_ptr,
    )
    _lib.check(rc, "fsb_spmv_csr_panel_groups")
    la.status.posted("fsb_spmv_csr_panel_groups")
