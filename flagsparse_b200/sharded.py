"""Row-sharded CSR SpMV and SpMM over the GPUs of one box: one process per GPU, x (or B) replicated, the
result assembled on every rank.

The reference is single-GPU (no torch.distributed, NCCL or multi-device code anywhere in its tree); these
drivers are what "run src/flagsparse/sparse_operations/spmv_csr.py:557-610 (or spmm_csr.py:1129-1183) on a row
shard per GPU and gather the result" becomes on an NVSwitch box.  Rows are independent, so the only exchange is
the all-gather of the result rows:

  * mode "nccl": every rank computes its rows straight into its slice of a full-size result, then one
    all-gather moves the slices -- NCCL over NVLink, or broadcasts on a CPU (gloo) group.
  * mode "peer": the result lives in symmetric memory.  A rank computes its shard in a few slices, one launch
    each; as soon as a slice is finished the copy engines push it into every peer's result (plain peer copies
    over NVLink, destinations taken in a per-rank rotated order so that no GPU is written by everybody at
    once) while the SMs are already on the next slice.  One symmetric-memory barrier ends the step; the result
    is double-buffered, so a rank may start the next product while its peers still read this one.
  * mode "fused" (SpMV with the vector or stream kernel only): the kernel's epilogue stores each finished
    value into every rank's y through peer-mapped pointers (fsb_spmv_csr_scatter).

Shard boundaries are contiguous row ranges holding about nnz / P entries each.
"""

import os

import torch
import torch.distributed as dist

from . import _lib
from ._common import _ITYPE, _VTYPE, _ptr, _stream_ptr

MAX_SLICES = 4      # launches per product in mode "peer" (FSB_SHARD_SLICES overrides)


def partition_rows_by_nnz(indptr, n_parts):
    """Row boundaries b[0..n_parts] (python ints, b[0] = 0, b[-1] = n_rows) such that shard p = rows
    [b[p], b[p+1]) holds about nnz / n_parts entries: b[p] is the first row whose indptr value is at
    least p * nnz / n_parts (integer division).  `indptr` is a torch tensor or a numpy array."""
    if n_parts < 1:
        raise ValueError("n_parts must be positive")
    n_rows = int(indptr.shape[0]) - 1
    if n_rows < 0:
        raise ValueError("indptr must have at least one entry")
    nnz = int(indptr[-1])
    targets = [(p * nnz) // n_parts for p in range(1, n_parts)]
    if torch.is_tensor(indptr):
        t = torch.tensor(targets, dtype=indptr.dtype, device=indptr.device)
        inner = torch.searchsorted(indptr.contiguous(), t, right=False).tolist() if targets else []
    else:
        import numpy as np

        inner = np.searchsorted(indptr, np.asarray(targets, dtype=indptr.dtype), side="left").tolist() if targets else []
    bounds = [0] + [min(int(b), n_rows) for b in inner] + [n_rows]
    for i in range(1, len(bounds)):  # monotone even for degenerate inputs
        bounds[i] = max(bounds[i], bounds[i - 1])
    return bounds


def slice_plan(n_units, units_per_wave, max_slices):
    """Cut n_units work units (row blocks of the panel kernel) into at most max_slices contiguous slices made of
    whole waves of units_per_wave, the later slices never larger than the earlier ones (the last slice's
    transfer is the one nothing overlaps).  Returns [(begin, end), ...] covering [0, n_units)."""
    if n_units <= 0:
        return []
    waves = -(-n_units // max(1, units_per_wave))
    k = max(1, min(max_slices, waves))
    per, extra = divmod(waves, k)
    out, w = [], 0
    for j in range(k):
        take = per + (1 if j < extra else 0)
        b, e = w * units_per_wave, min(n_units, (w + take) * units_per_wave)
        out.append((b, e))
        w += take
    return [s for s in out if s[1] > s[0]]


class _ShardedBase:
    """Bookkeeping shared by the sharded products: row ranges of every rank, the symmetric result buffers of
    mode "peer" and the copy-engine pushes."""

    def _init_ranges(self, n_local, row_start, shape, group):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.n_rows, self.n_cols = int(shape[0]), int(shape[1])
        self.n_local = int(n_local)
        self.row_start = int(row_start)
        mine = (self.row_start, self.n_local)
        if self.world > 1:
            ranges = [None] * self.world
            dist.all_gather_object(ranges, mine, group=group)
        else:
            ranges = [mine]
        self.row_ranges = [(int(s), int(n)) for s, n in ranges]
        pos = 0
        for s, n in self.row_ranges:
            if s != pos or n < 0:
                raise ValueError(f"row shards must be contiguous and ordered by rank, got {self.row_ranges}")
            pos += n
        if pos != self.n_rows:
            raise ValueError(f"row shards cover {pos} rows, the matrix has {self.n_rows}")

    # -- symmetric result buffers ------------------------------------------------------------------
    def _setup_symmetric(self, width):
        """Two full-size results (n_rows x width elements each) in symmetric memory, plus a view of every
        peer's copy."""
        import torch.distributed._symmetric_memory as symm_mem

        group = self.group if self.group is not None else dist.group.WORLD
        rows = (max(self.n_rows, 1) + 63) // 64 * 64
        self._stride = rows * width                       # elements per result buffer
        self._width = width
        self._buf = symm_mem.empty(2 * self._stride, dtype=self.dtype, device=self.device)
        self._symm = symm_mem.rendezvous(self._buf, group)
        self._peer_bufs = [self._buf if p == self.rank else self._symm.get_buffer(p, (2 * self._stride,), self.dtype)
                           for p in range(self.world)]
        self._peer_ptrs = torch.tensor([int(p) for p in self._symm.buffer_ptrs], dtype=torch.int64,
                                       device=self.device)
        self._parity = 0
        self._side = torch.cuda.Stream(self.device)       # carries the pushes
        self._aux = torch.cuda.Stream(self.device)        # carries every other slice's launch

    def _push(self, base, row_lo, row_hi, after):
        """Copy rows [row_lo, row_hi) of the result at element offset `base` into every peer, on the side stream,
        once `after` (an event) has passed.  Peer p is served k-th by rank (p - k) mod world."""
        if row_hi <= row_lo or self.world == 1:
            return
        lo, hi = base + row_lo * self._width, base + row_hi * self._width
        self._side.wait_event(after)
        src = self._buf[lo:hi]
        with torch.cuda.stream(self._side):
            for k in range(1, self.world):
                p = (self.rank + k) % self.world
                self._peer_bufs[p][lo:hi].copy_(src, non_blocking=True)

    def _finish_step(self):
        """Main stream: wait for the pushes, then the barrier after which every rank's rows are everywhere (it
        also orders this product after every peer's reads of the buffer written two products ago)."""
        main = torch.cuda.current_stream(self.device)
        done = torch.cuda.Event()
        done.record(self._side)
        main.wait_event(done)
        self._symm.barrier(channel=0)

    # -- the plain all-gather ------------------------------------------------------------------------
    def _all_gather_rows(self, full):
        """`full` holds this rank's rows in place; fetch everybody else's (rows along dimension 0)."""
        if self.world == 1:
            return
        views = [full[a:a + b] for a, b in self.row_ranges]
        backend = dist.get_backend(self.group)
        sizes = {b for _, b in self.row_ranges}
        if backend == "nccl" and len(sizes) == 1:
            dist.all_gather_into_tensor(full, views[self.rank], group=self.group)   # in place: one ring all-gather
        elif backend == "nccl":
            dist.all_gather(views, views[self.rank], group=self.group)              # uneven sizes: grouped broadcasts
        else:
            for r, v in enumerate(views):
                if v.numel() > 0:
                    dist.broadcast(v, src=dist.get_global_rank(self.group, r) if self.group is not None else r,
                                   group=self.group)


def _max_slices():
    return int(os.environ.get("FSB_SHARD_SLICES", "0")) or MAX_SLICES


class ShardedCsrSpmv(_ShardedBase):
    """y = A x with A split by rows over the ranks of a process group.

    Each rank constructs it with ITS rows only: `data`, `indices`, and `indptr` rebased so that
    indptr[0] == 0; `row_start` is the global index of its first row.  `matvec(x)` takes the full x
    (replicated on every rank) and returns the full y on every rank.

    local_spmv: optional callable (x, out) -> None that fills `out` (length = local rows) with the local
    product.  It exists so that the host logic (partition bookkeeping, assembly, collectives) can be
    exercised on CPU process groups; by default the CUDA kernels of this package do the work.
    """

    def __init__(self, data, indices, indptr, row_start, shape, group=None, mode="auto", local_spmv=None):
        self._init_ranges(int(indptr.numel()) - 1, row_start, shape, group)
        self.device = data.device
        self.dtype = data.dtype
        self._local_spmv = local_spmv
        native = local_spmv is None and data.is_cuda and data.dtype in (torch.float32, torch.float64)
        if mode == "auto":
            # pushing slices needs the CUDA kernels, several ranks and something to multiply
            mode = "peer" if (native and self.world > 1) else "nccl"
        if mode not in ("nccl", "peer", "fused"):
            raise ValueError("mode must be 'auto', 'nccl', 'peer' or 'fused'")
        if mode != "nccl" and local_spmv is not None:
            raise ValueError(f"mode '{mode}' runs the CUDA kernels of this package; it cannot take local_spmv")
        if mode != "nccl" and data.dtype not in (torch.float32, torch.float64):
            raise TypeError(f"mode '{mode}' needs float32 or float64 values")
        self.prepared = None
        if local_spmv is None:
            from .spmv_csr import _prepare_spmv_csr

            # the kernels with a peer-store epilogue are the vector and the stream kernel: no panel, no split
            self.prepared = _prepare_spmv_csr(data, indices, indptr, (self.n_local, self.n_cols), 256, None,
                                              reuse_expected=mode != "fused", allow_split=mode != "fused")
        self.mode = mode
        self._y = None
        self._slices = None
        self._nccl_chunks = None
        if mode in ("peer", "fused"):
            self._setup_symmetric(1)
        if mode == "peer":
            self._plan_slices()
        # Gathering slice j while slice j + 1 is computed is there to be measured (FSB_NCCL_CHUNKS=1), not the default:
        # NCCL's kernels need SMs and the panel kernel holds all of them until a wave of row blocks ends, so the
        # chunked form came out slower than one all-gather after the shard (2 GPUs 2.93 against 2.82 ms, 4 GPUs 2.45
        # against 1.91 ms on the 2.1 G-entry benchmark matrix)
        if mode == "nccl" and local_spmv is None and dist.is_initialized() and dist.get_backend(group) == "nccl" \
                and os.environ.get("FSB_NCCL_CHUNKS", "") not in ("", "0"):
            self._plan_nccl_chunks()

    def _plan_slices(self):
        """Row slices of this shard, one launch each.  Only the panel kernel can be launched on a sub-range of its
        row blocks; the other kernels run the shard in one piece."""
        p = self.prepared
        self._slices = [(0, 0, 0, self.n_local)]          # (block_begin, block_end, row_lo, row_hi)
        if p.algo == _lib.FSB_SPMV_PANEL and p.panel is not None and self.n_local > 0:
            la = p.panel
            # one wave = as many row blocks as the GPU runs at once (FSB_SHARD_WAVE_BLOCKS: smaller waves, for tests)
            sms = int(os.environ.get("FSB_SHARD_WAVE_BLOCKS", "0")) or \
                torch.cuda.get_device_properties(self.device).multi_processor_count
            self._slices = [(b, e, b * la.rb_rows, min(self.n_local, e * la.rb_rows))
                            for b, e in slice_plan(la.n_row_blocks, sms, _max_slices())]

    # -- the product -------------------------------------------------------------------------------
    def _local_into(self, x, out):
        if self._local_spmv is not None:
            self._local_spmv(x, out)
            return
        from .spmv_csr import flagsparse_spmv_csr

        flagsparse_spmv_csr(x=x, prepared=self.prepared, out=out)

    def matvec(self, x):
        """Full-length y on every rank.  The returned tensor is owned by this object: in mode "nccl" it is
        overwritten by the next call, in the other modes by the call after the next."""
        if self.mode == "peer":
            return self._matvec_peer(x)
        if self.mode == "fused":
            return self._matvec_fused(x)
        if self._y is None:
            self._y = torch.empty(self.n_rows, dtype=self.dtype, device=self.device)
        y = self._y
        if self._nccl_chunks is not None:
            return self._matvec_nccl_chunks(x, y)
        s, n = self.row_ranges[self.rank]
        self._local_into(x, y[s:s + n])
        self._all_gather_rows(y)
        return y

    def _plan_nccl_chunks(self):
        """Mode "nccl" on a panel layout: the shard is computed in the same slices of row blocks as in mode "peer",
        and slice j of every rank is gathered (on a stream of its own) while slice j+1 is computed.  Every rank needs
        every rank's slice boundaries, and all ranks must issue the same number of collectives: the tables are
        exchanged once, shorter ones padded with empty slices."""
        self._nccl_chunks = None
        p = self.prepared
        if self.world == 1 or p is None or not self.device.type == "cuda":
            return
        mine = []
        if p.algo == _lib.FSB_SPMV_PANEL and p.panel is not None and self.n_local > 0:
            la = p.panel
            sms = int(os.environ.get("FSB_SHARD_WAVE_BLOCKS", "0")) or \
                torch.cuda.get_device_properties(self.device).multi_processor_count
            mine = [(b, e, self.row_start + b * la.rb_rows, self.row_start + min(self.n_local, e * la.rb_rows))
                    for b, e in slice_plan(la.n_row_blocks, sms, _max_slices())]
        tables = [None] * self.world
        dist.all_gather_object(tables, mine, group=self.group)
        if any(len(t) == 0 for t in tables) or max(len(t) for t in tables) < 2:
            return                       # some shard has no panel layout, or nothing to overlap
        k = max(len(t) for t in tables)
        rows = []
        for r, t in enumerate(tables):
            end = self.row_ranges[r][0] + self.row_ranges[r][1]
            rows.append([(g0, g1) for _, _, g0, g1 in t] + [(end, end)] * (k - len(t)))
        self._nccl_chunks = [[rows[r][j] for r in range(self.world)] for j in range(k)]
        self._nccl_blocks = [(b, e) for b, e, _, _ in mine] + [(0, 0)] * (k - len(mine))
        self._side = torch.cuda.Stream(self.device)

    def _matvec_nccl_chunks(self, x, y):
        from . import panel
        from .spmv_csr import _validate_spmv_x

        p = self.prepared
        x = _validate_spmv_x(x, p)
        main = torch.cuda.current_stream(self.device)
        y_local = y[self.row_start: self.row_start + self.n_local]
        for (b0, b1), ranges in zip(self._nccl_blocks, self._nccl_chunks):
            if b1 > b0:
                with torch.cuda.device(self.device):
                    panel.launch_panel(p.panel, x, y_local, p.n_rows, p.n_cols, main.cuda_stream, b0, b1)
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(self._side):
                self._side.wait_event(ev)
                views = [y[g0:g1] for g0, g1 in ranges]
                sizes = {v.numel() for v in views}
                if len(sizes) == 1 and views[0].numel() > 0:
                    dist.all_gather(views, views[self.rank], group=self.group)
                else:
                    for r, v in enumerate(views):
                        if v.numel() > 0:
                            src = dist.get_global_rank(self.group, r) if self.group is not None else r
                            dist.broadcast(v, src=src, group=self.group)
        done = torch.cuda.Event()
        done.record(self._side)
        main.wait_event(done)
        return y

    def _matvec_peer(self, x):
        from . import panel
        from .spmv_csr import _spmv_launch, _validate_spmv_x

        p = self.prepared
        x = _validate_spmv_x(x, p)
        base = self._parity * self._stride
        self._parity ^= 1
        main = torch.cuda.current_stream(self.device)
        y_local = self._buf[base + self.row_start: base + self.row_start + self.n_local]
        if self.n_local > 0:
            if len(self._slices) == 1 and self._slices[0][1] == 0:
                _spmv_launch(p, x, y_local)
                ev = torch.cuda.Event()
                ev.record(main)
                self._push(base, self.row_start, self.row_start + self.n_local, ev)
            else:
                # consecutive slices go to two streams, so a slice's last row blocks and the next slice's first
                # ones share the SMs instead of waiting for each other; each push waits for its own slice only
                start = torch.cuda.Event()
                start.record(main)
                self._aux.wait_event(start)
                for j, (b0, b1, r0, r1) in enumerate(self._slices):
                    st = main if j % 2 == 0 else self._aux
                    with torch.cuda.device(self.device):
                        panel.launch_panel(p.panel, x, y_local, p.n_rows, p.n_cols, st.cuda_stream, b0, b1,
                                           record_on=st)
                    ev = torch.cuda.Event()
                    ev.record(st)
                    self._push(base, self.row_start + r0, self.row_start + r1, ev)
                back = torch.cuda.Event()
                back.record(self._aux)
                main.wait_event(back)
        self._finish_step()
        return self._buf[base: base + self.n_rows]

    def _matvec_fused(self, x):
        from .spmv_csr import _validate_spmv_x

        p = self.prepared
        x = _validate_spmv_x(x, p)
        L = _lib.lib()
        base = self._parity * self._stride
        self._parity ^= 1
        if self.n_local > 0:
            algo = _lib.FSB_SPMV_STREAM if (p.algo == _lib.FSB_SPMV_STREAM and p.tile_row is not None) \
                else _lib.FSB_SPMV_VECTOR
            with torch.cuda.device(self.device):
                rc = L.fsb_spmv_csr_scatter(
                    _VTYPE[p.data.dtype], _ITYPE[p.kernel_indices.dtype], _ITYPE[p.kernel_indptr.dtype],
                    _ptr(p.data), _ptr(p.kernel_indices), p.kernel_indptr.data_ptr(), _ptr(x),
                    self._peer_ptrs.data_ptr(), self.world, self.rank, base + self.row_start, p.n_rows, p.n_cols,
                    p.data.numel(), algo, p.tuning if algo == _lib.FSB_SPMV_STREAM else 0,
                    None if p.tile_row is None else p.tile_row.data_ptr(),
                    None if p.scratch is None else p.scratch.data_ptr(),
                    0 if p.scratch is None else p.scratch.numel(), _stream_ptr(self.device),
                )
            _lib.check(rc, "fsb_spmv_csr_scatter")
        self._symm.barrier(channel=0)
        return self._buf[base: base + self.n_rows]


class ShardedCsrSpmm(_ShardedBase):
    """C = A B with A split by rows over the ranks of a process group, B (n_cols x n_dense, row-major) replicated,
    the full C assembled on every rank.  Per-rank call being wrapped: flagsparse_spmm_csr_opt
    (src/flagsparse/sparse_operations/spmm_csr.py:1129-1183 in the reference).

    Each rank constructs it with ITS rows only (indptr rebased to start at 0) and the global index of its first
    row.  In mode "peer" the shard is cut into a few sub-shards of about equal nnz, each a prepared matrix of its
    own: sub-shard j is pushed to the peers while sub-shard j+1 is multiplied.

    local_spmm: optional callable (B, out) -> None for CPU process groups, as ShardedCsrSpmv's local_spmv.
    """

    def __init__(self, data, indices, indptr, row_start, shape, group=None, mode="auto", local_spmm=None):
        self._init_ranges(int(indptr.numel()) - 1, row_start, shape, group)
        self.device = data.device
        self.dtype = data.dtype
        self._local_spmm = local_spmm
        native = local_spmm is None and data.is_cuda and data.dtype in (torch.float32, torch.float64)
        if mode == "auto":
            mode = "peer" if (native and self.world > 1) else "nccl"
        if mode not in ("nccl", "peer"):
            raise ValueError("mode must be 'auto', 'nccl' or 'peer'")
        if mode == "peer" and not native:
            raise ValueError("mode 'peer' runs the CUDA kernels of this package on float32 / float64 values")
        self.mode = mode
        self.parts = []            # (row_lo, row_hi, prepared) of the sub-shards
        if local_spmm is None:
            from .spmm_csr import prepare_spmm_csr_opt

            k = _max_slices() if mode == "peer" else 1
            cuts = partition_rows_by_nnz(indptr, max(1, min(k, max(1, self.n_local))))
            for a, b in zip(cuts[:-1], cuts[1:]):
                if b <= a:
                    continue
                e0, e1 = int(indptr[a]), int(indptr[b])
                sub_ptr = (indptr[a:b + 1] - indptr[a]).contiguous()
                prep = prepare_spmm_csr_opt(data[e0:e1], indices[e0:e1], sub_ptr, (b - a, self.n_cols))
                self.parts.append((a, b, prep))
        self._c = None
        self._width_ready = None

    def _local_into(self, B, out):
        if self._local_spmm is not None:
            self._local_spmm(B, out)
            return
        from .spmm_csr import flagsparse_spmm_csr_opt

        for a, b, prep in self.parts:
            flagsparse_spmm_csr_opt(B=B, prepared=prep, out=out[a:b])

    def matmul(self, B):
        """Full C (n_rows x n_dense) on every rank; owned by this object like ShardedCsrSpmv.matvec's result."""
        if B.ndim != 2 or B.shape[0] != self.n_cols:
            raise ValueError(f"B must be 2D with {self.n_cols} rows")
        if B.dtype != self.dtype:
            raise TypeError("B dtype must match the sparse matrix dtype")
        n_dense = int(B.shape[1])
        if self.mode == "peer":
            return self._matmul_peer(B, n_dense)
        if self._c is None or self._c.shape[1] != n_dense:
            self._c = torch.empty((self.n_rows, n_dense), dtype=self.dtype, device=self.device)
        C = self._c
        s, n = self.row_ranges[self.rank]
        if n > 0 and n_dense > 0:
            self._local_into(B, C[s:s + n])
        if n_dense > 0:
            self._all_gather_rows(C)
        return C

    def _matmul_peer(self, B, n_dense):
        from .spmm_csr import flagsparse_spmm_csr_opt

        if n_dense == 0:
            return torch.empty((self.n_rows, 0), dtype=self.dtype, device=self.device)
        if self._width_ready != n_dense:
            self._setup_symmetric(n_dense)      # collective: every rank calls matmul with the same width
            self._width_ready = n_dense
        base = self._parity * self._stride
        self._parity ^= 1
        main = torch.cuda.current_stream(self.device)
        C = self._buf[base: base + self.n_rows * n_dense].view(self.n_rows, n_dense)
        for a, b, prep in self.parts:
            flagsparse_spmm_csr_opt(B=B, prepared=prep, out=C[self.row_start + a: self.row_start + b])
            ev = torch.cuda.Event()
            ev.record(main)
            self._push(base, self.row_start + a, self.row_start + b, ev)
        covered = sum(b - a for a, b, _ in self.parts)
        if covered != self.n_local:                 # rows of sub-shards without entries (nothing was launched)
            raise RuntimeError("sub-shards do not cover the local rows")
        self._finish_step()
        return C
