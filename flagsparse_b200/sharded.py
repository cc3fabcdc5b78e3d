"""Row-sharded CSR SpMV over the GPUs of one box: one process per GPU, x replicated, y assembled on every rank.

The reference is single-GPU (no torch.distributed, NCCL or multi-device code anywhere in its tree); this
driver is what "run src/flagsparse/sparse_operations/spmv_csr.py:557-610 on a row shard per GPU and gather
y" becomes on an NVSwitch box.  Rows are independent, so the only exchange is the all-gather of y:

  * mode "nccl": every rank computes its rows straight into its slice of a full-length y, then one
    (uneven) all-gather moves the slices -- NCCL over NVLink, or broadcasts on a CPU (gloo) group.
  * mode "peer": y lives in symmetric memory; the SpMV kernel's epilogue stores each finished value into
    every rank's y through peer-mapped pointers (plain stores, no TMA), so the transfer overlaps the
    streaming of A tile by tile, and a barrier ends the step.

Shard boundaries are contiguous row ranges holding about nnz / P entries each.
"""

import torch
import torch.distributed as dist

from . import _lib
from ._common import _ITYPE, _VTYPE, _ptr, _stream_ptr


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


class ShardedCsrSpmv:
    """y = A x with A split by rows over the ranks of a process group.

    Each rank constructs it with ITS rows only: `data`, `indices`, and `indptr` rebased so that
    indptr[0] == 0; `row_start` is the global index of its first row.  `matvec(x)` takes the full x
    (replicated on every rank) and returns the full y on every rank.

    local_spmv: optional callable (x, out) -> None that fills `out` (length = local rows) with the local
    product.  It exists so that the host logic (partition bookkeeping, assembly, collectives) can be
    exercised on CPU process groups; by default the CUDA kernels of this package do the work.
    """

    def __init__(self, data, indices, indptr, row_start, shape, group=None, mode="auto", local_spmv=None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.n_rows, self.n_cols = int(shape[0]), int(shape[1])
        self.n_local = int(indptr.numel()) - 1
        self.row_start = int(row_start)
        self.device = data.device
        self.dtype = data.dtype
        # every rank learns every shard's row range
        mine = (self.row_start, self.n_local)
        if self.world > 1:
            ranges = [None] * self.world
            dist.all_gather_object(ranges, mine, group=group)
        else:
            ranges = [mine]
        self.row_ranges = [(int(s), int(n)) for s, n in ranges]
        self._check_cover()
        self._local_spmv = local_spmv
        if mode == "auto":
            # the fused exchange needs the CUDA kernels, several ranks and something to multiply
            fused_ok = (local_spmv is None and self.world > 1 and data.is_cuda
                        and data.dtype in (torch.float32, torch.float64))
            mode = "peer" if fused_ok else "nccl"
        if mode not in ("nccl", "peer"):
            raise ValueError("mode must be 'auto', 'nccl' or 'peer'")
        if mode == "peer" and local_spmv is not None:
            raise ValueError("mode 'peer' fuses the exchange into the CUDA kernel; it cannot take local_spmv")
        if mode == "peer" and data.dtype not in (torch.float32, torch.float64):
            raise TypeError("mode 'peer' needs float32 or float64 values (the kernels with peer stores compute those)")
        self.prepared = None
        if local_spmv is None:
            from .spmv_csr import _prepare_spmv_csr

            # the peer-store epilogue exists for the vector, the stream and the panel kernel, not for the split
            # of long rows
            self.prepared = _prepare_spmv_csr(data, indices, indptr, (self.n_local, self.n_cols), 256, None,
                                              reuse_expected=True, allow_split=mode != "peer")
        self.mode = mode
        self._y = None
        self._symm = None
        self._peer_ptrs = None
        if mode == "peer":
            self._setup_peer()

    # -- bookkeeping -----------------------------------------------------------------------------
    def _check_cover(self):
        pos = 0
        for s, n in self.row_ranges:
            if s != pos or n < 0:
                raise ValueError(f"row shards must be contiguous and ordered by rank, got {self.row_ranges}")
            pos += n
        if pos != self.n_rows:
            raise ValueError(f"row shards cover {pos} rows, the matrix has {self.n_rows}")

    def _setup_peer(self):
        import torch.distributed._symmetric_memory as symm_mem

        # a shard prepared for the panel kernel has its own entry point with peer stores
        self._peer_algo = _lib.FSB_SPMV_STREAM if self.prepared.algo == _lib.FSB_SPMV_STREAM else _lib.FSB_SPMV_VECTOR
        group = self.group if self.group is not None else dist.group.WORLD
        # two result buffers used alternately: a rank may start the next product while its peers still
        # read the previous one, so a single barrier per product is enough
        self._stride = (max(self.n_rows, 1) + 63) // 64 * 64
        self._y = symm_mem.empty(2 * self._stride, dtype=self.dtype, device=self.device)
        self._symm = symm_mem.rendezvous(self._y, group)
        ptrs = [int(p) for p in self._symm.buffer_ptrs]
        self._peer_ptrs = torch.tensor(ptrs, dtype=torch.int64, device=self.device)
        self._parity = 0

    # -- the product -------------------------------------------------------------------------------
    def _local_into(self, x, out):
        if self._local_spmv is not None:
            self._local_spmv(x, out)
            return
        from .spmv_csr import flagsparse_spmv_csr

        flagsparse_spmv_csr(x=x, prepared=self.prepared, out=out)

    def matvec(self, x):
        """Full-length y on every rank.  The returned tensor is owned by this object: in mode "nccl" it is
        overwritten by the next call, in mode "peer" by the call after the next."""
        if self.mode == "peer":
            return self._matvec_peer(x)
        if self._y is None:
            self._y = torch.empty(self.n_rows, dtype=self.dtype, device=self.device)
        y = self._y
        s, n = self.row_ranges[self.rank]
        self._local_into(x, y[s:s + n])
        if self.world > 1:
            views = [y[a:a + b] for a, b in self.row_ranges]
            backend = dist.get_backend(self.group)
            if backend == "nccl":
                dist.all_gather(views, views[self.rank], group=self.group)  # uneven sizes: grouped broadcasts
            else:
                for r, v in enumerate(views):
                    if v.numel() > 0:
                        dist.broadcast(v, src=dist.get_global_rank(self.group, r) if self.group is not None else r,
                                       group=self.group)
        return y

    def _matvec_peer(self, x):
        from .spmv_csr import _validate_spmv_x

        p = self.prepared
        x = _validate_spmv_x(x, p)
        L = _lib.lib()
        base = self._parity * self._stride
        self._parity ^= 1
        if self.n_local > 0 and p.algo == _lib.FSB_SPMV_PANEL and p.panel is not None:
            la = p.panel
            with torch.cuda.device(self.device):
                rc = L.fsb_spmv_csr_panel_scatter(
                    _VTYPE[la.val.dtype], la.val.data_ptr(), la.rc.data_ptr(), la.unit_piece_ptr.data_ptr(),
                    la.unit_chunk.data_ptr(), la.rb_unit_ptr.data_ptr(), la.n_row_blocks, la.rb_rows, la.chunk_cols,
                    la.n_buffers, _ptr(x), self._peer_ptrs.data_ptr(), self.world, base + self.row_start, p.n_rows,
                    p.n_cols, la.status.data_ptr(), _stream_ptr(self.device),
                )
            _lib.check(rc, "fsb_spmv_csr_panel_scatter")
        elif self.n_local > 0:
            with torch.cuda.device(self.device):
                rc = L.fsb_spmv_csr_scatter(
                    _VTYPE[p.data.dtype], _ITYPE[p.kernel_indices.dtype], _ITYPE[p.kernel_indptr.dtype],
                    _ptr(p.data), _ptr(p.kernel_indices), p.kernel_indptr.data_ptr(), _ptr(x),
                    self._peer_ptrs.data_ptr(), self.world, base + self.row_start, p.n_rows, p.n_cols, p.data.numel(),
                    self._peer_algo, p.tuning if self._peer_algo == _lib.FSB_SPMV_STREAM else 0,
                    None if p.tile_row is None else p.tile_row.data_ptr(),
                    None if p.scratch is None else p.scratch.data_ptr(),
                    0 if p.scratch is None else p.scratch.numel(), _stream_ptr(self.device),
                )
            _lib.check(rc, "fsb_spmv_csr_scatter")
        # every rank's stores have landed everywhere once all ranks pass this barrier; it also orders this
        # product after every peer's reads of the buffer written two products ago
        self._symm.barrier(channel=0)
        return self._y[base: base + self.n_rows]
