#!/usr/bin/env python
"""Benchmark of the CSR SpMV / SpMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one product over the whole matrix of the workload, with the prepared matrix resident in HBM
(the steady state the reference's scripts time).  Rank 0 prints ONE JSON line.

Workloads (all synthetic, seeded; see flagsparse_b200/synthetic.py):
  c5       SpMV, 2^26 rows, Poisson(32), band +-2^20, int64 indptr (~2.1e9 nnz): the default at every --gpus N.
           One GPU holds the whole matrix; under torchrun it is row-sharded over the ranks (strong scaling: the
           matrix is fixed), so the per-N lines of one workload form the scaling curve
  c2       SpMV, 2^22 rows, Poisson(32) rows, band +-2^16, float32 / int32
  c2f64    the same matrix in float64 / int64
  c1, c3   SpMV 4096^2 with 16 nnz per row; SpMV 2^24 rows with Zipf(2) row lengths
  c4n32, c4n64, c4n128   SpMM, 2^20 rows x 16 nnz, dense width 32 / 64 / 128 (sharded under torchrun)
`value` is algorithmic bytes / device time in GB/s: A once (values + indices + indptr), x (or B) once, y (or
C) once, with the byte widths the kernels actually stream (never more than the caller's widths).

The default single-GPU run also times every other configuration briefly (`others`), next to cuSPARSE and the
reference's Triton kernels on the same GPU where those can be run, and checks results in the run itself
(`parity`): rank 0 regenerates row blocks of the matrix on the host and holds the device result to the
float64 bound; sharded runs also compare every rank's assembled result with rank 0's bit for bit.  A failed
check makes the run exit non-zero.
"""

import argparse
import datetime
import hashlib
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the step's dominant kernel, from the ncu captures
# summarised under profiles/, each tied to the sources it was taken on: workload -> (bytes, source files relative to
# the repository root, first 12 hex digits of the sha256 of their concatenation).  A capture of other sources is not
# reported (traffic: null).  c5: the capture is of the same matrix law at 2^22 rows (1/16 of the rows, of the units
# and of the entries), scaled by 16.
_PANEL_SOURCES = ("flagsparse_b200/csrc/spmv_panel.cu", "flagsparse_b200/panel.py")
NCU_TRAFFIC_BYTES = {
    "c2": (1_097_973_000 + 4_892_672, _PANEL_SOURCES, "2536da0b2366"),        # profiles/spmv_panel_c2_f32.md
    "c2f64": (1_673_750_000 + 4_101_376, _PANEL_SOURCES, "2536da0b2366"),     # profiles/spmv_panel_c2_f64.md
    "c5": (16 * (1_127_045_000 + 3_713_792), _PANEL_SOURCES, "2536da0b2366"),  # profiles/spmv_panel_c5like_f32.md
}

SPMV_WORKLOADS = {
    "c1": ("c1", "float32", "int32", "int32"),
    "c2": ("c2", "float32", "int32", "int32"),
    "c2f64": ("c2", "float64", "int64", "int64"),
    "c3": ("c3", "float32", "int32", "int32"),
    "c5": ("c5", "float32", "int32", "int64"),
}
SPMM_WORKLOADS = {"c4n32": 32, "c4n64": 64, "c4n128": 128}
OTHERS = ("c2", "c2f64", "c3", "c4n32", "c4n64", "c4n128", "c1")
TOL = {"float32": 1e-5, "float64": 1e-13}
PARITY_BLOCK_ROWS = 2048


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def spmv_bytes(n_rows, n_cols, nnz, sv, si, sp):
    return nnz * (sv + si) + (n_rows + 1) * sp + n_cols * sv + n_rows * sv


def spmm_bytes(n_rows, n_cols, nnz, n_dense, sv, si, sp):
    return nnz * (sv + si) + (n_rows + 1) * sp + n_cols * n_dense * sv + n_rows * n_dense * sv


def measured_traffic(workload):
    """DRAM bytes per launch from a committed ncu capture, if it was taken on the kernel source being run."""
    entry = NCU_TRAFFIC_BYTES.get(workload)
    if entry is None:
        return None
    nbytes, sources, sha = entry
    h = hashlib.sha256()
    try:
        for source in sources:
            with open(os.path.join(ROOT, source), "rb") as f:
                h.update(f.read())
    except OSError:
        return None
    return nbytes if h.hexdigest()[:12] == sha else None


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz, self._stop, self._thread = [], set(), None, False, None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "nvmlClocksThrottleReasonHwSlowdown": "hw_slowdown",
            "nvmlClocksThrottleReasonHwThermalSlowdown": "hw_thermal_slowdown",
            "nvmlClocksThrottleReasonSwThermalSlowdown": "sw_thermal_slowdown",
            "nvmlClocksThrottleReasonSwPowerCap": "sw_power_cap",
            "nvmlClocksThrottleReasonHwPowerBrakeSlowdown": "hw_power_brake_slowdown",
        }
        while not self._stop:
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for attr, label in names.items():
                    if mask & int(getattr(nv, attr, 0)):
                        self.reasons.add(label)
            except Exception:
                pass
            time.sleep(0.01)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop = True
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {
            "sm_mhz": (statistics.median(self.samples) if self.samples else None),
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def physical_gpu_index(local_index):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


# -------------------------------------------------------------------------------------------------------
# the CPU arms: the timed baseline of the default run and the whole of --impl reference
# -------------------------------------------------------------------------------------------------------
def cpu_sample(workload, rows_log2=None):
    """A bounded slice of the workload regenerated on the host: 2^rows_log2 consecutive rows (from the middle of
    a banded matrix, so that the band is not clipped by the matrix edge) and the full x / B."""
    from flagsparse_b200 import synthetic as S

    if workload in SPMM_WORKLOADS:
        spec = S.config_spec("c4")
        rows = min(spec.n_rows, 1 << (rows_log2 or 17))
        d, i, p = S.generate_csr(spec, None, row_range=(0, rows))
        dense = S.dense_vector(spec, spec.n_cols, n_dense=SPMM_WORKLOADS[workload])
        return spec, rows, (d, i, p), dense, f"rows [0, {rows}) of {spec.n_rows}, B full"
    cfg, vdt, idt, pdt = SPMV_WORKLOADS[workload]
    spec = S.config_spec(cfg)
    # c5: 1/16 of the rows (134 M entries, 1.1 GB of A; about a minute of generation on the host)
    rows = min(spec.n_rows, 1 << (rows_log2 or (22 if workload == "c5" else 19)))
    r0 = 0 if spec.columns[0] != "band" else (spec.n_rows - rows) // 2
    d, i, p = S.generate_csr(spec, None, value_dtype=vdt, index_dtype=idt, indptr_dtype=pdt, row_range=(r0, r0 + rows))
    dense = S.dense_vector(spec, spec.n_cols, value_dtype=vdt)
    return spec, rows, (d, i, p), dense, f"rows [{r0}, {r0 + rows}) of {spec.n_rows}, x full"


def sample_bytes(workload, spec, rows, csr):
    """Algorithmic bytes of a row slice: its part of A and of the output, and the part of x / B it can
    touch (all of it for uniform columns, the rows plus the band for a banded matrix)."""
    d, i, p = csr
    if spec.columns[0] == "band":
        dense_rows = min(spec.n_cols, rows + 2 * int(spec.columns[1]))
    else:
        dense_rows = spec.n_cols
    if workload in SPMM_WORKLOADS:
        return spmm_bytes(rows, dense_rows, d.size, SPMM_WORKLOADS[workload], d.itemsize, i.itemsize, p.itemsize)
    return spmv_bytes(rows, dense_rows, d.size, d.itemsize, i.itemsize, p.itemsize)


def time_cpu(fn, min_seconds, min_reps=3):
    fn()
    times = []
    t_end = time.perf_counter() + min_seconds
    while len(times) < min_reps or time.perf_counter() < t_end:
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return statistics.median(times)


def cpu_baseline_scipy(workload, rows_log2=None):
    """scipy.sparse (single-threaded CSR kernels) in the input dtype on a bounded sample -- the oracle's
    arithmetic, timed on one host core."""
    import scipy.sparse as sp

    spec, rows, (d, i, p), dense, what = cpu_sample(workload, rows_log2 or (20 if workload == "c5" else None))
    a = sp.csr_matrix((d, i, p), shape=(rows, spec.n_cols))
    t = time_cpu(lambda: a @ dense, min_seconds=3.0)
    nbytes = sample_bytes(workload, spec, rows, (d, i, p))
    flops = 2.0 * d.size * (dense.shape[1] if dense.ndim == 2 else 1)
    return {"value": nbytes / t / 1e9, "unit": "GB/s", "cores": 1, "kind": "port", "sample": what,
            "impl": "scipy.sparse csr @ dense", "ms": t * 1e3, "gflops": flops / t / 1e9,
            "host_cores_available": os.cpu_count()}


def run_reference_arm(args, workload):
    """--impl reference: the reference has no CPU implementation of its own (its kernels are Triton); the
    CPU arm is the plain-C restatement of its arithmetic (oracle/csr_ref.c) on every host thread."""
    from oracle import csr_ref as C

    threads = C.max_threads()
    spec, rows, (d, i, p), dense, what = cpu_sample(workload, args.cpu_rows_log2)
    shape = (rows, spec.n_cols)
    if workload in SPMM_WORKLOADS:
        fn = lambda: C.spmm(d, i, p, shape, dense, native=False, threads=threads)  # noqa: E731
    else:
        fn = lambda: C.spmv(d, i, p, shape, dense, native=False, threads=threads)  # noqa: E731
    for _ in range(max(args.warmup, 1)):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    dt = (time.perf_counter() - t0) / args.steps
    nbytes = sample_bytes(workload, spec, rows, (d, i, p))
    value = nbytes / dt / 1e9
    flops = 2.0 * d.size * (dense.shape[1] if dense.ndim == 2 else 1)
    line = {
        "impl": "reference", "metric": metric_name(workload), "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": "f32" if d.dtype == np.float32 else "f64", "data": "synthetic",
        "config": workload_config(workload, args.gpus),
        "gflops": flops / dt / 1e9,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": what,
                         "impl": "oracle/csr_ref.c (float64 accumulate, POSIX threads)"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def metric_name(workload):
    return "CSR SpMM HBM GB/s" if workload in SPMM_WORKLOADS else "CSR SpMV HBM GB/s"


def workload_config(workload, n_gpus):
    desc = {
        "c1": "CSR SpMV 4096x4096, 16 nnz/row, f32/i32 (latency-bound: 0.57 MB of traffic)",
        "c2": "CSR SpMV 2^22 rows, Poisson(32) rows (~134M nnz), band +-2^16, f32 values / i32 indices",
        "c2f64": "CSR SpMV 2^22 rows, Poisson(32) rows (~134M nnz), band +-2^16, f64 values / i64 indices",
        "c3": "CSR SpMV 2^24 rows, Zipf(2) row lengths clipped to [1,2^17] (~240M nnz), uniform columns, f32/i32",
        "c5": "CSR SpMV 2^26 rows, Poisson(32) rows (~2.1B nnz), band +-2^20, f32/i32, i64 indptr",
    }
    if workload in SPMM_WORKLOADS:
        w = f"CSR SpMM 2^20 rows x 16 nnz/row times dense 2^20 x {SPMM_WORKLOADS[workload]}, f32/i32"
    else:
        w = desc[workload]
    cfg = {"workload": w, "name": workload, "l2": "inputs larger than L2 (no flush needed)"}
    if workload == "c1":
        cfg["l2"] = "working set 0.57 MB: L2-resident after warm-up; GB/s is a latency figure"
    if n_gpus > 1:
        what = "B replicated, C" if workload in SPMM_WORKLOADS else "x replicated, y"
        cfg["parallelism"] = f"rows sharded by nnz over {n_gpus} GPUs, {what} assembled on every GPU"
    return cfg


# -------------------------------------------------------------------------------------------------------
# in-run parity: host-regenerated row blocks against a float64 product
# -------------------------------------------------------------------------------------------------------
def parity_blocks(n_rows, marks, block_rows=PARITY_BLOCK_ROWS, extra=3, seed=1):
    """Row blocks to check: the first and the last rows, one block around every row in `marks` (shard
    boundaries, the row where the entry count passes 2^31), and a few seeded random ones."""
    starts = {0, max(0, n_rows - block_rows)}
    for m in marks:
        starts.add(min(max(0, int(m) - block_rows // 2), max(0, n_rows - block_rows)))
    rng = np.random.default_rng(seed)
    for s in rng.integers(0, max(1, n_rows - block_rows), extra).tolist():
        starts.add(int(s))
    return [(s, min(n_rows, s + block_rows)) for s in sorted(starts)]


def check_blocks(workload, result_dev, dense_host, blocks):
    """Hold the device result (y or C, full size) to |r - r64| <= tol * (|A| |dense|) on the given row blocks,
    with A regenerated on the host from the row-keyed generator.  Returns the worst ratio |r - r64| / (|A||dense|)."""
    import scipy.sparse as sp

    from flagsparse_b200 import synthetic as S

    if workload in SPMM_WORKLOADS:
        spec, vdt, idt, pdt = S.config_spec("c4"), "float32", "int32", "int32"
    else:
        cfg, vdt, idt, pdt = SPMV_WORKLOADS[workload]
        spec = S.config_spec(cfg)
    dense64 = np.asarray(dense_host, dtype=np.float64)
    worst = 0.0
    for r0, r1 in blocks:
        d, i, p = S.generate_csr(spec, None, value_dtype=vdt, index_dtype=idt, indptr_dtype=pdt, row_range=(r0, r1))
        a = sp.csr_matrix((d.astype(np.float64), i, p), shape=(r1 - r0, spec.n_cols))
        ref = a @ dense64
        mag = abs(a) @ np.abs(dense64)
        got = result_dev[r0:r1].cpu().numpy().astype(np.float64)
        if got.shape != ref.shape:
            return float("inf")
        err = np.abs(got - ref)
        zero = mag == 0
        if np.any(err[zero] != 0):
            return float("inf")
        if np.any(~zero):
            worst = max(worst, float(np.max(err[~zero] / mag[~zero])))
    return worst


# -------------------------------------------------------------------------------------------------------
# the GPU arm
# -------------------------------------------------------------------------------------------------------
def timed_region(torch, fn, steps, barrier):
    """K calls of fn between two CUDA events on the current stream; barrier + synchronize on both sides."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    barrier()
    return start.elapsed_time(end) / 1e3  # seconds


def timed_pipeline(torch, api_call, host_in, host_out, steps, depth=2):
    """End-to-end steps with the three stages of consecutive steps overlapped: copy-in of step k+1, the product
    of step k and copy-out of step k-1 run on three streams with `depth` device buffers each.  Every step still
    moves its own input from pinned host memory and its own result back inside the timed region.
    api_call(dev_in, dev_out) is the package's public call, issued on the current (compute) stream."""
    dev = torch.cuda.current_device()
    s_in, s_run, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dev_in = [torch.empty(host_in.shape, dtype=host_in.dtype, device="cuda") for _ in range(depth)]
    dev_out = [torch.empty(host_out.shape, dtype=host_out.dtype, device="cuda") for _ in range(depth)]
    ev_in = [torch.cuda.Event() for _ in range(depth)]      # input b is on the device
    ev_used = [torch.cuda.Event() for _ in range(depth)]    # input b has been consumed
    ev_res = [torch.cuda.Event() for _ in range(depth)]     # result b is ready
    ev_read = [torch.cuda.Event() for _ in range(depth)]    # result b has been copied out
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    main = torch.cuda.current_stream()

    def run(n):
        for k in range(n):
            b = k % depth
            with torch.cuda.stream(s_in):
                if k >= depth:
                    s_in.wait_event(ev_used[b])
                dev_in[b].copy_(host_in, non_blocking=True)
                ev_in[b].record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_in[b])
                if k >= depth:
                    s_run.wait_event(ev_read[b])
                api_call(dev_in[b], dev_out[b])
                ev_used[b].record(s_run)
                ev_res[b].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_res[b])
                host_out.copy_(dev_out[b], non_blocking=True)
                ev_read[b].record(s_out)

    run(2 * depth)  # warm-up of the pipeline
    torch.cuda.synchronize()
    start.record(main)
    for st in (s_in, s_run, s_out):
        st.wait_event(start)
    run(steps)
    for st in (s_in, s_run, s_out):
        fin = torch.cuda.Event()
        fin.record(st)
        main.wait_event(fin)
    end.record(main)
    torch.cuda.synchronize()
    return start.elapsed_time(end) / 1e3


def timed_pipeline_sharded(torch, dist, run, host_in, host_out, dev_full, n_in, r0, r1, steps, barrier, lag):
    """Sharded end-to-end steps with the stages of consecutive steps overlapped: the upload of this rank's 1/N of
    the dense operand for step k+1 (its own stream, two device buffers) runs under the all-gather and the product of
    step k (current stream), and the read-back of this rank's rows of step k (a third stream) under step k+1.
    `lag`: how many products later the result buffer of a product is written again (the read-back of step k must be
    over before product k+lag starts).  Every step still moves its own input and its own result inside the timed
    region.  Returns seconds."""
    dev = torch.cuda.current_device()
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    main = torch.cuda.current_stream()
    slices = [torch.empty(host_in.shape, dtype=host_in.dtype, device="cuda") for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]      # slice b is on the device
    ev_used = [torch.cuda.Event() for _ in range(2)]    # slice b has been gathered
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def go(n):
        reads = []
        for k in range(n):
            b = k % 2
            with torch.cuda.stream(s_in):
                if k >= 2:
                    s_in.wait_event(ev_used[b])
                slices[b].copy_(host_in, non_blocking=True)
                ev_in[b].record(s_in)
            main.wait_event(ev_in[b])
            dist.all_gather_into_tensor(dev_full, slices[b])
            ev_used[b].record(main)
            if k >= lag:
                main.wait_event(reads[k - lag])
            res = run(dev_full[:n_in])
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                host_out.copy_(res[r0:r1], non_blocking=True)
                e = torch.cuda.Event()
                e.record(s_out)
                reads.append(e)
        for st in (s_in, s_out):
            fin = torch.cuda.Event()
            fin.record(st)
            main.wait_event(fin)

    go(4)   # warm-up of the pipeline
    barrier()
    torch.cuda.synchronize()
    start.record(main)
    s_in.wait_event(start)
    s_out.wait_event(start)
    go(steps)
    end.record(main)
    torch.cuda.synchronize()
    barrier()
    return start.elapsed_time(end) / 1e3


def event_time_ms(torch, fn, warm, iters):
    """Median over `iters` single calls, CUDA events around each (the protocol of the reference's own scripts)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def batch_time_ms(torch, fn, warm, iters):
    """Milliseconds per call over `iters` back-to-back calls between two CUDA events (what the headline uses)."""
    for _ in range(warm):
        fn()
    return timed_region(torch, fn, iters, lambda: None) * 1e3 / iters


def load_reference_package():
    """The unmodified reference package installed under baseline/_ref (Triton kernels), or None."""
    path = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(path, "flagsparse")):
        return None
    try:
        if path not in sys.path:
            sys.path.insert(0, path)
        import flagsparse as ref

        return ref
    except Exception:
        return None


class SingleGpuWorkload:
    """One workload on one GPU: the matrix, the prepared object, the step, and what is needed to check and to
    describe it."""

    def __init__(self, torch, workload, device):
        import flagsparse_b200 as fs
        from flagsparse_b200 import _lib
        from flagsparse_b200 import synthetic as S

        self.torch, self.fs, self.workload, self.device = torch, fs, workload, device
        self.is_spmm = workload in SPMM_WORKLOADS
        t0 = time.perf_counter()
        if self.is_spmm:
            self.n_dense = SPMM_WORKLOADS[workload]
            self.spec = spec = S.config_spec("c4")
            self.vdt = "float32"
            self.csr = S.generate_csr(spec, device)
            self.dense = S.dense_vector(spec, spec.n_cols, device, n_dense=self.n_dense)
        else:
            cfg, vdt, idt, pdt = SPMV_WORKLOADS[workload]
            self.spec = spec = S.config_spec(cfg)
            self.vdt = vdt
            self.csr = S.generate_csr(spec, device, value_dtype=vdt, index_dtype=idt, indptr_dtype=pdt)
            self.dense = S.dense_vector(spec, spec.n_cols, device, value_dtype=vdt)
        torch.cuda.synchronize()
        self.generate_s = time.perf_counter() - t0
        d, i, p = self.csr
        self.shape = (spec.n_rows, spec.n_cols)
        self.nnz = d.numel()
        # prepare, timed on its own (host clock around a synchronised region: it holds host syncs by design)
        t0 = time.perf_counter()
        if self.is_spmm:
            self.prep = fs.prepare_spmm_csr_opt(d, i, p, self.shape)
            self.out = torch.empty((spec.n_rows, self.n_dense), dtype=d.dtype, device=device)
            self.step = lambda: fs.flagsparse_spmm_csr_opt(B=self.dense, prepared=self.prep, out=self.out)
            self.api_call = lambda di, do: fs.flagsparse_spmm_csr_opt(B=di, prepared=self.prep, out=do)
            self.one_shot = lambda: fs.flagsparse_spmm_csr_opt(d, i, p, self.dense, self.shape)
            self.step()                       # the first call builds the width-dependent part of the prepared state
        else:
            self.prep = fs.prepare_spmv_csr(d, i, p, self.shape)
            self.out = torch.empty(spec.n_rows, dtype=d.dtype, device=device)
            self.step = lambda: fs.flagsparse_spmv_csr(x=self.dense, prepared=self.prep, out=self.out)
            self.api_call = lambda di, do: fs.flagsparse_spmv_csr(x=di, prepared=self.prep, out=do)
            self.one_shot = lambda: fs.flagsparse_spmv_csr(d, i, p, self.dense, self.shape)
        torch.cuda.synchronize()
        self.prepare_s = time.perf_counter() - t0
        sv = d.element_size()
        si, sp_ = self.prep.kernel_indices.element_size(), self.prep.kernel_indptr.element_size()
        if self.is_spmm:
            self.nbytes = spmm_bytes(spec.n_rows, spec.n_cols, self.nnz, self.n_dense, sv, si, sp_)
            self.flops = 2.0 * self.nnz * self.n_dense
            self.kernel = self.prep.row_buckets[0]["kind"]
            self.launches = getattr(self.prep, "launches_per_product", lambda n: 2)(self.n_dense)
        else:
            self.nbytes = spmv_bytes(spec.n_rows, spec.n_cols, self.nnz, sv, si, sp_)
            self.flops = 2.0 * self.nnz
            self.kernel = self.prep.opt_buckets[0]["kind"]
            self.launches = 2 if self.prep.algo == _lib.FSB_SPMV_STREAM else 1
            if self.prep.long_rows is not None:
                short = self.prep.long_rows[0]
                self.launches = (2 if short.algo == _lib.FSB_SPMV_STREAM and short.tile_row is not None else 1) + 2

    def describe(self):
        """Layout facts of the prepared matrix for the JSON line."""
        extra = {"kernel": self.kernel}
        if self.is_spmm:
            d = self.csr[0]
            extra["bytes_gather_model"] = (self.nnz * (d.element_size() + 4) + self.nnz * self.n_dense * d.element_size()
                                           + self.spec.n_rows * self.n_dense * d.element_size())
            plan = getattr(self.prep, "plan_summary", None)
            if plan is not None:
                extra["spmm_plan"] = plan(self.n_dense)
            return extra
        lay = self.prep.panel
        if lay is not None:
            extra["panel"] = {"rb_rows": lay.rb_rows, "chunk_cols": lay.chunk_cols, "units": lay.n_units,
                              "rounds": lay.rounds, "long_runs": bool(lay.flags & 1), "n_buffers": lay.n_buffers,
                              "x_overhead": round(lay.x_overhead, 3), "slot_overhead": round(lay.slot_overhead, 3),
                              "layout_bytes": lay.nbytes()}
        if self.prep.long_rows is not None:
            short, lay = self.prep.long_rows
            extra["long_rows"] = {"rows": lay.n_long, "nnz": lay.nnz, "groups": lay.n_groups, "ctas": lay.n_ctas,
                                  "units": lay.n_units, "x_overhead": round(lay.x_overhead, 3),
                                  "slot_overhead": round(lay.slot_overhead, 3), "layout_bytes": lay.nbytes(),
                                  "short_nnz": short.data.numel()}
        return extra

    def parity(self, extra_marks=()):
        """(blocks checked, worst ratio) of the result of one more step against host-regenerated row blocks."""
        torch = self.torch
        self.out.zero_()
        self.step()
        self.prep.check_status()
        torch.cuda.synchronize()
        marks = list(extra_marks)
        p = self.prep.kernel_indptr
        if self.nnz > 2**31:
            marks.append(int(torch.searchsorted(p, torch.tensor([2**31], dtype=p.dtype, device=p.device))[0]))
        n_blocks = 3 if self.workload != "c5" else 5
        blocks = parity_blocks(self.spec.n_rows, marks, extra=n_blocks)
        if self.is_spmm or self.workload == "c3":
            blocks = blocks[:4]               # wide or long rows: a few blocks are plenty of host work
        worst = check_blocks(self.workload, self.out, self.dense.cpu().numpy(), blocks)
        return len(blocks), worst

    def compare(self, ref, budget_s):
        """cuSPARSE (through torch) and the reference's Triton kernels on the same inputs; milliseconds or a
        short reason.  The 10 + 50 protocol of the reference's scripts, fewer repeats for its slow paths."""
        torch, out = self.torch, {}
        d, i, p = self.csr
        t_begin = time.perf_counter()
        try:
            if self.nnz >= 2**31:
                raise RuntimeError("skipped: torch wants int64 column indices here (+17 GB)")
            A = torch.sparse_csr_tensor(p.to(torch.int64), i.to(torch.int64), d, size=self.shape)
            fn = (lambda: torch.sparse.mm(A, self.dense)) if self.is_spmm else (lambda: torch.mv(A, self.dense))
            out["cusparse_ms"] = event_time_ms(torch, fn, 5, 20)
            del A
        except Exception as e:  # noqa: BLE001 -- one column failing must not lose the line
            out["cusparse_ms"] = f"unavailable: {type(e).__name__}: {str(e)[:80]}"
        if ref is None:
            out["ref_triton_opt_ms"] = "unavailable: baseline/_ref not importable"
        elif time.perf_counter() - t_begin > budget_s:
            out["ref_triton_opt_ms"] = "skipped: time budget of the run"
        else:
            try:
                if self.is_spmm:
                    rp = ref.prepare_spmm_csr_opt(d, i, p, self.shape)
                    fn = lambda: ref.flagsparse_spmm_csr_opt(B=self.dense, prepared=rp)  # noqa: E731
                else:
                    rp = ref.prepare_spmv_csr(d, i, p, self.shape)
                    fn = lambda: ref.flagsparse_spmv_csr(x=self.dense, prepared=rp, use_opt=True)  # noqa: E731
                out["ref_triton_opt_ms"] = event_time_ms(torch, fn, 3, 10)
                del rp
            except Exception as e:  # noqa: BLE001
                out["ref_triton_opt_ms"] = f"unavailable: {type(e).__name__}: {str(e)[:80]}"
        torch.cuda.empty_cache()
        return out

    def release(self):
        for name in ("csr", "dense", "prep", "out", "step", "api_call", "one_shot"):
            setattr(self, name, None)
        self.torch.cuda.empty_cache()


def run_others(torch, device, peak, ref, skip, deadline):
    """Every other configuration, briefly: device time (median of single calls), fraction of the roofline,
    in-run parity, cuSPARSE and the reference next to it."""
    res = {}
    for w in OTHERS:
        if w == skip:
            continue
        if time.perf_counter() > deadline:
            res[w] = {"skipped": "time budget of the run"}
            continue
        try:
            wl = SingleGpuWorkload(torch, w, device)
            ms = batch_time_ms(torch, wl.step, 10, 50)
            n_blocks, worst = wl.parity()
            tol = TOL[wl.vdt]
            entry = {"ms": ms, "gbs": wl.nbytes / ms / 1e6, "frac": wl.nbytes / ms / 1e6 / peak,
                     "gflops": wl.flops / ms / 1e6, "algorithmic_bytes": wl.nbytes, "kernel": wl.kernel,
                     "prepare_ms": wl.prepare_s * 1e3, "one_shot_ms": event_time_ms(torch, wl.one_shot, 1, 3),
                     "parity": {"blocks": n_blocks, "worst_ratio": worst, "tol": tol, "ok": bool(worst <= tol)}}
            entry.update(wl.compare(ref, max(0.0, deadline - time.perf_counter())))
            res[w] = entry
            wl.release()
        except Exception as e:  # noqa: BLE001 -- keep the headline even if a side measurement breaks
            res[w] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
            torch.cuda.empty_cache()
    return res


def run_single(args, workload, torch, device):
    t_start = time.perf_counter()
    wl = SingleGpuWorkload(torch, workload, device)
    setup_s = time.perf_counter() - t_start
    steps, warm = args.steps, max(args.warmup, 3)
    for _ in range(warm):
        wl.step()
    with ClockSampler(physical_gpu_index(0)) as clocks:
        elapsed = timed_region(torch, wl.step, steps, lambda: None)
        # keep the same load on the GPU until the sampler has seen enough of it (not part of any timing)
        t_more = time.perf_counter()
        while len(clocks.samples) < 12 and time.perf_counter() - t_more < 2.0:
            for _ in range(5):
                wl.step()
            torch.cuda.synchronize()
    # end to end through the public call: host -> device copy of the dense operand, product, device -> host copy
    dense, out = wl.dense, wl.out
    host_in = torch.empty(dense.shape, dtype=dense.dtype).pin_memory()
    host_in.copy_(dense)
    host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    dev_in = torch.empty_like(dense)

    def e2e_step():
        dev_in.copy_(host_in, non_blocking=True)
        r = wl.api_call(dev_in, out)
        host_out.copy_(r, non_blocking=True)

    for _ in range(3):
        e2e_step()
    e2e_serial = timed_region(torch, e2e_step, steps, lambda: None)
    e2e_elapsed = min(e2e_serial, timed_pipeline(torch, wl.api_call, host_in, host_out, steps))
    h2d = dense.numel() * dense.element_size()
    d2h = out.numel() * out.element_size()
    del dev_in, host_in, host_out, dense, out, e2e_step
    n_blocks, worst = wl.parity()
    tol = TOL[wl.vdt]
    per_step = elapsed / steps
    value = wl.nbytes / per_step / 1e9
    peak, peak_kind = measured_peak()
    line = {
        "metric": metric_name(workload), "value": value, "unit": "GB/s", "n_gpus": 1, "steps": steps,
        "warmup": warm, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32" if wl.vdt == "float32" else "f64", "data": "synthetic",
        "config": workload_config(workload, 1),
        "gflops": wl.flops / per_step / 1e9, "nnz": wl.nnz, "algorithmic_bytes": wl.nbytes,
        "frac_of_nominal_8tbs": value / 8000.0,
        "e2e": {"value": wl.nbytes / (e2e_elapsed / steps) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_elapsed / steps * 1e3, "serial_ms_per_step": e2e_serial / steps * 1e3,
                "how": ("copy-in, product and copy-out of consecutive steps overlapped on three streams"
                        if e2e_elapsed < e2e_serial else "copy-in, product, copy-out one after the other")},
        "gpu_launches": wl.launches * steps,
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "achieved": value, "peak": peak, "unit": "GB/s", "frac": value / peak,
                     "traffic": measured_traffic(workload), "peak_source": f"{peak_kind} copy bandwidth per GPU",
                     "per": "GPU, whole step (every kernel of the step)"},
        "parity": {"blocks": n_blocks, "block_rows": PARITY_BLOCK_ROWS, "worst_ratio": worst, "tol": tol,
                   "ranks_equal": True, "ok": bool(worst <= tol)},
        "setup_seconds": setup_s, "generate_ms": wl.generate_s * 1e3, "prepare_ms": wl.prepare_s * 1e3,
        "prepare_in_products": wl.prepare_s / per_step,
    }
    line.update(wl.describe())
    ok = line["parity"]["ok"]
    if not args.no_others:
        ref = load_reference_package()
        deadline = time.perf_counter() + args.others_seconds
        if workload != "c1" and workload not in SPMM_WORKLOADS and wl.nnz < 2**30:
            line["one_shot_ms"] = event_time_ms(torch, wl.one_shot, 1, 3)
        line["compare"] = wl.compare(ref, args.others_seconds / 3)
        wl.release()
        line["others"] = run_others(torch, device, peak, ref, workload, deadline)
        ok = ok and all(v.get("parity", {}).get("ok", True) for v in line["others"].values())
    else:
        wl.release()
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_scipy(workload)
    print(json.dumps(line), flush=True)
    if not ok:
        raise SystemExit("parity check failed: see the `parity` entries of the line above")


def run_sharded(args, workload, torch, device, rank, world):
    import torch.distributed as dist

    import flagsparse_b200 as fs
    from flagsparse_b200 import _lib
    from flagsparse_b200 import synthetic as S

    t_setup = time.perf_counter()
    is_spmm = workload in SPMM_WORKLOADS
    if is_spmm:
        n_dense = SPMM_WORKLOADS[workload]
        spec, vdt, idt, pdt = S.config_spec("c4"), "float32", "int32", "int32"
    else:
        cfg, vdt, idt, pdt = SPMV_WORKLOADS[workload]
        spec = S.config_spec(cfg)
    # every rank derives the row lengths (a pure function of the row index), hence the same partition
    if spec.dedup:
        raise SystemExit("sharded run needs a workload whose row lengths are known up front (c5, c4n*)")
    lens = S.row_lengths(spec, S._ops(device), 0, spec.n_rows)
    gptr = torch.zeros(spec.n_rows + 1, dtype=torch.int64, device=device)
    torch.cumsum(lens, 0, out=gptr[1:])
    bounds = fs.partition_rows_by_nnz(gptr, world)
    nnz = int(gptr[-1])
    marks = list(bounds[1:-1])
    if nnz > 2**31:
        marks.append(int(torch.searchsorted(gptr, torch.tensor([2**31], dtype=torch.int64, device=device))[0]))
    del lens, gptr
    r0, r1 = bounds[rank], bounds[rank + 1]
    d, i, p = S.generate_csr(spec, device, value_dtype=vdt, index_dtype=idt, indptr_dtype=pdt, row_range=(r0, r1))
    extra = {}
    if is_spmm:
        dense = S.dense_vector(spec, spec.n_cols, device, n_dense=n_dense)
        op = fs.ShardedCsrSpmm(d, i, p, r0, (spec.n_rows, spec.n_cols), mode=args.exchange if args.exchange != "fused" else "auto")
        run = op.matmul
        prep0 = op.parts[0][2]
        si, sp_ = prep0.kernel_indices.element_size(), prep0.kernel_indptr.element_size()
        nbytes = spmm_bytes(spec.n_rows, spec.n_cols, nnz, n_dense, d.element_size(), si, sp_)
        flops = 2.0 * nnz * n_dense
        launches = sum(getattr(pp, "launches_per_product", lambda n: 2)(n_dense) for _, _, pp in op.parts)
        extra["kernel"] = prep0.row_buckets[0]["kind"]
        extra["sub_shards"] = len(op.parts)
    else:
        dense = S.dense_vector(spec, spec.n_cols, device, value_dtype=vdt)
        op = fs.ShardedCsrSpmv(d, i, p, r0, (spec.n_rows, spec.n_cols), mode=args.exchange)
        run = op.matvec
        si, sp_ = op.prepared.kernel_indices.element_size(), op.prepared.kernel_indptr.element_size()
        nbytes = spmv_bytes(spec.n_rows, spec.n_cols, nnz, dense.element_size(), si, sp_)
        flops = 2.0 * nnz
        launches = 2 if op.prepared.algo == _lib.FSB_SPMV_STREAM else 1
        if op._slices is not None and op.prepared.algo == _lib.FSB_SPMV_PANEL:
            launches = len(op._slices)
            extra["slices"] = [e - b for b, e, _, _ in op._slices]
        elif getattr(op, "_nccl_chunks", None) is not None:
            launches = sum(1 for b, e in op._nccl_blocks if e > b)
            extra["slices"] = [e - b for b, e in op._nccl_blocks]
        extra["kernel"] = op.prepared.opt_buckets[0]["kind"]
        if op.prepared.panel is not None:
            lay = op.prepared.panel
            extra["panel"] = {"rb_rows": lay.rb_rows, "chunk_cols": lay.chunk_cols, "units": lay.n_units,
                              "rounds": lay.rounds, "row_blocks": lay.n_row_blocks,
                              "x_overhead": round(lay.x_overhead, 3), "slot_overhead": round(lay.slot_overhead, 3)}
    extra["exchange"] = op.mode
    extra["shard_nnz"] = d.numel()
    step = lambda: run(dense)  # noqa: E731
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t_setup

    def barrier():
        dist.barrier()

    steps, warm = args.steps, max(args.warmup, 3)
    for _ in range(warm):
        step()
    with ClockSampler(physical_gpu_index(int(os.environ.get("LOCAL_RANK", "0")))) as clocks:
        elapsed = timed_region(torch, step, steps, barrier)
        # keep the same load on the GPU until the sampler has seen enough of it (not part of any timing).  Every
        # sharded step holds a collective, so all ranks must run the SAME number of extra steps: derive it from
        # the slowest rank's step time, never from a rank's own clock or sampler
        t = torch.tensor([elapsed], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        slowest = max(float(t[0]) / steps, 1e-6)
        for _ in range(int(min(2000, max(20, 0.3 / slowest)))):
            step()
        torch.cuda.synchronize()

    # end to end: every rank uploads 1/world of the dense operand from pinned host memory, the slices are
    # all-gathered over NVLink, then the product, then every rank reads its own rows of the result back
    width = n_dense if is_spmm else 1
    n_in = dense.shape[0]
    per = -(-n_in // world)
    padded = per * world
    host_in = torch.empty((per,) + tuple(dense.shape[1:]), dtype=dense.dtype).pin_memory()
    lo, hi = min(n_in, rank * per), min(n_in, (rank + 1) * per)
    host_in.zero_()
    host_in[:hi - lo].copy_(dense[lo:hi])
    dev_slice = torch.empty_like(host_in, device=device)
    dev_full = torch.empty((padded,) + tuple(dense.shape[1:]), dtype=dense.dtype, device=device)
    host_out = torch.empty((r1 - r0,) + ((n_dense,) if is_spmm else ()), dtype=dense.dtype).pin_memory()

    def e2e_step():
        dev_slice.copy_(host_in, non_blocking=True)
        dist.all_gather_into_tensor(dev_full, dev_slice)
        res = run(dev_full[:n_in])
        host_out.copy_(res[r0:r1], non_blocking=True)

    for _ in range(3):
        e2e_step()
    e2e_serial = timed_region(torch, e2e_step, steps, barrier)
    lag = 2 if op.mode in ("peer", "fused") else 1
    e2e_piped = timed_pipeline_sharded(torch, dist, run, host_in, host_out, dev_full, n_in, r0, r1, steps, barrier, lag)

    # parity: rank 0's assembled result against host-regenerated blocks; every rank's result against rank 0's
    res = run(dense).clone()
    torch.cuda.synchronize()
    theirs = res.clone()
    dist.broadcast(theirs, src=0)
    same = torch.tensor([1 if torch.equal(theirs, res) else 0], dtype=torch.int32, device=device)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    del theirs
    t = torch.tensor([elapsed, e2e_serial, e2e_piped], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed, e2e_serial, e2e_piped = float(t[0]), float(t[1]), float(t[2])
    e2e_elapsed = min(e2e_serial, e2e_piped)
    per_step = elapsed / steps
    value = nbytes / per_step / 1e9
    peak, peak_kind = measured_peak()
    ok = True
    if rank == 0:
        blocks = parity_blocks(spec.n_rows, marks, extra=2)
        if is_spmm:
            blocks = blocks[:6]
        worst = check_blocks(workload, res, dense.cpu().numpy(), blocks)
        tol = TOL[vdt]
        ok = bool(worst <= tol) and bool(int(same[0]) == 1)
        line = {
            "metric": metric_name(workload), "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
            "warmup": warm, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32" if vdt == "float32" else "f64", "data": "synthetic",
            "config": workload_config(workload, world),
            "gflops": flops / per_step / 1e9, "nnz": nnz, "algorithmic_bytes": nbytes,
            "frac_of_nominal_8tbs": value / (8000.0 * world),
            "e2e": {"value": nbytes / (e2e_elapsed / steps) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": host_in.numel() * host_in.element_size() * world,
                    "d2h_bytes_per_step": spec.n_rows * width * dense.element_size(),
                    "ms_per_step": e2e_elapsed / steps * 1e3, "serial_ms_per_step": e2e_serial / steps * 1e3,
                    "how": "each rank uploads 1/N of the dense operand, NCCL all-gather, product with the exchange, "
                           "each rank reads back its own rows"
                           + ("; upload, product and read-back of consecutive steps overlapped on three streams"
                              if e2e_piped < e2e_serial else "; one after the other")},
            "gpu_launches": launches * steps,
            "clocks": clocks.summary(),
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s",
                         "frac": value / world / peak, "traffic": None,
                         "peak_source": f"{peak_kind} copy bandwidth per GPU",
                         "per": "GPU, whole step (every kernel of the step and the exchange)"},
            "parity": {"blocks": len(blocks), "block_rows": PARITY_BLOCK_ROWS, "worst_ratio": worst, "tol": tol,
                       "ranks_equal": bool(int(same[0]) == 1), "ok": ok},
            "setup_seconds": setup_s,
        }
        line.update(extra)
        print(json.dumps(line), flush=True)
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    dist.broadcast(flag, src=0)
    dist.barrier()
    if int(flag[0]) != 1:
        raise SystemExit("parity check failed: see the `parity` entry of rank 0's line")


def run_ours(args, workload):
    import torch

    from flagsparse_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the package has no CPU path")
    _lib.lib()  # fail loudly if libfsb.so is missing
    torch.cuda.set_device(local_rank)
    device = f"cuda:{local_rank}"
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if world == 1:
        run_single(args, workload, torch, device)
        return
    import torch.distributed as dist

    # a rank that never reaches a collective ends the run after three minutes instead of ten
    dist.init_process_group("nccl", device_id=torch.device(device), timeout=datetime.timedelta(seconds=180))
    try:
        run_sharded(args, workload, torch, device, rank, world)
    finally:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", default="auto", choices=["auto"] + sorted(SPMV_WORKLOADS) + sorted(SPMM_WORKLOADS))
    ap.add_argument("--exchange", default="auto", choices=("auto", "nccl", "peer", "fused"),
                    help="how a sharded run assembles the result: NCCL all-gather, slices pushed by the copy engines "
                         "while the next slice is computed, or peer stores fused into the kernel")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-others", action="store_true",
                    help="single GPU: skip the other configurations and the cuSPARSE / reference columns")
    ap.add_argument("--others-seconds", type=float, default=240.0,
                    help="time budget of the side measurements (what does not fit is reported as skipped)")
    ap.add_argument("--cpu-rows-log2", type=int, default=None, help="--impl reference: rows of the timed sample")
    args = ap.parse_args()
    workload = args.workload
    if workload == "auto":
        workload = "c5"
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            run_reference_arm(args, workload)
        return
    run_ours(args, workload)


if __name__ == "__main__":
    main()
