#!/usr/bin/env python
"""Benchmark of the CSR SpMV / SpMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one product over the whole matrix of the workload, with the prepared matrix resident in HBM
(the steady state the reference's scripts time).  Rank 0 prints ONE JSON line.

Workloads (all synthetic, seeded; see flagsparse_b200/synthetic.py):
  c2       SpMV, 2^22 rows, Poisson(32) rows, band +-2^16, float32 / int32      (default at --gpus 1)
  c2f64    the same matrix in float64 / int64
  c1, c3   SpMV 4096^2 with 16 nnz per row; SpMV 2^24 rows with Zipf(2) row lengths
  c4n32, c4n64, c4n128   SpMM, 2^20 rows x 16 nnz, dense width 32 / 64 / 128
  c5       SpMV, 2^26 rows, Poisson(32), band +-2^20, int64 indptr; row-sharded over the ranks when
           launched under torchrun (default at --gpus N > 1; strong scaling: the matrix is fixed)
`value` is algorithmic bytes / device time in GB/s: A once (values + indices + indptr), x (or B) once, y (or
C) once, with the byte widths the kernels actually stream (never more than the caller's widths).
"""

import argparse
import datetime
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
# dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel per launch, from the ncu captures
# summarised under profiles/ (None until a capture exists for the workload)
NCU_TRAFFIC_BYTES = {
    "c2": 1.102e9,      # profiles/spmv_panel_c2_f32.md
    "c2f64": 1.678e9,   # profiles/spmv_panel_c2_f64.md
    "c3": 2.950e9,      # profiles/spmv_panel_groups_c3_f32.md: stream kernel on the short rows + row-group panel kernel
    "c4n32": 1.290e9,   # profiles/spmm_tile_c4_f32.md
    "c4n128": 7.951e9,  # profiles/spmm_tile_c4_f32.md
}

SPMV_WORKLOADS = {
    "c1": ("c1", "float32", "int32", "int32"),
    "c2": ("c2", "float32", "int32", "int32"),
    "c2f64": ("c2", "float64", "int64", "int64"),
    "c3": ("c3", "float32", "int32", "int32"),
    "c5": ("c5", "float32", "int32", "int64"),
}
SPMM_WORKLOADS = {"c4n32": 32, "c4n64": 64, "c4n128": 128}


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
def cpu_sample(workload, rows_log2=19):
    """A bounded slice of the workload regenerated on the host: the first 2^rows_log2 rows, full x / B."""
    from flagsparse_b200 import synthetic as S

    if workload in SPMM_WORKLOADS:
        spec = S.config_spec("c4")
        rows = min(spec.n_rows, 1 << 17)
        d, i, p = S.generate_csr(spec, None, row_range=(0, rows))
        dense = S.dense_vector(spec, spec.n_cols, n_dense=SPMM_WORKLOADS[workload])
        return spec, rows, (d, i, p), dense, f"rows [0, {rows}) of {spec.n_rows}, B full"
    cfg, vdt, idt, pdt = SPMV_WORKLOADS[workload]
    spec = S.config_spec(cfg)
    rows = min(spec.n_rows, 1 << rows_log2)
    d, i, p = S.generate_csr(spec, None, value_dtype=vdt, index_dtype=idt, indptr_dtype=pdt, row_range=(0, rows))
    dense = S.dense_vector(spec, spec.n_cols, value_dtype=vdt)
    return spec, rows, (d, i, p), dense, f"rows [0, {rows}) of {spec.n_rows}, x full"


def sample_bytes(workload, spec, rows, csr):
    """Algorithmic bytes of a row slice: its part of A and of the output, and the part of x / B it can
    touch (all of it for uniform columns, the same fraction as the rows for a banded matrix)."""
    d, i, p = csr
    dense_rows = spec.n_cols if spec.columns[0] != "band" else max(1, spec.n_cols * rows // spec.n_rows)
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


def cpu_baseline_scipy(workload):
    """scipy.sparse (single-threaded CSR kernels) in the input dtype on a bounded sample -- the oracle's
    arithmetic, timed on one host core."""
    import scipy.sparse as sp

    spec, rows, (d, i, p), dense, what = cpu_sample(workload)
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
    spec, rows, (d, i, p), dense, what = cpu_sample(workload)
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
        cfg["parallelism"] = f"rows sharded by nnz over {n_gpus} GPUs, x replicated, y assembled on every GPU"
    return cfg


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


def run_ours(args, workload):
    import torch
    import torch.distributed as dist

    import flagsparse_b200 as fs
    from flagsparse_b200 import _lib
    from flagsparse_b200 import synthetic as S

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the package has no CPU path")
    _lib.lib()  # fail loudly if libfsb.so is missing
    torch.cuda.set_device(local_rank)
    device = f"cuda:{local_rank}"
    if world > 1:
        # a rank that never reaches a collective ends the run after three minutes instead of ten
        dist.init_process_group("nccl", device_id=torch.device(device), timeout=datetime.timedelta(seconds=180))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")

    def barrier():
        if world > 1:
            dist.barrier()

    t_setup = time.perf_counter()
    is_spmm = workload in SPMM_WORKLOADS
    launches_per_step = 2
    if is_spmm:
        n_dense = SPMM_WORKLOADS[workload]
        spec = S.config_spec("c4")
        d, i, p = S.generate_csr(spec, device)
        dense = S.dense_vector(spec, spec.n_cols, device, n_dense=n_dense)
        prep = fs.prepare_spmm_csr_opt(d, i, p, (spec.n_rows, spec.n_cols))
        out = torch.empty((spec.n_rows, n_dense), dtype=d.dtype, device=device)
        step = lambda: fs.flagsparse_spmm_csr_opt(B=dense, prepared=prep, out=out)  # noqa: E731
        nnz = d.numel()
        nbytes = spmm_bytes(spec.n_rows, spec.n_cols, nnz, n_dense, d.element_size(),
                            prep.kernel_indices.element_size(), prep.kernel_indptr.element_size())
        flops = 2.0 * nnz * n_dense
        extra = {"bytes_gather_model": nnz * (d.element_size() + 4) + nnz * n_dense * d.element_size()
                 + spec.n_rows * n_dense * d.element_size()}
        h2d, d2h = dense.numel() * dense.element_size(), out.numel() * out.element_size()
        host_in = torch.empty(dense.shape, dtype=dense.dtype).pin_memory()
        host_in.copy_(dense)
        host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        dev_in = torch.empty_like(dense)

        def e2e_step():
            dev_in.copy_(host_in, non_blocking=True)
            c = fs.flagsparse_spmm_csr_opt(B=dev_in, prepared=prep, out=out)
            host_out.copy_(c, non_blocking=True)

        api_call = lambda di, do: fs.flagsparse_spmm_csr_opt(B=di, prepared=prep, out=do)  # noqa: E731
    else:
        cfg, vdt, idt, pdt = SPMV_WORKLOADS[workload]
        spec = S.config_spec(cfg)
        x = S.dense_vector(spec, spec.n_cols, device, value_dtype=vdt)
        extra = {}
        if world == 1:
            d, i, p = S.generate_csr(spec, device, value_dtype=vdt, index_dtype=idt, indptr_dtype=pdt)
            prep = fs.prepare_spmv_csr(d, i, p, (spec.n_rows, spec.n_cols))
            out = torch.empty(spec.n_rows, dtype=d.dtype, device=device)
            step = lambda: fs.flagsparse_spmv_csr(x=x, prepared=prep, out=out)  # noqa: E731
            nnz = d.numel()
            launches_per_step = 2 if prep.algo == _lib.FSB_SPMV_STREAM else 1
            if prep.long_rows is not None:
                # short rows (stream kernel + fix-up, or one vector kernel), then the long-row panel kernel + its reduction
                short, lay = prep.long_rows
                launches_per_step = (2 if short.algo == _lib.FSB_SPMV_STREAM and short.tile_row is not None else 1) + 2
                extra["long_rows"] = {"rows": lay.n_long, "nnz": lay.nnz, "groups": lay.n_groups, "ctas": lay.n_ctas,
                                      "units": lay.n_units, "x_overhead": round(lay.x_overhead, 3),
                                      "slot_overhead": round(lay.slot_overhead, 3), "layout_bytes": lay.nbytes(),
                                      "short_nnz": short.data.numel()}
            si, sp_ = prep.kernel_indices.element_size(), prep.kernel_indptr.element_size()
            extra["kernel"] = prep.opt_buckets[0]["kind"]
            if prep.panel is not None:
                # bytes the panel kernel streams: entries (with padding), unit tables, x chunks, y
                lay = prep.panel
                extra["panel"] = {"rb_rows": lay.rb_rows, "chunk_cols": lay.chunk_cols, "units": lay.n_units,
                                  "x_overhead": round(lay.x_overhead, 3), "slot_overhead": round(lay.slot_overhead, 3),
                                  "layout_bytes": lay.nbytes()}
            my_rows = (0, spec.n_rows)
            run_y = lambda xv: fs.flagsparse_spmv_csr(x=xv, prepared=prep, out=out)  # noqa: E731
            api_call = lambda di, do: fs.flagsparse_spmv_csr(x=di, prepared=prep, out=do)  # noqa: E731
        else:
            # every rank derives the row lengths (a pure function of the row index), hence the same partition
            if spec.dedup:
                raise SystemExit("sharded run needs a workload whose row lengths are known up front (c5)")
            lens = S.row_lengths(spec, S._ops(device), 0, spec.n_rows)
            gptr = torch.zeros(spec.n_rows + 1, dtype=torch.int64, device=device)
            torch.cumsum(lens, 0, out=gptr[1:])
            bounds = fs.partition_rows_by_nnz(gptr, world)
            nnz = int(gptr[-1])
            del lens
            r0, r1 = bounds[rank], bounds[rank + 1]
            del gptr
            d, i, p = S.generate_csr(spec, device, value_dtype=vdt, index_dtype=idt, indptr_dtype=pdt, row_range=(r0, r1))
            op = fs.ShardedCsrSpmv(d, i, p, r0, (spec.n_rows, spec.n_cols), mode=args.exchange)
            step = lambda: op.matvec(x)  # noqa: E731
            # stream kernel + fix-up, or one vector / panel kernel (the barrier / NCCL kernels are not ours)
            launches_per_step = 2 if op.prepared.algo == _lib.FSB_SPMV_STREAM else 1
            extra["kernel"] = op.prepared.opt_buckets[0]["kind"]
            si, sp_ = op.prepared.kernel_indices.element_size(), op.prepared.kernel_indptr.element_size()
            extra["exchange"] = op.mode
            extra["shard_nnz"] = d.numel()
            my_rows = (r0, r1)
            run_y = op.matvec
        sv = x.element_size()
        nbytes = spmv_bytes(spec.n_rows, spec.n_cols, nnz, sv, si, sp_)
        flops = 2.0 * nnz
        h2d = x.numel() * sv * world
        d2h = spec.n_rows * sv
        host_in = torch.empty(x.shape, dtype=x.dtype).pin_memory()
        host_in.copy_(x)
        host_out = torch.empty(my_rows[1] - my_rows[0], dtype=x.dtype).pin_memory()
        dev_in = torch.empty_like(x)

        def e2e_step():
            dev_in.copy_(host_in, non_blocking=True)
            y = run_y(dev_in)
            host_out.copy_(y[my_rows[0]:my_rows[1]] if y.numel() != host_out.numel() else y, non_blocking=True)

    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t_setup

    for _ in range(max(args.warmup, 3)):
        step()
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        elapsed = timed_region(torch, step, args.steps, barrier)
        # keep the same load on the GPU until the sampler has seen enough of it (not part of any timing)
        if world > 1:
            # every sharded step holds a collective (the exchange of y), so all ranks must run the SAME number of
            # extra steps: derive it from the slowest rank's step time, never from a rank's own clock or sampler
            t = torch.tensor([elapsed], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            slowest = max(float(t[0]) / args.steps, 1e-6)
            for _ in range(int(min(2000, max(20, 0.3 / slowest)))):
                step()
            torch.cuda.synchronize()
        else:
            t_more = time.perf_counter()
            while len(clocks.samples) < 12 and time.perf_counter() - t_more < 2.0:
                for _ in range(20):
                    step()
                torch.cuda.synchronize()
    for _ in range(3):
        e2e_step()
    e2e_elapsed = timed_region(torch, e2e_step, args.steps, barrier)
    e2e_serial = e2e_elapsed
    if world == 1:
        # the same end-to-end step with copy-in, product and copy-out of consecutive steps overlapped
        e2e_elapsed = min(e2e_serial, timed_pipeline(torch, api_call, host_in, host_out, args.steps))

    if world > 1:
        t = torch.tensor([elapsed, e2e_elapsed], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed, e2e_elapsed = float(t[0]), float(t[1])
        if not args.no_single_gpu_baseline:
            # the strong-scaling reference: the SAME matrix on one GPU (rank 0 alone; the others wait)
            del op, d, i, p, step, run_y
            torch.cuda.empty_cache()
            if rank == 0:
                d, i, p = S.generate_csr(spec, device, value_dtype=vdt, index_dtype=idt, indptr_dtype=pdt)
                prep1 = fs.prepare_spmv_csr(d, i, p, (spec.n_rows, spec.n_cols))
                out1 = torch.empty(spec.n_rows, dtype=d.dtype, device=device)
                step1 = lambda: fs.flagsparse_spmv_csr(x=x, prepared=prep1, out=out1)  # noqa: E731
                for _ in range(3):
                    step1()
                n1 = max(3, min(args.steps, 50))
                t1 = timed_region(torch, step1, n1, lambda: None) / n1
                extra["scaling_reference"] = ("strong scaling of this workload: divide by single_gpu_same_workload "
                                              "(the same matrix on one GPU, timed by rank 0 in this run); the default "
                                              "--gpus 1 run is another workload (c2)")
                extra["single_gpu_same_workload"] = {"ms_per_step": t1 * 1e3, "value": nbytes / t1 / 1e9,
                                                     "unit": "GB/s", "kernel": prep1.opt_buckets[0]["kind"],
                                                     "steps": n1, "speedup_at_n_gpus": t1 / (elapsed / args.steps)}
            dist.barrier()
    per_step = elapsed / args.steps
    value = nbytes / per_step / 1e9
    peak, peak_kind = measured_peak()

    if rank == 0:
        line = {
            "metric": metric_name(workload), "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": per_step * 1e3, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "f32" if d.dtype == torch.float32 else "f64", "data": "synthetic",
            "config": workload_config(workload, world),
            "gflops": flops / per_step / 1e9, "nnz": nnz, "algorithmic_bytes": nbytes,
            "frac_of_nominal_8tbs": value / (8000.0 * world),
            "e2e": {"value": nbytes / (e2e_elapsed / args.steps) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_elapsed / args.steps * 1e3,
                    "serial_ms_per_step": e2e_serial / args.steps * 1e3,
                    "how": ("copy-in, product and copy-out of consecutive steps overlapped on three streams"
                            if e2e_elapsed < e2e_serial else "copy-in, product, copy-out one after the other")},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks.summary(),
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s",
                         "frac": value / world / peak, "traffic": NCU_TRAFFIC_BYTES.get(workload),
                         "peak_source": f"{peak_kind} copy bandwidth per GPU", "per": "GPU, whole step (every kernel of the step)"},
            "setup_seconds": setup_s,
        }
        line.update(extra)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_scipy(workload)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", default="auto", choices=["auto"] + sorted(SPMV_WORKLOADS) + sorted(SPMM_WORKLOADS))
    ap.add_argument("--exchange", default="auto", choices=("auto", "nccl", "peer"),
                    help="how the sharded run assembles y: NCCL all-gather, or peer stores fused into the kernel")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-single-gpu-baseline", action="store_true",
                    help="sharded runs: skip timing the same matrix on one GPU (rank 0) after the sharded measurement")
    args = ap.parse_args()
    workload = args.workload
    if workload == "auto":
        workload = "c2" if args.gpus == 1 else "c5"
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            run_reference_arm(args, workload)
        return
    run_ours(args, workload)


if __name__ == "__main__":
    main()
