"""Comparison on one GPU: this package vs cuSPARSE (through torch.sparse) vs the reference's Triton kernels.

    python -m flagsparse_b200.compare_bench [c1 c2 c2f64 c3 c4] [--reference-path DIR] [--out FILE]

For every workload: CUDA events, 10 warm-ups + 50 timed calls (the reference: 3 + 10, its base paths 2 + 5, which
take milliseconds per call), prepared matrices resident, the same seeded inputs for every implementation (the
generators of flagsparse_b200.synthetic).  The reference is imported from --reference-path (an installed copy of the
unmodified package; its columns are skipped when it cannot be imported).  Prints a markdown table per workload:
median and minimum milliseconds, GB/s of algorithmic bytes, GFLOP/s, fraction of the measured copy bandwidth.
"""

import argparse
import os
import statistics
import sys
import time

import torch

import flagsparse_b200 as fs
from flagsparse_b200 import synthetic as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _peak_gbs():
    """Measured copy bandwidth (GB/s) from MEASURED_PEAKS.json at the repository root; 6650 when the file is absent
    (an earlier measurement on the same kind of GPU).  Only the last column of the table depends on it."""
    import json

    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"])
    except (OSError, KeyError, ValueError, TypeError):
        return 6650.0


PEAK_GBS = _peak_gbs()


class Report:
    def __init__(self, path):
        self.lines, self.path = [], path

    def log(self, *parts):
        s = " ".join(str(x) for x in parts)
        print(s, flush=True)
        self.lines.append(s)
        if self.path:
            with open(self.path, "w") as f:
                f.write("\n".join(self.lines) + "\n")


def timeit(fn, warm=10, iters=50):
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
    return statistics.median(ts), min(ts)


def row(rep, label, fn, nbytes, flops, **kw):
    try:
        med, mn = timeit(fn, **kw)
        rep.log(f"| {label} | {med:.4f} | {mn:.4f} | {nbytes / med / 1e6:.0f} | {flops / med / 1e6:.0f} | "
                f"{nbytes / med / 1e6 / PEAK_GBS:.3f} |")
    except Exception as e:  # one implementation failing must not lose the others' rows
        rep.log(f"| {label} | failed: {type(e).__name__}: {str(e)[:120]} | | | | |")


def _torch_csr(d, i, p, shape):
    # torch wants both index arrays of one integer type
    return torch.sparse_csr_tensor(p.to(torch.int64), i.to(torch.int64), d, size=shape)


def spmv_case(rep, ref, name, spec, vdt, idt, pdt, base=True):
    d, i, p = S.generate_csr(spec, "cuda", value_dtype=vdt, index_dtype=idt, indptr_dtype=pdt)
    x = S.dense_vector(spec, spec.n_cols, "cuda", value_dtype=vdt)
    nnz, shape, sv = d.numel(), (spec.n_rows, spec.n_cols), d.element_size()
    prep = fs.prepare_spmv_csr(d, i, p, shape)
    si, sp = prep.kernel_indices.element_size(), prep.kernel_indptr.element_size()
    nbytes = nnz * (sv + si) + (spec.n_rows + 1) * sp + spec.n_cols * sv + spec.n_rows * sv
    rep.log(f"\n### {name}: rows {spec.n_rows}, nnz {nnz}, algorithmic bytes (as streamed) {nbytes / 1e9:.3f} GB")
    rep.log("| implementation | median ms | min ms | GB/s | GFLOP/s | of %.1f GB/s |" % PEAK_GBS)
    rep.log("|---|---|---|---|---|---|")
    out = torch.empty(spec.n_rows, dtype=d.dtype, device="cuda")
    row(rep, f"ours ({prep.opt_buckets[0]['kind']})", lambda: fs.flagsparse_spmv_csr(x=x, prepared=prep, out=out),
        nbytes, 2.0 * nnz)
    try:
        A = _torch_csr(d, i, p, shape)
        row(rep, "cuSPARSE via torch (A @ x)", lambda: torch.mv(A, x), nbytes, 2.0 * nnz)
        del A
    except Exception as e:
        rep.log(f"| cuSPARSE | failed {repr(e)[:100]} | | | | |")
    if ref is not None:
        try:
            rp = ref.prepare_spmv_csr(d, i, p, shape)
            row(rep, "reference Triton, use_opt=True", lambda: ref.flagsparse_spmv_csr(x=x, prepared=rp, use_opt=True),
                nbytes, 2.0 * nnz, warm=3, iters=10)
            if base:
                row(rep, "reference Triton, default (base path)", lambda: ref.flagsparse_spmv_csr(x=x, prepared=rp),
                    nbytes, 2.0 * nnz, warm=2, iters=5)
            del rp
        except Exception as e:
            rep.log(f"| reference | failed {repr(e)[:160]} | | | | |")
    del d, i, p, x, prep
    torch.cuda.empty_cache()


def spmm_case(rep, ref, n_dense):
    spec = S.config_spec("c4")
    d, i, p = S.generate_csr(spec, "cuda")
    B = S.dense_vector(spec, spec.n_cols, "cuda", n_dense=n_dense)
    nnz, shape = d.numel(), (spec.n_rows, spec.n_cols)
    nbytes = nnz * 8 + (spec.n_rows + 1) * 4 + 2 * spec.n_rows * n_dense * 4
    gather = nnz * 8 + nnz * n_dense * 4 + spec.n_rows * n_dense * 4
    rep.log(f"\n### c4 SpMM N={n_dense}: nnz {nnz}, compulsory bytes {nbytes / 1e9:.3f} GB "
            f"(gather model {gather / 1e9:.2f} GB)")
    rep.log("| implementation | median ms | min ms | GB/s (compulsory) | GFLOP/s | of %.1f GB/s |" % PEAK_GBS)
    rep.log("|---|---|---|---|---|---|")
    out = torch.empty((spec.n_rows, n_dense), dtype=d.dtype, device="cuda")
    prep = fs.prepare_spmm_csr_opt(d, i, p, shape)
    flops = 2.0 * nnz * n_dense
    row(rep, "ours", lambda: fs.flagsparse_spmm_csr_opt(B=B, prepared=prep, out=out), nbytes, flops)
    try:
        A = _torch_csr(d, i, p, shape)
        row(rep, "cuSPARSE via torch.sparse.mm", lambda: torch.sparse.mm(A, B), nbytes, flops, warm=5, iters=20)
        del A
    except Exception as e:
        rep.log(f"| cuSPARSE | failed {repr(e)[:100]} | | | | |")
    if ref is not None:
        try:
            rp = ref.prepare_spmm_csr_opt(d, i, p, shape)
            row(rep, "reference Triton opt", lambda: ref.flagsparse_spmm_csr_opt(B=B, prepared=rp), nbytes, flops,
                warm=3, iters=10)
            row(rep, "reference Triton base", lambda: ref.flagsparse_spmm_csr(d, i, p, B, shape), nbytes, flops,
                warm=2, iters=5)
        except Exception as e:
            rep.log(f"| reference | failed {repr(e)[:160]} | | | | |")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("workloads", nargs="*", default=["c1", "c2", "c2f64", "c3", "c4"])
    ap.add_argument("--reference-path", default=os.path.join(ROOT, "baseline", "_ref"),
                    help="directory that holds an installed copy of the reference package")
    ap.add_argument("--out", default=None, help="also write the tables to this file")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("compare_bench needs a CUDA device")
    rep = Report(args.out)
    ref = None
    try:
        sys.path.insert(0, args.reference_path)
        import flagsparse as ref
    except Exception as e:
        rep.log("reference import failed:", repr(e))
    rep.log("# comparison on", torch.cuda.get_device_name(0), time.strftime("%F %T"))
    for w in args.workloads:
        t0 = time.time()
        if w == "c1":
            spmv_case(rep, ref, "C1 SpMV 4096^2, 16/row, f32/i32", S.config_spec("c1"), "float32", "int32", "int32")
        elif w == "c2":
            spmv_case(rep, ref, "C2 SpMV f32/i32", S.config_spec("c2"), "float32", "int32", "int32")
        elif w == "c2f64":
            spmv_case(rep, ref, "C2 SpMV f64/i64", S.config_spec("c2"), "float64", "int64", "int64")
        elif w == "c3":
            spmv_case(rep, ref, "C3 SpMV power-law f32/i32", S.config_spec("c3"), "float32", "int32", "int32", base=False)
        elif w == "c4":
            for n in (32, 64, 128):
                spmm_case(rep, ref, n)
        else:
            raise SystemExit(f"unknown workload {w!r}")
        rep.log(f"({w}: {time.time() - t0:.0f} s)")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
