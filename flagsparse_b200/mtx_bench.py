"""SpMV over a batch of Matrix Market files: time, check, print a table, export CSV.

The counterpart of the reference's real-matrix workflow (tests/test_spmv.py of the reference: run_one_mtx
:106-383, run_mtx_batch :386-410, the table printer :413-471, run_all_dtypes_export_csv :474-520): every file is
loaded with load_mtx_to_csr_torch, multiplied through the prepared entry point (`warmup` untimed + `iters` timed
calls between CUDA events), compared with a float64 product of the same matrix (the reference's recipe for
float32: compute in float64, cast back), and timed against cuSPARSE through torch.sparse.  The reference's CuPy
and CSC columns are not reproduced (no CuPy here).

    python -m flagsparse_b200.mtx_bench a.mtx b.mtx --csv out.csv [--dtype float64] [--index-dtype int64]
"""

import argparse
import csv
import os
import time

import torch

from .mtx import load_mtx_to_csr_torch

CSV_FIELDS = ["matrix", "value_dtype", "index_dtype", "n_rows", "n_cols", "nnz", "kernel", "flagsparse_ms",
              "cusparse_ms", "speedup_vs_cusparse", "err", "status"]
# |y - y_ref| <= tol * (|A| |x|) per row, the bound the kernels are held to everywhere else
TOLERANCE = {torch.float32: 1e-5, torch.float64: 1e-13}


def _time_calls(fn, warmup, iters, device):
    """Milliseconds per call: CUDA events on the current stream (perf_counter for a CPU stand-in in tests)."""
    for _ in range(warmup):
        fn()
    if device.type == "cuda":
        torch.cuda.synchronize(device)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(iters):
            fn()
        end.record()
        torch.cuda.synchronize(device)
        return start.elapsed_time(end) / max(iters, 1)
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    return (time.perf_counter() - t0) * 1e3 / max(iters, 1)


def _reference_product(data, indices, indptr, x, shape):
    """(A x, |A| |x|) in float64 on the matrix's device, row by row sums through index_add."""
    n_rows = shape[0]
    rows = torch.repeat_interleave(torch.arange(n_rows, device=data.device), (indptr[1:] - indptr[:-1]).to(torch.int64))
    prod = data.to(torch.float64) * x.to(torch.float64)[indices.to(torch.int64)]
    y = torch.zeros(n_rows, dtype=torch.float64, device=data.device).index_add_(0, rows, prod)
    mag = torch.zeros(n_rows, dtype=torch.float64, device=data.device).index_add_(0, rows, prod.abs())
    return y, mag


def run_one_mtx(path, value_dtype=torch.float32, index_dtype=torch.int32, warmup=10, iters=50, run_cusparse=True,
                device=None, prepare=None, product=None):
    """One file -> result dict.  `prepare` / `product` default to prepare_spmv_csr / flagsparse_spmv_csr; tests
    substitute CPU stand-ins to exercise the bookkeeping without a GPU."""
    if prepare is None or product is None:
        from .spmv_csr import flagsparse_spmv_csr, prepare_spmv_csr

        prepare = prepare or prepare_spmv_csr
        product = product or (lambda prepared, x: flagsparse_spmv_csr(x=x, prepared=prepared))
    if device is None:
        device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    device = torch.device(device)
    data, indices, indptr, shape = load_mtx_to_csr_torch(path, dtype=value_dtype, device=device)
    indices = indices.to(index_dtype)
    nnz = int(data.numel())
    result = {"path": path, "shape": shape, "nnz": nnz, "value_dtype": value_dtype, "index_dtype": index_dtype,
              "kernel": None, "flagsparse_ms": None, "cusparse_ms": None, "err": None, "status": "FAIL", "error": None}
    gen = torch.Generator(device="cpu").manual_seed(nnz + shape[0])
    x = (torch.rand(shape[1], generator=gen, dtype=torch.float64) * 2 - 1).to(value_dtype).to(device)
    try:
        prepared = prepare(data, indices, indptr, shape)
        buckets = getattr(prepared, "opt_buckets", None)
        result["kernel"] = buckets[0]["kind"] if buckets else None
        y = product(prepared, x)
        result["flagsparse_ms"] = _time_calls(lambda: product(prepared, x), warmup, iters, device)
    except Exception as exc:  # a file the entry point refuses is reported, the batch goes on
        result["error"] = f"{type(exc).__name__}: {exc}"
        result["status"] = "ERROR"
        return result
    y_ref, mag = _reference_product(data, indices, indptr, x, shape)
    if shape[0] > 0:
        bound = torch.clamp(mag, min=torch.finfo(torch.float64).tiny)
        result["err"] = float(((y.to(torch.float64) - y_ref).abs() / bound).max().item()) if nnz else \
            float(y.abs().max().item())
    else:
        result["err"] = 0.0
    tol = TOLERANCE[value_dtype] if nnz else 0.0
    result["status"] = "PASS" if result["err"] <= tol and y.dtype == value_dtype and tuple(y.shape) == (shape[0],) \
        else "FAIL"
    if run_cusparse and device.type == "cuda" and nnz > 0:
        try:
            csr = torch.sparse_csr_tensor(indptr.to(torch.int64), indices.to(torch.int64), data, size=shape)
            result["cusparse_ms"] = _time_calls(lambda: torch.mv(csr, x), warmup, iters, device)
        except Exception:
            result["cusparse_ms"] = None
    return result


def run_mtx_batch(mtx_paths, value_dtype=torch.float32, index_dtype=torch.int32, warmup=10, iters=50, run_cusparse=True,
                  on_result=None, **kw):
    """Every file in turn; returns the list of result dicts (reference: run_mtx_batch, tests/test_spmv.py:386-410)."""
    results = []
    for path in mtx_paths:
        r = run_one_mtx(path, value_dtype=value_dtype, index_dtype=index_dtype, warmup=warmup, iters=iters,
                        run_cusparse=run_cusparse, **kw)
        results.append(r)
        if on_result is not None:
            on_result(r)
    return results


def _dtype_name(dtype):
    return str(dtype).replace("torch.", "")


def _fmt(v, spec):
    return "N/A" if v is None else format(v, spec)


def result_row(r):
    fs_ms, cu_ms = r.get("flagsparse_ms"), r.get("cusparse_ms")
    return {
        "matrix": os.path.basename(r["path"]), "value_dtype": _dtype_name(r["value_dtype"]),
        "index_dtype": _dtype_name(r["index_dtype"]), "n_rows": r["shape"][0], "n_cols": r["shape"][1],
        "nnz": r["nnz"], "kernel": r.get("kernel"), "flagsparse_ms": fs_ms, "cusparse_ms": cu_ms,
        "speedup_vs_cusparse": (cu_ms / fs_ms) if fs_ms and cu_ms else None, "err": r.get("err"),
        "status": r["status"] if not r.get("error") else f"{r['status']}: {r['error']}",
    }


def print_mtx_header():
    print(f"{'Matrix':<28} {'N_rows':>9} {'N_cols':>9} {'NNZ':>11} {'ours(ms)':>10} {'cuSPARSE(ms)':>13} {'speedup':>8} "
          f"{'err/bound':>10} {'status':>7}  kernel")
    print("-" * 128)


def print_mtx_row(r):
    row = result_row(r)
    print(f"{row['matrix'][:28]:<28} {row['n_rows']:>9} {row['n_cols']:>9} {row['nnz']:>11} "
          f"{_fmt(row['flagsparse_ms'], '.4f'):>10} {_fmt(row['cusparse_ms'], '.4f'):>13} "
          f"{_fmt(row['speedup_vs_cusparse'], '.2f'):>8} {_fmt(row['err'], '.2e'):>10} {row['status'][:7]:>7}  "
          f"{row['kernel'] or ''}")


def export_csv(results, csv_path):
    """One line per result (reference: run_all_dtypes_export_csv, tests/test_spmv.py:474-520)."""
    with open(csv_path, "w", newline="", encoding="utf-8") as f:
        w = csv.DictWriter(f, fieldnames=CSV_FIELDS, extrasaction="ignore")
        w.writeheader()
        for r in results:
            w.writerow({k: ("" if v is None else v) for k, v in result_row(r).items()})
    return len(results)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("paths", nargs="+", help=".mtx files")
    ap.add_argument("--csv", default=None, help="write the results to this CSV file")
    ap.add_argument("--dtype", choices=("float32", "float64", "all"), default="float32")
    ap.add_argument("--index-dtype", choices=("int32", "int64", "all"), default="int32")
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--no-cusparse", action="store_true")
    args = ap.parse_args(argv)
    vdts = [torch.float32, torch.float64] if args.dtype == "all" else [getattr(torch, args.dtype)]
    idts = [torch.int32, torch.int64] if args.index_dtype == "all" else [getattr(torch, args.index_dtype)]
    results = []
    for vdt in vdts:
        for idt in idts:
            print(f"Value dtype: {_dtype_name(vdt)}  |  Index dtype: {_dtype_name(idt)}")
            print_mtx_header()
            results += run_mtx_batch(args.paths, value_dtype=vdt, index_dtype=idt, warmup=args.warmup, iters=args.iters,
                                     run_cusparse=not args.no_cusparse, on_result=print_mtx_row)
            print("-" * 128)
    if args.csv:
        print(f"Wrote {export_csv(results, args.csv)} rows to {args.csv}")
    return 0 if all(r["status"] == "PASS" for r in results) else 1


if __name__ == "__main__":
    raise SystemExit(main())
