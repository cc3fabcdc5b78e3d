"""Generate the golden fixtures of tests/golden/ by running the REFERENCE's own code on small seeded cases.

Run from the repository root, in a container where the reference checkout is available:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --reference /path/to/flagsparse

The reference's public entry points insist on CUDA tensors, so this script calls the functions right
below them -- the same ones the entry points call -- on CPU tensors with Triton's interpreter executing
the reference's @triton.jit kernels:
  SpMV base path  _triton_spmv_csr_impl_prepared      (src/flagsparse/sparse_operations/spmv_csr.py:510-554)
  SpMV opt path   _triton_spmv_csr_impl_opt_prepared  (:329-376) with _build_spmv_opt_buckets (:281-327)
  SpMM base path  _triton_spmm_csr_impl               (src/flagsparse/sparse_operations/spmm_csr.py:525-599)
  SpMM opt path   _run_spmm_opt_bucket / _run_spmm_opt_split_bucket (:922-1030), driven as in :1046-1055
  COO SpMV       _triton_spmv_coo_kernel             (src/flagsparse/sparse_operations/spmv_coo.py:252-289), on
                 a PreparedCoo built as _prepare_coo_tensors (:183-222) builds it, row-run and atomic forms
  COO SpMM       _triton_spmm_coo_impl               (src/flagsparse/sparse_operations/spmm_coo.py:533-570) after
                 _prepare_spmm_coo_canonical_prepared (:78-105), as _run_spmm_coo_route (:626-668) does
plus the pure host helpers (_resolve_spmm_alg1_launch_config, _select_spmm_opt_block_n,
coo_to_csr_for_spmv), and the Matrix Market loader of the reference's benchmark scripts
  load_mtx_to_csr_torch  (tests/test_spmv.py:29-103 and tests/test_spmm.py:163-268 of the reference)
on the small files of tests/golden/mtx/, and the base SpMV / SpMM paths on float16, bfloat16, complex64 and
complex128 values (the same two launch helpers; the reference widens or takes real views there), and
  SDDMM          _sddmm_csr_real_kernel launched as _run_sddmm_prepared launches it
                 (src/flagsparse/sparse_operations/sddmm_csr.py:107-152, 265-347), on a pattern prepared by the
                 same steps as prepare_sddmm_csr (:83-104) without its CUDA check.
`--only coo` / `--only mtx` / `--only wide` / `--only sddmm` regenerate those fixtures alone.  Inputs and outputs are stored together, so the fixtures stay valid even if the
synthetic generator changes.  Nothing here is imported by the package, the tests or the benchmark.
"""

import argparse
import json
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from flagsparse_b200 import synthetic as S  # noqa: E402


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def handmade_csr(seed, row_lens, n_cols, value_dtype, index_dtype, indptr_dtype):
    rng = np.random.default_rng(seed)
    indptr = np.zeros(len(row_lens) + 1, dtype=np.int64)
    indptr[1:] = np.cumsum(row_lens)
    cols = np.concatenate([np.sort(rng.choice(n_cols, size=k, replace=False)) for k in row_lens] or [np.zeros(0)])
    data = rng.uniform(-1, 1, size=int(indptr[-1])).astype(value_dtype)
    return data, cols.astype(index_dtype), indptr.astype(indptr_dtype)


def spmv_cases():
    out = {}
    c1 = S.config_spec("c1").scaled(256)
    out["c1_small"] = (S.generate_csr(c1), (256, 256), S.dense_vector(c1, 256))
    c2 = S.config_spec("c2").scaled(512)
    out["c2_small_f32"] = (S.generate_csr(c2), (512, 512), S.dense_vector(c2, 512))
    out["c2_small_f64_i64"] = (
        S.generate_csr(c2, value_dtype="float64", index_dtype="int64", indptr_dtype="int64"),
        (512, 512), S.dense_vector(c2, 512, value_dtype="float64"))
    c3 = S.config_spec("c3").scaled(2048)
    out["c3_small"] = (S.generate_csr(c3), (2048, 2048), S.dense_vector(c3, 2048))
    lens = [0, 0, 3, 0, 1, 300, 0, 0, 64, 65, 0, 33, 32, 31, 1, 1, 0, 700, 0, 0, 2, 0]
    out["empty_rows_f32"] = (handmade_csr(11, lens, 1024, np.float32, np.int32, np.int32), (len(lens), 1024),
                             np.random.default_rng(12).uniform(-1, 1, 1024).astype(np.float32))
    out["empty_rows_f64"] = (handmade_csr(13, lens, 1024, np.float64, np.int32, np.int64), (len(lens), 1024),
                             np.random.default_rng(14).uniform(-1, 1, 1024).astype(np.float64))
    return out


def spmm_cases():
    out = {}
    c4 = S.config_spec("c4").scaled(192)
    csr = S.generate_csr(c4)
    for n in (5, 12, 32, 64, 128):
        out[f"c4_small_n{n}"] = (csr, (192, 192), S.dense_vector(c4, 192, n_dense=n))
    lens = [1536, 4, 0, 2500, 0, 40, 130, 600]
    out["long_rows_n48"] = (handmade_csr(21, lens, 4096, np.float32, np.int32, np.int64), (len(lens), 4096),
                            np.random.default_rng(22).uniform(-1, 1, (4096, 48)).astype(np.float32))
    out["long_rows_f64_n8"] = (handmade_csr(23, lens, 4096, np.float64, np.int64, np.int64), (len(lens), 4096),
                               np.random.default_rng(24).uniform(-1, 1, (4096, 8)).astype(np.float64))
    return out


def run_reference_spmv(R, data, indices, indptr, shape, x):
    """Mirror of prepare_spmv_csr (spmv_csr.py:455-495) minus the is_cuda gate, then both launch helpers."""
    data, indices, indptr, x = _t(data), _t(indices), _t(indptr), _t(x)
    n_rows, n_cols = shape
    nnz = data.numel()
    kernel_indices = indices.to(torch.int32) if indices.dtype == torch.int64 else indices
    kernel_indptr = indptr.to(torch.int32) if nnz <= 2**31 - 1 else indptr.to(torch.int64)
    row_lengths = kernel_indptr[1:] - kernel_indptr[:-1]
    max_row_nnz = int(row_lengths.max().item()) if n_rows > 0 else 0
    block_nnz = 256
    max_segments = max((max_row_nnz + block_nnz - 1) // block_nnz, 1)
    buckets = R._build_spmv_opt_buckets(row_lengths, max_row_nnz=max_row_nnz, row_index_dtype=torch.int32,
                                        max_segments=None, fp64=data.dtype == torch.float64)
    prepared = R.PreparedCsrSpmv(data=data, kernel_indices=kernel_indices, kernel_indptr=kernel_indptr, shape=shape,
                                 n_rows=n_rows, n_cols=n_cols, block_nnz=block_nnz, max_segments=max_segments,
                                 max_row_nnz=max_row_nnz, opt_buckets=buckets)
    y_base = R._triton_spmv_csr_impl_prepared(prepared, x)
    y_opt = R._triton_spmv_csr_impl_opt_prepared(prepared, x)
    meta = [{"n_rows": int(b["rows"].numel()), "block_size": b["block_size"], "max_segs": b["max_segs"],
             "batch_rows": b["batch_rows"]} for b in buckets]
    return y_base.numpy(), y_opt.numpy(), meta


def run_reference_spmm(M, data, indices, indptr, shape, B):
    data, indices, indptr, B = _t(data), _t(indices), _t(indptr), _t(B)
    n_rows, n_cols = shape
    n_dense = int(B.shape[1])
    kernel_indices = indices.to(torch.int32) if indices.dtype == torch.int64 else indices
    kernel_indptr = indptr.to(torch.int64)
    row_lengths = kernel_indptr[1:] - kernel_indptr[:-1]
    max_row_nnz = int(row_lengths.max().item())
    launch = M._resolve_spmm_alg1_launch_config(n_dense, max_row_nnz)
    C_base = M._triton_spmm_csr_impl(data, kernel_indices, kernel_indptr, B, n_rows, n_dense,
                                     block_n=launch["block_n"], block_nnz=launch["block_nnz"])
    # opt path, as prepare_spmm_csr_opt (:480-522) + _triton_spmm_csr_impl_opt_prepared (:1046-1055)
    buckets, long_rows = M._build_spmm_opt_buckets(row_lengths)
    parts = (torch.empty((0,), dtype=long_rows.dtype), torch.empty((0,), dtype=torch.int64),
             torch.empty((0,), dtype=torch.int64), torch.zeros(1, dtype=torch.int64))
    if long_rows.numel() > 0:
        parts = M._build_spmm_opt_split_metadata(kernel_indptr, long_rows, part_block_nnz=256)
    prepared = M.PreparedCsrSpmmOpt(data=data, kernel_indices=kernel_indices, kernel_indptr=kernel_indptr, shape=shape,
                                    n_rows=n_rows, n_cols=n_cols, row_lengths=row_lengths, max_row_nnz=max_row_nnz,
                                    row_buckets=buckets, long_part_rows=parts[0], long_part_starts=parts[1],
                                    long_part_ends=parts[2], long_row_ids=long_rows, long_row_part_ptr=parts[3],
                                    long_row_fallback_only=False)
    block_n = M._select_spmm_opt_block_n(n_dense)
    C_opt = torch.zeros((n_rows, n_dense), dtype=B.dtype)
    for bucket in buckets:
        if bucket["kind"] == "split":
            M._run_spmm_opt_split_bucket(prepared, B, C_opt, block_n)
        else:
            M._run_spmm_opt_bucket(prepared, bucket, B, C_opt, block_n)
    meta = [{"kind": b["kind"], "n_rows": int(b["rows"].numel())} for b in buckets]
    return C_base.numpy(), C_opt.numpy(), meta


def coo_cases():
    """Unsorted entries with duplicate (row, col) pairs and rows without entries."""
    out = {}
    for name, seed, n_rows, n_cols, nnz, vt, rt, ct, n_dense in (
            ("dups_f32", 31, 37, 29, 400, np.float32, np.int64, np.int32, 5),
            ("dups_f64", 32, 64, 300, 500, np.float64, np.int32, np.int64, 32),
            ("sparse_rows_f32", 33, 200, 64, 90, np.float32, np.int32, np.int32, 12)):
        rng = np.random.default_rng(seed)
        row = rng.integers(0, n_rows, nnz).astype(rt)
        row[row % 5 == 3] = 1  # a long row and a set of rows that stay empty
        col = rng.integers(0, n_cols, nnz).astype(ct)
        val = rng.uniform(-1, 1, nnz).astype(vt)
        x = rng.uniform(-1, 1, n_cols).astype(vt)
        B = rng.uniform(-1, 1, (n_cols, n_dense)).astype(vt)
        out[name] = (val, row, col, (n_rows, n_cols), x, B)
    return out


def run_reference_coo(V, MC, val, row, col, shape, x, B):
    n_rows, n_cols = shape
    val, row, col, x, B = _t(val), _t(row), _t(col), _t(x), _t(B)
    # SpMV, sort_by_row=True (row-run kernel) and False (atomic kernel): _prepare_coo_tensors minus is_cuda
    d, r64, c64 = V._sort_coo_lex_inplace(val, row, col, n_cols)
    seg = V._seg_starts_from_sorted_rows(r64.to(torch.int32), d.numel(), d.device)
    p_seg = V.PreparedCoo(d, r64.to(torch.int32), c64.to(torch.int32), shape, seg_starts=seg)
    y_seg = V._triton_spmv_coo_kernel(p_seg, x, block_size=256, num_warps=4, block_inner=128)
    p_at = V.PreparedCoo(val.contiguous(), row.to(torch.int32), col.to(torch.int32), shape, seg_starts=None)
    y_atomic = V._triton_spmv_coo_kernel(p_at, x, block_size=256, num_warps=4, block_inner=128)
    # SpMM, as _run_spmm_coo_route: coalesce + sort, then the row-run kernel
    kr = row.to(torch.int32)
    kc = col.to(torch.int32)
    n_dense = int(B.shape[1])
    (cd, cr, cc, cB, _, _, _, out_dtype, _) = MC._prepare_spmm_coo_canonical_prepared(val, kr, kc, B, n_rows, n_cols,
                                                                                      n_dense)
    launch = MC._resolve_spmm_coo_launch_config(n_dense, cd.numel())
    C = MC._triton_spmm_coo_impl(cd, cr, cc, cB, n_rows, n_dense, block_n=launch["block_n"],
                                 block_nnz=launch["block_nnz"], route="rowrun", output_dtype=out_dtype)
    return (y_seg.numpy(), y_atomic.numpy(), C.numpy(), d.numpy(), r64.numpy(), c64.numpy(), seg.numpy(), launch)


def make_coo(index, V, MC):
    index["coo"] = {}
    for name, (val, row, col, shape, x, B) in coo_cases().items():
        y_seg, y_atomic, C, d, r, c, seg, launch = run_reference_coo(V, MC, val, row, col, shape, x, B)
        np.savez_compressed(os.path.join(HERE, f"coo_{name}.npz"), data=val, row=row, col=col, shape=np.asarray(shape),
                            x=x, B=B, y_seg=y_seg, y_atomic=y_atomic, C=C, sorted_data=d, sorted_row=r, sorted_col=c,
                            seg_starts=seg)
        index["coo"][name] = {"nnz": int(val.size), "n_segs": int(seg.size - 1), "launch": launch}
        print("coo", name, val.size, index["coo"][name], flush=True)


WIDE = {"f16": torch.float16, "bf16": torch.bfloat16, "c64": torch.complex64, "c128": torch.complex128}


def _storable(t):
    """numpy has no bfloat16: store it (and float16) widened to float32, which is exact."""
    return t.to(torch.float32).numpy() if t.dtype in (torch.float16, torch.bfloat16) else t.numpy()


def make_wide(index, R, M):
    """Outputs of the reference's base SpMV and SpMM helpers for the four value types it widens or splits."""
    index["wide"] = {}
    lens = [0, 3, 17, 1, 0, 40, 5, 9, 64, 2, 0, 31]
    _, indices, indptr = handmade_csr(41, lens, 96, np.float32, np.int32, np.int32)
    n_rows, n_cols, nnz = len(lens), 96, int(indptr[-1])
    rng = np.random.default_rng(42)
    for tag, dt in WIDE.items():
        def values(shape):
            v = rng.uniform(-1, 1, shape)
            if dt.is_complex:
                v = v + 1j * rng.uniform(-1, 1, shape)
            return torch.from_numpy(v).to(dt)
        data, x, B = values(nnz), values(n_cols), values((n_cols, 6))
        ti, tp = _t(indices), _t(indptr)
        prepared = R.PreparedCsrSpmv(data=data, kernel_indices=ti, kernel_indptr=tp, shape=(n_rows, n_cols),
                                     n_rows=n_rows, n_cols=n_cols, block_nnz=256, max_segments=1, max_row_nnz=max(lens),
                                     opt_buckets=[])
        y = R._triton_spmv_csr_impl_prepared(prepared, x)
        launch = M._resolve_spmm_alg1_launch_config(6, max(lens))
        C = M._triton_spmm_csr_impl(data, ti, tp.to(torch.int64), B, n_rows, 6, block_n=launch["block_n"],
                                    block_nnz=launch["block_nnz"])
        assert y.dtype == dt and C.dtype == dt
        np.savez_compressed(os.path.join(HERE, f"wide_{tag}.npz"), data=_storable(data), indices=indices, indptr=indptr,
                            shape=np.asarray((n_rows, n_cols)), x=_storable(x), B=_storable(B), y=_storable(y),
                            C=_storable(C))
        index["wide"][tag] = {"dtype": str(dt), "nnz": nnz}
        print("wide", tag, index["wide"][tag], flush=True)


def make_sddmm(index, D):
    """Outputs of the reference's SDDMM kernel (value-dtype accumulation, its default variant)."""
    import triton
    import triton.language as tl

    index["sddmm"] = {}
    lens = [0, 3, 0, 17, 1, 64, 0, 0, 5, 140, 2, 0]
    cases = {
        "k8_f32": (handmade_csr(41, lens, 150, np.float32, np.int32, np.int32), 150, 8, 1.0, 0.0, False),
        "k33_f32_beta": (handmade_csr(42, lens, 150, np.float32, np.int32, np.int64), 150, 33, 0.5, -2.0, True),
        "k64_f32": (handmade_csr(43, [16] * 40, 97, np.float32, np.int32, np.int32), 97, 64, -1.25, 0.0, False),
        "k130_f64_beta": (handmade_csr(44, lens, 150, np.float64, np.int32, np.int32), 150, 130, 2.0, 0.75, True),
        "k4_f64": (handmade_csr(45, [7] * 30, 64, np.float64, np.int32, np.int64), 64, 4, 1.0, 0.0, False),
    }
    for name, ((data, indices, indptr), n_cols, k, alpha, beta, has_in) in cases.items():
        n_rows = indptr.shape[0] - 1
        rng = np.random.default_rng(sum(ord(ch) for ch in name))
        x = rng.uniform(-1, 1, (n_rows, k)).astype(data.dtype)
        y = rng.uniform(-1, 1, (n_cols, k)).astype(data.dtype)
        t_idx, t_ptr = _t(indices), _t(indptr).to(torch.int64)
        row_ids = D._build_row_ids(t_ptr)
        tx, ty, td = _t(x), _t(y), _t(data)
        nnz = int(t_idx.numel())
        out = torch.empty(nnz, dtype=tx.dtype)
        block_k, num_warps = D._resolve_sddmm_launch_config(k)
        acc = tl.float64 if tx.dtype == torch.float64 else tl.float32
        D._sddmm_csr_real_kernel[(triton.cdiv(nnz, 128),)](
            t_idx, row_ids, tx, ty, td if has_in else out, out, nnz, k, tx.stride(0), tx.stride(1), ty.stride(0),
            ty.stride(1), float(alpha), float(beta), HAS_IN=has_in, BLOCK_P=128, BLOCK_K=block_k, ACC_DTYPE=acc,
            num_warps=num_warps)
        np.savez_compressed(os.path.join(HERE, f"sddmm_{name}.npz"), data=data, indices=indices, indptr=indptr,
                            shape=np.asarray((n_rows, n_cols)), x=x, y=y, alpha=np.float64(alpha),
                            beta=np.float64(beta), has_in=np.asarray(has_in), out=out.numpy(),
                            row_ids=row_ids.numpy())
        index["sddmm"][name] = {"nnz": nnz, "k": k, "block_k": block_k, "num_warps": num_warps}
        print("sddmm", name, nnz, k, flush=True)


def make_mtx(index, reference_root):
    """CSR arrays the reference's two loaders produce for tests/golden/mtx/*.mtx (float32 and float64, on CPU)."""
    import glob
    import importlib.util

    loaders = {}
    for name in ("test_spmv", "test_spmm"):
        spec = importlib.util.spec_from_file_location(f"ref_{name}", os.path.join(reference_root, "tests", f"{name}.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        loaders[name] = mod.load_mtx_to_csr_torch
    index["mtx"] = {}
    for path in sorted(glob.glob(os.path.join(HERE, "mtx", "*.mtx"))):
        name = os.path.splitext(os.path.basename(path))[0]
        out = {}
        for dt, tag in ((torch.float32, "f32"), (torch.float64, "f64")):
            a = loaders["test_spmv"](path, dtype=dt, device=torch.device("cpu"))
            b = loaders["test_spmm"](path, dtype=dt, device=torch.device("cpu"))
            assert a[3] == b[3] and all(torch.equal(u, v) for u, v in zip(a[:3], b[:3])), "the two loaders disagree"
            out[f"data_{tag}"] = a[0].numpy()
            out["indices"], out["indptr"], out["shape"] = a[1].numpy(), a[2].numpy(), np.asarray(a[3])
        np.savez_compressed(os.path.join(HERE, f"mtx_{name}.npz"), **out)
        index["mtx"][name] = {"nnz": int(out["indices"].size), "shape": [int(v) for v in out["shape"]]}
        print("mtx", name, index["mtx"][name], flush=True)


def host_helper_goldens(R, M):
    g = {"alg1": [], "opt_block_n": {}, "coo": {}}
    for n in (1, 4, 5, 8, 9, 16, 17, 24, 32, 33, 48, 64, 65, 96, 128, 256):
        g["opt_block_n"][str(n)] = M._select_spmm_opt_block_n(n)
        for max_row in (0, 1, 31, 32, 33, 1536, 5000):
            for kw in ({}, {"block_nnz": 128}, {"block_n": 16, "block_nnz": 8}, {"block_nnz": 128, "max_segments": 4},
                       {"max_segments": 1}, {"block_n": 0}, {"max_segments": 0}):
                try:
                    res = M._resolve_spmm_alg1_launch_config(n, max_row, **kw)
                except Exception as exc:  # the exception TYPE is the contract
                    res = {"raises": type(exc).__name__}
                g["alg1"].append({"n": n, "max_row_nnz": max_row, "kw": kw, "result": res})
    rng = np.random.default_rng(5)
    row = rng.integers(0, 9, 40)
    col = rng.integers(0, 7, 40)
    val = rng.uniform(-1, 1, 40).astype(np.float32)
    d, i, p = R.coo_to_csr_for_spmv(_t(val), _t(row), _t(col), (9, 7))
    g["coo"] = {"row": row.tolist(), "col": col.tolist(), "val": val.tolist(), "data": d.tolist(),
                "indices": i.tolist(), "indptr": p.tolist(), "indices_dtype": str(i.dtype), "indptr_dtype": str(p.dtype)}
    return g


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    ap.add_argument("--only", choices=("all", "coo", "mtx", "wide", "sddmm"), default="all")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src"))
    from flagsparse.sparse_operations import spmm_coo as MC  # noqa: E402
    from flagsparse.sparse_operations import spmm_csr as M  # noqa: E402
    from flagsparse.sparse_operations import spmv_coo as V  # noqa: E402
    from flagsparse.sparse_operations import spmv_csr as R  # noqa: E402
    from flagsparse.sparse_operations import sddmm_csr as D  # noqa: E402

    index_path = os.path.join(HERE, "index.json")
    if args.only in ("coo", "mtx", "wide", "sddmm"):
        with open(index_path) as f:
            index = json.load(f)
        if args.only == "coo":
            make_coo(index, V, MC)
        elif args.only == "wide":
            make_wide(index, R, M)
        elif args.only == "sddmm":
            make_sddmm(index, D)
        else:
            make_mtx(index, args.reference)
        with open(index_path, "w") as f:
            json.dump(index, f, indent=1, sort_keys=True)
        return
    index = {"spmv": {}, "spmm": {}}
    for name, ((data, indices, indptr), shape, x) in spmv_cases().items():
        y_base, y_opt, meta = run_reference_spmv(R, data, indices, indptr, shape, x)
        np.savez_compressed(os.path.join(HERE, f"spmv_{name}.npz"), data=data, indices=indices, indptr=indptr,
                            shape=np.asarray(shape), x=x, y_base=y_base, y_opt=y_opt)
        index["spmv"][name] = {"nnz": int(data.size), "buckets": meta}
        print("spmv", name, data.size, meta, flush=True)
    for name, ((data, indices, indptr), shape, B) in spmm_cases().items():
        C_base, C_opt, meta = run_reference_spmm(M, data, indices, indptr, shape, B)
        np.savez_compressed(os.path.join(HERE, f"spmm_{name}.npz"), data=data, indices=indices, indptr=indptr,
                            shape=np.asarray(shape), B=B, C_base=C_base, C_opt=C_opt)
        index["spmm"][name] = {"nnz": int(data.size), "buckets": meta}
        print("spmm", name, data.size, meta, flush=True)
    make_coo(index, V, MC)
    make_mtx(index, args.reference)
    make_wide(index, R, M)
    make_sddmm(index, D)
    index["host"] = host_helper_goldens(R, M)
    with open(index_path, "w") as f:
        json.dump(index, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
