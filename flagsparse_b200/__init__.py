"""flagsparse_b200: the CSR SpMV / CSR SpMM path of flagsparse on hand-written sm_100a CUDA kernels.

The public names are the reference's (src/flagsparse/__init__.py:65-136 re-exports them from
sparse_operations): CSR arrays as torch tensors, float32/float64 values, int32/int64 indices, a dense x or a
row-major B.  Compute goes through libfsb.so (include/fsb.h); there is no Triton path and no CPU path.
"""

from ._common import SUPPORTED_INDEX_DTYPES, SUPPORTED_VALUE_DTYPES, _tolerance_for_dtype
from .coo import PreparedCoo, flagsparse_spmm_coo, flagsparse_spmv_coo, prepare_spmv_coo
from .mtx import load_mtx_to_csr_torch
from .sddmm_csr import SDDMMPrepared, flagsparse_sddmm_csr, prepare_sddmm_csr
from .sharded import ShardedCsrSpmm, ShardedCsrSpmv, partition_rows_by_nnz
from .spmm_csr import (
    PreparedCsrSpmmOpt,
    flagsparse_spmm_csr,
    flagsparse_spmm_csr_opt,
    prepare_spmm_csr_opt,
)
from .spmv_csr import (
    PreparedCsrSpmv,
    coo_to_csr_for_spmv,
    flagsparse_spmv_coo_tocsr,
    flagsparse_spmv_csr,
    prepare_spmv_coo_tocsr,
    prepare_spmv_csr,
)

__all__ = [
    "SUPPORTED_VALUE_DTYPES",
    "SUPPORTED_INDEX_DTYPES",
    "PreparedCsrSpmv",
    "prepare_spmv_csr",
    "flagsparse_spmv_csr",
    "coo_to_csr_for_spmv",
    "prepare_spmv_coo_tocsr",
    "flagsparse_spmv_coo_tocsr",
    "PreparedCoo",
    "prepare_spmv_coo",
    "flagsparse_spmv_coo",
    "flagsparse_spmm_coo",
    "PreparedCsrSpmmOpt",
    "prepare_spmm_csr_opt",
    "flagsparse_spmm_csr",
    "flagsparse_spmm_csr_opt",
    "SDDMMPrepared",
    "prepare_sddmm_csr",
    "flagsparse_sddmm_csr",
    "load_mtx_to_csr_torch",
    "ShardedCsrSpmv",
    "ShardedCsrSpmm",
    "partition_rows_by_nnz",
]
