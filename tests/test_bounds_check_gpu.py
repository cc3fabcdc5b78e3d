"""The checking build of the library (libfsb_check.so, the sources compiled with -DFSB_BOUNDS_CHECK): the edge-case
tests of every product pass under it, and index arrays that would take a kernel out of bounds are refused with a
record instead of being launched.  The library is chosen when the package is imported, so both run in child
processes with FSB_BOUNDS_CHECK=1."""

import os
import subprocess
import sys

import pytest

from flagsparse_b200 import build

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

EDGE_TESTS = ("test_edge_cases or test_panel_kernel_edge_cases or test_golden_fixtures or test_edge_shapes_and_strides "
              "or test_tiny_and_empty or test_coo_empty_and_degenerate or test_many_short_rows_and_tile_edges "
              "or test_rows_with_many_entries_per_chunk_and_several_groups or test_duplicates_unsorted_and_index_widths "
              "or test_panel_kernel_with_long_runs or test_stream_rows_across_many_tiles")
EDGE_FILES = ("test_spmv_gpu.py", "test_spmm_gpu.py", "test_sddmm_gpu.py", "test_widetypes_gpu.py", "test_coo_gpu.py",
              "test_longrows_gpu.py")


def _child(args, timeout):
    assert os.path.exists(build.CHECK_LIB), "build it with `python -m flagsparse_b200.build --check`"
    env = dict(os.environ, FSB_BOUNDS_CHECK="1")
    return subprocess.run([sys.executable, *args], env=env, cwd=ROOT, capture_output=True, text=True, timeout=timeout)


@pytest.mark.gpu
def test_out_of_range_indices_are_refused_with_a_record(cuda):
    r = _child([os.path.join(HERE, "bounds_check_cases.py")], 600)
    assert r.returncode == 0, (r.stdout + r.stderr)[-4000:]
    assert "all cases ok" in r.stdout


@pytest.mark.gpu
def test_edge_case_tests_pass_under_the_checking_build(cuda):
    r = _child(["-c", "from flagsparse_b200 import _lib; print('checking', _lib.lib().fsb_bounds_check_enabled())"], 300)
    assert r.returncode == 0 and "checking 1" in r.stdout, r.stdout + r.stderr
    r = _child(["-m", "pytest", *[os.path.join(HERE, f) for f in EDGE_FILES], "-m", "gpu", "-q", "-x", "-k", EDGE_TESTS,
                "-p", "no:cacheprovider"], 1500)
    assert r.returncode == 0, (r.stdout + r.stderr)[-4000:]
    assert " passed" in r.stdout and " failed" not in r.stdout
