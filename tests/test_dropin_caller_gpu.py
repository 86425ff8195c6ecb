"""A program compiled against the REFERENCE's own header (build/SpMM_API.cuh of the reference tree) and linked with
-lSpMM_API against this repository's library: encode -> SpMM_SplitK_API through the C++ names the reference's consumers
use (kernel_benchmark/spmm_test.cu:251-306, third_party/ft.patch:2833-2843), checked against a host GEMM inside the
program.  The binary is built by oracle/Makefile where the reference tree is present (source: tests/dropin/caller.cu)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CALLER = os.path.join(ROOT, "oracle", "_ref", "dropin_caller")

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not os.path.exists(CALLER), reason="oracle/_ref/dropin_caller not built")]


@pytest.mark.parametrize("args", [("1024", "2048", "16", "4"), ("512", "1024", "8", "1"), ("256", "4096", "64", "7")])
def test_reference_header_caller_links_and_runs(args):
    run = subprocess.run([CALLER, *args], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert run.stdout.count("DROPIN PASS") == 2, run.stdout  # reordered and scan-order encodings
