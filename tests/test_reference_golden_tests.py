"""The reference's own golden tests for the quantized path (test/ref/quantizelinear.cpp,
dequantizelinear.cpp, unpack_int4.cpp, pack_int4.cpp, pack_unpack_int4.cpp, dot_op.cpp) compiled
where they lie and run against the ref target this repository's oracle is pinned to
(oracle/run_reference_tests.py).  Skipped where the MIGraphX sources or the oracle build are absent."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import build_ref  # noqa: E402

REF = build_ref.reference_dir()


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "test", "ref")) or
                    not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "lib", "libmigraphx_ref.so")),
                    reason="MIGraphX sources or the oracle build are not present")
def test_reference_golden_tests_pass_on_the_oracle_build():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "run_reference_tests.py"), "--ref", REF],
                       capture_output=True, text=True, timeout=1500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    lines = r.stdout.splitlines()
    ran = [l for l in lines if l.startswith("test cases run:")]
    failed = [l for l in lines if l.startswith("lines containing FAILED:")]
    assert ran and int(ran[0].split(":")[1]) >= 70
    assert failed and int(failed[0].split(":")[1]) == 0


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "test", "ref")) or
                    not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "lib", "libmigraphx_ref.so")),
                    reason="MIGraphX sources or the oracle build are not present")
def test_reference_pass_tests_pass_on_the_host_library_the_plugin_links():
    """test/simplify_qdq_test.cpp, quantization.cpp, fuse_pointwise.cpp, memory_coloring_test.cpp,
    schedule_test.cpp, replace_allocate.cpp, eliminate_allocation_test.cpp, dead_code_elimination_test.cpp,
    eval_test.cpp, op_shape_test.cpp, half.cpp, fp8e4m3fn.cpp: the target-independent passes, shape rules
    and number types the `cuda` target compiles programs with, in the build it links."""
    r = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "run_reference_tests.py"), "--ref", REF,
                        "--passes"], capture_output=True, text=True, timeout=1500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    lines = r.stdout.splitlines()
    ran = [l for l in lines if l.startswith("test cases run:")]
    failed = [l for l in lines if l.startswith("lines containing FAILED:")]
    assert ran and int(ran[0].split(":")[1]) >= 700
    assert failed and int(failed[0].split(":")[1]) == 0
