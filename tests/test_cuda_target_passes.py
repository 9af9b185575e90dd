"""CPU tests of the MIGraphX `cuda` target plug-in: the target registers through MIGraphX's
own make_target(), and its pass pipeline (simplify_qdq, lowering, replace_allocate,
memory_coloring, ...) turns the quantized-GEMM programs into cuda:: operators.  Nothing is
executed on a device here: the pipeline stops before finalize."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECK = os.path.join(ROOT, "amdmigraphx_b200", "bin", "cuda_target_check")

pytestmark = pytest.mark.skipif(not os.path.exists(CHECK), reason="plug-in driver not built")


def _passes(case, mode=None):
    cmd = [CHECK, "passes", case] + ([mode] if mode else [])
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


def test_cases_are_listed():
    out = subprocess.run([CHECK, "list"], capture_output=True, text=True).stdout.split()
    assert {"c1", "fp8_gelu", "int4_decode", "raw_quant_dot"} <= set(out)


@pytest.mark.parametrize("mode", [None, "prefused"])
def test_qdq_linear_becomes_one_fused_qgemm(mode):
    out = _passes("c1_small", mode)
    lines = [l for l in out.splitlines() if "cuda::qgemm" in l]
    assert len(lines) == 1
    # per-column scale, relu, bias, weights re-laid out [N,K] at compile time, fp32 out
    assert "scale_mode=2" in lines[0] and "act=1" in lines[0] and "has_bias=1" in lines[0]
    assert "b_nk=1" in lines[0]
    assert "cuda::quantizelinear" in out
    for gone in ("dequantizelinear", " dot(", "relu", "pointwise"):
        assert gone not in out.replace("cuda::dequantizelinear", "")
    # buffers come from one preallocated arena, the result is written to the output parameter
    assert "cuda::preallocate" in out and "load[" in out and "main:#output_0" in out


def test_gelu_chain_and_fp8_are_fused():
    out = _passes("int8_gelu")
    assert "act=2" in out and "erf" not in out
    out = _passes("fp8_gelu")
    line = [l for l in out.splitlines() if "cuda::qgemm" in l][0]
    assert "scale_mode=1" in line and "act=2" in line and "fp8e4m3fn_type" in out


def test_int4_linear_keeps_weights_packed():
    out = _passes("int4_decode")
    assert "cuda::w4a16[group=128,zp_const=8,has_zp=0" in out
    assert "unpack_int4" not in out and "uint8_type, {256, 256}" in out  # [N, K/2] stays packed
    out = _passes("int4_batch16_zp")
    assert "cuda::w4a16[group=32" in out and "has_zp=1" in out


def test_offload_copy_inserts_copies():
    out = _passes("int8_gelu", "offload")
    assert "cuda::copy_to" in out and "cuda::copy_from" in out


def test_non_constant_right_operand_gets_a_workspace():
    out = _passes("raw_quant_dot")
    assert "has_workspace=1" in out and "int32_type, {2, 72, 48}" in out


def test_quantizelinear_between_two_linears_is_fused_into_the_first():
    out = _passes("mlp_fused_q")
    gemms = [l for l in out.splitlines() if "cuda::qgemm" in l]
    assert len(gemms) == 2
    # first GEMM: relu + trailing quantizelinear (int8, scale 0.05), only the int8 tensor is written
    assert "q_type=5" in gemms[0] and "write_d=0" in gemms[0] and "int8_type, {96, 320}" in gemms[0]
    assert out.count("cuda::quantizelinear") == 1  # only the one on the program input is left
    out = _passes("mlp_two_outputs")
    assert "cuda::second_output" in out and "write_d=1" in out
