"""MIGraphX's own cross-target verify harness (test/verify/run_verify.cpp) on its verify programs
for the quantized path, with the `cuda` plug-in as the target under test: every program is compiled
for `cuda`, round-tripped through program save / load, evaluated, compared with the ref target by
the harness's own tolerance, and checked for stream races (oracle/verify_cuda_main.cpp).  The
binary is built by oracle/build_verify.py from the reference's sources where they lie."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
VERIFY = os.path.join(ROOT, "oracle", "_ref", "bin", "test_verify_cuda")

pytestmark = pytest.mark.gpu

I8 = "<signed char, int>"
F8 = "<migraphx::fp8::float8<migraphx::fp8::f8_type::fp8, false>, float>"
GROUPS = {
    "quant_dot_int8": [f"test_quant_dot_3args_{i}{I8}" for i in range(1, 6)] +
                      [f"test_batch_quant_dot_{i}{I8}" for i in (1, 2)] +
                      [f"test_batch_quant_dot_{i}<migraphx::shape::int8_type>" for i in (3, 4, 5)],
    "quant_dot_fp8": [f"test_quant_dot_3args_{i}{F8}" for i in range(1, 6)] +
                     [f"test_batch_quant_dot_{i}{F8}" for i in (1, 2)] +
                     [f"test_batch_quant_dot_{i}<migraphx::shape::fp8e4m3fn_type>" for i in (3, 4, 5)],
    "q_dq_int4": ["test_unpack_int4<migraphx::shape::uint8_type>", "test_unpack_int4<migraphx::shape::int8_type>",
                  "test_quantizelinear", "test_quantizelinear_int32", "test_dequantizelinear"],
    "epilogues": ["test_gemm_pointwise<migraphx::shape::half_type>", "test_add_gelu", "test_add_gelu_half"],
    "layernorm_softmax": ["test_softmax<3, migraphx::shape::half_type>", "test_layernorm", "test_layernorm2",
                          "test_layernorm_large", "test_layernorm_fp16", "test_layernorm_eps",
                          "test_layernorm_triadd", "test_layernorm_triadd_large"],
    "movers_attention": [f"test_gather<{a}, migraphx::shape::{t}>" for a in ("0", "-2")
                         for t in ("float_type", "half_type", "int8_type")] +
                        ["test_concat_axis_1", "test_gemm_softmax_gemm_relu<bias::without>",
                         "test_gemm_softmax_gemm_relu<bias::with>",
                         "test_gemm_softmax_gemm_relu<bias::with_standard_shape>"],
}

# Verify programs of the same source files that are outside this target's types: the fnuz and e5m2
# fp8 formats (no tensor-core kind on sm_100a takes them and the target has no emulation), fp32 /
# bf16 dot and softmax on fp32 with non-last axes.  They are not run.


@pytest.mark.parametrize("nstreams", [1, 2])
@pytest.mark.parametrize("group", sorted(GROUPS))
def test_reference_verify_programs_pass_on_the_cuda_target(group, nstreams):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not os.path.exists(VERIFY):
        pytest.fail("oracle/_ref/bin/test_verify_cuda is missing: run oracle/build_verify.py where the MIGraphX "
                    "sources are present")
    names = GROUPS[group]
    if nstreams == 2 and group not in ("movers_attention", "quant_dot_int8"):
        pytest.skip("the two-stream schedule (and the harness's stream-race analysis) on two groups only")
    r = subprocess.run([VERIFY, "-c"] + names, capture_output=True, text=True, timeout=900,
                       env=dict(os.environ, MIGRAPHX_CUDA_NSTREAMS=str(nstreams)))
    out = r.stdout + r.stderr
    done = [l for l in out.splitlines() if l.startswith("[ COMPLETE ]")]
    failed = [l for l in out.splitlines() if l.startswith("[  FAILED  ]")]
    assert not failed, "\n".join(failed) + "\n" + out[-3000:]
    assert len(done) == len(names), out[-3000:]
    assert r.returncode == 0, out[-3000:]
