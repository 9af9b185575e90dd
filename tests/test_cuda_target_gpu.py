"""GPU tests of the MIGraphX `cuda` target plug-in: MIGraphX programs built with the public
module API are compiled and evaluated on MIGraphX's CPU `ref` target and on `cuda`
(make_target("cuda") -> program::compile -> program::eval) and compared, the scheme of the
reference's test/verify harness.  int8 results are bit-exact against ref running the same
simplify_qdq-rewritten program; fp8 / int4 results within rtol 2e-2 / atol 1e-2."""
import json
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECK = os.path.join(ROOT, "amdmigraphx_b200", "bin", "cuda_target_check")

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.exists(CHECK), reason="plug-in driver not built")]

CASES = ["c1_small", "c1_semantic", "int8_gelu", "int8_per_tensor", "fp8_gelu", "int4_decode",
         "int4_batch16_zp", "int4_batch8_zp", "int4_prefill", "q_dq_ops", "raw_quant_dot", "mlp_fused_q", "mlp_two_outputs",
         "pw_gelu_f16", "pw_arith_f32", "pw_transcendental_f32",
         "layernorm_f32", "layernorm_f16", "softmax_f32", "softmax_f16", "softmax_f32_long",
         "attention_f16", "dot_f16_const", "dot_f16_batched", "bert_layer_int8", "embed_rope_f16",
         "dot_f16_odd_k", "dot_f16_odd_k_const", "reduce_axes"]


def _run(case, mode=None):
    cmd = [CHECK, "run", case] + ([mode] if mode else [])
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert lines, r.stdout + r.stderr
    return json.loads(lines[-1])


@pytest.mark.parametrize("case", CASES)
def test_program_matches_ref(cuda_device, case):
    res = _run(case)
    assert res.get("pass"), res


@pytest.mark.parametrize("case", ["c1_small", "int8_gelu", "int4_decode", "attention_f16", "bert_layer_int8",
                                  "embed_rope_f16"])
def test_program_matches_ref_with_offload_copy(cuda_device, case):
    res = _run(case, "offload")
    assert res.get("pass"), res


def test_prefused_pointwise_program_matches_ref(cuda_device):
    res = _run("c1_small", "prefused")
    assert res.get("pass"), res


def test_config1_full_size_bit_exact(cuda_device):
    """config 1: int8 QDQ linear 256x1024x1024, per-channel scales, bias, relu."""
    res = _run("c1")
    assert res.get("pass") and res["exact"], res
    assert res["outputs"][0]["mismatched"] == 0
