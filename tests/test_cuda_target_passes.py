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


def _passes(case, mode=None, env=None):
    cmd = [CHECK, "passes", case] + ([mode] if mode else [])
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, **env) if env else None)
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


def test_layernorm_chain_becomes_one_kernel():
    out = _passes("layernorm_f32")
    assert out.count("cuda::layernorm[") == 1 and "has_gamma=1,has_beta=1" in out
    assert "cuda::reduce[mode=1]" not in out and "rsqrt" not in out
    for mode in (0, 2, 3):  # the max / min / sum the case also returns stay reductions
        assert "cuda::reduce[mode=%d]" % mode in out


def test_layernorm_with_unaligned_rows_lowers_to_reductions_and_fused_pointwise():
    out = _passes("layernorm_f32_odd")
    assert "cuda::layernorm" not in out
    # two reduce_mean of the decomposition plus the max / min / sum the case also returns
    assert out.count("cuda::reduce[mode=1]") == 2
    for mode in (0, 2, 3):
        assert "cuda::reduce[mode=%d]" % mode in out
    # scale + shift + normalise end up in one launch
    assert any(l.count(",") > 8 and "cuda::pointwise[ops={2, 2, 0}" in l for l in out.splitlines())
    assert "reduce_mean" not in out


def test_attention_lowers_to_fp16_gemms_softmax_and_packed_copies():
    out = _passes("attention_f16")
    gemms = [l for l in out.splitlines() if "cuda::qgemm" in l]
    assert len(gemms) == 2 and all("scale_mode=0" in g and "out_type=1" in g for g in gemms)
    assert out.count("cuda::softmax") == 1
    # reshape of the packed parameters is a view; the head transposes are copied once
    assert "reshape_lazy" in out and " reshape[" not in out and "contiguous" not in out
    assert out.count("cuda::pointwise[ops={32}") >= 3
    # everything runs inside the submodule of one cuda::graph_run, which takes all parameters
    call = [l for l in out.splitlines() if "= cuda::graph_run[" in l]
    assert len(call) == 1 and all(p in call[0] for p in ("main:#output_0", "q", "k", "v"))


def test_constant_fp16_weight_is_relaid_out_once():
    out = _passes("dot_f16_const")
    line = [l for l in out.splitlines() if "cuda::qgemm" in l][0]
    assert "b_nk=1" in line and "has_workspace=0" in line
    assert "half_type, {136, 264}" in out  # the [K,N] literal became [N,K]
    out = _passes("dot_f16_batched")
    line = [l for l in out.splitlines() if "cuda::qgemm" in l][0]
    assert "b_nk=0" in line and "has_workspace=1" in line


def test_bert_layer_compiles_into_one_graph():
    out = _passes("bert_layer_int8")
    # the Q, K and V projections as one GEMM over the concatenated weights, then O, FFN1, FFN2
    assert out.count("cuda::qgemm") == 4 and "half_type, {128, 768}, {768, 1}" in out
    assert out.count("slice[axes={1}") == 3
    assert out.count("= cuda::graph_run[") == 1 and 'module: "main:graph"' in out
    # FFN1: GELU and the quantizelinear feeding FFN2 run in its epilogue
    assert any("act=2" in l and "q_type=5" in l and "write_d=0" in l for l in out.splitlines())
    # the attention block and the two LayerNorms are one launch each
    assert out.count("cuda::attention[") == 1 and "cuda::softmax" not in out
    assert out.count("cuda::layernorm[") == 2 and "cuda::reduce" not in out


def test_attention_block_with_64_wide_heads_becomes_one_kernel():
    out = _passes("attention_f16_d64")
    assert out.count("cuda::attention[batch=2,seq=200,heads=3,head_dim=64") == 1
    assert "cuda::qgemm" not in out and "cuda::softmax" not in out and "cuda::pointwise" not in out


def test_embedding_rope_and_cache_append_lower_to_movers():
    out = _passes("embed_rope_f16")
    assert "cuda::gather[axis=0]" in out
    assert "cuda::concat[axis=2]" in out and "cuda::concat[axis=1]" in out
    # the two halves are views (slice) read by the element-wise kernel, not copies of x
    assert out.count("slice[") == 2
    # cos / sin mix in one launch
    assert "cuda::pointwise[ops={2, 2, 0}" in out


def test_fp16_dot_with_unaligned_inner_dimension_pads_rows():
    out = _passes("dot_f16_odd_k")
    assert "cuda::pad_rows" in out and "{2, 50, 197}, {10000, 200, 1}" in out
    out = _passes("dot_f16_odd_k_const")
    # 13 is no multiple of 8: the constant stays [K,N] and is re-laid out per evaluation
    line = [l for l in out.splitlines() if "cuda::qgemm" in l][0]
    assert "b_nk=0" in line and "has_workspace=1" in line and "cuda::pad_rows" in out


def test_reductions_over_other_axes_use_a_transposed_copy():
    out = _passes("reduce_axes")
    # trailing axes {1, 2}: reduced in place; axis 1, axis 0 and axes {0, 2}: transposed copy first
    assert out.count("cuda::reduce[") == 4
    assert out.count("transpose[") == 3 and out.count("cuda::pointwise[ops={32}") == 3
    assert "reshape_lazy[dims={6, 1, 48}]" in out and "reshape_lazy[dims={1, 20, 1}]" in out


def test_int4_group_size_when_k_over_group_is_not_a_power_of_two():
    # K = 28672 (Llama-2-70B down projection) with groups of 128: 224 groups per row
    out = _passes("int4_group_k28672")
    assert "cuda::w4a16[group=128,zp_const=8,has_zp=0" in out and "half_type, {64, 224}" in out
    out = _passes("int4_group_k96")
    assert "cuda::w4a16[group=32" in out and "has_zp=1" in out and "half_type, {64, 3}" in out


def test_transposed_batched_left_operand_is_packed_first():
    out = _passes("quant_dot_transposed_a")
    lines = out.splitlines()
    gemm = [l for l in lines if "cuda::qgemm" in l][0]
    # the transposed view goes through a packed copy; quant_dot reads the copy, not the view
    copy = [l for l in lines if "cuda::pointwise[ops={32}" in l and "int8_type, {2, 3, 24, 32}, {2304, 768, 32, 1}" in l]
    assert len(copy) == 1
    assert copy[0].split(" = ")[0] in gemm


def test_offload_copy_program_keeps_host_copies_around_the_graph_run():
    out = _passes("int8_gelu", "offload")
    main, sub = out.split('module: "main:graph"')
    order = [n for l in main.splitlines() for n in ("cuda::copy_to", "cuda::graph_run", "cuda::copy_from")
             if "= " + n in l]
    # host copies stay in the main module around the one call; the launches live in the submodule
    assert order == ["cuda::copy_to", "cuda::graph_run", "cuda::copy_from"]
    assert "cuda::qgemm" in sub and "cuda::qgemm" not in main and "cuda::copy" not in sub.replace("cuda::copy_", "")


def test_config2_layer_lowers_at_real_dimensions():
    out = _passes("c2_layer")
    gemms = [l for l in out.splitlines() if "cuda::qgemm" in l]
    assert any("half_type, {384, 768}" in l for l in gemms)
    assert "cuda::gather" in out and "cuda::softmax" in out or "cuda::attention" in out


def test_gqa_decode_step_becomes_cache_appends_and_one_attention_kernel():
    # the parser's decomposition of a GroupQueryAttention node at a decode step (rotary embedding by
    # the builder, concat_past_present, KV-head broadcast, dot / mul / where / softmax / dot)
    out = _passes("gqa_decode_d64_f4")
    assert out.count("cuda::concat_past_present") == 2
    assert out.count("cuda::gqa_decode_attention[num_heads=8,kv_num_heads=2") == 1
    assert "cuda::softmax" not in out and "cuda::qgemm" not in out
    # the rotary-embedding builder's chain (gathernd of cos / sin rows, rotate-half, three muls, add)
    assert out.count("cuda::rotary_embedding") == 1 and "cuda::gather" not in out and "cuda::concat[" not in out


def test_gqa_prompt_and_unsupported_head_sizes_keep_the_operator_chain():
    for case in ("gqa_prompt_small", "gqa_decode_small"):
        out = _passes(case)
        assert "cuda::gqa_decode_attention" not in out
        assert out.count("cuda::concat_past_present") == 2 and out.count("cuda::softmax") == 1
        assert out.count("cuda::qgemm") == 2


def test_gqa_rotary_embedding_operator_is_lowered():
    out = _passes("gqa_decode_rotary_op")
    assert out.count("cuda::gqa_rotary_embedding[num_heads=4,kv_num_heads=2,interleaved=0]") == 1


def test_two_streams_schedule_parallel_branches_with_events():
    # MIGRAPHX_CUDA_NSTREAMS=2: MIGraphX's schedule pass (src/schedule.cpp) places the independent
    # Q / K / V projections on two streams through the target's schedule model; every cross-stream
    # read is ordered by a record / wait pair
    out = _passes("bert_layer_int8", env={"MIGRAPHX_CUDA_NSTREAMS": "2",
                                          "MIGRAPHX_CUDA_DISABLE_FUSION": "horizontal,attention"})
    assert "cuda::set_stream[stream=1]" in out and "cuda::set_stream[stream=0]" in out
    records = [l for l in out.splitlines() if "cuda::record_event" in l]
    waits = [l for l in out.splitlines() if "cuda::wait_event" in l]
    assert len(records) >= 2 and len(waits) >= len(records)
    # several streams: evaluated instruction by instruction, no graph submodule
    assert "cuda::graph_run" not in out


def test_make_target_loads_the_plugin_by_name_and_fails_loudly_without_a_device():
    # an application linked with libmigraphx.so only; the plug-in and the ref target come through
    # dlopen (src/register_target.cpp:56-80).  Without a GPU the first device call throws: the
    # target has no CPU fallback.
    import json
    import torch
    exe = os.path.join(os.path.dirname(CHECK), "cuda_dlopen_check")
    root = os.path.dirname(os.path.dirname(os.path.dirname(exe)))
    libs = [os.path.join(root, "amdmigraphx_b200", "lib"), os.path.join(root, "oracle", "_ref", "lib")]
    env = dict(os.environ, LD_LIBRARY_PATH=":".join(libs + [os.environ.get("LD_LIBRARY_PATH", "")]))
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=env)
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert lines and lines[0] == {"targets_before": 0, "cuda": "cuda", "ref": "ref"}, r.stdout + r.stderr
    if not torch.cuda.is_available():
        assert r.returncode == 2 and "cuda target: cudaSetDevice" in lines[-1]["error"]


def test_activation_and_quantizelinear_table_is_opt_in():
    # fp16 chain whose only result is the int8 tensor (FFN1 of an encoder layer): with
    # MIGRAPHX_CUDA_QGEMM_LUT=1 the erf-GELU and the quantizelinear become a 65536-entry table input
    plain = _passes("c2_layer")
    assert "has_lut=1" not in plain
    out = _passes("c2_layer", env={"MIGRAPHX_CUDA_QGEMM_LUT": "1"})
    lines = [l for l in out.splitlines() if "cuda::qgemm" in l and "has_lut=1" in l]
    assert len(lines) == 1 and "act=2" in lines[0] and "write_d=0" in lines[0]
    assert "int8_type, {65536}" in out


def test_llama_decoder_layer_lowers_to_int4_linears_cache_appends_and_decode_attention():
    # RMSNorm (parser decomposition), five MatMulNBits linears, GroupQueryAttention decomposition with
    # KV cache, SwiGLU, residual adds: every operator has a kernel, the layer is one graph_run
    out = _passes("llama_layer_small")
    # packed QKV, O, gate + up as one operator over the concatenated weights, down
    assert out.count("cuda::w4a16[") == 4
    assert "-> half_type, {2, 1024}, {1024, 1}" in out and out.count("slice[axes={1},starts={512},ends={1024}]") == 1
    assert out.count("cuda::concat_past_present") == 2 and out.count("cuda::gqa_decode_attention") == 1
    assert out.count("cuda::layernorm[rms=1") == 2 and out.count("cuda::rotary_embedding") == 1
    assert "cuda::reduce[" not in out and "cuda::graph_run" in out
    assert "cuda::qgemm" not in out and "cuda::softmax" not in out
    # 13 launches: 4 linears, 2 RMSNorms, rotary, 2 cache appends, attention, residual add,
    # SwiGLU, residual add
    assert out.count("cuda::pointwise[") == 3
