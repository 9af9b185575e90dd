// Builders of the MIGraphX programs this repository checks and measures: the quantized-GEMM
// path (QDQ linears, weight-only int4 linears), its neighbours (LayerNorm, softmax, attention,
// embeddings) and whole encoder layers / stacks assembled from them with MIGraphX's public
// module API.  Shared by the parity driver (check_main.cpp) and the benchmark runner
// (runner.cpp); header-only.
#ifndef MGX_CUDA_PROGRAMS_HPP
#define MGX_CUDA_PROGRAMS_HPP
#include <migraphx/program.hpp>
#include <migraphx/module.hpp>
#include <migraphx/make_op.hpp>
#include <migraphx/register_target.hpp>
#include <migraphx/literal.hpp>
#include <migraphx/instruction.hpp>
#include <migraphx/pass_manager.hpp>
#include <migraphx/fuse_pointwise.hpp>
#include <migraphx/dead_code_elimination.hpp>
#include <migraphx/simplify_qdq.hpp>
#include <migraphx/generate.hpp>
#include <migraphx/half.hpp>
#include <migraphx/quantization.hpp>
#include <migraphx/common.hpp>
#include <migraphx/op/builder/insert.hpp>
#include <chrono>
#include <cmath>
#include <cstring>
#include <iostream>
#include <map>
#include <random>
#include <functional>
#include <algorithm>
#include <numeric>
#include <limits>

namespace mgx_programs {

using migraphx::shape;
using migraphx::instruction_ref;


struct test_case
{
    migraphx::program prog;
    migraphx::parameter_map params; // host arguments
    bool exact    = false;          // bit-exact comparison
    // run simplify_qdq on the program ref evaluates too (always done for exact cases): the pass
    // is part of every GPU target's pipeline and changes values on purpose, e.g. a residual read
    // of a tensor that is also quantised becomes a read of its dequantised int8 copy
    // (match_qlinear_reused, src/simplify_qdq.cpp:401-432)
    bool ref_simplify_qdq = false;
    double rtol   = 1e-5;
    double atol   = 1e-6;
    // atol is meant for results of order one; with atol_row_rms it is scaled, row by row, by the
    // root mean square of the reference row (at least 1): |d| <= atol * max(1, rms) + rtol * |ref|.
    // For inputs with outliers, whose results are sums of large terms that partly cancel: an
    // element-wise bound relative to a near-cancelled sum is met by no inexact method, the
    // reference's own cross-target check included (it bounds the RMS error against the largest
    // magnitude, src/include/migraphx/verify.hpp:174-195).
    bool atol_row_rms = false;
    // Whole layers with quantizers inside: where the target's kernels round an intermediate value
    // differently from the reference's operator chain (a fused attention that keeps fp32 where the
    // chain rounds to half, fp32 sums in another order), a value next to a rounding boundary of a
    // following quantizelinear lands in the neighbouring int8 bucket, and the layer's result moves
    // by (activation scale) x (weight) for every such flip.  Up to `outlier_fraction` of the
    // elements may therefore miss (rtol, atol) as long as they stay within `outlier_atol`.
    double outlier_fraction = 0.0;
    double outlier_atol     = 0.0;
    // Cases too large for the CPU interpreter to evaluate in full: the rows of the left operand
    // are independent, so ref evaluates `ref_prog` - the same program built for fewer rows (same
    // seed, hence the same weights) - on `ref_params`, whose rows are rows `sample_rows` of the
    // full input; row i of its outputs is compared with row sample_rows[i] of the cuda outputs.
    bool sampled = false;
    migraphx::program ref_prog;
    migraphx::parameter_map ref_params;
    std::vector<std::size_t> sample_rows;
};

// rows `pick` of a [rows, cols] host argument as a packed argument
inline migraphx::argument take_rows(const migraphx::argument& a, const std::vector<std::size_t>& pick)
{
    const auto& s          = a.get_shape();
    const std::size_t cols = s.lens().back();
    const std::size_t rb   = cols * s.type_size();
    migraphx::argument out{shape{s.type(), {pick.size(), cols}}};
    for(std::size_t i = 0; i < pick.size(); ++i)
        std::memcpy(out.data() + i * rb, a.data() + pick[i] * rb, rb);
    return out;
}

// n distinct rows out of m, seeded, ascending; always includes the first and the last row
inline std::vector<std::size_t> pick_rows(std::size_t m, std::size_t n, unsigned seed)
{
    std::vector<std::size_t> all(m);
    for(std::size_t i = 0; i < m; ++i)
        all[i] = i;
    if(n >= m)
        return all;
    std::mt19937 g(seed);
    std::shuffle(all.begin() + 1, all.end() - 1, g);
    std::vector<std::size_t> r(all.begin(), all.begin() + (n - 1));
    r.push_back(m - 1);
    std::sort(r.begin(), r.end());
    return r;
}

template <class T>
std::vector<T> rand_ints(std::mt19937& g, std::size_t n, int lo, int hi)
{
    std::uniform_int_distribution<int> d(lo, hi);
    std::vector<T> v(n);
    for(auto& x : v)
        x = static_cast<T>(d(g));
    return v;
}

inline std::vector<float> rand_normal(std::mt19937& g, std::size_t n, float sd)
{
    std::normal_distribution<float> d(0.0f, sd);
    std::vector<float> v(n);
    for(auto& x : v)
        x = d(g);
    return v;
}

inline std::vector<float> rand_uniform(std::mt19937& g, std::size_t n, float lo, float hi)
{
    std::uniform_real_distribution<float> d(lo, hi);
    std::vector<float> v(n);
    for(auto& x : v)
        x = d(g);
    return v;
}

inline instruction_ref mbcast(migraphx::module* mm, instruction_ref x, const std::vector<std::size_t>& lens)
{
    return mm->add_instruction(migraphx::make_op("multibroadcast", {{"out_lens", lens}}), x);
}

inline instruction_ref bcast_axis(migraphx::module* mm, instruction_ref x, std::size_t axis,
                           const std::vector<std::size_t>& lens)
{
    return mm->add_instruction(migraphx::make_op("broadcast", {{"axis", axis}, {"out_lens", lens}}), x);
}

// Q -> DQ on the activation, DQ on the int8/fp8 weight literal, dot, + bias, activation:
// the fake-quantised form quantize_int8 / quantize_fp8 leave behind.
inline test_case qdq_linear(std::size_t m, std::size_t k, std::size_t n, shape::type_t qtype,
                     const std::string& act, bool per_channel, unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    auto* mm = t.prog.get_main_module();
    const bool fp8 = qtype == shape::fp8e4m3fn_type;
    auto x       = mm->add_parameter("x", shape{shape::float_type, {m, k}});
    auto xs      = mm->add_literal(migraphx::literal{shape{shape::float_type}, {fp8 ? 0.01f : 0.02f}});
    instruction_ref xz, wq, wz;
    if(fp8)
    {
        std::vector<migraphx::fp8::fp8e4m3fn> z1 = {migraphx::fp8::fp8e4m3fn(0.0f)};
        xz = mm->add_literal(migraphx::literal{shape{qtype}, z1});
        auto wf = rand_normal(g, k * n, 60.0f);
        std::vector<migraphx::fp8::fp8e4m3fn> wv(k * n);
        for(std::size_t i = 0; i < wv.size(); ++i)
            wv[i] = migraphx::fp8::fp8e4m3fn(std::max(-448.0f, std::min(448.0f, wf[i])));
        wq = mm->add_literal(migraphx::literal{shape{qtype, {k, n}}, wv});
    }
    else
    {
        xz = mm->add_literal(migraphx::literal{shape{qtype}, std::vector<int8_t>{0}});
        wq = mm->add_literal(migraphx::literal{shape{qtype, {k, n}}, rand_ints<int8_t>(g, k * n, -127, 127)});
    }
    auto xq  = mm->add_instruction(migraphx::make_op("quantizelinear"), x, mbcast(mm, xs, {m, k}),
                                  mbcast(mm, xz, {m, k}));
    auto xdq = mm->add_instruction(migraphx::make_op("dequantizelinear"), xq, mbcast(mm, xs, {m, k}),
                                   mbcast(mm, xz, {m, k}));
    instruction_ref wdq;
    if(per_channel)
    {
        auto ws = mm->add_literal(migraphx::literal{shape{shape::float_type, {n}}, rand_uniform(g, n, 0.001f, 0.01f)});
        instruction_ref wzl;
        if(fp8)
            wzl = mm->add_literal(migraphx::literal{shape{qtype, {n}}, std::vector<migraphx::fp8::fp8e4m3fn>(n, migraphx::fp8::fp8e4m3fn(0.0f))});
        else
            wzl = mm->add_literal(migraphx::literal{shape{qtype, {n}}, std::vector<int8_t>(n, 0)});
        wdq = mm->add_instruction(migraphx::make_op("dequantizelinear"), wq, bcast_axis(mm, ws, 1, {k, n}),
                                  bcast_axis(mm, wzl, 1, {k, n}));
    }
    else
    {
        auto ws = mm->add_literal(migraphx::literal{shape{shape::float_type}, {0.005f}});
        wdq = mm->add_instruction(migraphx::make_op("dequantizelinear"), wq, mbcast(mm, ws, {k, n}),
                                  mbcast(mm, xz, {k, n}));
    }
    auto d    = mm->add_instruction(migraphx::make_op("dot"), xdq, wdq);
    auto bias = mm->add_literal(migraphx::literal{shape{shape::float_type, {n}}, rand_normal(g, n, 0.1f)});
    instruction_ref y = mm->add_instruction(migraphx::make_op("add"), d, bcast_axis(mm, bias, 1, {m, n}));
    if(act == "relu")
        y = mm->add_instruction(migraphx::make_op("relu"), y);
    else if(act == "gelu")
    {
        auto half  = mm->add_literal(migraphx::literal{shape{shape::float_type}, {0.5f}});
        auto one   = mm->add_literal(migraphx::literal{shape{shape::float_type}, {1.0f}});
        auto sqrt2 = mm->add_literal(migraphx::literal{shape{shape::float_type}, {static_cast<float>(M_SQRT2)}});
        auto mh    = mm->add_instruction(migraphx::make_op("mul"), y, mbcast(mm, half, {m, n}));
        auto dv    = mm->add_instruction(migraphx::make_op("div"), y, mbcast(mm, sqrt2, {m, n}));
        auto er    = mm->add_instruction(migraphx::make_op("erf"), dv);
        auto ao    = mm->add_instruction(migraphx::make_op("add"), er, mbcast(mm, one, {m, n}));
        y          = mm->add_instruction(migraphx::make_op("mul"), mh, ao);
    }
    mm->add_return({y});
    auto xv = rand_normal(g, m * k, fp8 ? 1.5f : 1.0f);
    migraphx::argument xa{shape{shape::float_type, {m, k}}};
    std::memcpy(xa.data(), xv.data(), xv.size() * sizeof(float));
    t.params["x"] = xa;
    // ref evaluates the fake-quantised program (fp32 dot of dequantised operands); the cuda
    // target runs quant_dot + fused dequantise.  int8: products are exact either way and only
    // the fp32 rounding of the scaled sum differs; fp8: fp32 accumulation order.
    t.rtol = fp8 ? 2e-2 : 1e-5;
    t.atol = fp8 ? 1e-2 : 2e-5;
    return t;
}

// Two chained QDQ linears (an MLP): the quantizelinear between them is fed by the first GEMM's
// epilogue.  keep_hidden also returns the un-quantised hidden tensor (two outputs of one GEMM).
inline test_case qdq_mlp(std::size_t m, std::size_t k, std::size_t h, std::size_t n, bool keep_hidden, unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    auto* mm  = t.prog.get_main_module();
    auto x    = mm->add_parameter("x", shape{shape::float_type, {m, k}});
    auto zero = mm->add_literal(migraphx::literal{shape{shape::int8_type}, std::vector<int8_t>{0}});
    auto qdq  = [&](instruction_ref v, float sc, const std::vector<std::size_t>& lens) {
        auto s  = mm->add_literal(migraphx::literal{shape{shape::float_type}, {sc}});
        auto q  = mm->add_instruction(migraphx::make_op("quantizelinear"), v, mbcast(mm, s, lens), mbcast(mm, zero, lens));
        return mm->add_instruction(migraphx::make_op("dequantizelinear"), q, mbcast(mm, s, lens), mbcast(mm, zero, lens));
    };
    auto weight = [&](std::size_t kk, std::size_t nn) {
        auto wq = mm->add_literal(migraphx::literal{shape{shape::int8_type, {kk, nn}}, rand_ints<int8_t>(g, kk * nn, -127, 127)});
        auto ws = mm->add_literal(migraphx::literal{shape{shape::float_type, {nn}}, rand_uniform(g, nn, 0.001f, 0.01f)});
        auto wz = mm->add_literal(migraphx::literal{shape{shape::int8_type, {nn}}, std::vector<int8_t>(nn, 0)});
        return mm->add_instruction(migraphx::make_op("dequantizelinear"), wq, bcast_axis(mm, ws, 1, {kk, nn}),
                                   bcast_axis(mm, wz, 1, {kk, nn}));
    };
    auto d1 = mm->add_instruction(migraphx::make_op("dot"), qdq(x, 0.02f, {m, k}), weight(k, h));
    auto b1 = mm->add_literal(migraphx::literal{shape{shape::float_type, {h}}, rand_normal(g, h, 0.1f)});
    auto a1 = mm->add_instruction(migraphx::make_op("add"), d1, bcast_axis(mm, b1, 1, {m, h}));
    auto r1 = mm->add_instruction(migraphx::make_op("relu"), a1);
    auto d2 = mm->add_instruction(migraphx::make_op("dot"), qdq(r1, 0.05f, {m, h}), weight(h, n));
    auto b2 = mm->add_literal(migraphx::literal{shape{shape::float_type, {n}}, rand_normal(g, n, 0.1f)});
    auto y  = mm->add_instruction(migraphx::make_op("add"), d2, bcast_axis(mm, b2, 1, {m, n}));
    if(keep_hidden)
        mm->add_return({y, r1});
    else
        mm->add_return({y});
    auto xv = rand_normal(g, m * k, 1.0f);
    migraphx::argument xa{shape{shape::float_type, {m, k}}};
    std::memcpy(xa.data(), xv.data(), xv.size() * sizeof(float));
    t.params["x"] = xa;
    t.exact       = true;
    return t;
}

// The MatMulNBits IR (src/onnx/parse_matmulnbits.cpp:85-158): packed uint8 weights [N,K/2],
// fp16 scales [N,K/g] broadcast over the group, zero point 8 (or explicit), transpose, dot.
inline test_case int4_linear(std::size_t m, std::size_t n, std::size_t k, std::size_t g, bool with_zp,
                      unsigned seed)
{
    test_case t;
    std::mt19937 gen(seed);
    auto* mm   = t.prog.get_main_module();
    auto a     = mm->add_parameter("a", shape{shape::half_type, {m, k}});
    auto bp    = mm->add_literal(migraphx::literal{shape{shape::uint8_type, {n, k / 2}},
                                                rand_ints<uint8_t>(gen, n * k / 2, 0, 255)});
    auto sf    = rand_uniform(gen, n * (k / g), 0.005f, 0.02f);
    std::vector<migraphx::half> sh(sf.size());
    for(std::size_t i = 0; i < sf.size(); ++i)
        sh[i] = migraphx::half(sf[i]);
    auto scales = mm->add_literal(migraphx::literal{shape{shape::half_type, {n, k / g}}, sh});
    auto expand = [&](instruction_ref v) {
        auto u  = mm->add_instruction(migraphx::make_op("unsqueeze", {{"axes", {2}}}), v);
        auto mb = mm->add_instruction(
            migraphx::make_op("multibroadcast", {{"out_lens", {n, k / g, g}}}), u);
        return mm->add_instruction(migraphx::make_op("reshape", {{"dims", {n, k}}}), mb);
    };
    auto unpacked = mm->add_instruction(migraphx::make_op("unpack_int4"), bp);
    instruction_ref zp;
    if(with_zp)
    {
        auto zl = mm->add_literal(migraphx::literal{shape{shape::uint8_type, {n, k / g}},
                                                    rand_ints<uint8_t>(gen, n * (k / g), 0, 15)});
        zp = expand(zl);
    }
    else
    {
        auto z8 = mm->add_literal(migraphx::literal{shape{shape::uint8_type}, std::vector<uint8_t>{8}});
        zp      = mbcast(mm, z8, {n, k});
    }
    auto dq = mm->add_instruction(migraphx::make_op("dequantizelinear"), unpacked, expand(scales), zp);
    auto bt = mm->add_instruction(migraphx::make_op("transpose", {{"permutation", {1, 0}}}), dq);
    auto y  = mm->add_instruction(migraphx::make_op("dot"), a, bt);
    mm->add_return({y});
    auto av = rand_normal(gen, m * k, 1.0f);
    migraphx::argument aa{shape{shape::half_type, {m, k}}};
    auto* ah = reinterpret_cast<migraphx::half*>(aa.data());
    for(std::size_t i = 0; i < av.size(); ++i)
        ah[i] = migraphx::half(av[i]);
    t.params["a"] = aa;
    t.rtol = 2e-2;
    t.atol = 1e-2;
    return t;
}

// quantizelinear and dequantizelinear alone, on parameters.
inline test_case q_dq_ops(unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    const std::size_t r = 48, c = 160;
    auto* mm = t.prog.get_main_module();
    auto x   = mm->add_parameter("x", shape{shape::float_type, {r, c}});
    auto s   = mm->add_literal(migraphx::literal{shape{shape::float_type, {c}}, rand_uniform(g, c, 0.01f, 0.05f)});
    auto z   = mm->add_literal(migraphx::literal{shape{shape::int8_type, {c}}, rand_ints<int8_t>(g, c, -20, 20)});
    auto q   = mm->add_instruction(migraphx::make_op("quantizelinear"), x, bcast_axis(mm, s, 1, {r, c}),
                                 bcast_axis(mm, z, 1, {r, c}));
    // dequantizelinear on its own int8 parameter (a DQ fed by the Q above would be removed
    // as a Q/DQ pair by simplify_qdq)
    auto q2 = mm->add_parameter("q2", shape{shape::int8_type, {r, c}});
    auto d  = mm->add_instruction(migraphx::make_op("dequantizelinear"), q2, bcast_axis(mm, s, 1, {r, c}),
                                 bcast_axis(mm, z, 1, {r, c}));
    mm->add_return({q, d});
    auto xv = rand_normal(g, r * c, 2.0f);
    migraphx::argument xa{shape{shape::float_type, {r, c}}};
    std::memcpy(xa.data(), xv.data(), xv.size() * sizeof(float));
    t.params["x"] = xa;
    auto qv = rand_ints<int8_t>(g, r * c, -128, 127);
    migraphx::argument qa{shape{shape::int8_type, {r, c}}};
    std::memcpy(qa.data(), qv.data(), qv.size());
    t.params["q2"] = qa;
    t.exact       = true;
    return t;
}

// Element-wise operators outside the GEMM patterns (the "next" part of the path): an fp16
// bias + erf-GELU + residual chain as a BERT layer has it between its linears.
inline test_case pw_gelu_f16(unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    const std::size_t r = 96, c = 320;
    auto* mm  = t.prog.get_main_module();
    const shape xs{shape::half_type, {r, c}};
    auto x    = mm->add_parameter("x", xs);
    auto res  = mm->add_parameter("res", xs);
    auto bv   = rand_normal(g, c, 0.3f);
    std::vector<migraphx::half> bh(bv.begin(), bv.end());
    auto bias = mm->add_literal(migraphx::literal{shape{shape::half_type, {c}}, bh});
    auto lit  = [&](float v) {
        auto l = mm->add_literal(migraphx::literal{shape{shape::half_type}, {migraphx::half(v)}});
        return mm->add_instruction(migraphx::make_op("multibroadcast", {{"out_lens", xs.lens()}}), l);
    };
    auto xb   = mm->add_instruction(migraphx::make_op("add"), x, bcast_axis(mm, bias, 1, {r, c}));
    auto u    = mm->add_instruction(migraphx::make_op("mul"), xb, lit(0.70710678f));
    auto e    = mm->add_instruction(migraphx::make_op("erf"), u);
    auto e1   = mm->add_instruction(migraphx::make_op("add"), e, lit(1.0f));
    auto h    = mm->add_instruction(migraphx::make_op("mul"), xb, lit(0.5f));
    auto ge   = mm->add_instruction(migraphx::make_op("mul"), h, e1);
    auto y    = mm->add_instruction(migraphx::make_op("add"), ge, res);
    mm->add_return({y});
    auto fill = [&](const char* name, float sd) {
        auto v = rand_normal(g, r * c, sd);
        std::vector<migraphx::half> hv(v.begin(), v.end());
        migraphx::argument a{xs};
        std::memcpy(a.data(), hv.data(), hv.size() * sizeof(migraphx::half));
        t.params[name] = a;
    };
    fill("x", 1.5f);
    fill("res", 1.0f);
    // libm and CUDA erf differ in the last place; every fp16 operator truncates like the reference
    t.rtol = 4e-3;
    t.atol = 2e-3;
    return t;
}

// fp32 operators with exactly rounded results: bit-exact against ref.
inline test_case pw_arith_f32(unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    const std::size_t b = 3, r = 40, c = 72;
    auto* mm = t.prog.get_main_module();
    const shape xs{shape::float_type, {b, r, c}};
    auto x   = mm->add_parameter("x", xs);
    auto y   = mm->add_parameter("y", xs);
    auto sv  = rand_uniform(g, c, 0.5f, 2.0f);
    auto s   = mm->add_literal(migraphx::literal{shape{shape::float_type, {c}}, sv});
    auto sb  = mm->add_instruction(migraphx::make_op("broadcast", {{"axis", 2}, {"out_lens", xs.lens()}}), s);
    auto d   = mm->add_instruction(migraphx::make_op("div"), x, sb);
    auto a   = mm->add_instruction(migraphx::make_op("abs"), d);
    auto q   = mm->add_instruction(migraphx::make_op("sqrt"), a);
    auto gt  = mm->add_instruction(migraphx::make_op("greater"), x, y);
    auto mn  = mm->add_instruction(migraphx::make_op("min"), x, y);
    auto w   = mm->add_instruction(migraphx::make_op("where"), gt, q, mn);
    auto rl  = mm->add_instruction(migraphx::make_op("relu"), w);
    auto rs  = mm->add_instruction(migraphx::make_op("sub"), rl, y);
    auto n   = mm->add_instruction(migraphx::make_op("neg"), rs);
    auto rc  = mm->add_instruction(migraphx::make_op("recip"), mm->add_instruction(migraphx::make_op("add"), a, sb));
    auto out = mm->add_instruction(migraphx::make_op("mul"), n, rc);
    auto hf  = mm->add_instruction(migraphx::make_op("convert", {{"target_type", migraphx::to_value(shape::half_type)}}), out);
    mm->add_return({out, hf});
    for(const char* name : {"x", "y"})
    {
        auto v = rand_normal(g, b * r * c, 2.0f);
        migraphx::argument arg{xs};
        std::memcpy(arg.data(), v.data(), v.size() * sizeof(float));
        t.params[name] = arg;
    }
    t.exact = true;
    return t;
}

// transcendental operators in fp32: within rtol 1e-5 of ref (libm vs CUDA math library).
inline test_case pw_transcendental_f32(unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    const std::size_t r = 64, c = 200;
    auto* mm = t.prog.get_main_module();
    const shape xs{shape::float_type, {r, c}};
    auto x   = mm->add_parameter("x", xs);
    auto th  = mm->add_instruction(migraphx::make_op("tanh"), x);
    auto sg  = mm->add_instruction(migraphx::make_op("sigmoid"), x);
    auto ex  = mm->add_instruction(migraphx::make_op("exp"), th);
    auto lg  = mm->add_instruction(migraphx::make_op("log"), mm->add_instruction(migraphx::make_op("add"), ex, sg));
    auto er  = mm->add_instruction(migraphx::make_op("erf"), x);
    auto rq  = mm->add_instruction(migraphx::make_op("rsqrt"), mm->add_instruction(migraphx::make_op("add"), ex, ex));
    auto o1  = mm->add_instruction(migraphx::make_op("mul"), lg, er);
    auto o2  = mm->add_instruction(migraphx::make_op("add"), o1, rq);
    mm->add_return({o2});
    auto v = rand_normal(g, r * c, 1.5f);
    migraphx::argument arg{xs};
    std::memcpy(arg.data(), v.data(), v.size() * sizeof(float));
    t.params["x"] = arg;
    t.rtol = 1e-5;
    t.atol = 1e-6;
    return t;
}

// LayerNorm as the ONNX parser decomposes it (reduce_mean, sub, mul, reduce_mean, add eps,
// rsqrt, mul, scale, bias) over the innermost axis of a [batch, seq, hidden] tensor.
inline test_case layernorm(shape::type_t type, std::size_t b, std::size_t sq, std::size_t hid, unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    auto* mm = t.prog.get_main_module();
    const shape xs{type, {b, sq, hid}};
    auto x    = mm->add_parameter("x", xs);
    auto make = [&](const std::vector<float>& v, const std::vector<std::size_t>& lens) {
        if(type == shape::half_type)
        {
            std::vector<migraphx::half> h(v.begin(), v.end());
            return mm->add_literal(migraphx::literal{shape{type, lens}, h});
        }
        return mm->add_literal(migraphx::literal{shape{type, lens}, v});
    };
    auto full = [&](migraphx::instruction_ref r) {
        return mm->add_instruction(migraphx::make_op("multibroadcast", {{"out_lens", xs.lens()}}), r);
    };
    auto gamma = make(rand_uniform(g, hid, 0.5f, 1.5f), {hid});
    auto beta  = make(rand_normal(g, hid, 0.2f), {hid});
    auto eps   = make({1e-5f}, {1});
    auto mean  = mm->add_instruction(migraphx::make_op("reduce_mean", {{"axes", {2}}}), x);
    auto d     = mm->add_instruction(migraphx::make_op("sub"), x, full(mean));
    auto d2    = mm->add_instruction(migraphx::make_op("mul"), d, d);
    auto var   = mm->add_instruction(migraphx::make_op("reduce_mean", {{"axes", {-1}}}), d2);
    auto lens1 = var->get_shape().lens();
    auto epsb  = mm->add_instruction(migraphx::make_op("multibroadcast", {{"out_lens", lens1}}), eps);
    auto rs    = mm->add_instruction(migraphx::make_op("rsqrt"), mm->add_instruction(migraphx::make_op("add"), var, epsb));
    auto nrm   = mm->add_instruction(migraphx::make_op("mul"), d, full(rs));
    auto sc    = mm->add_instruction(migraphx::make_op("mul"), nrm, full(gamma));
    auto y     = mm->add_instruction(migraphx::make_op("add"), sc, full(beta));
    auto mx    = mm->add_instruction(migraphx::make_op("reduce_max", {{"axes", {2}}}), x);
    auto mn    = mm->add_instruction(migraphx::make_op("reduce_min", {{"axes", {2}}}), x);
    auto sm    = mm->add_instruction(migraphx::make_op("reduce_sum", {{"axes", {2}}}), x);
    mm->add_return({y, mx, mn, sm});
    auto v = rand_normal(g, b * sq * hid, 1.0f);
    migraphx::argument arg{xs};
    if(type == shape::half_type)
    {
        std::vector<migraphx::half> h(v.begin(), v.end());
        std::memcpy(arg.data(), h.data(), h.size() * sizeof(migraphx::half));
    }
    else
        std::memcpy(arg.data(), v.data(), v.size() * sizeof(float));
    t.params["x"] = arg;
    // the reference sums sequentially in double, the kernel as an fp32 tree
    t.rtol = type == shape::half_type ? 1e-2 : 1e-5;
    t.atol = type == shape::half_type ? 1e-2 : 2e-5;
    return t;
}

// reductions over axes other than the innermost one: global average pooling over two trailing
// axes, a sum over the middle axis, a maximum over the outermost.
inline test_case reduce_axes(unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    auto* mm = t.prog.get_main_module();
    const shape xs{shape::float_type, {6, 20, 48}};
    auto x  = mm->add_parameter("x", xs);
    auto gp = mm->add_instruction(migraphx::make_op("reduce_mean", {{"axes", {1, 2}}}), x);
    auto sm = mm->add_instruction(migraphx::make_op("reduce_sum", {{"axes", {1}}}), x);
    auto mx = mm->add_instruction(migraphx::make_op("reduce_max", {{"axes", {0}}}), x);
    auto mn = mm->add_instruction(migraphx::make_op("reduce_min", {{"axes", {0, 2}}}), x);
    // consumers, so that the views are read by kernels too
    auto s2 = mm->add_instruction(migraphx::make_op("add"), sm, mbcast(mm, gp, sm->get_shape().lens()));
    mm->add_return({s2, mx, mn, gp});
    auto v = rand_normal(g, xs.elements(), 1.0f);
    migraphx::argument arg{xs};
    std::memcpy(arg.data(), v.data(), v.size() * sizeof(float));
    t.params["x"] = arg;
    t.rtol = 1e-5;
    t.atol = 2e-5;
    return t;
}

// softmax over the innermost axis of attention-score shaped input [batch, heads, q, k].
inline test_case softmax_rows(shape::type_t type, std::size_t b, std::size_t h, std::size_t q, std::size_t k, unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    auto* mm = t.prog.get_main_module();
    const shape xs{type, {b, h, q, k}};
    auto x   = mm->add_parameter("x", xs);
    mm->add_return({mm->add_instruction(migraphx::make_op("softmax", {{"axis", 3}}), x)});
    auto v = rand_normal(g, xs.elements(), 3.0f);
    migraphx::argument arg{xs};
    if(type == shape::half_type)
    {
        std::vector<migraphx::half> hv(v.begin(), v.end());
        std::memcpy(arg.data(), hv.data(), hv.size() * sizeof(migraphx::half));
    }
    else
        std::memcpy(arg.data(), v.data(), v.size() * sizeof(float));
    t.params["x"] = arg;
    t.rtol = type == shape::half_type ? 4e-3 : 1e-5;
    t.atol = type == shape::half_type ? 1e-5 : 1e-8;
    return t;
}

// Multi-head attention on fp16 tensors as the ONNX parser lays it out: [batch, seq, heads * dim]
// projections reshaped and transposed into heads, Q.K^T scaled, softmax, P.V, heads merged back.
inline test_case attention_f16(std::size_t b, std::size_t h, std::size_t sq, std::size_t d, unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    auto* mm = t.prog.get_main_module();
    const shape xs{shape::half_type, {b, sq, h * d}};
    auto heads = [&](const char* name, std::vector<int64_t> perm) {
        auto p = mm->add_parameter(name, xs);
        auto r = mm->add_instruction(migraphx::make_op("reshape", {{"dims", {b, sq, h, d}}}), p);
        return mm->add_instruction(migraphx::make_op("transpose", {{"permutation", perm}}), r);
    };
    auto q  = heads("q", {0, 2, 1, 3});
    auto kt = heads("k", {0, 2, 3, 1});
    auto v  = heads("v", {0, 2, 1, 3});
    auto sc = mm->add_instruction(migraphx::make_op("dot"), q, kt);
    auto l  = mm->add_literal(migraphx::literal{shape{shape::half_type}, {migraphx::half(1.0f / std::sqrt(static_cast<float>(d)))}});
    auto lb = mm->add_instruction(migraphx::make_op("multibroadcast", {{"out_lens", sc->get_shape().lens()}}), l);
    auto ss = mm->add_instruction(migraphx::make_op("mul"), sc, lb);
    auto p  = mm->add_instruction(migraphx::make_op("softmax", {{"axis", 3}}), ss);
    auto o  = mm->add_instruction(migraphx::make_op("dot"), p, v);
    auto ot = mm->add_instruction(migraphx::make_op("transpose", {{"permutation", {0, 2, 1, 3}}}), o);
    auto oc = mm->add_instruction(migraphx::make_op("contiguous"), ot);
    auto y  = mm->add_instruction(migraphx::make_op("reshape", {{"dims", {b, sq, h * d}}}), oc);
    mm->add_return({y});
    for(const char* name : {"q", "k", "v"})
    {
        auto vals = rand_normal(g, xs.elements(), 1.0f);
        std::vector<migraphx::half> hv(vals.begin(), vals.end());
        migraphx::argument arg{xs};
        std::memcpy(arg.data(), hv.data(), hv.size() * sizeof(migraphx::half));
        t.params[name] = arg;
    }
    // fp32 accumulation on the tensor cores against the reference's double, every fp16 result truncated
    t.rtol = 2e-2;
    t.atol = 1e-2;
    return t;
}

// dot on fp16 operands: a constant [K,N] weight (re-laid out once) and a non-constant one.
inline test_case dot_f16(std::size_t bt, std::size_t m, std::size_t n, std::size_t k, bool const_b, unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    auto* mm = t.prog.get_main_module();
    const shape as{shape::half_type, bt > 1 ? std::vector<std::size_t>{bt, m, k} : std::vector<std::size_t>{m, k}};
    const shape bs{shape::half_type, bt > 1 ? std::vector<std::size_t>{bt, k, n} : std::vector<std::size_t>{k, n}};
    auto fill = [&](const shape& s, float sd) {
        auto vals = rand_normal(g, s.elements(), sd);
        std::vector<migraphx::half> hv(vals.begin(), vals.end());
        migraphx::argument arg{s};
        std::memcpy(arg.data(), hv.data(), hv.size() * sizeof(migraphx::half));
        return arg;
    };
    auto a = mm->add_parameter("a", as);
    migraphx::instruction_ref bi;
    if(const_b)
    {
        auto barg = fill(bs, 0.5f);
        bi        = mm->add_literal(migraphx::literal{bs, barg.data()});
    }
    else
    {
        bi            = mm->add_parameter("b", bs);
        t.params["b"] = fill(bs, 0.5f);
    }
    mm->add_return({mm->add_instruction(migraphx::make_op("dot"), a, bi)});
    t.params["a"] = fill(as, 1.0f);
    t.rtol = 2e-2;
    t.atol = 1e-2;
    return t;
}

// One int8 BERT encoder layer end to end: QDQ linears (quant_dot + fused epilogues) for Q, K, V,
// the output projection and the two feed-forward GEMMs, fp16 attention in between, residual adds
// and the decomposed LayerNorms - every operator class of the quantised-GEMM path and its
// neighbours in one program.
inline test_case bert_layer_int8(std::size_t b, std::size_t sq, std::size_t h, std::size_t d, std::size_t ffn, unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    auto* mm            = t.prog.get_main_module();
    const std::size_t m = b * sq, hid = h * d;
    auto x    = mm->add_parameter("x", shape{shape::float_type, {m, hid}});
    auto zero = mm->add_literal(migraphx::literal{shape{shape::int8_type}, std::vector<int8_t>{0}});
    auto flit = [&](float v) { return mm->add_literal(migraphx::literal{shape{shape::float_type}, {v}}); };
    auto qdq  = [&](instruction_ref v, float sc) {
        const auto lens = v->get_shape().lens();
        auto s = flit(sc);
        auto q = mm->add_instruction(migraphx::make_op("quantizelinear"), v, mbcast(mm, s, lens), mbcast(mm, zero, lens));
        return mm->add_instruction(migraphx::make_op("dequantizelinear"), q, mbcast(mm, s, lens), mbcast(mm, zero, lens));
    };
    auto linear = [&](instruction_ref v, float in_scale, std::size_t kk, std::size_t nn) {
        auto wq = mm->add_literal(migraphx::literal{shape{shape::int8_type, {kk, nn}}, rand_ints<int8_t>(g, kk * nn, -127, 127)});
        auto ws = mm->add_literal(migraphx::literal{shape{shape::float_type, {nn}},
                                                    rand_uniform(g, nn, 0.4f / (127.0f * std::sqrt(static_cast<float>(kk))),
                                                                 1.2f / (127.0f * std::sqrt(static_cast<float>(kk))))});
        auto wz = mm->add_literal(migraphx::literal{shape{shape::int8_type, {nn}}, std::vector<int8_t>(nn, 0)});
        auto w  = mm->add_instruction(migraphx::make_op("dequantizelinear"), wq, bcast_axis(mm, ws, 1, {kk, nn}),
                                     bcast_axis(mm, wz, 1, {kk, nn}));
        auto dt = mm->add_instruction(migraphx::make_op("dot"), qdq(v, in_scale), w);
        auto bi = mm->add_literal(migraphx::literal{shape{shape::float_type, {nn}}, rand_normal(g, nn, 0.1f)});
        return mm->add_instruction(migraphx::make_op("add"), dt, bcast_axis(mm, bi, 1, {m, nn}));
    };
    auto layer_norm = [&](instruction_ref v) {
        const auto lens = v->get_shape().lens();
        auto gamma = mm->add_literal(migraphx::literal{shape{shape::float_type, {hid}}, rand_uniform(g, hid, 0.8f, 1.2f)});
        auto beta  = mm->add_literal(migraphx::literal{shape{shape::float_type, {hid}}, rand_normal(g, hid, 0.1f)});
        auto mean  = mm->add_instruction(migraphx::make_op("reduce_mean", {{"axes", {1}}}), v);
        auto dv    = mm->add_instruction(migraphx::make_op("sub"), v, mbcast(mm, mean, lens));
        auto var   = mm->add_instruction(migraphx::make_op("reduce_mean", {{"axes", {1}}}),
                                       mm->add_instruction(migraphx::make_op("mul"), dv, dv));
        auto ve    = mm->add_instruction(migraphx::make_op("add"), var, mbcast(mm, flit(1e-5f), var->get_shape().lens()));
        auto rs    = mm->add_instruction(migraphx::make_op("rsqrt"), ve);
        auto nv    = mm->add_instruction(migraphx::make_op("mul"), dv, mbcast(mm, rs, lens));
        auto sv    = mm->add_instruction(migraphx::make_op("mul"), nv, bcast_axis(mm, gamma, 1, lens));
        return mm->add_instruction(migraphx::make_op("add"), sv, bcast_axis(mm, beta, 1, lens));
    };
    auto heads = [&](instruction_ref v, std::vector<int64_t> perm) {
        auto hv = mm->add_instruction(migraphx::make_op("convert", {{"target_type", migraphx::to_value(shape::half_type)}}), v);
        auto r  = mm->add_instruction(migraphx::make_op("reshape", {{"dims", {b, sq, h, d}}}), hv);
        return mm->add_instruction(migraphx::make_op("transpose", {{"permutation", perm}}), r);
    };
    auto q   = heads(linear(x, 0.03f, hid, hid), {0, 2, 1, 3});
    auto kt  = heads(linear(x, 0.03f, hid, hid), {0, 2, 3, 1});
    auto v   = heads(linear(x, 0.03f, hid, hid), {0, 2, 1, 3});
    auto sc  = mm->add_instruction(migraphx::make_op("dot"), q, kt);
    auto isd = mm->add_literal(migraphx::literal{shape{shape::half_type}, {migraphx::half(1.0f / std::sqrt(static_cast<float>(d)))}});
    auto ss  = mm->add_instruction(migraphx::make_op("mul"), sc, mbcast(mm, isd, sc->get_shape().lens()));
    auto pr  = mm->add_instruction(migraphx::make_op("softmax", {{"axis", 3}}), ss);
    auto cx  = mm->add_instruction(migraphx::make_op("dot"), pr, v);
    auto ct  = mm->add_instruction(migraphx::make_op("transpose", {{"permutation", {0, 2, 1, 3}}}), cx);
    auto cr  = mm->add_instruction(migraphx::make_op("reshape", {{"dims", {m, hid}}}),
                                  mm->add_instruction(migraphx::make_op("contiguous"), ct));
    auto cf  = mm->add_instruction(migraphx::make_op("convert", {{"target_type", migraphx::to_value(shape::float_type)}}), cr);
    auto ao  = mm->add_instruction(migraphx::make_op("add"), linear(cf, 0.02f, hid, hid), x);
    auto h1  = layer_norm(ao);
    // feed-forward: erf-GELU between the two GEMMs
    auto f1  = linear(h1, 0.03f, hid, ffn);
    auto mh  = mm->add_instruction(migraphx::make_op("mul"), f1, mbcast(mm, flit(0.5f), {m, ffn}));
    auto dv  = mm->add_instruction(migraphx::make_op("div"), f1, mbcast(mm, flit(static_cast<float>(M_SQRT2)), {m, ffn}));
    auto er  = mm->add_instruction(migraphx::make_op("erf"), dv);
    auto e1  = mm->add_instruction(migraphx::make_op("add"), er, mbcast(mm, flit(1.0f), {m, ffn}));
    auto ge  = mm->add_instruction(migraphx::make_op("mul"), mh, e1);
    auto f2  = mm->add_instruction(migraphx::make_op("add"), linear(ge, 0.02f, ffn, hid), h1);
    mm->add_return({layer_norm(f2)});
    auto xv = rand_normal(g, m * hid, 1.0f);
    migraphx::argument xa{shape{shape::float_type, {m, hid}}};
    std::memcpy(xa.data(), xv.data(), xv.size() * sizeof(float));
    t.params["x"] = xa;
    // The attention block runs as one kernel that keeps fp32 where the reference's operator chain
    // rounds to half: its results differ by ~1e-3 relative, and this case quantises them with a
    // coarse scale (a handful of int8 levels), so some values land in the neighbouring bucket; each
    // such flip moves an output by about scale_x * |w| before the LayerNorm.  With the attention
    // fusion disabled (MIGRAPHX_CUDA_DISABLE_FUSION=attention) the measured max abs error is 7e-7.
    t.ref_simplify_qdq = true;
    t.rtol = 1e-2;
    t.atol = 2e-3;
    t.outlier_fraction = 3e-2;
    t.outlier_atol     = 6e-2;
    return t;
}

// Token embedding, rotary position embedding (rotate-half form: slice, neg, concat) and the
// KV-cache append of a decoder layer: gather, strided views, element-wise fp16 and concat.
inline test_case embed_rope_f16(std::size_t b, std::size_t sq, std::size_t past, std::size_t hid, std::size_t vocab, unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    auto* mm = t.prog.get_main_module();
    auto half_lit = [&](const std::vector<float>& v, const std::vector<std::size_t>& lens) {
        std::vector<migraphx::half> h(v.begin(), v.end());
        return mm->add_literal(migraphx::literal{shape{shape::half_type, lens}, h});
    };
    auto ids   = mm->add_parameter("ids", shape{shape::int64_type, {b, sq}});
    auto cache = mm->add_parameter("cache", shape{shape::half_type, {b, past, hid}});
    auto table = half_lit(rand_normal(g, vocab * hid, 1.0f), {vocab, hid});
    std::vector<float> cv(sq * hid), sv(sq * hid);
    for(std::size_t p = 0; p < sq; ++p)
        for(std::size_t i = 0; i < hid; ++i)
        {
            const double ang = static_cast<double>(past + p) * std::pow(10000.0, -2.0 * static_cast<double>(i % (hid / 2)) / hid);
            cv[p * hid + i]  = static_cast<float>(std::cos(ang));
            sv[p * hid + i]  = static_cast<float>(std::sin(ang));
        }
    auto cosl = half_lit(cv, {sq, hid});
    auto sinl = half_lit(sv, {sq, hid});
    auto x    = mm->add_instruction(migraphx::make_op("gather", {{"axis", 0}}), table, ids);
    const std::vector<std::size_t> lens = {b, sq, hid};
    auto x1   = mm->add_instruction(migraphx::make_op("slice", {{"axes", {2}}, {"starts", {0}}, {"ends", {hid / 2}}}), x);
    auto x2   = mm->add_instruction(migraphx::make_op("slice", {{"axes", {2}}, {"starts", {hid / 2}}, {"ends", {hid}}}), x);
    auto rot  = mm->add_instruction(migraphx::make_op("concat", {{"axis", 2}}), mm->add_instruction(migraphx::make_op("neg"), x2), x1);
    auto xc   = mm->add_instruction(migraphx::make_op("mul"), x, mbcast(mm, cosl, lens));
    auto rs   = mm->add_instruction(migraphx::make_op("mul"), rot, mbcast(mm, sinl, lens));
    auto y    = mm->add_instruction(migraphx::make_op("add"), xc, rs);
    auto kv   = mm->add_instruction(migraphx::make_op("concat", {{"axis", 1}}), cache, y);
    mm->add_return({kv, y});
    std::uniform_int_distribution<int64_t> pick(-static_cast<int64_t>(vocab), static_cast<int64_t>(vocab) - 1);
    migraphx::argument ia{shape{shape::int64_type, {b, sq}}};
    for(std::size_t i = 0; i < b * sq; ++i)
        reinterpret_cast<int64_t*>(ia.data())[i] = pick(g); // negative indices count from the end
    t.params["ids"] = ia;
    auto cvv = rand_normal(g, b * past * hid, 1.0f);
    std::vector<migraphx::half> ch(cvv.begin(), cvv.end());
    migraphx::argument ca{shape{shape::half_type, {b, past, hid}}};
    std::memcpy(ca.data(), ch.data(), ch.size() * sizeof(migraphx::half));
    t.params["cache"] = ca;
    t.exact = true; // exactly rounded fp16 operators and byte moves
    return t;
}

// An un-quantised fp32 MLP (dot + bias + relu, dot + bias) taken through MIGraphX's own
// quantize_int8 / quantize_fp8 (src/quantization.cpp:88-210: capture operators, a calibration run
// on `calib_target`, then Q/DQ pairs with the measured scales) - the program a user of the
// reference would hand to a target.
inline test_case quantized_mlp(std::size_t mrows, std::size_t k, std::size_t h, std::size_t n, bool fp8,
                               const std::string& calib_target, unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    auto* mm = t.prog.get_main_module();
    auto x   = mm->add_parameter("x", shape{shape::float_type, {mrows, k}});
    auto w1  = mm->add_literal(migraphx::literal{shape{shape::float_type, {k, h}}, rand_normal(g, k * h, 0.06f)});
    auto b1  = mm->add_literal(migraphx::literal{shape{shape::float_type, {h}}, rand_normal(g, h, 0.1f)});
    auto w2  = mm->add_literal(migraphx::literal{shape{shape::float_type, {h, n}}, rand_normal(g, h * n, 0.06f)});
    auto b2  = mm->add_literal(migraphx::literal{shape{shape::float_type, {n}}, rand_normal(g, n, 0.1f)});
    auto d1  = mm->add_instruction(migraphx::make_op("dot"), x, w1);
    auto a1  = mm->add_instruction(migraphx::make_op("add"), d1, bcast_axis(mm, b1, 1, {mrows, h}));
    auto r1  = mm->add_instruction(migraphx::make_op("relu"), a1);
    auto d2  = mm->add_instruction(migraphx::make_op("dot"), r1, w2);
    auto y   = mm->add_instruction(migraphx::make_op("add"), d2, bcast_axis(mm, b2, 1, {mrows, n}));
    mm->add_return({y});
    auto fill = [&](unsigned sd) {
        std::mt19937 gg(sd);
        auto v = rand_normal(gg, mrows * k, 1.0f);
        migraphx::argument a{shape{shape::float_type, {mrows, k}}};
        std::memcpy(a.data(), v.data(), v.size() * sizeof(float));
        return a;
    };
    // calibration data: two seeded batches
    std::vector<migraphx::parameter_map> calib = {{{"x", fill(seed + 1)}}, {{"x", fill(seed + 2)}}};
    auto ct = migraphx::make_target(calib_target);
    if(fp8)
        migraphx::quantize_fp8(t.prog, ct, calib);
    else
        migraphx::quantize_int8(t.prog, ct, calib);
    t.params["x"] = fill(seed + 3);
    // both targets run the quantised program; ref after simplify_qdq, like every GPU pipeline
    t.ref_simplify_qdq = true;
    t.rtol = fp8 ? 2e-2 : 1e-5;
    t.atol = fp8 ? 1e-2 : 2e-5;
    return t;
}

// An fp16 linear whose weight literal went through MIGraphX's quantize_int4_weights
// (src/quantization.cpp:189-192, src/quantize_int4.cpp:38-103): per-tensor scale and zero point,
// [K, N] weight, nibbles packed along N.
inline test_case int4_weights_pass_linear(std::size_t mrows, std::size_t k, std::size_t n, unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    auto* mm = t.prog.get_main_module();
    auto a   = mm->add_parameter("a", shape{shape::half_type, {mrows, k}});
    auto wf  = rand_normal(g, k * n, 0.05f);
    std::vector<migraphx::half> wh(wf.begin(), wf.end());
    auto w   = mm->add_literal(migraphx::literal{shape{shape::half_type, {k, n}}, wh});
    mm->add_return({mm->add_instruction(migraphx::make_op("dot"), a, w)});
    migraphx::quantize_int4_weights(t.prog);
    auto av = rand_normal(g, mrows * k, 1.0f);
    std::vector<migraphx::half> ah(av.begin(), av.end());
    migraphx::argument aa{shape{shape::half_type, {mrows, k}}};
    std::memcpy(aa.data(), ah.data(), ah.size() * sizeof(migraphx::half));
    t.params["a"] = aa;
    t.rtol = 2e-2;
    t.atol = 1e-2;
    return t;
}

// quant_dot whose left operand is a transposed 4-D view ([B,S,H,D] seen as [B,H,S,D], the heads
// of an attention block): its batch entries are not evenly spaced in memory.
inline test_case quant_dot_transposed_a(unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    const std::size_t b = 2, sq = 24, h = 3, d = 32, n = 16;
    auto* mm = t.prog.get_main_module();
    auto a   = mm->add_parameter("a", shape{shape::int8_type, {b, sq, h, d}});
    auto at  = mm->add_instruction(migraphx::make_op("transpose", {{"permutation", {0, 2, 1, 3}}}), a);
    auto w   = mm->add_parameter("b", shape{shape::int8_type, {b, h, d, n}});
    mm->add_return({mm->add_instruction(migraphx::make_op("quant_dot"), at, w)});
    auto av = rand_ints<int8_t>(g, b * sq * h * d, -128, 127);
    auto bv = rand_ints<int8_t>(g, b * h * d * n, -128, 127);
    migraphx::argument aa{shape{shape::int8_type, {b, sq, h, d}}}, ba{shape{shape::int8_type, {b, h, d, n}}};
    std::memcpy(aa.data(), av.data(), av.size());
    std::memcpy(ba.data(), bv.data(), bv.size());
    t.params["a"] = aa;
    t.params["b"] = ba;
    t.exact       = true;
    return t;
}

// quant_dot alone at GEMM-benchmark size, the reference evaluated on a sample of rows.
inline test_case raw_quant_dot_sampled(std::size_t m, std::size_t k, std::size_t n, unsigned seed, std::size_t ref_rows)
{
    auto build = [&](std::size_t rows) {
        migraphx::program p;
        auto* mm = p.get_main_module();
        auto x   = mm->add_parameter("a", shape{shape::int8_type, {rows, k}});
        auto w   = mm->add_parameter("b", shape{shape::int8_type, {k, n}});
        mm->add_return({mm->add_instruction(migraphx::make_op("quant_dot"), x, w)});
        return p;
    };
    test_case t;
    std::mt19937 g(seed);
    t.prog  = build(m);
    auto av = rand_ints<int8_t>(g, m * k, -128, 127);
    auto bv = rand_ints<int8_t>(g, k * n, -128, 127);
    migraphx::argument aa{shape{shape::int8_type, {m, k}}}, ba{shape{shape::int8_type, {k, n}}};
    std::memcpy(aa.data(), av.data(), av.size());
    std::memcpy(ba.data(), bv.data(), bv.size());
    t.params["a"] = aa;
    t.params["b"] = ba;
    t.exact       = true;
    if(ref_rows < m)
    {
        t.sampled         = true;
        t.sample_rows     = pick_rows(m, ref_rows, seed + 1000);
        t.ref_prog        = build(ref_rows);
        t.ref_params["a"] = take_rows(aa, t.sample_rows);
        t.ref_params["b"] = ba;
    }
    return t;
}

// quant_dot alone on int8 parameters (batched, non-constant right operand).
inline test_case raw_quant_dot(unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    const std::size_t b = 2, m = 72, k = 160, n = 48;
    auto* mm = t.prog.get_main_module();
    auto x   = mm->add_parameter("a", shape{shape::int8_type, {b, m, k}});
    auto w   = mm->add_parameter("b", shape{shape::int8_type, {b, k, n}});
    mm->add_return({mm->add_instruction(migraphx::make_op("quant_dot"), x, w)});
    auto av = rand_ints<int8_t>(g, b * m * k, -128, 127);
    auto bv = rand_ints<int8_t>(g, b * k * n, -128, 127);
    migraphx::argument aa{shape{shape::int8_type, {b, m, k}}}, ba{shape{shape::int8_type, {b, k, n}}};
    std::memcpy(aa.data(), av.data(), av.size());
    std::memcpy(ba.data(), bv.data(), bv.size());
    t.params["a"] = aa;
    t.params["b"] = ba;
    t.exact       = true;
    return t;
}

// ---------------------------------------------------------------------------------------------
// A QDQ linear whose reference is evaluated on a seeded sample of rows (see test_case::sampled):
// the large points of the fp8 / int8 GEMM sweeps.
inline test_case qdq_linear_sampled(std::size_t m, std::size_t k, std::size_t n, shape::type_t qtype,
                                    const std::string& act, bool per_channel, unsigned seed,
                                    std::size_t ref_rows)
{
    test_case t = qdq_linear(m, k, n, qtype, act, per_channel, seed);
    if(ref_rows >= m)
        return t;
    test_case small = qdq_linear(ref_rows, k, n, qtype, act, per_channel, seed);
    t.sampled       = true;
    t.sample_rows   = pick_rows(m, ref_rows, seed + 1000);
    t.ref_prog      = small.prog;
    t.ref_params["x"] = take_rows(t.params.at("x"), t.sample_rows);
    return t;
}

// heavy_tail: a few activations per row are hundreds of times larger than the rest, as the
// outlier channels of real decoder activations are.
inline test_case int4_linear_sampled(std::size_t m, std::size_t n, std::size_t k, std::size_t g, bool with_zp,
                                     unsigned seed, std::size_t ref_rows, bool heavy_tail = false)
{
    test_case t = int4_linear(m, n, k, g, with_zp, seed);
    t.atol_row_rms = heavy_tail;
    if(heavy_tail)
    {
        std::mt19937 gen(seed + 77);
        std::uniform_int_distribution<std::size_t> col(0, k - 1);
        std::uniform_real_distribution<float> mag(100.0f, 1000.0f);
        auto* ah = reinterpret_cast<migraphx::half*>(t.params.at("a").data());
        for(std::size_t r = 0; r < m; ++r)
            for(int j = 0; j < 6; ++j)
                ah[r * k + col(gen)] = migraphx::half((j % 2 == 0 ? 1.0f : -1.0f) * mag(gen));
    }
    if(ref_rows >= m)
        return t;
    test_case small = int4_linear(ref_rows, n, k, g, with_zp, seed);
    t.sampled       = true;
    t.sample_rows   = pick_rows(m, ref_rows, seed + 1000);
    t.ref_prog      = small.prog;
    t.ref_params["a"] = take_rows(t.params.at("a"), t.sample_rows);
    return t;
}

// ---------------------------------------------------------------------------------------------
// BERT-shaped int8 encoder stack in fp16 (BASELINE config 2): token + position embedding,
// LayerNorm, then `layers` encoder layers.  Every linear (Q, K, V, attention output, the two
// feed-forward GEMMs) is a QDQ int8 linear in the form an fp16 model with ONNX-style Q/DQ nodes
// has after parsing: quantizelinear(x, s_x) -> dequantizelinear(fp32 scale) -> convert(half) on the
// activation (per-tensor scale), dequantizelinear(per-output-channel scale) -> convert(half) on the
// int8 weight literal, dot in half, bias add in half (src/simplify_qdq.cpp:140-146, 283-287 is the
// "fp16 model" form simplify_qdq recognises).  Softmax, GELU, residual adds and the LayerNorms (in
// the ONNX parser's decomposition) are fp16.
struct bert_config
{
    std::size_t batch = 1, seq = 384, layers = 12, hidden = 768, heads = 12, ffn = 3072, vocab = 30522;
    unsigned seed = 0;
    // activation scales, four per layer in the order q/k/v input (shared), attention-output
    // projection input, ffn1 input, ffn2 input.  Empty: calibrate - the linears stay un-quantised fp16
    // dots and the program returns, after the encoder output, the per-row max |x| of every
    // linear's input (four [tokens, 1] tensors per layer).
    std::vector<float> act_scales;
    bool calibrate() const { return act_scales.empty(); }
};

struct bert_program
{
    migraphx::program prog;
    std::size_t tokens     = 0;
    double quant_ops       = 0; // sum of 2*M*N*K over the QDQ linears
};

inline bert_program bert_encoder_int8(const bert_config& c)
{
    bert_program bp;
    std::mt19937 g(c.seed);
    auto* mm             = bp.prog.get_main_module();
    const std::size_t m  = c.batch * c.seq, hid = c.hidden, d = c.hidden / c.heads;
    bp.tokens            = m;
    const auto half_t    = shape::half_type;
    auto to_half = [&](instruction_ref v) {
        return mm->add_instruction(migraphx::make_op("convert", {{"target_type", migraphx::to_value(half_t)}}), v);
    };
    auto half_lit = [&](const std::vector<float>& v, const std::vector<std::size_t>& lens) {
        std::vector<migraphx::half> h(v.begin(), v.end());
        return mm->add_literal(migraphx::literal{shape{half_t, lens}, h});
    };
    auto hscalar = [&](float v, const std::vector<std::size_t>& lens) {
        auto l = mm->add_literal(migraphx::literal{shape{half_t}, {migraphx::half(v)}});
        return mbcast(mm, l, lens);
    };
    auto zero8 = mm->add_literal(migraphx::literal{shape{shape::int8_type}, std::vector<int8_t>{0}});
    std::vector<instruction_ref> calib_out;
    std::size_t scale_idx = 0;

    // activation side of a QDQ linear: quantised once per distinct input (q, k, v share it)
    auto quantise_act = [&](instruction_ref v) -> instruction_ref {
        const auto lens = v->get_shape().lens();
        if(c.calibrate())
        {
            auto ab = mm->add_instruction(migraphx::make_op("abs"), v);
            calib_out.push_back(mm->add_instruction(migraphx::make_op("reduce_max", {{"axes", {1}}}), ab));
            return v;
        }
        const float sc = c.act_scales.at(scale_idx++);
        const migraphx::half sh(sc);
        auto s_h = mm->add_literal(migraphx::literal{shape{half_t}, {sh}});
        auto s_f = mm->add_literal(migraphx::literal{shape{shape::float_type}, {static_cast<float>(sh)}});
        auto q   = mm->add_instruction(migraphx::make_op("quantizelinear"), v, mbcast(mm, s_h, lens), mbcast(mm, zero8, lens));
        auto dq  = mm->add_instruction(migraphx::make_op("dequantizelinear"), q, mbcast(mm, s_f, lens), mbcast(mm, zero8, lens));
        return to_half(dq);
    };
    // weight side + dot + bias: weights ~ N(0, 0.02), int8 per output channel (scale = max|w| / 127)
    auto linear = [&](instruction_ref xq, std::size_t kk, std::size_t nn) {
        std::normal_distribution<float> nd(0.0f, 0.02f);
        std::vector<float> w(kk * nn), colmax(nn, 0.0f);
        for(std::size_t i = 0; i < kk; ++i)
            for(std::size_t j = 0; j < nn; ++j)
            {
                const float v = nd(g);
                w[i * nn + j] = v;
                colmax[j]     = std::max(colmax[j], std::fabs(v));
            }
        std::vector<float> ws(nn);
        std::vector<int8_t> wq(kk * nn);
        for(std::size_t j = 0; j < nn; ++j)
            ws[j] = colmax[j] / 127.0f;
        for(std::size_t i = 0; i < kk; ++i)
            for(std::size_t j = 0; j < nn; ++j)
                wq[i * nn + j] = static_cast<int8_t>(std::max(-127.0f, std::min(127.0f, std::nearbyint(w[i * nn + j] / ws[j]))));
        auto wl  = mm->add_literal(migraphx::literal{shape{shape::int8_type, {kk, nn}}, wq});
        auto wsl = mm->add_literal(migraphx::literal{shape{shape::float_type, {nn}}, ws});
        auto wzl = mm->add_literal(migraphx::literal{shape{shape::int8_type, {nn}}, std::vector<int8_t>(nn, 0)});
        auto wdq = mm->add_instruction(migraphx::make_op("dequantizelinear"), wl, bcast_axis(mm, wsl, 1, {kk, nn}),
                                       bcast_axis(mm, wzl, 1, {kk, nn}));
        auto dt  = mm->add_instruction(migraphx::make_op("dot"), xq, to_half(wdq));
        auto bi  = half_lit(rand_normal(g, nn, 0.02f), {nn});
        bp.quant_ops += 2.0 * static_cast<double>(m) * static_cast<double>(kk) * static_cast<double>(nn);
        return mm->add_instruction(migraphx::make_op("add"), dt, bcast_axis(mm, bi, 1, {m, nn}));
    };
    // LayerNorm over the innermost axis as the ONNX parser decomposes it (src/onnx/parse_layernorm.cpp)
    auto layer_norm = [&](instruction_ref v) {
        const auto lens = v->get_shape().lens();
        auto gamma = half_lit(rand_uniform(g, hid, 0.8f, 1.2f), {hid});
        auto beta  = half_lit(rand_normal(g, hid, 0.1f), {hid});
        auto mean  = mm->add_instruction(migraphx::make_op("reduce_mean", {{"axes", {1}}}), v);
        auto dv    = mm->add_instruction(migraphx::make_op("sub"), v, mbcast(mm, mean, lens));
        auto var   = mm->add_instruction(migraphx::make_op("reduce_mean", {{"axes", {1}}}),
                                       mm->add_instruction(migraphx::make_op("mul"), dv, dv));
        auto ve    = mm->add_instruction(migraphx::make_op("add"), var, hscalar(1e-5f, var->get_shape().lens()));
        auto rs    = mm->add_instruction(migraphx::make_op("rsqrt"), ve);
        auto nv    = mm->add_instruction(migraphx::make_op("mul"), dv, mbcast(mm, rs, lens));
        auto sv    = mm->add_instruction(migraphx::make_op("mul"), nv, bcast_axis(mm, gamma, 1, lens));
        return mm->add_instruction(migraphx::make_op("add"), sv, bcast_axis(mm, beta, 1, lens));
    };
    auto heads = [&](instruction_ref v, std::vector<int64_t> perm) {
        auto r = mm->add_instruction(migraphx::make_op("reshape", {{"dims", {c.batch, c.seq, c.heads, d}}}), v);
        return mm->add_instruction(migraphx::make_op("transpose", {{"permutation", perm}}), r);
    };

    // embeddings
    auto ids   = mm->add_parameter("ids", shape{shape::int32_type, {c.batch, c.seq}});
    auto table = half_lit(rand_normal(g, c.vocab * hid, 0.5f), {c.vocab, hid});
    auto pos   = half_lit(rand_normal(g, c.seq * hid, 0.5f), {c.seq, hid});
    auto tok   = mm->add_instruction(migraphx::make_op("gather", {{"axis", 0}}), table, ids); // [B,S,H]
    auto emb   = mm->add_instruction(migraphx::make_op("add"), tok,
                                     mm->add_instruction(migraphx::make_op("broadcast", {{"axis", 1}, {"out_lens", tok->get_shape().lens()}}), pos));
    instruction_ref x = layer_norm(mm->add_instruction(migraphx::make_op("reshape", {{"dims", {m, hid}}}), emb));

    for(std::size_t l = 0; l < c.layers; ++l)
    {
        auto xq  = quantise_act(x);
        auto q   = heads(linear(xq, hid, hid), {0, 2, 1, 3});
        auto kt  = heads(linear(xq, hid, hid), {0, 2, 3, 1});
        auto v   = heads(linear(xq, hid, hid), {0, 2, 1, 3});
        auto sc  = mm->add_instruction(migraphx::make_op("dot"), q, kt);
        auto ss  = mm->add_instruction(migraphx::make_op("mul"), sc,
                                       hscalar(1.0f / std::sqrt(static_cast<float>(d)), sc->get_shape().lens()));
        auto pr  = mm->add_instruction(migraphx::make_op("softmax", {{"axis", 3}}), ss);
        auto cx  = mm->add_instruction(migraphx::make_op("dot"), pr, v);
        auto ct  = mm->add_instruction(migraphx::make_op("transpose", {{"permutation", {0, 2, 1, 3}}}), cx);
        auto cr  = mm->add_instruction(migraphx::make_op("reshape", {{"dims", {m, hid}}}),
                                       mm->add_instruction(migraphx::make_op("contiguous"), ct));
        auto ao  = mm->add_instruction(migraphx::make_op("add"), linear(quantise_act(cr), hid, hid), x);
        auto h1  = layer_norm(ao);
        auto f1  = linear(quantise_act(h1), hid, c.ffn);
        // erf-GELU (src/op/builder/gelu.cpp:58-74)
        const std::vector<std::size_t> fl = {m, c.ffn};
        auto mh  = mm->add_instruction(migraphx::make_op("mul"), f1, hscalar(0.5f, fl));
        auto dv  = mm->add_instruction(migraphx::make_op("div"), f1, hscalar(static_cast<float>(M_SQRT2), fl));
        auto er  = mm->add_instruction(migraphx::make_op("erf"), dv);
        auto e1  = mm->add_instruction(migraphx::make_op("add"), er, hscalar(1.0f, fl));
        auto ge  = mm->add_instruction(migraphx::make_op("mul"), mh, e1);
        auto f2  = mm->add_instruction(migraphx::make_op("add"), linear(quantise_act(ge), c.ffn, hid), h1);
        x        = layer_norm(f2);
    }
    std::vector<instruction_ref> rets = {x};
    rets.insert(rets.end(), calib_out.begin(), calib_out.end());
    mm->add_return(rets);
    return bp;
}

// ---------------------------------------------------------------------------------------------
// GroupQueryAttention of a decoder layer exactly as the ONNX parser decomposes it
// (src/onnx/parse_group_query_attention.cpp:113-268): packed QKV -> heads, rotary embedding of Q
// and K through the rotary_embedding builder (src/op/builder/rotary_embedding.cpp: gathernd of the
// cos / sin caches at the positions, rotate-half, mul, add), concat_past_present of K and V into
// the fp16 caches, grouped-query broadcast of the KV heads, Q K^T over the whole cache length,
// masks by position and by past length, softmax, P V, heads merged.  seq = 1: a decode step at the
// past lengths `seqlens`; seq > 1: the prompt.  Returns {attention output, K cache, V cache}.
inline std::vector<instruction_ref> add_gqa(migraphx::module* mm, instruction_ref qkv, instruction_ref past_k,
                                            instruction_ref past_v, instruction_ref slk, instruction_ref cos_cache,
                                            instruction_ref sin_cache, std::size_t num_heads,
                                            std::size_t kv_num_heads, bool use_rotary_op = false)
{
    using migraphx::make_op;
    const auto& q_lens                = qkv->get_shape().lens();
    const std::size_t batch_size      = q_lens[0];
    const std::size_t sequence_length = q_lens[1];
    const std::size_t head_size       = q_lens[2] / (num_heads + 2 * kv_num_heads);
    const auto dtype                  = qkv->get_shape().type();
    std::vector<std::size_t> bsnh{batch_size, sequence_length, num_heads + 2 * kv_num_heads, head_size};
    auto tq = mm->add_instruction(make_op("reshape", {{"dims", bsnh}}), qkv);
    tq      = mm->add_instruction(make_op("transpose", {{"permutation", {0, 2, 1, 3}}}), tq);
    instruction_ref qk, cur_v;
    if(use_rotary_op)
    {
        // the single-operator form (op::gqa_rotary_embedding rotates Q and K of the packed tensor)
        auto rot = mm->add_instruction(
            make_op("gqa_rotary_embedding",
                    {{"num_heads", num_heads}, {"kv_num_heads", kv_num_heads}, {"interleaved", false}}),
            mm->add_instruction(make_op("contiguous"), tq), slk, cos_cache, sin_cache);
        qk    = mm->add_instruction(make_op("slice", {{"axes", {1}}, {"starts", {0}}, {"ends", {num_heads + kv_num_heads}}}), rot);
        cur_v = mm->add_instruction(make_op("slice", {{"axes", {1}}, {"starts", {num_heads + kv_num_heads}}, {"ends", {num_heads + 2 * kv_num_heads}}}), rot);
    }
    else
    {
        qk    = mm->add_instruction(make_op("slice", {{"axes", {1}}, {"starts", {0}}, {"ends", {num_heads + kv_num_heads}}}), tq);
        cur_v = mm->add_instruction(make_op("slice", {{"axes", {1}}, {"starts", {num_heads + kv_num_heads}}, {"ends", {num_heads + 2 * kv_num_heads}}}), tq);
        auto pos_ids = slk;
        if(sequence_length > 1)
            pos_ids = mm->add_literal(migraphx::literal{shape{slk->get_shape().type(), {1}}, {0}});
        qk = migraphx::op::builder::add("rotary_embedding", *mm, {qk, pos_ids, cos_cache, sin_cache},
                                        {{"interleaved", false}})
                 .at(0);
    }
    auto q     = mm->add_instruction(make_op("slice", {{"axes", {1}}, {"starts", {0}}, {"ends", {num_heads}}}), qk);
    auto cur_k = mm->add_instruction(make_op("slice", {{"axes", {1}}, {"starts", {num_heads}}, {"ends", {num_heads + kv_num_heads}}}), qk);
    auto k = mm->add_instruction(make_op("concat_past_present", {{"kv_num_heads", kv_num_heads}}), cur_k, slk, past_k);
    auto v = mm->add_instruction(make_op("concat_past_present", {{"kv_num_heads", kv_num_heads}}), cur_v, slk, past_v);
    auto k_out = k, v_out = v;
    const auto factor      = num_heads / kv_num_heads;
    const auto max_seq_len = k->get_shape().lens()[2];
    auto past_sl = mm->add_instruction(make_op("multibroadcast", {{"out_lens", {batch_size, num_heads}}}), slk);
    if(factor != 1)
    {
        auto kv_new_lens  = k->get_shape().lens();
        kv_new_lens.at(1) = num_heads;
        k = mm->add_instruction(make_op("unsqueeze", {{"axes", {2}}}), k);
        v = mm->add_instruction(make_op("unsqueeze", {{"axes", {2}}}), v);
        auto ul  = k->get_shape().lens();
        ul.at(2) = factor;
        k = mm->add_instruction(make_op("multibroadcast", {{"out_lens", ul}}), k);
        v = mm->add_instruction(make_op("multibroadcast", {{"out_lens", ul}}), v);
        k = mm->add_instruction(make_op("reshape", {{"dims", kv_new_lens}}), k);
        v = mm->add_instruction(make_op("reshape", {{"dims", kv_new_lens}}), v);
    }
    auto kt    = mm->add_instruction(make_op("transpose", {{"permutation", {0, 1, 3, 2}}}), k);
    auto gemm1 = mm->add_instruction(make_op("dot"), q, kt);
    std::vector<int> range_vec(max_seq_len);
    std::iota(range_vec.begin(), range_vec.end(), 0);
    auto range = mm->add_literal(migraphx::literal{shape{past_sl->get_shape().type(), {max_seq_len}}, range_vec});
    std::vector<std::size_t> bnsm{batch_size, num_heads, sequence_length, max_seq_len};
    auto bc_range = mm->add_instruction(make_op("multibroadcast", {{"out_lens", bnsm}}), range);
    const shape scalar_s{dtype, {1}};
    auto ninf = mm->add_literal(migraphx::literal{scalar_s, {-std::numeric_limits<float>::infinity()}});
    ninf      = mm->add_instruction(make_op("multibroadcast", {{"out_lens", bnsm}}), ninf);
    auto scale_ins = mm->add_literal(migraphx::literal{scalar_s, {1.0f / std::sqrt(static_cast<float>(head_size))}});
    scale_ins      = mm->add_instruction(make_op("multibroadcast", {{"out_lens", bnsm}}), scale_ins);
    auto mul       = mm->add_instruction(make_op("mul"), gemm1, scale_ins);
    if(sequence_length > 1)
    {
        std::vector<int> sr(sequence_length);
        std::iota(sr.begin(), sr.end(), 0);
        auto seq_range = mm->add_literal(migraphx::literal{shape{past_sl->get_shape().type(), {sequence_length}}, sr});
        seq_range = mm->add_instruction(make_op("reshape", {{"dims", {sequence_length, 1}}}), seq_range);
        seq_range = mm->add_instruction(make_op("multibroadcast", {{"out_lens", bnsm}}), seq_range);
        auto causal = mm->add_instruction(make_op("greater"), bc_range, seq_range);
        causal = mm->add_instruction(make_op("convert", {{"target_type", migraphx::to_value(shape::bool_type)}}), causal);
        mul    = mm->add_instruction(make_op("where"), causal, ninf, mul);
    }
    auto bc_past_sl = mm->add_instruction(make_op("reshape", {{"dims", {batch_size, num_heads, 1, 1}}}), past_sl);
    auto mask_comp  = mm->add_instruction(make_op("multibroadcast", {{"out_lens", bnsm}}), bc_past_sl);
    auto mask       = mm->add_instruction(make_op("greater"), bc_range, mask_comp);
    mask = mm->add_instruction(make_op("convert", {{"target_type", migraphx::to_value(shape::bool_type)}}), mask);
    auto where   = mm->add_instruction(make_op("where"), mask, ninf, mul);
    auto softmax = mm->add_instruction(make_op("softmax", {{"axis", 3}}), where);
    auto scores  = mm->add_instruction(make_op("dot"), softmax, v);
    auto out     = mm->add_instruction(make_op("transpose", {{"permutation", {0, 2, 1, 3}}}), scores);
    out = mm->add_instruction(make_op("reshape", {{"dims", {batch_size, sequence_length, head_size * num_heads}}}), out);
    return {out, k_out, v_out};
}

// The attention block of a decoder layer by itself, on parameters.  For a decode step the past
// lengths differ per batch entry; the caches hold random history.
inline test_case gqa_attention(std::size_t batch, std::size_t num_heads, std::size_t kv_heads, std::size_t head,
                               std::size_t seq, std::size_t cache_len, bool use_rotary_op, unsigned seed)
{
    test_case t;
    std::mt19937 g(seed);
    auto* mm = t.prog.get_main_module();
    const std::size_t width = (num_heads + 2 * kv_heads) * head;
    auto half_arg = [&](const shape& s, float sd) {
        auto v = rand_normal(g, s.elements(), sd);
        std::vector<migraphx::half> h(v.begin(), v.end());
        migraphx::argument a{s};
        std::memcpy(a.data(), h.data(), h.size() * sizeof(migraphx::half));
        return a;
    };
    const shape qkv_s{shape::half_type, {batch, seq, width}};
    const shape kv_s{shape::half_type, {batch, kv_heads, cache_len, head}};
    const shape slk_s{shape::int32_type, {batch, 1}};
    auto qkv    = mm->add_parameter("qkv", qkv_s);
    auto past_k = mm->add_parameter("past_k", kv_s);
    auto past_v = mm->add_parameter("past_v", kv_s);
    auto slk    = mm->add_parameter("seqlens_k", slk_s);
    std::vector<migraphx::half> cosv(cache_len * head / 2), sinv(cache_len * head / 2);
    for(std::size_t p = 0; p < cache_len; ++p)
        for(std::size_t i = 0; i < head / 2; ++i)
        {
            const double ang = static_cast<double>(p) * std::pow(10000.0, -2.0 * static_cast<double>(i) / head);
            cosv[p * head / 2 + i] = migraphx::half(static_cast<float>(std::cos(ang)));
            sinv[p * head / 2 + i] = migraphx::half(static_cast<float>(std::sin(ang)));
        }
    auto cosl = mm->add_literal(migraphx::literal{shape{shape::half_type, {cache_len, head / 2}}, cosv});
    auto sinl = mm->add_literal(migraphx::literal{shape{shape::half_type, {cache_len, head / 2}}, sinv});
    mm->add_return(add_gqa(mm, qkv, past_k, past_v, slk, cosl, sinl, num_heads, kv_heads, use_rotary_op));
    t.params["qkv"]    = half_arg(qkv_s, 1.0f);
    t.params["past_k"] = half_arg(kv_s, 1.0f);
    t.params["past_v"] = half_arg(kv_s, 1.0f);
    migraphx::argument sa{slk_s};
    std::uniform_int_distribution<int32_t> pick(static_cast<int32_t>(cache_len / 2), static_cast<int32_t>(cache_len - seq - 1));
    for(std::size_t b = 0; b < batch; ++b)
        reinterpret_cast<int32_t*>(sa.data())[b] = seq == 1 ? pick(g) : static_cast<int32_t>(seq - 1);
    t.params["seqlens_k"] = sa;
    t.rtol = 2e-2;
    t.atol = 1e-2;
    return t;
}

// ---------------------------------------------------------------------------------------------
// One Llama-shaped decoder layer at a decode step, as a front end hands it over: RMSNorm in the
// parser's decomposition (src/onnx/parse_simplified_layer_normalization.cpp:91-106: convert to
// float, mul, reduce_mean, convert back, add eps, rsqrt, mul, mul), weight-only int4 linears in the
// MatMulNBits IR (src/onnx/parse_matmulnbits.cpp:85-158; packed QKV, O, gate, up, down),
// GroupQueryAttention in the parser's decomposition (add_gqa above) against fp16 KV caches, SwiGLU
// (mul(gate, sigmoid(gate)) * up) and the two residual adds.  Returns {layer output, K cache, V cache}.
inline instruction_ref add_int4_matmul(migraphx::module* mm, instruction_ref a, std::size_t n, std::size_t k,
                                       std::size_t g, std::mt19937& gen)
{
    auto bp = mm->add_literal(
        migraphx::literal{shape{shape::uint8_type, {n, k / 2}}, rand_ints<uint8_t>(gen, n * k / 2, 0, 255)});
    // scales that keep the result of order one for inputs of order one (nibbles - 8 have rms 4.6)
    const float s0 = 1.0f / (4.6f * std::sqrt(static_cast<float>(k)));
    auto sf        = rand_uniform(gen, n * (k / g), 0.6f * s0, 1.4f * s0);
    std::vector<migraphx::half> sh(sf.begin(), sf.end());
    auto scales = mm->add_literal(migraphx::literal{shape{shape::half_type, {n, k / g}}, sh});
    auto u      = mm->add_instruction(migraphx::make_op("unsqueeze", {{"axes", {2}}}), scales);
    auto mb     = mm->add_instruction(migraphx::make_op("multibroadcast", {{"out_lens", {n, k / g, g}}}), u);
    auto se     = mm->add_instruction(migraphx::make_op("reshape", {{"dims", {n, k}}}), mb);
    auto z8     = mm->add_literal(migraphx::literal{shape{shape::uint8_type}, std::vector<uint8_t>{8}});
    auto zp     = mbcast(mm, z8, {n, k});
    auto unpacked = mm->add_instruction(migraphx::make_op("unpack_int4"), bp);
    auto dq       = mm->add_instruction(migraphx::make_op("dequantizelinear"), unpacked, se, zp);
    auto bt       = mm->add_instruction(migraphx::make_op("transpose", {{"permutation", {1, 0}}}), dq);
    return mm->add_instruction(migraphx::make_op("dot"), a, bt);
}

inline instruction_ref add_rmsnorm(migraphx::module* mm, instruction_ref x, std::size_t hidden, std::mt19937& gen)
{
    using migraphx::make_op;
    auto gv = rand_uniform(gen, hidden, 0.8f, 1.2f);
    std::vector<migraphx::half> gh(gv.begin(), gv.end());
    auto gamma = mm->add_literal(migraphx::literal{shape{shape::half_type, {hidden}}, gh});
    auto fx    = mm->add_instruction(make_op("convert", {{"target_type", migraphx::to_value(shape::float_type)}}), x);
    auto sq    = migraphx::add_common_op(*mm, make_op("mul"), {fx, fx});
    auto rms   = mm->add_instruction(make_op("reduce_mean", {{"axes", {1}}}), sq);
    rms        = mm->add_instruction(make_op("convert", {{"target_type", migraphx::to_value(shape::half_type)}}), rms);
    auto eps   = mm->add_literal(migraphx::literal{shape{shape::half_type}, {1e-5f}});
    rms        = migraphx::add_common_op(*mm, make_op("add"), {rms, eps});
    auto rrms  = mm->add_instruction(make_op("rsqrt"), rms);
    auto y     = migraphx::add_common_op(*mm, make_op("mul"), {x, rrms});
    return migraphx::add_common_op(*mm, make_op("mul"), {y, gamma});
}

inline test_case llama_decoder_layer(std::size_t batch, std::size_t hidden, std::size_t heads, std::size_t kv_heads,
                                     std::size_t head, std::size_t ffn, std::size_t cache_len, std::size_t group,
                                     unsigned seed)
{
    using migraphx::make_op;
    test_case t;
    std::mt19937 g(seed);
    auto* mm = t.prog.get_main_module();
    const std::size_t width = (heads + 2 * kv_heads) * head;
    const shape x_s{shape::half_type, {batch, hidden}}; // one token per batch entry
    const shape kv_s{shape::half_type, {batch, kv_heads, cache_len, head}};
    const shape slk_s{shape::int32_type, {batch, 1}};
    auto x      = mm->add_parameter("x", x_s);
    auto past_k = mm->add_parameter("past_k", kv_s);
    auto past_v = mm->add_parameter("past_v", kv_s);
    auto slk    = mm->add_parameter("seqlens_k", slk_s);
    std::vector<migraphx::half> cosv(cache_len * head / 2), sinv(cache_len * head / 2);
    for(std::size_t p = 0; p < cache_len; ++p)
        for(std::size_t i = 0; i < head / 2; ++i)
        {
            const double ang = static_cast<double>(p) * std::pow(10000.0, -2.0 * static_cast<double>(i) / head);
            cosv[p * head / 2 + i] = migraphx::half(static_cast<float>(std::cos(ang)));
            sinv[p * head / 2 + i] = migraphx::half(static_cast<float>(std::sin(ang)));
        }
    auto cosl = mm->add_literal(migraphx::literal{shape{shape::half_type, {cache_len, head / 2}}, cosv});
    auto sinl = mm->add_literal(migraphx::literal{shape{shape::half_type, {cache_len, head / 2}}, sinv});

    auto h1   = add_rmsnorm(mm, x, hidden, g);
    auto qkv  = add_int4_matmul(mm, h1, width, hidden, group, g);
    auto qkv3 = mm->add_instruction(make_op("reshape", {{"dims", {batch, std::size_t{1}, width}}}), qkv);
    auto att  = add_gqa(mm, qkv3, past_k, past_v, slk, cosl, sinl, heads, kv_heads);
    auto a2   = mm->add_instruction(make_op("reshape", {{"dims", {batch, heads * head}}}), att[0]);
    auto o    = add_int4_matmul(mm, a2, hidden, heads * head, group, g);
    auto r1   = mm->add_instruction(make_op("add"), x, o);
    auto h2   = add_rmsnorm(mm, r1, hidden, g);
    auto gate = add_int4_matmul(mm, h2, ffn, hidden, group, g);
    auto up   = add_int4_matmul(mm, h2, ffn, hidden, group, g);
    auto sg   = mm->add_instruction(make_op("sigmoid"), gate);
    auto act  = mm->add_instruction(make_op("mul"), mm->add_instruction(make_op("mul"), gate, sg), up);
    auto down = add_int4_matmul(mm, act, hidden, ffn, group, g);
    auto y    = mm->add_instruction(make_op("add"), r1, down);
    mm->add_return({y, att[1], att[2]});

    auto half_arg = [&](const shape& s, float sd) {
        auto v = rand_normal(g, s.elements(), sd);
        std::vector<migraphx::half> h(v.begin(), v.end());
        migraphx::argument a{s};
        std::memcpy(a.data(), h.data(), h.size() * sizeof(migraphx::half));
        return a;
    };
    t.params["x"]      = half_arg(x_s, 1.0f);
    t.params["past_k"] = half_arg(kv_s, 1.0f);
    t.params["past_v"] = half_arg(kv_s, 1.0f);
    migraphx::argument sa{slk_s};
    std::uniform_int_distribution<int32_t> pick(static_cast<int32_t>(cache_len / 2), static_cast<int32_t>(cache_len - 2));
    for(std::size_t b = 0; b < batch; ++b)
        reinterpret_cast<int32_t*>(sa.data())[b] = pick(g);
    t.params["seqlens_k"] = sa;
    t.rtol = 2e-2;
    t.atol = 1e-2;
    return t;
}

// ---------------------------------------------------------------------------------------------
// Tensor-parallel int4 MLP of one rank (config 5's sharding): up projection split by output
// columns, down projection by input rows, the partial result summed over the ranks by
// cuda::all_reduce inside the compiled program.  ref_prog is the unsharded MLP (the oracle);
// every rank builds the same seeded full weights and keeps its slice.
inline test_case tp_int4_mlp(std::size_t rank, std::size_t world, std::size_t m, std::size_t hidden, std::size_t ffn,
                             std::size_t g, unsigned seed)
{
    using migraphx::make_op;
    test_case t;
    std::mt19937 gen(seed);
    const auto up_w = rand_ints<uint8_t>(gen, ffn * hidden / 2, 0, 255);    // [ffn, hidden / 2]
    const auto dn_w = rand_ints<uint8_t>(gen, hidden * ffn / 2, 0, 255);    // [hidden, ffn / 2]
    auto to_half    = [](const std::vector<float>& v) { return std::vector<migraphx::half>(v.begin(), v.end()); };
    const auto up_s = to_half(rand_uniform(gen, ffn * (hidden / g), 0.6f / (4.6f * std::sqrt(float(hidden))),
                                           1.4f / (4.6f * std::sqrt(float(hidden)))));
    const auto dn_s = to_half(rand_uniform(gen, hidden * (ffn / g), 0.6f / (4.6f * std::sqrt(float(ffn))),
                                           1.4f / (4.6f * std::sqrt(float(ffn)))));
    auto linear = [&](migraphx::module* mm, instruction_ref a, const std::vector<uint8_t>& w,
                      const std::vector<migraphx::half>& sc, std::size_t n, std::size_t k) {
        auto bp     = mm->add_literal(migraphx::literal{shape{shape::uint8_type, {n, k / 2}}, w});
        auto scales = mm->add_literal(migraphx::literal{shape{shape::half_type, {n, k / g}}, sc});
        auto u      = mm->add_instruction(make_op("unsqueeze", {{"axes", {2}}}), scales);
        auto mb     = mm->add_instruction(make_op("multibroadcast", {{"out_lens", {n, k / g, g}}}), u);
        auto se     = mm->add_instruction(make_op("reshape", {{"dims", {n, k}}}), mb);
        auto z8     = mm->add_literal(migraphx::literal{shape{shape::uint8_type}, std::vector<uint8_t>{8}});
        auto dq     = mm->add_instruction(make_op("dequantizelinear"), mm->add_instruction(make_op("unpack_int4"), bp),
                                      se, mbcast(mm, z8, {n, k}));
        return mm->add_instruction(make_op("dot"), a,
                                   mm->add_instruction(make_op("transpose", {{"permutation", {1, 0}}}), dq));
    };
    const shape xs{shape::half_type, {m, hidden}};
    {
        // the unsharded MLP
        auto* mm = t.ref_prog.get_main_module();
        auto x   = mm->add_parameter("x", xs);
        auto h   = linear(mm, x, up_w, up_s, ffn, hidden);
        mm->add_return({linear(mm, h, dn_w, dn_s, hidden, ffn)});
    }
    {
        const std::size_t fr = ffn / world; // this rank's columns of the hidden layer
        std::vector<uint8_t> uw(up_w.begin() + rank * fr * hidden / 2, up_w.begin() + (rank + 1) * fr * hidden / 2);
        std::vector<migraphx::half> us(up_s.begin() + rank * fr * (hidden / g), up_s.begin() + (rank + 1) * fr * (hidden / g));
        std::vector<uint8_t> dw(hidden * fr / 2);
        std::vector<migraphx::half> ds(hidden * (fr / g));
        for(std::size_t r = 0; r < hidden; ++r)
        {
            std::copy_n(dn_w.begin() + r * ffn / 2 + rank * fr / 2, fr / 2, dw.begin() + r * fr / 2);
            std::copy_n(dn_s.begin() + r * (ffn / g) + rank * (fr / g), fr / g, ds.begin() + r * (fr / g));
        }
        auto* mm = t.prog.get_main_module();
        auto x   = mm->add_parameter("x", xs);
        auto h   = linear(mm, x, uw, us, fr, hidden);
        auto y   = linear(mm, h, dw, ds, hidden, fr);
        mm->add_return({mm->add_instruction(make_op("cuda::all_reduce"), y)});
    }
    auto xv = rand_normal(gen, m * hidden, 1.0f);
    std::vector<migraphx::half> xh(xv.begin(), xv.end());
    migraphx::argument xa{xs};
    std::memcpy(xa.data(), xh.data(), xh.size() * sizeof(migraphx::half));
    t.params["x"]     = xa;
    t.ref_params["x"] = xa;
    t.sampled         = true;
    t.sample_rows.resize(m);
    std::iota(t.sample_rows.begin(), t.sample_rows.end(), std::size_t{0});
    t.rtol = 2e-2;
    t.atol = 1e-2;
    return t;
}

// seeded token ids in [0, vocab)
inline migraphx::argument bert_ids(const bert_config& c, unsigned seed)
{
    std::mt19937 g(seed);
    std::uniform_int_distribution<int32_t> pick(0, static_cast<int32_t>(c.vocab) - 1);
    migraphx::argument a{shape{shape::int32_type, {c.batch, c.seq}}};
    auto* p = reinterpret_cast<int32_t*>(a.data());
    for(std::size_t i = 0; i < c.batch * c.seq; ++i)
        p[i] = pick(g);
    return a;
}

// Activation scales (max |x| / 127 per linear input) from the outputs of the calibration program.
inline std::vector<float> bert_scales_from_calibration(const std::vector<migraphx::argument>& host_outputs)
{
    std::vector<float> scales;
    for(std::size_t i = 1; i < host_outputs.size(); ++i)
    {
        float amax = 0.0f;
        host_outputs[i].visit([&](auto v) {
            for(auto x : v)
                amax = std::max(amax, static_cast<float>(x));
        });
        scales.push_back(std::max(amax, 1e-3f) / 127.0f);
    }
    return scales;
}

// The calibrated config-2 program: runs the calibration program once on `calib_target` (device
// buffers through the target's copy_to / copy_from) with seeded token ids and builds the
// quantised program with the activation scales it measured.  use_device = false (a machine
// without a GPU, where only the pass pipeline is exercised): typical fixed scales instead.
inline bert_program bert_encoder_int8_calibrated(bert_config c, bool use_device, std::vector<float>* scales_out = nullptr,
                                                 const std::string& calib_target = "cuda")
{
    if(not use_device)
    {
        for(std::size_t l = 0; l < c.layers; ++l)
            c.act_scales.insert(c.act_scales.end(), {0.04f, 0.006f, 0.04f, 0.03f});
        return bert_encoder_int8(c);
    }
    bert_config cc = c;
    cc.act_scales.clear();
    auto cal = bert_encoder_int8(cc);
    auto t   = migraphx::make_target(calib_target);
    cal.prog.compile(t);
    migraphx::parameter_map pm;
    for(const auto& ps : cal.prog.get_parameter_shapes())
        pm[ps.first] = ps.first == "ids" ? t.copy_to(bert_ids(cc, cc.seed + 4242)) : t.allocate(ps.second);
    auto outs = cal.prog.eval(pm);
    std::vector<migraphx::argument> host;
    for(const auto& o : outs)
        host.push_back(t.copy_from(o));
    c.act_scales = bert_scales_from_calibration(host);
    if(scales_out != nullptr)
        *scales_out = c.act_scales;
    return bert_encoder_int8(c);
}

} // namespace mgx_programs
#endif

