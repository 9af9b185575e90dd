// cuda_target_check: builds MIGraphX programs of the quantized-GEMM path with the public
// module API, runs them on MIGraphX's CPU `ref` target and on the `cuda` target and compares
// the results - the same scheme as the reference's cross-target verify harness
// (test/verify/run_verify.cpp:176-259), for the programs this target supports.
//
//   cuda_target_check passes <case>          print the program after the cuda pass pipeline
//                                            (no GPU needed: finalize is not run)
//   cuda_target_check run <case> [offload]   compile + eval on ref and cuda, print one JSON line
//   cuda_target_check list
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
#include <chrono>
#include <cmath>
#include <cstring>
#include <iostream>
#include <map>
#include <random>
#include <functional>

using migraphx::shape;
using migraphx::instruction_ref;

namespace {

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
};

template <class T>
std::vector<T> rand_ints(std::mt19937& g, std::size_t n, int lo, int hi)
{
    std::uniform_int_distribution<int> d(lo, hi);
    std::vector<T> v(n);
    for(auto& x : v)
        x = static_cast<T>(d(g));
    return v;
}

std::vector<float> rand_normal(std::mt19937& g, std::size_t n, float sd)
{
    std::normal_distribution<float> d(0.0f, sd);
    std::vector<float> v(n);
    for(auto& x : v)
        x = d(g);
    return v;
}

std::vector<float> rand_uniform(std::mt19937& g, std::size_t n, float lo, float hi)
{
    std::uniform_real_distribution<float> d(lo, hi);
    std::vector<float> v(n);
    for(auto& x : v)
        x = d(g);
    return v;
}

instruction_ref mbcast(migraphx::module* mm, instruction_ref x, const std::vector<std::size_t>& lens)
{
    return mm->add_instruction(migraphx::make_op("multibroadcast", {{"out_lens", lens}}), x);
}

instruction_ref bcast_axis(migraphx::module* mm, instruction_ref x, std::size_t axis,
                           const std::vector<std::size_t>& lens)
{
    return mm->add_instruction(migraphx::make_op("broadcast", {{"axis", axis}, {"out_lens", lens}}), x);
}

// Q -> DQ on the activation, DQ on the int8/fp8 weight literal, dot, + bias, activation:
// the fake-quantised form quantize_int8 / quantize_fp8 leave behind.
test_case qdq_linear(std::size_t m, std::size_t k, std::size_t n, shape::type_t qtype,
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
test_case qdq_mlp(std::size_t m, std::size_t k, std::size_t h, std::size_t n, bool keep_hidden, unsigned seed)
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
test_case int4_linear(std::size_t m, std::size_t n, std::size_t k, std::size_t g, bool with_zp,
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
test_case q_dq_ops(unsigned seed)
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
test_case pw_gelu_f16(unsigned seed)
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
test_case pw_arith_f32(unsigned seed)
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
test_case pw_transcendental_f32(unsigned seed)
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
test_case layernorm(shape::type_t type, std::size_t b, std::size_t sq, std::size_t hid, unsigned seed)
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
test_case reduce_axes(unsigned seed)
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
test_case softmax_rows(shape::type_t type, std::size_t b, std::size_t h, std::size_t q, std::size_t k, unsigned seed)
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
test_case attention_f16(std::size_t b, std::size_t h, std::size_t sq, std::size_t d, unsigned seed)
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
test_case dot_f16(std::size_t bt, std::size_t m, std::size_t n, std::size_t k, bool const_b, unsigned seed)
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
test_case bert_layer_int8(std::size_t b, std::size_t sq, std::size_t h, std::size_t d, std::size_t ffn, unsigned seed)
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
    // measured: max abs error 7e-7.  The bound leaves room for one int8 value of the output
    // projection's input landing in the neighbouring bucket (fp16 attention: fp32 against double
    // accumulation), which moves an output by about scale_x * scale_w * |w| before the LayerNorm
    t.ref_simplify_qdq = true;
    t.rtol = 1e-2;
    t.atol = 2e-3;
    return t;
}

// Token embedding, rotary position embedding (rotate-half form: slice, neg, concat) and the
// KV-cache append of a decoder layer: gather, strided views, element-wise fp16 and concat.
test_case embed_rope_f16(std::size_t b, std::size_t sq, std::size_t past, std::size_t hid, std::size_t vocab, unsigned seed)
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

// quant_dot alone on int8 parameters (batched, non-constant right operand).
test_case raw_quant_dot(unsigned seed)
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

std::map<std::string, std::function<test_case()>> cases()
{
    return {
        {"c1", [] { auto t = qdq_linear(256, 1024, 1024, shape::int8_type, "relu", true, 0); t.exact = true; return t; }},
        {"c1_small", [] { auto t = qdq_linear(64, 256, 96, shape::int8_type, "relu", true, 1); t.exact = true; return t; }},
        {"c1_semantic", [] { return qdq_linear(64, 256, 96, shape::int8_type, "relu", true, 1); }},
        {"int8_gelu", [] { return qdq_linear(128, 256, 320, shape::int8_type, "gelu", true, 2); }},
        {"int8_per_tensor", [] { auto t = qdq_linear(100, 128, 72, shape::int8_type, "none", false, 3); t.exact = true; return t; }},
        {"fp8_gelu", [] { return qdq_linear(128, 512, 256, shape::fp8e4m3fn_type, "gelu", false, 4); }},
        {"int4_decode", [] { return int4_linear(1, 256, 512, 128, false, 5); }},
        {"int4_batch16_zp", [] { return int4_linear(16, 128, 1024, 32, true, 6); }},
        {"int4_batch8_zp", [] { return int4_linear(8, 384, 1024, 128, true, 7); }},
        {"int4_prefill", [] { return int4_linear(96, 256, 512, 128, true, 8); }},
        {"pw_gelu_f16", [] { return pw_gelu_f16(9); }},
        {"pw_arith_f32", [] { return pw_arith_f32(10); }},
        {"pw_transcendental_f32", [] { return pw_transcendental_f32(11); }},
        {"layernorm_f32", [] { return layernorm(shape::float_type, 2, 48, 768, 12); }},
        {"layernorm_f16", [] { return layernorm(shape::half_type, 3, 20, 1000, 13); }},
        {"reduce_axes", [] { return reduce_axes(24); }},
        {"softmax_f32", [] { return softmax_rows(shape::float_type, 2, 4, 56, 200, 14); }},
        {"softmax_f16", [] { return softmax_rows(shape::half_type, 1, 3, 40, 1500, 15); }},
        {"softmax_f32_long", [] { return softmax_rows(shape::float_type, 1, 1, 6, 9000, 16); }},
        {"attention_f16", [] { return attention_f16(2, 4, 64, 32, 17); }},
        {"dot_f16_const", [] { return dot_f16(1, 200, 136, 264, true, 18); }},
        {"dot_f16_batched", [] { return dot_f16(3, 72, 50, 96, false, 19); }},
        {"dot_f16_odd_k", [] { return dot_f16(2, 50, 64, 197, false, 22); }},
        {"dot_f16_odd_k_const", [] { return dot_f16(1, 33, 40, 13, true, 23); }},
        {"bert_layer_int8", [] { return bert_layer_int8(2, 64, 4, 64, 1024, 20); }},
        {"embed_rope_f16", [] { return embed_rope_f16(2, 24, 40, 128, 500, 21); }},
        {"q_dq_ops", [] { return q_dq_ops(7); }},
        {"mlp_fused_q", [] { return qdq_mlp(96, 256, 320, 128, false, 9); }},
        {"mlp_two_outputs", [] { return qdq_mlp(96, 256, 320, 128, true, 10); }},
        {"raw_quant_dot", [] { return raw_quant_dot(8); }},
    };
}

struct cmp_result
{
    double max_abs = 0, max_rel = 0;
    std::size_t mismatched = 0, n = 0;
};

cmp_result compare(const migraphx::argument& ref, const migraphx::argument& got, bool exact, double rtol,
                   double atol)
{
    cmp_result r;
    if(ref.get_shape().lens() != got.get_shape().lens() or ref.get_shape().type() != got.get_shape().type())
    {
        r.mismatched = 1u << 30;
        return r;
    }
    r.n = ref.get_shape().elements();
    if(exact)
    {
        const auto es = ref.get_shape().type_size();
        for(std::size_t i = 0; i < r.n; ++i)
            if(std::memcmp(ref.data() + i * es, got.data() + i * es, es) != 0)
                ++r.mismatched;
        return r;
    }
    std::vector<double> a(r.n), b(r.n);
    ref.visit([&](auto v) { std::size_t i = 0; for(auto x : v) a[i++] = static_cast<double>(x); });
    got.visit([&](auto v) { std::size_t i = 0; for(auto x : v) b[i++] = static_cast<double>(x); });
    for(std::size_t i = 0; i < r.n; ++i)
    {
        const double d = std::fabs(a[i] - b[i]);
        r.max_abs      = std::max(r.max_abs, d);
        if(std::fabs(a[i]) > 0)
            r.max_rel = std::max(r.max_rel, d / std::fabs(a[i]));
        if(not(d <= atol + rtol * std::fabs(a[i])))
            ++r.mismatched;
    }
    return r;
}

} // namespace

int main(int argc, char** argv)
{
    const auto all = cases();
    if(argc < 2 or std::string(argv[1]) == "list")
    {
        for(const auto& c : all)
            std::cout << c.first << "\n";
        return 0;
    }
    const std::string mode = argv[1];
    const std::string name = argc > 2 ? argv[2] : "c1_small";
    const bool offload     = argc > 3 and std::string(argv[3]) == "offload";
    const bool prefused    = argc > 3 and std::string(argv[3]) == "prefused";
    if(all.count(name) == 0)
    {
        std::cerr << "unknown case " << name << "\n";
        return 2;
    }
    try
    {
        test_case t = all.at(name)();
        auto cuda_t = migraphx::make_target("cuda");
        if(mode == "passes")
        {
            migraphx::program p = t.prog;
            auto ctx            = cuda_t.get_context();
            migraphx::compile_options opts;
            opts.offload_copy = offload;
            if(prefused)
                migraphx::run_passes(p, {migraphx::simplify_qdq{}, migraphx::dead_code_elimination{},
                                         migraphx::fuse_pointwise{}, migraphx::dead_code_elimination{}});
            migraphx::run_passes(p, cuda_t.get_passes(ctx, opts));
            std::cout << p << std::endl;
            return 0;
        }
        // reference result
        migraphx::program pr = t.prog;
        if(t.exact or t.ref_simplify_qdq)
            migraphx::run_passes(pr, {migraphx::simplify_qdq{}, migraphx::dead_code_elimination{}});
        pr.compile(migraphx::make_target("ref"));
        auto t0       = std::chrono::steady_clock::now();
        auto ref_out  = pr.eval(t.params);
        double ref_s  = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        // cuda result
        migraphx::program pc = t.prog;
        if(prefused)
            migraphx::run_passes(pc, {migraphx::simplify_qdq{}, migraphx::dead_code_elimination{},
                                      migraphx::fuse_pointwise{}, migraphx::dead_code_elimination{}});
        migraphx::compile_options opts;
        opts.offload_copy = offload;
        pc.compile(cuda_t, opts);
        migraphx::parameter_map pm;
        for(const auto& ps : pc.get_parameter_shapes())
        {
            if(t.params.count(ps.first) > 0)
                pm[ps.first] = offload ? t.params.at(ps.first) : cuda_t.copy_to(t.params.at(ps.first));
            else
                pm[ps.first] = cuda_t.allocate(ps.second);
        }
        auto cuda_out = pc.eval(pm);
        // the target runs the first evals instruction by instruction and then records them as
        // a CUDA graph: time the steady state
        for(int i = 0; i < 4; ++i)
            cuda_out = pc.eval(pm);
        pc.finish();
        auto t1 = std::chrono::steady_clock::now();
        const int reps = 100;
        for(int i = 0; i < reps; ++i)
            cuda_out = pc.eval(pm);
        pc.finish();
        double cuda_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t1).count() / reps;
        bool ok = ref_out.size() == cuda_out.size();
        std::cout << "{\"case\": \"" << name << "\", \"offload\": " << (offload ? "true" : "false")
                  << ", \"prefused\": " << (prefused ? "true" : "false") << ", \"outputs\": [";
        for(std::size_t i = 0; i < ref_out.size() and i < cuda_out.size(); ++i)
        {
            auto host = offload ? cuda_out[i] : cuda_t.copy_from(cuda_out[i]);
            auto c    = compare(ref_out[i], host, t.exact, t.rtol, t.atol);
            ok        = ok and c.mismatched == 0;
            std::cout << (i ? ", " : "") << "{\"n\": " << c.n << ", \"mismatched\": " << c.mismatched
                      << ", \"max_abs\": " << c.max_abs << ", \"max_rel\": " << c.max_rel << "}";
        }
        // the same program with other parameter buffers (the recorded graph does not apply:
        // the target has to notice, run instruction by instruction and record again)
        bool rebind_ok = true;
        if(not offload)
        {
            migraphx::parameter_map pm2;
            for(const auto& ps : pc.get_parameter_shapes())
            {
                if(t.params.count(ps.first) > 0)
                    pm2[ps.first] = cuda_t.copy_to(t.params.at(ps.first));
                else
                    pm2[ps.first] = cuda_t.allocate(ps.second);
            }
            std::vector<migraphx::argument> out2;
            for(int i = 0; i < 5; ++i)
                out2 = pc.eval(pm2);
            pc.finish();
            rebind_ok = out2.size() == ref_out.size();
            for(std::size_t i = 0; i < ref_out.size() and i < out2.size(); ++i)
                rebind_ok = rebind_ok and
                            compare(ref_out[i], cuda_t.copy_from(out2[i]), t.exact, t.rtol, t.atol).mismatched == 0;
            ok = ok and rebind_ok;
        }
        std::cout << "], \"exact\": " << (t.exact ? "true" : "false") << ", \"ref_seconds\": " << ref_s
                  << ", \"cuda_seconds\": " << cuda_s << ", \"rebind\": " << (rebind_ok ? "true" : "false")
                  << ", \"pass\": " << (ok ? "true" : "false") << "}"
                  << std::endl;
        return ok ? 0 : 1;
    }
    catch(const std::exception& e)
    {
        std::cout << "{\"case\": \"" << name << "\", \"error\": \"" << e.what() << "\", \"pass\": false}"
                  << std::endl;
        return 3;
    }
}
