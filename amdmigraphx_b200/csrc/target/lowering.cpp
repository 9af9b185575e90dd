// cuda::lowering - replaces the quantized-GEMM sub-graphs of a MIGraphX module by the
// operators of the `cuda` target and refuses everything else (no CPU fallback).
//
// What arrives here (after simplify_qdq, src/simplify_qdq.cpp:225-290):
//   quant_dot(xq, wq) -> dequantizelinear(acc, mul(bcast(x_scale), bcast(w_scale)))
//        [-> convert(half)] [-> add(broadcast(bias))] [-> relu | erf-GELU] [-> add(residual)]
// and, for weight-only int4 (src/onnx/parse_matmulnbits.cpp:85-158):
//   dot(A, transpose(dequantizelinear(unpack_int4(packed), scales[N,K], zero_points[N,K])))
// The HIP target does the equivalent in src/targets/gpu/lowering.cpp:62-613 (operator
// replacement + output allocation) and src/targets/gpu/fuse_mlir.cpp:709-807, 1161-1276
// (GEMM + pointwise / dequantize / unpack_int4 fusion); nothing is shared with that code.
#include "cuda_ops.hpp"
#include <migraphx/errors.hpp>
#include <migraphx/dead_code_elimination.hpp>
#include <migraphx/instruction.hpp>
#include <migraphx/iterator_for.hpp>
#include <migraphx/builtin.hpp>
#include <migraphx/literal.hpp>
#include <migraphx/make_op.hpp>
#include <migraphx/module.hpp>
#include <migraphx/pass_manager.hpp>
#include <migraphx/ranges.hpp>
#include <migraphx/stringutils.hpp>
#include <migraphx/half.hpp>
#include "../../../include/mgx_cuda.h"
#include <algorithm>
#include <functional>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <set>
#include <unordered_map>
#include <unordered_set>

namespace migraphx {
inline namespace MIGRAPHX_INLINE_NS {
namespace cuda {

namespace {

// Context-free operators whose compute() only re-describes the buffer (no data is read):
// they work on device pointers unchanged.
bool is_view_op(const std::string& n)
{
    static const std::set<std::string> views = {
        "broadcast", "multibroadcast", "transpose", "reshape_lazy", "squeeze", "unsqueeze",
        "flatten", "slice", "identity", "load", "get_tuple_elem", "step"};
    return views.count(n) > 0;
}

bool is_builtin(const std::string& n) { return not n.empty() and n.front() == '@'; }

instruction_ref insert_allocation(module& m, instruction_ref pos, const shape& s)
{
    return m.insert_instruction(pos, make_op("allocate", {{"shape", to_value(s)}}));
}

// Host copy of a constant instruction's value as fp32, element by element in logical order.
std::vector<float> eval_as_floats(instruction_ref ins)
{
    argument a = ins->eval();
    if(a.empty())
        MIGRAPHX_THROW("cuda::lowering: expected a compile-time constant");
    std::vector<float> out(a.get_shape().elements());
    a.visit([&](auto v) {
        std::size_t i = 0;
        for(auto x : v)
            out[i++] = static_cast<float>(x);
    });
    return out;
}

enum class bcast_kind
{
    scalar,
    per_col,
    per_row,
    full
};

struct const_vector
{
    bcast_kind kind = bcast_kind::full;
    std::vector<float> values; // 1, cols or rows values
};

// Classifies a constant of the data tensor's dims seen as [rows, cols] by evaluating all of it.
const_vector classify_constant_dense(instruction_ref ins)
{
    const auto& s    = ins->get_shape();
    const auto vals  = eval_as_floats(ins);
    const_vector r;
    if(vals.empty())
        return r;
    const std::size_t cols = s.ndim() == 0 ? 1 : s.lens().back();
    const std::size_t rows = vals.size() / cols;
    auto same              = [](float a, float b) { return std::memcmp(&a, &b, sizeof(float)) == 0; };
    bool all_same = true, col_const = true, row_const = true;
    for(std::size_t i = 0; i < vals.size() and (all_same or col_const or row_const); ++i)
    {
        const std::size_t rr = i / cols, cc = i % cols;
        if(not same(vals[i], vals[0]))
            all_same = false;
        if(not same(vals[i], vals[cc]))
            col_const = false; // differs from row 0 in the same column
        if(not same(vals[i], vals[rr * cols]))
            row_const = false; // differs from column 0 in the same row
    }
    if(all_same)
    {
        r.kind   = bcast_kind::scalar;
        r.values = {vals[0]};
    }
    else if(col_const)
    {
        r.kind = bcast_kind::per_col;
        r.values.assign(vals.begin(), vals.begin() + cols);
    }
    else if(row_const and s.ndim() == 2)
    {
        r.kind = bcast_kind::per_row;
        r.values.resize(rows);
        for(std::size_t i = 0; i < rows; ++i)
            r.values[i] = vals[i * cols];
    }
    return r;
}

// The same answer read off the structure of the expression where that is possible - broadcasts
// of small literals and fp32 products of them, which is what simplify_qdq builds for scales
// (src/simplify_qdq.cpp:243-248) and what biases and scalar constants look like - so that a
// [tokens, features] view of a handful of numbers is never materialised.  false: not recognised.
bool classify_structural(instruction_ref ins, const_vector& out)
{
    const auto& s  = ins->get_shape();
    const auto nd  = s.ndim();
    const auto name = ins->name();
    if(nd == 0 or s.elements() == 0)
        return false;
    if(name == "multibroadcast" or name == "broadcast")
    {
        auto x = ins->inputs().front();
        if(not x->can_eval() or ins->inputs().size() != 1)
            return false;
        const auto& st = s.strides();
        const auto& ln = s.lens();
        std::size_t moving = 0, axis = 0; // axes the view actually steps along
        for(std::size_t i = 0; i < nd; ++i)
            if(ln[i] != 1 and st[i] != 0)
            {
                ++moving;
                axis = i;
            }
        if(moving > 1)
            return false;
        const auto vals = eval_as_floats(x);
        if(moving == 0)
        {
            if(vals.empty())
                return false;
            out.kind   = bcast_kind::scalar;
            out.values = {vals[0]};
            return true;
        }
        if(vals.size() != ln[axis] or st[axis] != 1)
            return false;
        if(axis == nd - 1)
            out.kind = bcast_kind::per_col;
        else if(axis == nd - 2 and nd == 2)
            out.kind = bcast_kind::per_row;
        else
            return false;
        out.values = vals;
        return true;
    }
    if(name == "mul" and s.type() == shape::float_type and ins->inputs().size() == 2)
    {
        const_vector a, b;
        if(not classify_structural(ins->inputs()[0], a) or not classify_structural(ins->inputs()[1], b))
            return false;
        if(a.kind == bcast_kind::scalar)
            std::swap(a, b);
        if(b.kind != bcast_kind::scalar and b.kind != a.kind)
            return false;
        out.kind = a.kind;
        out.values.resize(a.values.size());
        for(std::size_t i = 0; i < a.values.size(); ++i)
            out.values[i] = a.values[i] * (b.kind == bcast_kind::scalar ? b.values[0] : b.values[i]);
        // a vector whose entries are all equal is a scalar to the kernels
        return true;
    }
    return false;
}

const_vector classify_constant(instruction_ref ins)
{
    const_vector r;
    if(classify_structural(ins, r))
    {
        if(r.kind != bcast_kind::scalar and not r.values.empty() and
           std::all_of(r.values.begin(), r.values.end(), [&](float v) {
               return std::memcmp(&v, &r.values[0], sizeof(float)) == 0;
           }))
        {
            r.kind   = bcast_kind::scalar;
            r.values = {r.values[0]};
        }
        return r;
    }
    return classify_constant_dense(ins);
}

bool is_const_scalar(instruction_ref ins, float expect, float tol)
{
    if(not ins->can_eval())
        return false;
    auto c = classify_constant(ins);
    return c.kind == bcast_kind::scalar and std::fabs(c.values[0] - expect) <= tol;
}

instruction_ref other_input(instruction_ref ins, instruction_ref x)
{
    return ins->inputs()[0] == x ? ins->inputs()[1] : ins->inputs()[0];
}

instruction_ref single_user(const module& m, instruction_ref ins)
{
    return ins->outputs().size() == 1 ? ins->outputs().front() : m.end();
}

bool valid(instruction_ref ins, const module& m) { return ins != m.end(); }

// Matches the erf-GELU instruction sequence of src/op/builder/gelu.cpp:58-74 rooted at x:
//   mul(x, 0.5), div(x, sqrt(2)) -> erf -> add(., 1), mul(mul_half, add_one).
// Returns the final mul, or m.end().
instruction_ref match_gelu_erf(const module& m, instruction_ref x, std::vector<instruction_ref>& chain)
{
    if(x->outputs().size() != 2)
        return m.end();
    instruction_ref mul_half = m.end(), div = m.end();
    for(auto u : x->outputs())
    {
        if(u->name() == "mul" and is_const_scalar(other_input(u, x), 0.5f, 1e-6f))
            mul_half = u;
        else if(u->name() == "div" and u->inputs()[0] == x and
                is_const_scalar(u->inputs()[1], 1.41421356f, 1e-3f))
            div = u;
    }
    if(mul_half == m.end() or div == m.end())
        return m.end();
    auto erf = single_user(m, div);
    if(not valid(erf, m) or erf->name() != "erf")
        return m.end();
    auto add_one = single_user(m, erf);
    if(not valid(add_one, m) or add_one->name() != "add" or
       not is_const_scalar(other_input(add_one, erf), 1.0f, 1e-6f))
        return m.end();
    auto fin = single_user(m, add_one);
    if(not valid(fin, m) or fin->name() != "mul" or single_user(m, mul_half) != fin)
        return m.end();
    chain.insert(chain.end(), {mul_half, div, erf, add_one, fin});
    return fin;
}

instruction_ref add_float_literal(module& m, const std::vector<float>& v)
{
    return m.add_literal(literal{shape{shape::float_type, {v.size()}}, v});
}

// A constant 8-bit matrix [.., K, N] (any strides) as a standard [.., N, K] literal.
// [.., K, N] constant -> [.., N, K] literal (8- or 16-bit elements)
instruction_ref add_transposed_8bit_literal(module& m, instruction_ref b)
{
    argument a    = b->eval();
    const auto& s = a.get_shape();
    const auto nd = s.ndim();
    auto lens     = s.lens();
    const std::size_t k = lens[nd - 2], n = lens[nd - 1];
    std::size_t batch = 1;
    for(std::size_t i = 0; i + 2 < nd; ++i)
        batch *= lens[i];
    const std::size_t es = s.type_size();
    std::vector<char> out(batch * n * k * es);
    const char* src = a.data();
    if(s.standard() and (es == 1 or es == 2))
    {
        // packed input: a blocked transpose per batch entry
        constexpr std::size_t tb = 64;
        auto run = [&](auto* dst, const auto* sp) {
            for(std::size_t bi = 0; bi < batch; ++bi)
                for(std::size_t k0 = 0; k0 < k; k0 += tb)
                    for(std::size_t n0 = 0; n0 < n; n0 += tb)
                        for(std::size_t nn = n0; nn < std::min(n, n0 + tb); ++nn)
                            for(std::size_t kk = k0; kk < std::min(k, k0 + tb); ++kk)
                                dst[(bi * n + nn) * k + kk] = sp[(bi * k + kk) * n + nn];
        };
        if(es == 1)
            run(reinterpret_cast<uint8_t*>(out.data()), reinterpret_cast<const uint8_t*>(src));
        else
            run(reinterpret_cast<uint16_t*>(out.data()), reinterpret_cast<const uint16_t*>(src));
    }
    else
    {
        std::vector<std::size_t> idx(nd, 0);
        for(std::size_t bi = 0; bi < batch; ++bi)
        {
            std::size_t rem = bi;
            for(std::size_t d = nd - 2; d-- > 0;)
            {
                idx[d] = rem % lens[d];
                rem /= lens[d];
            }
            for(std::size_t kk = 0; kk < k; ++kk)
            {
                idx[nd - 2] = kk;
                for(std::size_t nn = 0; nn < n; ++nn)
                {
                    idx[nd - 1] = nn;
                    std::memcpy(&out[((bi * n + nn) * k + kk) * es], src + s.index(idx) * es, es);
                }
            }
        }
    }
    std::swap(lens[nd - 2], lens[nd - 1]);
    return m.add_literal(literal{shape{s.type(), lens}, out.data()});
}

} // namespace

namespace {

struct lowerer
{
    module& m;
    std::unordered_set<instruction*> consumed; // fused into an earlier replacement

    void consume(instruction_ref ins) { consumed.insert(&*ins); }
    bool is_consumed(instruction_ref ins) const { return consumed.count(&*ins) > 0; }

    [[noreturn]] void unsupported(instruction_ref ins, const std::string& why) const
    {
        MIGRAPHX_THROW("cuda target: cannot run '" + ins->name() + "' (" + why +
                       "); the target has no CPU fallback");
    }

    // MIGRAPHX_CUDA_DISABLE_FUSION: comma-separated list out of layernorm, attention, horizontal -
    // the multi-operator fusions listed are not applied (their operators are lowered one by one),
    // for bisecting a numerical difference or a performance change
    static bool fusion_disabled(const std::string& what)
    {
        const char* e = std::getenv("MIGRAPHX_CUDA_DISABLE_FUSION");
        return e != nullptr and contains(split_string(e, ','), what);
    }

    // ---------------------------------------------------------------- quant_dot chain
    void lower_quant_dot(instruction_ref qd)
    {
        if(qd->inputs().size() != 2)
            unsupported(qd, "only the two-operand form is supported");
        auto a = qd->inputs()[0];
        auto b = qd->inputs()[1];
        const auto in_type = a->get_shape().type();
        if(in_type != shape::int8_type and in_type != shape::fp8e4m3fn_type)
            unsupported(qd, "operands must be int8 or fp8e4m3fn");

        op_qgemm op;
        op.out_type = static_cast<int>(qd->get_shape().type()); // int32 or float
        std::vector<instruction_ref> chain; // instructions folded into the epilogue
        instruction_ref last  = qd;
        instruction_ref scale = m.end(), bias = m.end(), residual = m.end();

        // dequantizelinear(acc, constant scale) without zero point
        auto dq = single_user(m, last);
        if(valid(dq, m) and dq->name() == "dequantizelinear" and dq->inputs().size() == 2 and
           dq->inputs()[0] == last and dq->inputs()[1]->can_eval() and
           dq->get_shape().type() == shape::float_type)
        {
            auto c = classify_constant(dq->inputs()[1]);
            if(c.kind != bcast_kind::full)
            {
                op.scale_mode = c.kind == bcast_kind::scalar
                                    ? MGX_SCALE_PER_TENSOR
                                    : (c.kind == bcast_kind::per_col ? MGX_SCALE_PER_COL
                                                                     : MGX_SCALE_PER_ROW);
                scale       = add_float_literal(m, c.values);
                op.out_type = static_cast<int>(shape::float_type);
                chain.push_back(dq);
                last = dq;
            }
        }
        if(last != qd or in_type == shape::fp8e4m3fn_type)
        {
            // the rest of the epilogue only follows a float value
            bool progress = true;
            bool seen_act = false;
            while(progress)
            {
                progress = false;
                auto u   = single_user(m, last);
                if(not valid(u, m) or last->get_shape().type() == shape::int32_type)
                    break;
                if(u->name() == "convert" and u->get_shape().type() == shape::half_type and
                   residual == m.end() and
                   static_cast<shape::type_t>(op.out_type) == shape::float_type)
                {
                    op.out_type = static_cast<int>(shape::half_type);
                    // what follows the convert is half arithmetic; what came before it was fp32
                    op.half_math = bias == m.end() and not seen_act;
                    chain.push_back(u);
                    last     = u;
                    progress = true;
                    continue;
                }
                if(u->name() == "add" and residual == m.end())
                {
                    auto other = other_input(u, last);
                    if(other->can_eval() and bias == m.end() and not seen_act)
                    {
                        auto c = classify_constant(other);
                        if(c.kind == bcast_kind::per_col or c.kind == bcast_kind::scalar)
                        {
                            std::vector<float> v = c.values;
                            if(c.kind == bcast_kind::scalar)
                                v.assign(u->get_shape().lens().back(), c.values[0]);
                            bias = add_float_literal(m, v);
                            chain.push_back(u);
                            last     = u;
                            progress = true;
                            continue;
                        }
                    }
                    else if(not other->can_eval() and other->get_shape() == u->get_shape() and
                            other->get_shape().standard())
                    {
                        residual = other;
                        chain.push_back(u);
                        last     = u;
                        progress = true;
                        continue;
                    }
                }
                if(u->name() == "relu" and not seen_act and residual == m.end())
                {
                    op.act   = MGX_ACT_RELU;
                    seen_act = true;
                    chain.push_back(u);
                    last     = u;
                    progress = true;
                    continue;
                }
            }
            if(not seen_act and residual == m.end())
            {
                std::vector<instruction_ref> g;
                auto fin = match_gelu_erf(m, last, g);
                // in half arithmetic the kernel divides by the half value of sqrt(2)
                if(fin != m.end() and op.half_math and
                   not is_const_scalar(g[1]->inputs()[1], 1.4140625f, 0.0f))
                    fin = m.end();
                if(fin != m.end())
                {
                    op.act = MGX_ACT_GELU_ERF;
                    chain.insert(chain.end(), g.begin(), g.end());
                    last = fin;
                    // a residual add may still follow the activation
                    auto u = single_user(m, last);
                    if(valid(u, m) and u->name() == "add")
                    {
                        auto other = other_input(u, last);
                        if(not other->can_eval() and other->get_shape() == u->get_shape() and
                           other->get_shape().standard())
                        {
                            residual = other;
                            chain.push_back(u);
                            last = u;
                        }
                    }
                }
            }
        }
        if(static_cast<shape::type_t>(op.out_type) != last->get_shape().type())
            op.out_type = static_cast<int>(last->get_shape().type());
        if(residual != m.end() and residual->get_shape().type() != last->get_shape().type())
            unsupported(last, "residual type differs from the output type");

        // A: K-contiguous rows; with batch dimensions the entries must be evenly spaced, so a
        // transposed / sliced view (heads of an attention block) is packed first; rows whose length
        // is no multiple of 16 bytes (the tensor maps' pitch rule) are copied into padded rows
        {
            const auto as = a->get_shape();
            const auto nd = as.ndim();
            const auto k  = as.lens()[nd - 1];
            const bool rows_ok = as.strides()[nd - 1] == 1 and as.strides()[nd - 2] % 16 == 0;
            if(not as.standard() and (nd > 2 or not rows_ok))
                a = standard_copy(qd, a);
            if(k % 16 != 0)
            {
                if(not a->get_shape().standard())
                    a = standard_copy(qd, a);
                const std::size_t kp = (k + 15) / 16 * 16;
                auto lens            = as.lens();
                std::vector<std::size_t> strides(nd, 1);
                strides[nd - 2] = kp;
                for(std::size_t j = nd - 2; j-- > 0;)
                    strides[j] = strides[j + 1] * lens[j + 1];
                auto buf = insert_allocation(m, qd, shape{in_type, lens, strides});
                a        = m.insert_instruction(qd, op_pad_rows{}, a, buf);
                consume(a);
            }
        }
        // B operand: constants are re-laid out K-contiguous once, here
        std::vector<instruction_ref> args = {a, b};
        instruction_ref workspace = m.end();
        const bool k_aligned = a->get_shape().lens().back() % 16 == 0;
        if(b->can_eval() and k_aligned)
        {
            args[1]  = add_transposed_8bit_literal(m, b);
            op.b_nk  = true;
            // decode-sized launches (at most 16 rows) stream the weights once through the
            // skinny-M kernel, which wants room for partial sums
            const auto& al = a->get_shape().lens();
            const auto& bl = b->get_shape().lens();
            if(al.size() == 2 and bl.size() == 2 and residual == m.end())
            {
                mgx_qgemm_desc d{};
                d.M          = static_cast<int64_t>(al[0]);
                d.K          = static_cast<int64_t>(al[1]);
                d.N          = static_cast<int64_t>(bl[1]);
                d.batch      = 1;
                d.b_layout   = MGX_B_NK;
                d.scale_mode = op.scale_mode;
                const std::size_t ws = mgx_cuda_qgemm_workspace(&d);
                if(ws > 0)
                {
                    workspace        = insert_allocation(m, last, shape{shape::int8_type, {ws}});
                    op.has_workspace = true;
                }
            }
        }
        else
        {
            // re-laid out per evaluation into the workspace (rows padded to 16 bytes); a strided
            // view (a transposed parameter) is packed first
            if(not b->get_shape().standard())
                args[1] = standard_copy(qd, b);
            const auto& bl       = b->get_shape().lens();
            const std::size_t k  = bl[bl.size() - 2];
            const std::size_t kp = (k + 15) / 16 * 16;
            const std::size_t ws = b->get_shape().elements() / k * kp;
            workspace            = insert_allocation(m, last, shape{shape::int8_type, {ws}});
            op.has_workspace     = true;
        }
        if(op.scale_mode != MGX_SCALE_NONE)
            args.push_back(scale);
        if(bias != m.end())
        {
            op.has_bias = true;
            args.push_back(bias);
        }
        if(residual != m.end())
        {
            op.has_residual = true;
            args.push_back(residual);
        }
        if(workspace != m.end())
            args.push_back(workspace);
        // a trailing per-tensor quantizelinear (the next quantized operator's input) is done
        // by the same epilogue
        instruction_ref qz = m.end();
        if(last != qd and last->get_shape().type() != shape::int32_type)
        {
            for(auto u : last->outputs())
            {
                if(u->name() != "quantizelinear" or u->inputs().size() != 3 or u->inputs()[0] != last)
                    continue;
                const auto qt = u->get_shape().type();
                if(qt != shape::int8_type and qt != shape::fp8e4m3fn_type)
                    continue;
                if(not u->inputs()[1]->can_eval() or not u->inputs()[2]->can_eval())
                    continue;
                auto cs = classify_constant(u->inputs()[1]);
                auto cz = classify_constant(u->inputs()[2]);
                if(cs.kind != bcast_kind::scalar or cz.kind != bcast_kind::scalar or not(cs.values[0] > 0))
                    continue;
                op.q_type  = static_cast<int>(qt);
                op.q_scale = cs.values[0];
                op.q_zp    = cz.values[0];
                qz         = u;
                break;
            }
        }
        const bool only_q = qz != m.end() and last->outputs().size() == 1;
        // fp16 chain whose only result is the int8 tensor: activation + quantizelinear of the half
        // the chain holds after the bias is a function of 16 bits - one table look-up in the epilogue
        // (MIGRAPHX_CUDA_QGEMM_LUT=1.  Off by default: the table is the reference's own arithmetic, but
        // one uncoalesced byte load per element costs the FFN1 launch of a BERT-base layer more than the
        // ~30 instructions it saves - 29.6 us against 24.4 us per cold launch.)
        const char* lut_env = std::getenv("MIGRAPHX_CUDA_QGEMM_LUT");
        if(lut_env != nullptr and std::string(lut_env) == "1" and only_q and op.half_math and not op.has_residual and
           op.q_type == static_cast<int>(shape::int8_type) and
           (op.act == MGX_ACT_GELU_ERF or op.act == MGX_ACT_RELU))
        {
            op.has_lut = true;
            auto lut   = m.add_literal(act_quant_table(op.act, op.q_scale, op.q_zp));
            // the table sits after the residual slot and before the workspace
            args.insert(workspace != m.end() ? args.end() - 1 : args.end(), lut);
        }
        if(only_q)
        {
            op.write_d = false;
            args.push_back(insert_allocation(m, qz, qz->get_shape().as_standard()));
        }
        else
        {
            if(qz != m.end())
                args.push_back(insert_allocation(m, last, qz->get_shape().as_standard()));
            args.push_back(insert_allocation(m, last, last->get_shape().as_standard()));
        }
        for(auto c : chain)
        {
            consume(c);
            // constant operands used only by the fused chain need no folding of their own
            for(auto i : c->inputs())
                if(i->can_eval() and i->outputs().size() == 1 and not is_builtin(i->name()))
                    consume(i);
        }
        consume(qd);
        if(only_q)
        {
            consume(last);
            consume(m.replace_instruction(qz, op, args));
            return;
        }
        auto rep = m.replace_instruction(last, op, args);
        consume(rep);
        if(qz != m.end())
            consume(m.replace_instruction(qz, op_second_output{}, rep, args[args.size() - 2]));
    }

    // int8 quantizelinear(activation(x), scale, zero point) for every half x, indexed by x's bit
    // pattern, evaluated with migraphx::half exactly as a chain of half operators on the ref target
    // evaluates it: every operator computes in fp32 and stores (truncates to) half
    // (erf-GELU: src/op/builder/gelu.cpp:58-74; quantizelinear: src/include/migraphx/op/quantizelinear.hpp:71-108)
    static literal act_quant_table(int act, float q_scale, float q_zp)
    {
        auto h = [](float f) { return static_cast<float>(migraphx::half(f)); };
        std::vector<int8_t> table(65536);
        const float sqrt2 = h(static_cast<float>(M_SQRT2));
        for(std::uint32_t bits = 0; bits < 65536; ++bits)
        {
            const auto b16 = static_cast<std::uint16_t>(bits);
            migraphx::half xh;
            std::memcpy(&xh, &b16, sizeof(b16));
            const float x = static_cast<float>(xh);
            float v       = x;
            if(act == MGX_ACT_GELU_ERF)
            {
                const float mh = h(x * 0.5f);
                const float dv = h(x / sqrt2);
                const float e1 = h(h(std::erf(dv)) + 1.0f);
                v              = h(mh * e1);
            }
            else if(act == MGX_ACT_RELU)
                v = std::max(x, 0.0f);
            else if(act == MGX_ACT_GELU_TANH or act == MGX_ACT_SILU)
                MIGRAPHX_THROW("cuda: no table form of this activation");
            // quantizelinear of a half tensor: the quotient is a half, then nearbyint + zero point, saturated
            const double q = static_cast<double>(std::nearbyint(h(v / q_scale))) + static_cast<double>(q_zp);
            // std::max(lowest, std::min(max, q)) as the reference writes it: a NaN compares false and gives max
            table[bits] = static_cast<int8_t>(std::max(-128.0, std::min(127.0, q)));
        }
        return literal{shape{shape::int8_type, {65536}}, table.data()};
    }

    // ---------------------------------------------------------------- weight-only int4
    // dot(A, transpose(dequantizelinear(unpack_int4(packed), scales, [zero points])))
    bool lower_w4a16(instruction_ref dot)
    {
        if(dot->inputs().size() != 2)
            return false;
        auto a  = dot->inputs()[0];
        auto bt = dot->inputs()[1];
        if(a->get_shape().type() != shape::half_type or bt->name() != "transpose" or
           bt->get_shape().ndim() != 2)
            return false;
        auto dq = bt->inputs()[0];
        if(dq->name() != "dequantizelinear" or dq->get_shape().type() != shape::half_type)
            return false;
        auto unpack = dq->inputs()[0];
        if(unpack->name() != "unpack_int4" or unpack->get_shape().type() != shape::uint8_type)
            return false;
        auto packed = unpack->inputs()[0];
        if(not packed->get_shape().standard() or packed->get_shape().ndim() != 2)
            return false;
        if(not dq->inputs()[1]->can_eval())
            unsupported(dot, "int4 scales must be compile-time constants");
        if(dq->inputs().size() == 3 and not dq->inputs()[2]->can_eval())
            unsupported(dot, "int4 zero points must be compile-time constants");
        const std::size_t n = unpack->get_shape().lens()[0];
        const std::size_t k = unpack->get_shape().lens()[1];
        if(a->get_shape().lens().back() != k or not a->get_shape().standard())
            return false;

        // group size: the largest divisor g of K (a multiple of 32) for which scales and
        // zero points are constant inside every run of g columns
        const auto sv = eval_as_floats(dq->inputs()[1]);
        std::vector<float> zv;
        if(dq->inputs().size() == 3)
            zv = eval_as_floats(dq->inputs()[2]);
        auto blocks_const = [&](const std::vector<float>& v, std::size_t g) {
            for(std::size_t r = 0; r < n; ++r)
                for(std::size_t c = 0; c < k; ++c)
                    if(v[r * k + c] != v[r * k + (c / g) * g])
                        return false;
            return true;
        };
        // every multiple of 32 that divides K is a candidate, largest first (K / group need
        // not be a power of two: K = 11008 or 28672 with groups of 128)
        std::size_t group = 0;
        for(std::size_t g = k / 32 * 32; g >= 32; g -= 32)
        {
            if(k % g != 0)
                continue;
            if(blocks_const(sv, g) and (zv.empty() or blocks_const(zv, g)))
            {
                group = g;
                break;
            }
        }
        if(group == 0)
            unsupported(dot, "int4 group size must be a multiple of 32 dividing K");
        const std::size_t gpr = k / group;
        std::vector<half> scales(n * gpr);
        for(std::size_t r = 0; r < n; ++r)
            for(std::size_t g = 0; g < gpr; ++g)
                scales[r * gpr + g] = half(sv[r * k + g * group]);
        op_w4a16 op;
        op.group = static_cast<int>(group);
        std::vector<instruction_ref> args = {
            a, packed, m.add_literal(literal{shape{shape::half_type, {n, gpr}}, scales})};
        if(not zv.empty())
        {
            bool uniform = true;
            for(auto z : zv)
                if(z != zv[0])
                    uniform = false;
            if(uniform)
                op.zp_const = static_cast<int>(zv[0]);
            else
            {
                std::vector<uint8_t> zps(n * gpr);
                for(std::size_t r = 0; r < n; ++r)
                    for(std::size_t g = 0; g < gpr; ++g)
                        zps[r * gpr + g] = static_cast<uint8_t>(zv[r * k + g * group]);
                op.has_zp = true;
                args.push_back(m.add_literal(literal{shape{shape::uint8_type, {n, gpr}}, zps}));
            }
        }
        else
            op.zp_const = 0;
        mgx_w4_desc d{};
        d.M = static_cast<int64_t>(a->get_shape().elements() / k);
        d.N = static_cast<int64_t>(n);
        d.K = static_cast<int64_t>(k);
        d.group = op.group;
        const std::size_t ws = mgx_cuda_w4a16_workspace(&d);
        if(ws > 0)
        {
            op.has_workspace = true;
            args.push_back(insert_allocation(m, dot, shape{shape::int8_type, {ws}}));
        }
        args.push_back(insert_allocation(m, dot, dot->get_shape().as_standard()));
        consume(bt);
        consume(dq);
        consume(unpack);
        for(std::size_t i = 1; i < dq->inputs().size(); ++i)
            if(dq->inputs()[i]->outputs().size() == 1 and not is_builtin(dq->inputs()[i]->name()))
                consume(dq->inputs()[i]);
        auto rep = m.replace_instruction(dot, op, args);
        consume(rep);
        return true;
    }

    // dot(A, dequantizelinear(unpack_int4(P), scale, zero point)) with P a compile-time constant
    // packed along N - the form quantize_int4_weights leaves (src/quantize_int4.cpp:69-95: a
    // per-tensor scale and zero point on the [K, N] weight, no transpose).  The weights stay int4 in
    // device memory (the reference never folds through unpack_int4 either,
    // src/propagate_constant.cpp:39-54); they are re-packed once, here, along K into the [N, K/2]
    // layout the kernels stream.
    bool lower_w4a16_kn(instruction_ref dot)
    {
        if(dot->inputs().size() != 2)
            return false;
        auto a  = dot->inputs()[0];
        auto dq = dot->inputs()[1];
        if(a->get_shape().type() != shape::half_type or dq->name() != "dequantizelinear" or
           dq->get_shape().type() != shape::half_type or dq->get_shape().ndim() != 2 or dq->inputs().size() != 3)
            return false;
        auto unpack = dq->inputs()[0];
        if(unpack->name() != "unpack_int4" or unpack->get_shape().type() != shape::uint8_type or
           not unpack->inputs()[0]->can_eval() or not dq->inputs()[1]->can_eval() or not dq->inputs()[2]->can_eval())
            return false;
        const std::size_t k = dq->get_shape().lens()[0];
        const std::size_t n = dq->get_shape().lens()[1];
        if(a->get_shape().lens().back() != k or not a->get_shape().standard() or k % 32 != 0)
            return false;
        auto cs = classify_constant(dq->inputs()[1]);
        auto cz = classify_constant(dq->inputs()[2]);
        if(cs.kind != bcast_kind::scalar or cz.kind != bcast_kind::scalar)
            return false;
        // the unpacked [K, N] values (0..15), then nibbles paired along K, row n of the result
        argument u = unpack->eval();
        if(u.empty() or not u.get_shape().standard())
            return false;
        const auto* q = reinterpret_cast<const uint8_t*>(u.data());
        std::vector<uint8_t> packed(n * (k / 2));
        for(std::size_t kk = 0; kk < k; kk += 2)
            for(std::size_t nn = 0; nn < n; ++nn)
                packed[nn * (k / 2) + kk / 2] =
                    static_cast<uint8_t>((q[kk * n + nn] & 0xF) | ((q[(kk + 1) * n + nn] & 0xF) << 4));
        std::size_t group = k % 128 == 0 ? 128 : 32;
        const std::size_t gpr = k / group;
        std::vector<half> scales(n * gpr, half(cs.values[0]));
        op_w4a16 op;
        op.group    = static_cast<int>(group);
        op.zp_const = static_cast<int>(cz.values[0]);
        std::vector<instruction_ref> args = {
            a, m.add_literal(literal{shape{shape::uint8_type, {n, k / 2}}, packed}),
            m.add_literal(literal{shape{shape::half_type, {n, gpr}}, scales})};
        mgx_w4_desc d{};
        d.M     = static_cast<int64_t>(a->get_shape().elements() / k);
        d.N     = static_cast<int64_t>(n);
        d.K     = static_cast<int64_t>(k);
        d.group = op.group;
        const std::size_t ws = mgx_cuda_w4a16_workspace(&d);
        if(ws > 0)
        {
            op.has_workspace = true;
            args.push_back(insert_allocation(m, dot, shape{shape::int8_type, {ws}}));
        }
        args.push_back(insert_allocation(m, dot, dot->get_shape().as_standard()));
        consume(dq);
        consume(unpack);
        for(auto i : {unpack->inputs()[0], dq->inputs()[1], dq->inputs()[2]})
        {
            // the constant chain behind the packed weights (pack_int4(quantizelinear(W))) is dead now
            auto c = i;
            while(c->outputs().size() == 1 and not is_builtin(c->name()))
            {
                consume(c);
                if(c->inputs().empty())
                    break;
                c = c->inputs()[0];
            }
        }
        consume(m.replace_instruction(dot, op, args));
        return true;
    }

    // ---------------------------------------------------------------- horizontal fusion
    // Quantized linears that read the same activations with the same kind of epilogue (the Q, K and
    // V projections of an attention block) become one cuda::qgemm over the concatenated weights;
    // the former results are column slices of its output.  Only done when every reader takes
    // row-strided matrices (cuda::attention), so no slice ever has to be packed again.
    // cuda::w4a16 operators that read the same activations (gate and up projections of a SwiGLU
    // block) and whose results only element-wise kernels read (which take strided operands) become
    // one operator over the concatenated packed weights, scales and zero points: one stream over the
    // weights instead of two launches' fixed costs.
    void fuse_horizontal_w4a16()
    {
        if(fusion_disabled("horizontal"))
            return;
        std::vector<instruction_ref> lins;
        for(auto ins : iterator_for(m))
            if(ins->name() == "cuda::w4a16")
                lins.push_back(ins);
        std::unordered_set<instruction*> done;
        for(auto first : lins)
        {
            if(done.count(&*first) > 0)
                continue;
            const auto fop = any_cast<op_w4a16>(first->get_operator());
            auto eligible  = [&](instruction_ref g) {
                const auto op  = any_cast<op_w4a16>(g->get_operator());
                const auto& in = g->inputs();
                if(op.group != fop.group or op.zp_const != fop.zp_const or op.has_zp != fop.has_zp)
                    return false;
                if(in[0]->get_shape().ndim() != 2 or in[1]->name() != "@literal" or in[2]->name() != "@literal" or
                   (op.has_zp and in[3]->name() != "@literal"))
                    return false;
                bool any = false;
                for(auto o : g->outputs())
                {
                    if(o->name() == "cuda::pointwise" and o->inputs().back() != g)
                        any = true;
                    else if(not is_consumed(o))
                        return false;
                }
                return any;
            };
            if(not eligible(first))
                continue;
            std::vector<instruction_ref> group = {first};
            for(auto g : lins)
                if(g != first and done.count(&*g) == 0 and g->inputs()[0] == first->inputs()[0] and eligible(g) and
                   g->inputs()[1]->get_shape().lens()[1] == first->inputs()[1]->get_shape().lens()[1])
                    group.push_back(g);
            if(group.size() < 2)
                continue;
            const std::size_t k2  = first->inputs()[1]->get_shape().lens()[1]; // K / 2
            const std::size_t gpr = first->inputs()[2]->get_shape().lens()[1]; // groups per row
            std::vector<char> w, sc, zp;
            std::vector<std::size_t> widths;
            for(auto g : group)
            {
                auto wl = g->inputs()[1]->get_literal();
                auto sl = g->inputs()[2]->get_literal();
                w.insert(w.end(), wl.data(), wl.data() + wl.get_shape().bytes());
                sc.insert(sc.end(), sl.data(), sl.data() + sl.get_shape().bytes());
                if(fop.has_zp)
                {
                    auto zl = g->inputs()[3]->get_literal();
                    zp.insert(zp.end(), zl.data(), zl.data() + zl.get_shape().bytes());
                }
                widths.push_back(wl.get_shape().lens()[0]);
            }
            std::size_t n = 0;
            for(auto wd : widths)
                n += wd;
            const std::size_t mm = first->inputs()[0]->get_shape().lens()[0];
            std::vector<instruction_ref> args = {
                first->inputs()[0], m.add_literal(literal{shape{shape::uint8_type, {n, k2}}, w.data()}),
                m.add_literal(literal{shape{shape::half_type, {n, gpr}}, sc.data()})};
            if(fop.has_zp)
                args.push_back(m.add_literal(literal{shape{shape::uint8_type, {n, gpr}}, zp.data()}));
            instruction_ref pos = group.front();
            for(auto ins : iterator_for(m))
                if(std::find(group.begin(), group.end(), ins) != group.end())
                {
                    pos = ins;
                    break;
                }
            op_w4a16 op = fop;
            mgx_w4_desc d{};
            d.M     = static_cast<int64_t>(mm);
            d.N     = static_cast<int64_t>(n);
            d.K     = static_cast<int64_t>(k2 * 2);
            d.group = op.group;
            const std::size_t ws = mgx_cuda_w4a16_workspace(&d);
            op.has_workspace     = ws > 0;
            if(ws > 0)
                args.push_back(insert_allocation(m, pos, shape{shape::int8_type, {ws}}));
            args.push_back(insert_allocation(m, pos, shape{shape::half_type, {mm, n}}));
            auto fused = m.insert_instruction(pos, op, args);
            consume(fused);
            std::size_t c0 = 0;
            for(std::size_t i = 0; i < group.size(); ++i)
            {
                done.insert(&*group[i]);
                m.replace_instruction(group[i],
                                      make_op("slice", {{"axes", {1}}, {"starts", {c0}}, {"ends", {c0 + widths[i]}}}),
                                      fused);
                c0 += widths[i];
            }
        }
    }

    void fuse_horizontal_qgemms()
    {
        if(fusion_disabled("horizontal"))
            return;
        std::vector<instruction_ref> gemms;
        for(auto ins : iterator_for(m))
            if(ins->name() == "cuda::qgemm")
                gemms.push_back(ins);
        std::unordered_set<instruction*> done;
        for(auto first : gemms)
        {
            if(done.count(&*first) > 0)
                continue;
            const auto fop = any_cast<op_qgemm>(first->get_operator());
            auto eligible  = [&](instruction_ref g) {
                const auto op = any_cast<op_qgemm>(g->get_operator());
                const auto& in = g->inputs();
                if(not op.b_nk or op.has_residual or op.has_workspace or op.q_type != 0 or not op.has_bias or
                   op.scale_mode != MGX_SCALE_PER_COL or in.size() != 5 or in[0]->get_shape().ndim() != 2)
                    return false;
                if(in[1]->name() != "@literal" or in[2]->name() != "@literal" or in[3]->name() != "@literal")
                    return false;
                // readers: attention operators only (instructions already folded into an earlier
                // replacement are dead and do not count)
                bool any = false;
                for(auto o : g->outputs())
                {
                    if(o->name() == "cuda::attention")
                        any = true;
                    else if(not is_consumed(o))
                        return false;
                }
                return any;
            };
            if(not eligible(first))
                continue;
            std::vector<instruction_ref> group = {first};
            for(auto g : gemms)
            {
                if(g == first or done.count(&*g) > 0 or not eligible(g) or g->inputs()[0] != first->inputs()[0])
                    continue;
                const auto op = any_cast<op_qgemm>(g->get_operator());
                if(op.act == fop.act and op.out_type == fop.out_type and
                   g->inputs()[1]->get_shape().type() == first->inputs()[1]->get_shape().type())
                    group.push_back(g);
            }
            if(group.size() < 2)
                continue;
            // concatenated [N, K] weights, scales and biases
            const std::size_t k = first->inputs()[1]->get_shape().lens()[1];
            std::vector<char> w;
            std::vector<float> sc, bi;
            std::vector<std::size_t> widths;
            for(auto g : group)
            {
                auto wl = g->inputs()[1]->get_literal();
                auto sl = g->inputs()[2]->get_literal();
                auto bl = g->inputs()[3]->get_literal();
                w.insert(w.end(), wl.data(), wl.data() + wl.get_shape().bytes());
                const auto* sp = reinterpret_cast<const float*>(sl.data());
                const auto* bp = reinterpret_cast<const float*>(bl.data());
                sc.insert(sc.end(), sp, sp + sl.get_shape().elements());
                bi.insert(bi.end(), bp, bp + bl.get_shape().elements());
                widths.push_back(wl.get_shape().lens()[0]);
            }
            const std::size_t n  = sc.size();
            const std::size_t mm = first->inputs()[0]->get_shape().lens()[0];
            auto wlit = m.add_literal(literal{shape{first->inputs()[1]->get_shape().type(), {n, k}}, w.data()});
            auto slit = add_float_literal(m, sc);
            auto blit = add_float_literal(m, bi);
            // in front of the earliest member, so that every reader comes later
            instruction_ref pos = group.front();
            for(auto ins : iterator_for(m))
                if(std::find(group.begin(), group.end(), ins) != group.end())
                {
                    pos = ins;
                    break;
                }
            auto out   = insert_allocation(m, pos, shape{static_cast<shape::type_t>(fop.out_type), {mm, n}});
            auto fused = m.insert_instruction(pos, fop, {first->inputs()[0], wlit, slit, blit, out});
            consume(fused);
            std::size_t c0 = 0;
            for(std::size_t i = 0; i < group.size(); ++i)
            {
                done.insert(&*group[i]);
                m.replace_instruction(group[i],
                                      make_op("slice", {{"axes", {1}}, {"starts", {c0}}, {"ends", {c0 + widths[i]}}}),
                                      fused);
                c0 += widths[i];
            }
        }
    }

    // ---------------------------------------------------------------- attention
    // softmax(mul(dot(Qh, Kh^T), scale)) . Vh with Qh / Kh / Vh the head views
    // transpose(reshape[B,S,H,D](X)) of [B*S, H*D] fp16 matrices, and the result merged back by
    // transpose -> contiguous -> reshape: one cuda::attention that reads the heads in place.
    bool lower_attention(instruction_ref sm)
    {
        if(fusion_disabled("attention"))
            return false;
        const auto& ps = sm->get_shape();
        if(ps.type() != shape::half_type or ps.ndim() != 4)
            return false;
        const auto ax = sm->get_operator().to_value().at("axis").to<int64_t>();
        if(ax != 3 and ax != -1)
            return false;
        auto is_transpose = [](instruction_ref t, std::vector<int64_t> perm) {
            return t->name() == "transpose" and
                   t->get_operator().to_value().at("permutation").to_vector<int64_t>() == perm;
        };
        // [B,S,H,D] view of a [B*S, H*D] (or [B,S,H*D]) matrix; returns the matrix
        auto head_source = [&](instruction_ref t, std::vector<int64_t> perm, std::size_t b, std::size_t sq,
                               std::size_t h, std::size_t d) -> instruction_ref {
            if(not is_transpose(t, perm) or t->outputs().size() != 1)
                return m.end();
            auto r = t->inputs().front();
            if((r->name() != "reshape" and r->name() != "reshape_lazy") or r->outputs().size() != 1 or
               r->get_shape().lens() != std::vector<std::size_t>{b, sq, h, d})
                return m.end();
            auto x         = r->inputs().front();
            const auto& xs = x->get_shape();
            if(xs.type() != shape::half_type or xs.elements() != b * sq * h * d or xs.lens().back() != h * d or
               xs.strides().back() != 1)
                return m.end();
            // rows evenly spaced: a packed tensor, or a 2-D view with a row stride (a column slice)
            if(not xs.standard() and not(xs.ndim() == 2 and xs.strides()[0] % 8 == 0))
                return m.end();
            return x;
        };
        auto ss = sm->inputs().front();
        instruction_ref sc = ss;
        float scale        = 1.0f;
        std::vector<instruction_ref> chain = {sm};
        if(ss->name() == "mul" and ss->outputs().size() == 1)
        {
            instruction_ref c = m.end();
            for(auto i : ss->inputs())
                if(i->can_eval())
                    c = i;
            if(c == m.end())
                return false;
            auto cv = classify_constant(c);
            if(cv.kind != bcast_kind::scalar)
                return false;
            scale = cv.values[0];
            sc    = other_input(ss, c);
            chain.push_back(ss);
        }
        if(sc->name() != "dot" or sc->outputs().size() != 1)
            return false;
        const auto& sl = ps.lens(); // [B, H, S, S]
        const std::size_t b = sl[0], h = sl[1], sq = sl[2];
        if(sl[3] != sq)
            return false;
        const std::size_t d = sc->inputs()[0]->get_shape().lens().back();
        if(d != 64)
            return false;
        auto qx = head_source(sc->inputs()[0], {0, 2, 1, 3}, b, sq, h, d);
        auto kx = head_source(sc->inputs()[1], {0, 2, 3, 1}, b, sq, h, d);
        if(qx == m.end() or kx == m.end())
            return false;
        auto cx = single_user(m, sm);
        if(not valid(cx, m) or cx->name() != "dot" or cx->inputs()[0] != sm)
            return false;
        auto vx = head_source(cx->inputs()[1], {0, 2, 1, 3}, b, sq, h, d);
        if(vx == m.end())
            return false;
        auto ct = single_user(m, cx);
        if(not valid(ct, m) or not is_transpose(ct, {0, 2, 1, 3}))
            return false;
        auto cc = single_user(m, ct);
        if(not valid(cc, m) or cc->name() != "contiguous")
            return false;
        auto cr = single_user(m, cc);
        if(not valid(cr, m) or (cr->name() != "reshape" and cr->name() != "reshape_lazy") or
           cr->get_shape().lens().back() != h * d)
            return false;
        chain.insert(chain.end(), {sc, cx, ct, cc, sc->inputs()[0], sc->inputs()[1], cx->inputs()[1],
                                   sc->inputs()[0]->inputs()[0], sc->inputs()[1]->inputs()[0],
                                   cx->inputs()[1]->inputs()[0]});
        op_attention op;
        op.batch = b, op.seq = sq, op.heads = h, op.head_dim = d;
        op.scale = scale;
        // MIGRAPHX_CUDA_ATTENTION=fp32: the faster kernel that does not make the chain's half roundings
        const char* att = std::getenv("MIGRAPHX_CUDA_ATTENTION");
        op.fp32_softmax = att != nullptr and std::string(att) == "fp32";
        std::vector<instruction_ref> args = {qx, kx, vx};
        instruction_ref last = cr;
        instruction_ref qz   = m.end();
        for(auto o : last->outputs())
        {
            if(o->name() != "quantizelinear" or o->inputs().size() != 3 or o->inputs()[0] != last or
               o->get_shape().type() != shape::int8_type or not o->inputs()[1]->can_eval() or
               not o->inputs()[2]->can_eval())
                continue;
            auto cs = classify_constant(o->inputs()[1]);
            auto cz = classify_constant(o->inputs()[2]);
            if(cs.kind != bcast_kind::scalar or cz.kind != bcast_kind::scalar or not(cs.values[0] > 0))
                continue;
            op.q_type  = static_cast<int>(shape::int8_type);
            op.q_scale = cs.values[0];
            op.q_zp    = cz.values[0];
            qz         = o;
            break;
        }
        for(auto c : chain)
        {
            consume(c);
            for(auto i : c->inputs())
                if(i->can_eval() and i->outputs().size() == 1 and not is_builtin(i->name()))
                    consume(i);
        }
        const bool only_q = qz != m.end() and last->outputs().size() == 1;
        if(only_q)
        {
            op.write_o = false;
            args.push_back(insert_allocation(m, qz, qz->get_shape().as_standard()));
            consume(last);
            consume(m.replace_instruction(qz, op, args));
            return true;
        }
        if(qz != m.end())
            args.push_back(insert_allocation(m, last, qz->get_shape().as_standard()));
        args.push_back(insert_allocation(m, last, last->get_shape().as_standard()));
        auto rep = m.replace_instruction(last, op, args);
        consume(rep);
        if(qz != m.end())
            consume(m.replace_instruction(qz, op_second_output{}, rep, args[args.size() - 2]));
        return true;
    }

    // ---------------------------------------------------------------- rotary embedding (builder form)
    // add(mul(X, C), mul(concat(X[half:], X[:half]), mul(signs, S))) with C / S the cos / sin rows
    // gathernd-ed at the positions, doubled along the last axis and broadcast over the heads
    // (src/op/builder/rotary_embedding.cpp:60-230, non-interleaved): one cuda::rotary_embedding.
    bool lower_rotary(instruction_ref add)
    {
        if(fusion_disabled("rotary") or add->name() != "add" or add->inputs().size() != 2)
            return false;
        const auto& os = add->get_shape();
        if(os.ndim() != 4 or (os.type() != shape::half_type and os.type() != shape::float_type) or os.lens()[3] % 2 != 0)
            return false;
        const std::size_t d = os.lens()[3], half = d / 2;
        auto is_axis_last = [&](instruction_ref c) {
            const auto ax = c->get_operator().to_value().at("axis").to<int64_t>();
            return ax == -1 or ax == static_cast<int64_t>(c->get_shape().ndim()) - 1;
        };
        // multibroadcast(reshape[B,1,S,D](concat(G, G))), G = gathernd(cache, idx); returns {cache, idx}
        std::vector<instruction_ref> chain = {add};
        auto cache_rows = [&](instruction_ref x) -> std::pair<instruction_ref, instruction_ref> {
            const std::pair<instruction_ref, instruction_ref> none{m.end(), m.end()};
            if(x->name() == "multibroadcast")
            {
                chain.push_back(x);
                x = x->inputs().front();
            }
            if(x->name() != "reshape" and x->name() != "reshape_lazy")
                return none;
            const auto& rl = x->get_shape().lens();
            if(rl.size() != 4 or rl[0] != os.lens()[0] or rl[1] != 1 or rl[2] != os.lens()[2] or rl[3] != d)
                return none;
            auto cc = x->inputs().front();
            if(cc->name() != "concat" or not is_axis_last(cc) or cc->inputs().size() != 2 or
               cc->inputs()[0] != cc->inputs()[1])
                return none;
            auto gn = cc->inputs()[0];
            if(gn->name() != "gathernd" or gn->get_operator().to_value().at("batch_dims").to<int64_t>() != 0)
                return none;
            chain.insert(chain.end(), {x, cc, gn});
            return {gn->inputs()[0], gn->inputs()[1]};
        };
        for(int swap = 0; swap < 2; ++swap)
        {
            auto mc = add->inputs()[swap], ms2 = add->inputs()[1 - swap];
            if(mc->name() != "mul" or ms2->name() != "mul" or mc->outputs().size() != 1 or ms2->outputs().size() != 1)
                continue;
            // ms2 = mul(rotated, mul(signs, sin))
            instruction_ref rot = m.end(), msin = m.end();
            for(auto i : ms2->inputs())
            {
                if(i->name() == "concat")
                    rot = i;
                else if(i->name() == "mul")
                    msin = i;
            }
            if(rot == m.end() or msin == m.end() or not is_axis_last(rot) or rot->inputs().size() != 2)
                continue;
            auto s2 = rot->inputs()[0], s1 = rot->inputs()[1];
            auto is_slice = [&](instruction_ref sl, std::size_t lo, std::size_t hi) {
                if(sl->name() != "slice")
                    return false;
                const auto v  = sl->get_operator().to_value();
                const auto ax = v.at("axes").to_vector<int64_t>();
                return ax.size() == 1 and (ax[0] == -1 or ax[0] == 3) and
                       v.at("starts").to_vector<int64_t>() == std::vector<int64_t>{static_cast<int64_t>(lo)} and
                       v.at("ends").to_vector<int64_t>() == std::vector<int64_t>{static_cast<int64_t>(hi)};
            };
            if(not is_slice(s2, half, d) or not is_slice(s1, 0, half) or s1->inputs()[0] != s2->inputs()[0])
                continue;
            auto x = s1->inputs()[0];
            if(x->get_shape().lens() != os.lens() or x->get_shape().strides().back() != 1)
                continue;
            // mc = mul(x, cos rows)
            if(mc->inputs()[0] != x and mc->inputs()[1] != x)
                continue;
            auto cosb = mc->inputs()[0] == x ? mc->inputs()[1] : mc->inputs()[0];
            // msin = mul(signs, sin rows): signs constant, -1 on the first half of every row, +1 on the second
            instruction_ref sg = m.end(), sinb = m.end();
            for(auto i : msin->inputs())
            {
                if(i->can_eval())
                    sg = i;
                else
                    sinb = i;
            }
            if(sg == m.end() or sinb == m.end() or sg->get_shape().lens() != os.lens())
                continue;
            bool signs_ok = true;
            sg->eval().visit([&](auto view) {
                for(std::size_t i = 0; i < view.size() and signs_ok; ++i)
                    signs_ok = static_cast<float>(view[i]) == ((i % d) < half ? -1.0f : 1.0f);
            });
            if(not signs_ok)
                continue;
            const std::size_t mark = chain.size();
            auto cr = cache_rows(cosb);
            auto sr = cache_rows(sinb);
            if(cr.first == m.end() or sr.first == m.end() or cr.second != sr.second)
            {
                chain.resize(mark);
                continue;
            }
            auto idx       = cr.second;
            const auto& is = idx->get_shape();
            const auto& cs = cr.first->get_shape();
            if(is.elements() != os.lens()[0] * os.lens()[2] or is.lens().back() != 1 or
               (is.type() != shape::int32_type and is.type() != shape::int64_type) or cs.type() != os.type() or
               cs.ndim() != 2 or cs.lens()[1] != half or sr.first->get_shape().lens() != cs.lens() or
               sr.first->get_shape().type() != os.type())
            {
                chain.resize(mark);
                continue;
            }
            chain.insert(chain.end(), {mc, ms2, rot, s1, s2, msin});
            for(auto c : chain)
            {
                consume(c);
                for(auto i : c->inputs())
                    if(i->can_eval() and i->outputs().size() == 1 and not is_builtin(i->name()))
                        consume(i);
            }
            auto pos = idx;
            if(not is.standard())
                pos = standard_copy(add, idx);
            auto cosc = cr.first, sinc = sr.first;
            if(not cosc->get_shape().standard())
                cosc = standard_copy(add, cosc);
            if(not sinc->get_shape().standard())
                sinc = standard_copy(add, sinc);
            auto buf = insert_allocation(m, add, os.as_standard());
            consume(m.replace_instruction(add, op_rotary_embedding{}, x, pos, cosc, sinc, buf));
            return true;
        }
        return false;
    }

    // ---------------------------------------------------------------- decode-step GQA attention
    // softmax(where(position > seqlens_k, -inf, mul(dot(Q, transpose(K')), scale))) followed by
    // dot(P, V'), K' / V' the caches with their KV heads broadcast to the query heads, one query
    // row per head (src/onnx/parse_group_query_attention.cpp:184-262): one cuda::gqa_decode_attention
    // in place of the second dot.  Anything else (a prompt, another mask) keeps the operators.
    bool lower_gqa_decode(instruction_ref sm)
    {
        if(fusion_disabled("attention"))
            return false;
        const auto& ps = sm->get_shape(); // [B, heads, 1, T]
        if(ps.type() != shape::half_type or ps.ndim() != 4 or ps.lens()[2] != 1)
            return false;
        const auto ax = sm->get_operator().to_value().at("axis").to<int64_t>();
        if(ax != 3 and ax != -1)
            return false;
        const std::size_t b = ps.lens()[0], nh = ps.lens()[1], t = ps.lens()[3];
        auto is_transpose = [](instruction_ref x, std::vector<int64_t> perm) {
            return x->name() == "transpose" and
                   x->get_operator().to_value().at("permutation").to_vector<int64_t>() == perm;
        };
        // the cache behind the grouped-query broadcast: reshape(multibroadcast(unsqueeze(cache, 2)))
        std::vector<instruction_ref> chain = {sm};
        auto cache_of = [&](instruction_ref x, std::size_t d) -> instruction_ref {
            if(x->name() == "reshape" or x->name() == "reshape_lazy")
            {
                auto mb = x->inputs().front();
                if(mb->name() != "multibroadcast" or mb->get_shape().ndim() != 5)
                    return m.end();
                auto us = mb->inputs().front();
                if(us->name() != "unsqueeze" or
                   us->get_operator().to_value().at("axes").to_vector<int64_t>() != std::vector<int64_t>{2})
                    return m.end();
                chain.insert(chain.end(), {x, mb, us});
                x = us->inputs().front();
            }
            const auto& xs = x->get_shape();
            if(xs.type() != shape::half_type or xs.ndim() != 4 or not xs.standard() or xs.lens()[0] != b or
               xs.lens()[2] != t or xs.lens()[3] != d or nh % xs.lens()[1] != 0)
                return m.end();
            return x;
        };
        // where(mask, -inf, scores)
        auto wh = sm->inputs().front();
        if(wh->name() != "where" or wh->outputs().size() != 1)
            return false;
        auto mask = wh->inputs()[0], fill = wh->inputs()[1], mul = wh->inputs()[2];
        if(not fill->can_eval())
            return false;
        {
            auto fv = classify_constant(fill);
            if(fv.kind != bcast_kind::scalar or not(std::isinf(fv.values[0]) and fv.values[0] < 0))
                return false;
        }
        if(mask->name() == "convert")
        {
            chain.push_back(mask);
            mask = mask->inputs().front();
        }
        if(mask->name() != "greater")
            return false;
        // greater(positions 0 .. T-1 along the last axis, seqlens_k of the batch entry)
        auto range = mask->inputs()[0], lens = mask->inputs()[1];
        if(not range->can_eval())
            return false;
        {
            auto rv = range->eval();
            const auto& rs = rv.get_shape();
            if(rs.lens() != ps.lens() or rs.strides()[0] != 0 or rs.strides()[1] != 0 or rs.strides()[3] != 1)
                return false;
            bool iota = true;
            rv.visit([&](auto view) {
                for(std::size_t j = 0; j < t and iota; ++j)
                    iota = static_cast<std::size_t>(view[j]) == j;
            });
            if(not iota)
                return false;
        }
        chain.push_back(mask);
        // the past lengths behind broadcasts and reshapes: one value per batch entry
        while(lens->name() == "multibroadcast" or lens->name() == "reshape" or lens->name() == "reshape_lazy")
        {
            const auto& ls = lens->get_shape();
            // every view on the way must vary along the batch only
            if(ls.lens()[0] != b)
                return false;
            chain.push_back(lens);
            lens = lens->inputs().front();
        }
        const auto& lsh = lens->get_shape();
        if(lsh.elements() != b or not lsh.standard() or
           (lsh.type() != shape::int32_type and lsh.type() != shape::int64_type))
            return false;
        // scores = mul(dot(Q, K'^T), scale)
        if(mul->name() != "mul" or mul->outputs().size() != 1)
            return false;
        instruction_ref c = m.end();
        for(auto i : mul->inputs())
            if(i->can_eval())
                c = i;
        if(c == m.end())
            return false;
        auto cv = classify_constant(c);
        if(cv.kind != bcast_kind::scalar)
            return false;
        auto d1 = other_input(mul, c);
        if(d1->name() != "dot" or d1->outputs().size() != 1)
            return false;
        auto q  = d1->inputs()[0];
        auto kt = d1->inputs()[1];
        const auto& qs = q->get_shape();
        if(qs.type() != shape::half_type or qs.ndim() != 4 or qs.lens()[0] != b or qs.lens()[1] != nh or
           qs.lens()[2] != 1 or qs.strides().back() != 1)
            return false;
        const std::size_t d = qs.lens()[3];
        if(not is_transpose(kt, {0, 1, 3, 2}))
            return false;
        auto kc = cache_of(kt->inputs().front(), d);
        auto d2 = single_user(m, sm);
        if(kc == m.end() or not valid(d2, m) or d2->name() != "dot" or d2->inputs()[0] != sm)
            return false;
        auto vc = cache_of(d2->inputs()[1], d);
        if(vc == m.end() or vc->get_shape() != kc->get_shape())
            return false;
        const std::size_t kvh = kc->get_shape().lens()[1];
        if(mgx_cuda_gqa_decode_supported(static_cast<int64_t>(b), static_cast<int64_t>(nh), static_cast<int64_t>(kvh),
                                         static_cast<int64_t>(d), static_cast<int64_t>(t)) == 0)
            return false;
        chain.insert(chain.end(), {wh, mul, d1, kt});
        for(auto x : chain)
        {
            consume(x);
            for(auto i : x->inputs())
                if(i->can_eval() and i->outputs().size() == 1 and not is_builtin(i->name()))
                    consume(i);
        }
        op_gqa_decode_attention op;
        op.num_heads    = nh;
        op.kv_num_heads = kvh;
        op.scale        = cv.values[0];
        auto buf = insert_allocation(m, d2, d2->get_shape().as_standard());
        consume(m.replace_instruction(d2, op, q, kc, vc, lens, buf));
        return true;
    }

    // ---------------------------------------------------------------- LayerNorm
    // mean = reduce_mean(x, last axis); d = sub(x, bcast(mean)); var = reduce_mean(mul(d, d) |
    // sqdiff(x, bcast(mean))); rs = rsqrt(add(var, eps)); y = mul(d, bcast(rs)) [* gamma] [+ beta]
    // (src/onnx/parse_layernorm.cpp:100-140) becomes one cuda::layernorm; a per-tensor
    // quantizelinear of y joins it.  Anything that does not match exactly is left to the
    // single-operator lowering.
    bool lower_layernorm(instruction_ref mean)
    {
        if(fusion_disabled("layernorm"))
            return false;
        auto x         = mean->inputs().front();
        const auto& xs = x->get_shape();
        const auto nd  = xs.ndim();
        if(nd < 2 or not xs.standard() or (xs.type() != shape::float_type and xs.type() != shape::half_type))
            return false;
        if(not mgx_cuda_layernorm_supported(xs.type() == shape::half_type ? MGX_F16 : MGX_F32,
                                            static_cast<int64_t>(xs.lens().back())))
            return false;
        auto last_axis_only = [&](instruction_ref r) {
            auto axes = r->get_operator().to_value().at("axes").to_vector<int64_t>();
            return axes.size() == 1 and (axes[0] == -1 or axes[0] == static_cast<int64_t>(nd) - 1);
        };
        auto is_bcast_of = [&](instruction_ref b, instruction_ref src) {
            return b->name() == "multibroadcast" and b->inputs().size() == 1 and b->inputs()[0] == src and
                   b->get_shape().lens() == xs.lens();
        };
        auto users = [](instruction_ref i) {
            std::set<instruction*> u;
            for(auto o : i->outputs())
                u.insert(&*o);
            return u;
        };
        if(not last_axis_only(mean) or mean->outputs().size() != 1)
            return false;
        auto mb = mean->outputs().front();
        if(not is_bcast_of(mb, mean))
            return false;
        instruction_ref d = m.end(), sq = m.end();
        for(auto u : mb->outputs())
        {
            if(u->name() == "sub" and u->inputs()[0] == x and u->inputs()[1] == mb)
                d = u;
            else if(u->name() == "sqdiff" and u->inputs()[0] == x and u->inputs()[1] == mb)
                sq = u;
            else
                return false;
        }
        if(d == m.end())
            return false;
        instruction_ref nv = m.end();
        for(auto u : d->outputs())
        {
            if(u->name() == "mul" and u->inputs()[0] == d and u->inputs()[1] == d and sq == m.end())
                sq = u;
            else if(u->name() == "mul" and u->inputs()[0] == d and u != sq)
                nv = u;
            else if(u != sq)
                return false;
        }
        if(sq == m.end() or nv == m.end() or users(d).size() != (sq->name() == "mul" ? 2u : 1u))
            return false;
        auto var = single_user(m, sq);
        if(not valid(var, m) or var->name() != "reduce_mean" or not last_axis_only(var))
            return false;
        auto ve = single_user(m, var);
        if(not valid(ve, m) or ve->name() != "add" or not other_input(ve, var)->can_eval())
            return false;
        auto ec = classify_constant(other_input(ve, var));
        if(ec.kind != bcast_kind::scalar)
            return false;
        auto rs = single_user(m, ve);
        if(not valid(rs, m) or rs->name() != "rsqrt")
            return false;
        auto mb2 = single_user(m, rs);
        if(not valid(mb2, m) or not is_bcast_of(mb2, rs) or single_user(m, mb2) != nv or nv->inputs()[1] != mb2)
            return false;
        op_layernorm op;
        op.eps = ec.values[0];
        std::vector<instruction_ref> chain = {mean, mb, d, sq, var, ve, rs, mb2, nv};
        instruction_ref last = nv;
        std::vector<instruction_ref> args = {x};
        auto per_col_literal = [&](instruction_ref c) {
            auto cv = classify_constant(c);
            if(cv.kind == bcast_kind::scalar)
                cv.values.assign(xs.lens().back(), cv.values[0]);
            else if(cv.kind != bcast_kind::per_col)
                return m.end();
            if(xs.type() == shape::half_type)
            {
                std::vector<half> h(cv.values.begin(), cv.values.end());
                return m.add_literal(literal{shape{shape::half_type, {h.size()}}, h});
            }
            return add_float_literal(m, cv.values);
        };
        auto u = single_user(m, last);
        if(valid(u, m) and u->name() == "mul" and other_input(u, last)->can_eval())
        {
            auto g = per_col_literal(other_input(u, last));
            if(g != m.end())
            {
                op.has_gamma = true;
                args.push_back(g);
                chain.push_back(u);
                last = u;
                u    = single_user(m, last);
            }
        }
        if(valid(u, m) and u->name() == "add" and other_input(u, last)->can_eval())
        {
            auto b = per_col_literal(other_input(u, last));
            if(b != m.end())
            {
                op.has_beta = true;
                args.push_back(b);
                chain.push_back(u);
                last = u;
            }
        }
        // a per-tensor quantizelinear of the result is done by the same kernel
        instruction_ref qz = m.end();
        for(auto o : last->outputs())
        {
            if(o->name() != "quantizelinear" or o->inputs().size() != 3 or o->inputs()[0] != last)
                continue;
            const auto qt = o->get_shape().type();
            if((qt != shape::int8_type and qt != shape::fp8e4m3fn_type) or not o->inputs()[1]->can_eval() or
               not o->inputs()[2]->can_eval())
                continue;
            auto cs = classify_constant(o->inputs()[1]);
            auto cz = classify_constant(o->inputs()[2]);
            if(cs.kind != bcast_kind::scalar or cz.kind != bcast_kind::scalar or not(cs.values[0] > 0))
                continue;
            op.q_type  = static_cast<int>(qt);
            op.q_scale = cs.values[0];
            op.q_zp    = cz.values[0];
            qz         = o;
            break;
        }
        // ... and so is a dequantizelinear of that quantised tensor with the same zero point (what
        // simplify_qdq turns other reads of the un-quantised tensor into, src/simplify_qdq.cpp:401-432)
        instruction_ref dqz = m.end();
        if(qz != m.end() and qz->get_shape().type() == shape::int8_type)
        {
            for(auto o : qz->outputs())
            {
                if(o->name() != "dequantizelinear" or o->inputs()[0] != qz or o->get_shape().type() != xs.type() or
                   not o->inputs()[1]->can_eval())
                    continue;
                auto ds = classify_constant(o->inputs()[1]);
                if(ds.kind != bcast_kind::scalar)
                    continue;
                float zp = 0.0f;
                if(o->inputs().size() == 3)
                {
                    if(not o->inputs()[2]->can_eval())
                        continue;
                    auto dz = classify_constant(o->inputs()[2]);
                    if(dz.kind != bcast_kind::scalar)
                        continue;
                    zp = dz.values[0];
                }
                if(zp != op.q_zp)
                    continue;
                op.has_dq   = true;
                op.dq_scale = ds.values[0];
                dqz         = o;
                break;
            }
        }
        const bool only_q = qz != m.end() and last->outputs().size() == 1;
        for(auto c : chain)
        {
            consume(c);
            for(auto i : c->inputs())
                if(i->can_eval() and i->outputs().size() == 1 and not is_builtin(i->name()))
                    consume(i);
        }
        instruction_ref dqbuf = m.end();
        auto first_result     = only_q ? qz : last;
        if(dqz != m.end())
        {
            dqbuf = insert_allocation(m, first_result, dqz->get_shape().as_standard());
            args.push_back(dqbuf);
        }
        instruction_ref rep;
        if(only_q)
        {
            op.write_y = false;
            args.push_back(insert_allocation(m, qz, qz->get_shape().as_standard()));
            rep = m.replace_instruction(qz, op, args);
            consume(rep);
        }
        else
        {
            instruction_ref qbuf = m.end();
            if(qz != m.end())
            {
                qbuf = insert_allocation(m, last, qz->get_shape().as_standard());
                args.push_back(qbuf);
            }
            args.push_back(insert_allocation(m, last, last->get_shape().as_standard()));
            rep = m.replace_instruction(last, op, args);
            consume(rep);
            if(qz != m.end())
                consume(m.replace_instruction(qz, op_second_output{}, rep, qbuf));
        }
        if(dqz != m.end())
            consume(m.replace_instruction(dqz, op_second_output{}, rep, dqbuf));
        return true;
    }

    // ---------------------------------------------------------------- RMSNorm
    // SimplifiedLayerNormalization as the parser decomposes it
    // (src/onnx/parse_simplified_layer_normalization.cpp:91-106): fx = convert<float>(x);
    // ms = convert<T>(reduce_mean(mul(fx, fx))); rr = rsqrt(add(ms, eps)); y = mul(mul(x, bcast(rr)), gamma)
    // becomes one cuda::layernorm with rms set.
    bool lower_rmsnorm(instruction_ref rm)
    {
        if(fusion_disabled("layernorm") or rm->inputs().size() != 1 or rm->outputs().size() != 1)
            return false;
        auto sq = rm->inputs().front();
        if(sq->name() != "mul" or sq->inputs()[0] != sq->inputs()[1] or sq->outputs().size() != 1)
            return false;
        auto fx = sq->inputs()[0];
        auto x  = fx;
        std::vector<instruction_ref> chain = {rm, sq};
        if(fx->name() == "convert" and fx->get_shape().type() == shape::float_type)
        {
            if(fx->outputs().size() != 1)
                return false;
            x = fx->inputs().front();
            chain.push_back(fx);
        }
        const auto& xs = x->get_shape();
        const auto nd  = xs.ndim();
        if(nd < 2 or not xs.standard() or (xs.type() != shape::float_type and xs.type() != shape::half_type))
            return false;
        if(not mgx_cuda_layernorm_supported(xs.type() == shape::half_type ? MGX_F16 : MGX_F32,
                                            static_cast<int64_t>(xs.lens().back())))
            return false;
        auto axes = rm->get_operator().to_value().at("axes").to_vector<int64_t>();
        if(axes.size() != 1 or (axes[0] != -1 and axes[0] != static_cast<int64_t>(nd) - 1))
            return false;
        auto cur = single_user(m, rm);
        if(valid(cur, m) and cur->name() == "convert" and cur->get_shape().type() == xs.type())
        {
            chain.push_back(cur);
            cur = single_user(m, cur);
        }
        else if(xs.type() != shape::float_type)
            return false;
        if(not valid(cur, m) or cur->name() != "add")
            return false;
        auto ve = cur;
        instruction_ref ecst = m.end();
        for(auto i : ve->inputs())
            if(i->can_eval())
                ecst = i;
        if(ecst == m.end())
            return false;
        auto ec = classify_constant(ecst);
        if(ec.kind != bcast_kind::scalar)
            return false;
        auto rs = single_user(m, ve);
        if(not valid(rs, m) or rs->name() != "rsqrt")
            return false;
        auto mb = single_user(m, rs);
        if(not valid(mb, m) or mb->name() != "multibroadcast" or mb->get_shape().lens() != xs.lens())
            return false;
        auto nv = single_user(m, mb);
        if(not valid(nv, m) or nv->name() != "mul" or other_input(nv, mb) != x)
            return false;
        chain.insert(chain.end(), {ve, rs, mb, nv});
        op_layernorm op;
        op.rms = true;
        op.eps = ec.values[0];
        instruction_ref last = nv;
        std::vector<instruction_ref> args = {x};
        auto u = single_user(m, last);
        if(valid(u, m) and u->name() == "mul" and other_input(u, last)->can_eval())
        {
            auto cv = classify_constant(other_input(u, last));
            if(cv.kind == bcast_kind::scalar)
                cv.values.assign(xs.lens().back(), cv.values[0]);
            if(cv.kind == bcast_kind::scalar or cv.kind == bcast_kind::per_col)
            {
                instruction_ref g;
                if(xs.type() == shape::half_type)
                {
                    std::vector<half> h(cv.values.begin(), cv.values.end());
                    g = m.add_literal(literal{shape{shape::half_type, {h.size()}}, h});
                }
                else
                    g = add_float_literal(m, cv.values);
                op.has_gamma = true;
                args.push_back(g);
                chain.push_back(u);
                last = u;
            }
        }
        for(auto c : chain)
        {
            consume(c);
            for(auto i : c->inputs())
                if(i->can_eval() and i->outputs().size() == 1 and not is_builtin(i->name()))
                    consume(i);
        }
        args.push_back(insert_allocation(m, last, last->get_shape().as_standard()));
        consume(m.replace_instruction(last, op, args));
        return true;
    }

    // ---------------------------------------------------------------- single operators
    template <class Op>
    void lower_elementwise(instruction_ref ins, Op op)
    {
        auto args = ins->inputs();
        op.has_zp = args.size() == 3;
        if(not args[0]->get_shape().standard() and args[0]->get_shape().ndim() != 2)
            unsupported(ins, "input must be standard or a 2-D row-strided view");
        args.push_back(insert_allocation(m, ins, ins->get_shape().as_standard()));
        consume(m.replace_instruction(ins, op, args));
    }

    // A single element-wise operator (src/include/migraphx/op/{unary,binary}.hpp and friends)
    // becomes a one-instruction cuda::pointwise.
    bool lower_elementwise_op(instruction_ref ins)
    {
        static const std::unordered_map<std::string, int> table = {
            {"add", MGX_PW_ADD},       {"sub", MGX_PW_SUB},         {"mul", MGX_PW_MUL},
            {"div", MGX_PW_DIV},       {"min", MGX_PW_MIN},         {"max", MGX_PW_MAX},
            {"pow", MGX_PW_POW},       {"neg", MGX_PW_NEG},         {"abs", MGX_PW_ABS},
            {"exp", MGX_PW_EXP},       {"log", MGX_PW_LOG},         {"sqrt", MGX_PW_SQRT},
            {"rsqrt", MGX_PW_RSQRT},   {"recip", MGX_PW_RECIP},     {"tanh", MGX_PW_TANH},
            {"sigmoid", MGX_PW_SIGMOID}, {"erf", MGX_PW_ERF},       {"relu", MGX_PW_RELU},
            {"sin", MGX_PW_SIN},       {"cos", MGX_PW_COS},         {"floor", MGX_PW_FLOOR},
            {"ceil", MGX_PW_CEIL},     {"round", MGX_PW_ROUND},     {"nearbyint", MGX_PW_NEARBYINT},
            {"convert", MGX_PW_CONVERT}, {"where", MGX_PW_WHERE},   {"clip", MGX_PW_CLIP},
            {"equal", MGX_PW_EQUAL},   {"greater", MGX_PW_GREATER}, {"less", MGX_PW_LESS},
            {"leaky_relu", MGX_PW_LEAKY_RELU}, {"identity", MGX_PW_IDENTITY},
            {"contiguous", MGX_PW_IDENTITY}};
        auto it = table.find(ins->name());
        if(it == table.end())
            return false;
        auto args = ins->inputs();
        if(args.empty() or args.size() > 3)
            return false;
        const auto& os = ins->get_shape();
        for(auto a : args)
            if(a->get_shape().lens() != os.lens())
                unsupported(ins, "operands must have the output's dimensions");
        op_pointwise op;
        op.ops   = {it->second};
        op.types = {static_cast<int>(os.type())};
        op.srcs  = {0, args.size() > 1 ? 1 : 0, args.size() > 2 ? 2 : 0};
        op.imms  = {0.0f};
        if(ins->name() == "leaky_relu")
            op.imms[0] = ins->get_operator().to_value().at("alpha").to<float>();
        args.push_back(insert_allocation(m, ins, os.as_standard()));
        consume(m.replace_instruction(ins, op, args));
        return true;
    }

    // the decoder's cache / rotary operators and gathernd over single row indices
    bool lower_decoder_op(instruction_ref ins)
    {
        const auto name = ins->name();
        if(name == "concat_past_present")
        {
            auto args = ins->inputs();
            if(args.size() != 3)
                unsupported(ins, "expects present, seqlens_k and the cache");
            const auto& pr = args[0]->get_shape();
            if(pr.ndim() != 4 or pr.strides().back() != 1)
                args[0] = standard_copy(ins, args[0]);
            if(not args[1]->get_shape().standard())
                args[1] = standard_copy(ins, args[1]);
            if(not args[2]->get_shape().standard())
                unsupported(ins, "the cache must be a packed tensor");
            op_concat_past_present op;
            op.kv_num_heads = ins->get_operator().to_value().at("kv_num_heads").to<std::size_t>();
            consume(m.replace_instruction(ins, op, args));
            return true;
        }
        if(name == "gqa_rotary_embedding")
        {
            auto args = ins->inputs();
            if(args.size() != 4)
                unsupported(ins, "expects packed QKV, seqlens_k and the cos / sin caches");
            for(auto& a : args)
                if(not a->get_shape().standard())
                    a = standard_copy(ins, a);
            const auto v = ins->get_operator().to_value();
            op_gqa_rotary_embedding op;
            op.num_heads    = v.at("num_heads").to<std::size_t>();
            op.kv_num_heads = v.at("kv_num_heads").to<std::size_t>();
            op.interleaved  = v.at("interleaved").to<bool>();
            args.push_back(insert_allocation(m, ins, ins->get_shape().as_standard()));
            consume(m.replace_instruction(ins, op, args));
            return true;
        }
        if(name == "gathernd")
        {
            // indices [.., 1] without batch dimensions select whole slices along axis 0: a gather
            // (src/include/migraphx/op/gathernd.hpp); what the rotary-embedding builder uses to pick the
            // cos / sin rows of the positions (src/op/builder/rotary_embedding.cpp:151-154)
            const auto v   = ins->get_operator().to_value();
            auto data      = ins->inputs()[0];
            auto idx       = ins->inputs()[1];
            const auto& is = idx->get_shape();
            if(v.at("batch_dims").to<int64_t>() != 0 or is.lens().back() != 1)
                unsupported(ins, "only indices of one component without batch dimensions");
            if(is.type() != shape::int32_type and is.type() != shape::int64_type)
                unsupported(ins, "indices must be int32 or int64");
            if(not data->get_shape().standard())
                data = standard_copy(ins, data);
            if(not is.standard())
                idx = standard_copy(ins, idx);
            auto il = is.lens();
            il.pop_back();
            if(il.empty())
                il.push_back(1);
            auto flat = m.insert_instruction(ins, make_op("reshape_lazy", {{"dims", il}}), idx);
            auto buf  = insert_allocation(m, ins, ins->get_shape().as_standard());
            consume(m.replace_instruction(ins, op_gather{0}, data, flat, buf));
            return true;
        }
        return false;
    }

    // gather and concat: byte movers on packed tensors (strided operands are packed first)
    bool lower_mover(instruction_ref ins)
    {
        const auto name = ins->name();
        if(name != "gather" and name != "concat")
            return false;
        auto v        = ins->get_operator().to_value();
        auto axis     = v.at("axis").to<int64_t>();
        const auto nd = static_cast<int64_t>(ins->inputs()[0]->get_shape().ndim());
        if(axis < 0)
            axis += nd;
        auto args = ins->inputs();
        for(auto& a : args)
            if(not a->get_shape().standard())
                a = standard_copy(ins, a);
        if(name == "gather")
        {
            const auto it = args[1]->get_shape().type();
            if(it != shape::int32_type and it != shape::int64_type)
                unsupported(ins, "indices must be int32 or int64");
        }
        args.push_back(insert_allocation(m, ins, ins->get_shape().as_standard()));
        if(name == "gather")
            consume(m.replace_instruction(ins, op_gather{axis}, args));
        else
            consume(m.replace_instruction(ins, op_concat{axis}, args));
        return true;
    }

    // reduce_* and softmax over the innermost axis
    bool lower_row_op(instruction_ref ins)
    {
        static const std::unordered_map<std::string, int> modes = {{"reduce_sum", MGX_REDUCE_SUM},
                                                                   {"reduce_mean", MGX_REDUCE_MEAN},
                                                                   {"reduce_max", MGX_REDUCE_MAX},
                                                                   {"reduce_min", MGX_REDUCE_MIN}};
        const auto name    = ins->name();
        const bool softmax = name == "softmax";
        auto it            = modes.find(name);
        if(not softmax and it == modes.end())
            return false;
        if(ins->inputs().size() != 1)
            unsupported(ins, "variable axes are not supported");
        const auto& xs = ins->inputs()[0]->get_shape();
        const auto nd  = static_cast<int64_t>(xs.ndim());
        const auto v   = ins->get_operator().to_value();
        if(softmax)
        {
            const auto ax = v.at("axis").to<int64_t>();
            if(ax != -1 and ax != nd - 1)
                unsupported(ins, "only the innermost axis is supported");
        }
        if(xs.type() != shape::float_type and xs.type() != shape::half_type)
            unsupported(ins, "float and half only");
        auto args = ins->inputs();
        if(softmax)
        {
            if(not xs.standard())
                args[0] = standard_copy(ins, args[0]);
            args.push_back(insert_allocation(m, ins, ins->get_shape().as_standard()));
            consume(m.replace_instruction(ins, op_softmax{}, args));
            return true;
        }
        // reductions: the reduced axes become the trailing ones of a packed tensor
        std::vector<bool> reduced(nd, false);
        for(auto a : v.at("axes").to_vector<int64_t>())
        {
            a = a < 0 ? a + nd : a;
            if(a < 0 or a >= nd)
                unsupported(ins, "axis out of range");
            reduced[a] = true;
        }
        std::vector<int64_t> perm;
        for(int64_t d = 0; d < nd; ++d)
            if(not reduced[d])
                perm.push_back(d);
        const std::size_t kept = perm.size();
        for(int64_t d = 0; d < nd; ++d)
            if(reduced[d])
                perm.push_back(d);
        if(kept == static_cast<std::size_t>(nd))
            unsupported(ins, "no axis to reduce");
        bool trailing = true;
        for(int64_t d = 0; d < nd; ++d)
            if(perm[d] != d)
                trailing = false;
        if(trailing)
        {
            if(not xs.standard())
                args[0] = standard_copy(ins, args[0]);
            args.push_back(insert_allocation(m, ins, ins->get_shape().as_standard()));
            consume(m.replace_instruction(ins, op_reduce{it->second}, args));
            return true;
        }
        // other axes: a transposed packed copy first; the result (reduced dimensions of length 1)
        // has the element order of the operator's output, so a view gives it its dimensions
        auto xt = m.insert_instruction(ins, make_op("transpose", {{"permutation", perm}}), args[0]);
        auto xc = standard_copy(ins, xt);
        auto ol = xc->get_shape().lens();
        for(std::size_t d = kept; d < ol.size(); ++d)
            ol[d] = 1;
        auto buf = insert_allocation(m, ins, shape{xs.type(), ol});
        auto red = m.insert_instruction(ins, op_reduce{it->second}, xc, buf);
        consume(red);
        m.replace_instruction(ins, make_op("reshape_lazy", {{"dims", ins->get_shape().lens()}}), red);
        return true;
    }

    // packed copy of a strided view (what op::contiguous computes), made by the element-wise kernel
    instruction_ref standard_copy(instruction_ref pos, instruction_ref x)
    {
        op_pointwise op;
        op.ops   = {MGX_PW_IDENTITY};
        op.types = {static_cast<int>(x->get_shape().type())};
        op.srcs  = {0, 0, 0};
        op.imms  = {0.0f};
        auto buf = insert_allocation(m, pos, x->get_shape().as_standard());
        auto c   = m.insert_instruction(pos, op, x, buf);
        consume(c);
        return c;
    }

    // reshape copies its input in logical order (src/include/migraphx/op/reshape.hpp:207-217):
    // a view of the packed tensor
    void lower_reshape(instruction_ref ins)
    {
        if(ins->inputs().size() != 1)
            unsupported(ins, "only the one-operand form is supported");
        auto x = ins->inputs()[0];
        if(not x->get_shape().standard())
            x = standard_copy(ins, x);
        m.replace_instruction(ins, make_op("reshape_lazy", {{"dims", ins->get_shape().lens()}}), x);
    }

    // dot on fp16 operands (attention's Q.K^T and P.V, un-quantised linears): the tiled GEMM with
    // kind::f16 operands and fp32 accumulation, result truncated to fp16 (the reference's gemm
    // accumulates in double, src/include/migraphx/gemm.hpp).
    bool lower_half_dot(instruction_ref ins)
    {
        if(ins->inputs().size() != 2)
            return false;
        auto a = ins->inputs()[0];
        auto b = ins->inputs()[1];
        const auto& as = a->get_shape();
        const auto& bs = b->get_shape();
        if(as.type() != shape::half_type or bs.type() != shape::half_type or as.ndim() < 2 or
           bs.ndim() != as.ndim())
            return false;
        const auto nd = as.ndim();
        const auto k  = as.lens()[nd - 1];
        for(std::size_t j = 0; j + 2 < nd; ++j)
            if(as.lens()[j] != bs.lens()[j])
                return false;
        // a transposed / sliced left operand (attention heads) is packed first
        const bool a_ok = as.strides()[nd - 1] == 1 and as.strides()[nd - 2] % 8 == 0 and
                          (nd == 2 or as.standard());
        if(not a_ok and not as.standard())
            a = standard_copy(ins, a);
        if(k % 8 != 0)
        {
            // rows of 16-byte multiples (the tensor maps' stride rule): copy into padded rows
            const std::size_t kp = (k + 7) / 8 * 8;
            auto lens            = as.lens();
            std::vector<std::size_t> strides(nd, 1);
            strides[nd - 2] = kp;
            for(std::size_t j = nd - 2; j-- > 0;)
                strides[j] = strides[j + 1] * lens[j + 1];
            auto buf = insert_allocation(m, ins, shape{shape::half_type, lens, strides});
            a        = m.insert_instruction(ins, op_pad_rows{}, a, buf);
            consume(a);
        }
        op_qgemm op;
        op.out_type = static_cast<int>(shape::half_type);
        std::vector<instruction_ref> args = {a, b};
        instruction_ref workspace         = m.end();
        bool transposed_view = bs.strides()[nd - 1] != 1 and bs.strides()[nd - 2] == 1 and
                               bs.strides()[nd - 1] % 8 == 0;
        // every batch entry evenly spaced, like a standard tensor's
        for(std::size_t j = 0; j + 3 < nd; ++j)
            if(bs.strides()[j] != bs.strides()[j + 1] * bs.lens()[j + 1])
                transposed_view = false;
        if(nd > 2 and bs.strides()[nd - 3] % 8 != 0)
            transposed_view = false;
        if(b->can_eval() and k % 8 == 0)
        {
            args[1] = add_transposed_8bit_literal(m, b);
            op.b_nk = true;
        }
        else if(transposed_view)
        {
        }
        else
        {
            if(not bs.standard())
                args[1] = standard_copy(ins, b);
            const std::size_t kp = (k + 7) / 8 * 8;
            const std::size_t ws = bs.elements() / k * kp * 2;
            workspace            = insert_allocation(m, ins, shape{shape::int8_type, {ws}});
            op.has_workspace     = true;
        }
        if(workspace != m.end())
            args.push_back(workspace);
        args.push_back(insert_allocation(m, ins, ins->get_shape().as_standard()));
        consume(m.replace_instruction(ins, op, args));
        return true;
    }

    template <class Op>
    void lower_int4(instruction_ref ins, Op op)
    {
        const auto v  = ins->get_operator().to_value();
        const auto nd = static_cast<int64_t>(ins->get_shape().ndim());
        const auto ax = v.contains("axis") ? v.at("axis").template to<int64_t>() : -1;
        if(ax != -1 and ax != nd - 1)
            unsupported(ins, "only the last axis is supported");
        if(not ins->inputs()[0]->get_shape().standard())
            unsupported(ins, "input must be a standard tensor");
        auto args = ins->inputs();
        args.push_back(insert_allocation(m, ins, ins->get_shape().as_standard()));
        consume(m.replace_instruction(ins, op, args));
    }

    bool skip(instruction_ref ins) const
    {
        if(is_consumed(ins))
            return true;
        const auto name = ins->name();
        if(is_builtin(name) or is_view_op(name) or name == "allocate" or starts_with(name, "cuda::"))
            return true;
        // dead: removed by dead_code_elimination
        return ins->outputs().empty() and ins != std::prev(m.end());
    }

    void run()
    {
        std::vector<instruction_ref> order;
        for(auto ins : iterator_for(m))
            order.push_back(ins);
        // whole attention blocks first (their two dots must not be lowered one by one)
        for(auto ins : order)
            if(not skip(ins) and ins->name() == "softmax")
            {
                if(not lower_gqa_decode(ins))
                    lower_attention(ins);
            }
        // the rotary-embedding builder's rotation
        for(auto ins : order)
            if(not skip(ins) and ins->name() == "add")
                lower_rotary(ins);
        // GEMM sub-graphs next: their operands (packed int4 weights, scale expressions) must
        // still be in their original form, not folded into dense constants
        for(auto ins : order)
        {
            if(skip(ins))
                continue;
            if(ins->name() == "quant_dot")
                lower_quant_dot(ins);
            else if(ins->name() == "dot")
            {
                if(not lower_w4a16(ins) and not lower_w4a16_kn(ins) and not lower_half_dot(ins))
                    unsupported(ins, "only fp16 operands and the weight-only int4 form "
                                     "dot(A, transpose(dequantizelinear(unpack_int4(W)))) are supported");
            }
        }
        for(auto ins : order)
        {
            if(skip(ins))
                continue;
            if(ins->name() == "reduce_mean" and ins->inputs().size() == 1)
            {
                if(not lower_rmsnorm(ins))
                    lower_layernorm(ins);
            }
        }
        for(auto ins : order)
        {
            if(skip(ins))
                continue;
            const auto name = ins->name();
            if(ins->can_eval())
            {
                // a constant sub-graph (e.g. quantizelinear of a weight literal) is
                // evaluated once, now, and becomes a literal
                argument v = ins->eval();
                argument sv = v.get_shape().standard() ? v : make_standard(v);
                m.replace_instruction(ins, m.add_literal(literal{sv.get_shape(), sv.data()}));
                continue;
            }
            if(name == "quantizelinear")
                lower_elementwise(ins, op_quantizelinear{});
            else if(name == "dequantizelinear")
                lower_elementwise(ins, op_dequantizelinear{});
            else if(name == "unpack_int4")
                lower_int4(ins, op_unpack_int4{});
            else if(name == "pack_int4")
                lower_int4(ins, op_pack_int4{});
            else if(name == "reshape")
                lower_reshape(ins);
            else if(lower_elementwise_op(ins))
                continue;
            else if(lower_row_op(ins))
                continue;
            else if(lower_mover(ins))
                continue;
            else if(lower_decoder_op(ins))
                continue;
            else
                unsupported(ins, "no kernel");
        }
        // the folded chains are dead: remove them, so that no stale reader sees the column slices
        // the horizontal fusion turns some results into
        dead_code_elimination{}.apply(m);
        fuse_horizontal_qgemms();
        fuse_horizontal_w4a16();
    }

    // packed row-major copy of a host argument with arbitrary strides
    static argument make_standard(const argument& v)
    {
        argument out{v.get_shape().as_standard()};
        const auto& s      = v.get_shape();
        const std::size_t es = s.type_size();
        for(std::size_t i = 0; i < s.elements(); ++i)
            std::memcpy(out.data() + i * es, v.data() + s.index(i) * es, es);
        return out;
    }
};

} // namespace

void lowering::apply(module_pass_manager& mpm) const
{
    module& m = mpm.get_module();
    lowerer l{m, {}};
    l.run();
    // every arena offset a multiple of 32 bytes (see op_align_anchor)
    {
        auto ret = std::prev(m.end());
        bool any = false;
        for(auto ins : iterator_for(m))
            any = any or ins->name() == "allocate";
        if(any and ret->name() == "@return" and not ret->inputs().empty())
        {
            auto x      = ret->inputs().front();
            auto anchor = insert_allocation(m, ret, shape{shape::double_type, {8}});
            auto a      = m.insert_instruction(ret, op_align_anchor{}, x, anchor);
            instruction::replace_argument(ret, x, a);
        }
        else if(any and not is_builtin(ret->name()))
        {
            // no @return: the last instruction is the program's result
            auto anchor = insert_allocation(m, m.end(), shape{shape::double_type, {8}});
            m.add_instruction(op_align_anchor{}, ret, anchor);
        }
    }
    if(not offload_copy)
        return;
    // offload_copy: parameters arrive as host buffers and results are returned on the host
    // (compile_options.hpp:33-45; the HIP target does this in src/targets/gpu/lowering.cpp:122-161)
    std::vector<instruction_ref> params;
    for(auto ins : iterator_for(m))
        if(ins->name() == "@param" and not ins->outputs().empty())
            params.push_back(ins);
    for(auto p : params)
    {
        auto pos   = std::next(p);
        auto alloc = insert_allocation(m, pos, p->get_shape());
        auto c     = m.insert_instruction(pos, op_copy_to{}, p, alloc);
        m.replace_instruction(p, c);
    }
    auto ret = std::prev(m.end());
    if(ret->name() == "@return")
    {
        for(const auto& in : std::vector<instruction_ref>(ret->inputs()))
        {
            auto h = m.insert_instruction(ret, op_copy_from{}, in);
            instruction::replace_argument(ret, in, h);
        }
    }
    else
        m.add_instruction(op_copy_from{}, ret);
}

// ------------------------------------------------------------------ inline_pointwise
void inline_pointwise::apply(module& m) const
{
    std::vector<instruction_ref> pws;
    for(auto ins : iterator_for(m))
        if(ins->name() == "pointwise")
            pws.push_back(ins);
    for(auto ins : pws)
    {
        auto* pm    = ins->module_inputs().front();
        auto pnames = pm->get_parameter_names();
        std::sort(pnames.begin(), pnames.end());
        std::unordered_map<instruction_ref, instruction_ref> map;
        const auto& inputs = ins->inputs();
        const auto lens    = ins->get_shape().lens();
        instruction_ref result = m.end();
        for(auto sub : iterator_for(*pm))
        {
            if(sub->name() == "@param")
            {
                const auto pname = any_cast<builtin::param>(sub->get_operator()).parameter;
                const auto pos   = std::find(pnames.begin(), pnames.end(), pname) - pnames.begin();
                map[sub]         = inputs.at(pos);
            }
            else if(sub->name() == "@literal")
            {
                auto l   = m.add_literal(sub->get_literal());
                map[sub] = m.insert_instruction(
                    ins, make_op("multibroadcast", {{"out_lens", lens}}), l);
            }
            else if(sub->name() == "@return")
            {
                result = map.at(sub->inputs().front());
            }
            else
            {
                std::vector<instruction_ref> args;
                for(auto i : sub->inputs())
                    args.push_back(map.at(i));
                map[sub] = m.insert_instruction(ins, sub->get_operator(), args);
                result   = map[sub];
            }
        }
        if(result == m.end())
            MIGRAPHX_THROW("cuda::inline_pointwise: empty pointwise module");
        m.replace_instruction(ins, result);
    }
}

// ------------------------------------------------------------------ write_literals
void write_literals::apply(module& m) const
{
    std::size_t n = 0;
    for(auto ins : iterator_for(m))
    {
        if(ins->name() != "@literal")
            continue;
        if(ins->outputs().empty())
            continue;
        op_literal op;
        op.l  = ins->get_literal();
        op.id = m.name() + ":@literal:" + std::to_string(n++);
        m.replace_instruction(ins, op);
    }
}

// ------------------------------------------------------------------ sync_device
// ------------------------------------------------------------------ fuse_cuda_pointwise
void fuse_cuda_pointwise::apply(module& m) const
{
    bool changed = true;
    while(changed)
    {
        changed = false;
        for(auto user : iterator_for(m))
        {
            if(user->name() != "cuda::pointwise")
                continue;
            auto uop = any_cast<op_pointwise>(user->get_operator());
            auto uin = user->inputs(); // operands..., output buffer
            // an operand produced by another cuda::pointwise that nothing else reads
            std::size_t which = uin.size();
            for(std::size_t i = 0; i + 1 < uin.size(); ++i)
                if(uin[i]->name() == "cuda::pointwise" and
                   std::all_of(uin[i]->outputs().begin(), uin[i]->outputs().end(),
                               [&](auto o) { return o == user; }) and
                   std::count(uin.begin(), uin.end(), uin[i]) == 1)
                {
                    which = i;
                    break;
                }
            if(which == uin.size())
                continue;
            auto prod = uin[which];
            auto pop  = any_cast<op_pointwise>(prod->get_operator());
            auto pin  = prod->inputs();
            // merged operand list: the producer's operands, then the user's other operands
            std::vector<instruction_ref> operands(pin.begin(), pin.end() - 1);
            std::vector<int> umap(uin.size() - 1, -1); // user's operand index -> merged value index
            for(std::size_t i = 0; i + 1 < uin.size(); ++i)
            {
                if(i == which)
                    continue;
                auto it = std::find(operands.begin(), operands.end(), uin[i]);
                if(it == operands.end())
                {
                    operands.push_back(uin[i]);
                    it = std::prev(operands.end());
                }
                umap[i] = static_cast<int>(it - operands.begin());
            }
            const std::size_t nin = operands.size();
            const std::size_t np  = pop.ops.size();
            if(nin > MGX_PW_MAXIN or np + uop.ops.size() > MGX_PW_MAXINSN)
                continue;
            op_pointwise f;
            const int pin_n = static_cast<int>(pin.size() - 1);
            auto pmap = [&](int v) { return v < pin_n ? v : static_cast<int>(nin) + (v - pin_n); };
            for(std::size_t n = 0; n < np; ++n)
            {
                f.ops.push_back(pop.ops[n]);
                f.types.push_back(pop.types[n]);
                f.imms.push_back(pop.imms[n]);
                for(int j = 0; j < 3; ++j)
                    f.srcs.push_back(pmap(pop.srcs[3 * n + j]));
            }
            const int uin_n   = static_cast<int>(uin.size() - 1);
            const int presult = static_cast<int>(nin + np - 1);
            auto umapv        = [&](int v) {
                if(v >= uin_n)
                    return static_cast<int>(nin + np) + (v - uin_n);
                return v == static_cast<int>(which) ? presult : umap[static_cast<std::size_t>(v)];
            };
            for(std::size_t n = 0; n < uop.ops.size(); ++n)
            {
                f.ops.push_back(uop.ops[n]);
                f.types.push_back(uop.types[n]);
                f.imms.push_back(uop.imms[n]);
                for(int j = 0; j < 3; ++j)
                    f.srcs.push_back(umapv(uop.srcs[3 * n + j]));
            }
            operands.push_back(uin.back());
            m.replace_instruction(user, f, operands);
            // the producer is dead now; while it exists it still counts as a user of its operands
            if(prod->outputs().empty())
                m.remove_instruction(prod);
            changed = true;
            break; // the instruction list changed under the iterator
        }
    }
}

// ------------------------------------------------------------------ insert_graph_ops
void insert_graph_ops::apply(module_pass_manager& mpm) const
{
    module& m       = mpm.get_module();
    const char* env = std::getenv("MIGRAPHX_CUDA_GRAPH");
    if(ctx == nullptr or &m != mpm.get_root_module() or ctx->nstreams() > 1 or
       (env != nullptr and env[0] == '0'))
        return;
    auto launches = [](const std::string& n) {
        return n == "cuda::quantizelinear" or n == "cuda::dequantizelinear" or n == "cuda::qgemm" or
               n == "cuda::w4a16" or n == "cuda::unpack_int4" or n == "cuda::pack_int4" or
               n == "cuda::copy" or n == "cuda::pointwise" or n == "cuda::reduce" or n == "cuda::softmax" or
               n == "cuda::gather" or n == "cuda::concat" or n == "cuda::pad_rows" or
               n == "cuda::layernorm" or n == "cuda::attention" or n == "cuda::concat_past_present" or
               n == "cuda::gqa_rotary_embedding";
    };
    auto last = std::prev(m.end());
    if(last->name() != "@return" or last->inputs().empty())
        return;
    // What stays in the main module: parameters, the return, host copies and the final
    // synchronisation (none of them may run inside a stream capture), and whatever the
    // host-to-device copies need (their arena buffers).  Everything else moves.
    std::unordered_set<instruction*> stays;
    bool seen_launch = false, seen_copy_from = false;
    std::size_t nlaunch = 0;
    for(auto ins : iterator_for(m))
    {
        const auto n = ins->name();
        // explicit stream scheduling and collectives are not captured
        if(n == "cuda::all_reduce" or n == "cuda::set_stream" or n == "cuda::record_event" or
           n == "cuda::wait_event" or not ins->module_inputs().empty())
            return;
        if(n == "cuda::copy_to" and seen_launch)
            return; // a host-to-device copy after the first launch: the launches are not one contiguous run
        if(n == "cuda::copy_from" or n == "cuda::sync_stream")
            seen_copy_from = true;
        if(launches(n))
        {
            if(seen_copy_from)
                return; // a launch after the first device-to-host copy
            seen_launch = true;
            ++nlaunch;
        }
        if(n == "@param" or n == "@return" or n == "cuda::copy_to" or n == "cuda::copy_from" or
           n == "cuda::sync_stream")
            stays.insert(&*ins);
    }
    if(nlaunch == 0)
        return;
    std::function<void(instruction_ref)> keep_inputs = [&](instruction_ref ins) {
        for(auto i : ins->inputs())
            if(stays.insert(&*i).second)
                keep_inputs(i);
    };
    for(auto ins : iterator_for(m))
        if(ins->name() == "cuda::copy_to")
            keep_inputs(ins);

    // the submodule: the moved instructions in their order; values they read from instructions
    // that stay become its parameters, values the staying instructions read from it its results
    module* sub = mpm.create_module(m.name() + ":graph");
    std::unordered_map<instruction*, instruction_ref> inside; // moved instruction -> its clone
    std::unordered_map<instruction*, instruction_ref> as_param;
    std::vector<instruction_ref> ext_inputs;
    std::vector<std::string> ext_names;
    std::vector<instruction_ref> moved;
    for(auto ins : iterator_for(m))
    {
        if(stays.count(&*ins) > 0)
            continue;
        std::vector<instruction_ref> args;
        for(auto i : ins->inputs())
        {
            if(stays.count(&*i) == 0)
            {
                args.push_back(inside.at(&*i));
                continue;
            }
            auto it = as_param.find(&*i);
            if(it == as_param.end())
            {
                const std::string name = i->name() == "@param"
                                             ? any_cast<builtin::param>(i->get_operator()).parameter
                                             : "#in" + std::to_string(ext_inputs.size());
                it = as_param.emplace(&*i, sub->add_parameter(name, i->get_shape())).first;
                ext_inputs.push_back(i);
                ext_names.push_back(name);
            }
            args.push_back(it->second);
        }
        inside[&*ins] = sub->add_instruction(ins->get_operator(), args);
        moved.push_back(ins);
    }
    // results: moved instructions some staying instruction reads, in program order
    std::vector<instruction_ref> results;
    for(auto ins : moved)
        if(std::any_of(ins->outputs().begin(), ins->outputs().end(),
                       [&](auto o) { return stays.count(&*o) > 0; }))
            results.push_back(ins);
    if(results.empty())
        return;
    std::vector<instruction_ref> sub_results;
    for(auto r : results)
        sub_results.push_back(inside.at(&*r));
    sub->add_return(sub_results);
    // the call, in front of the first staying reader of a result
    instruction_ref pos = m.end();
    for(auto ins : iterator_for(m))
        if(stays.count(&*ins) > 0 and std::any_of(ins->inputs().begin(), ins->inputs().end(), [&](auto i) {
               return std::find(results.begin(), results.end(), i) != results.end();
           }))
        {
            pos = ins;
            break;
        }
    op_graph_run call;
    call.params = ext_names;
    auto gr     = m.insert_instruction(pos, call, ext_inputs, {sub});
    for(std::size_t k = 0; k < results.size(); ++k)
    {
        auto elem = m.insert_instruction(pos, make_op("get_tuple_elem", {{"index", k}}), gr);
        for(auto user : std::vector<instruction_ref>(results[k]->outputs()))
            if(stays.count(&*user) > 0)
                instruction::replace_argument(user, results[k], elem);
    }
    for(auto it = moved.rbegin(); it != moved.rend(); ++it)
        m.remove_instruction(*it);
    ctx->enable_graph();
}

void sync_device::apply(module& m) const
{
    auto last = std::prev(m.end());
    if(last->name() != "@return")
        return;
    // results that stay on the device: make sure the work that produces them has been
    // submitted and finished before eval() hands the buffers back
    auto inputs = last->inputs();
    if(inputs.empty())
        return;
    const bool all_host = std::all_of(inputs.begin(), inputs.end(), [](auto i) {
        return i->name() == "cuda::copy_from";
    });
    if(all_host)
        return; // copy_from already synchronises
    auto sync = m.insert_instruction(last, op_sync_stream{}, inputs.front());
    instruction::replace_argument(last, inputs.front(), sync);
}

} // namespace cuda
} // namespace MIGRAPHX_INLINE_NS
} // namespace migraphx
