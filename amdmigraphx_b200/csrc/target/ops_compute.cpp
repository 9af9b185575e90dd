// The compute operators of the `cuda` target: thin host wrappers that turn MIGraphX
// arguments (shapes with strides, broadcast views) into calls of the C ABI in
// include/mgx_cuda.h on the context's stream.
#include "cuda_ops.hpp"
#include <migraphx/check_shapes.hpp>
#include <migraphx/errors.hpp>
#include <migraphx/register_op.hpp>
#include "../../../include/mgx_cuda.h"

namespace migraphx {
inline namespace MIGRAPHX_INLINE_NS {
namespace cuda {

namespace {

int mgx_type(shape::type_t t)
{
    switch(t)
    {
    case shape::float_type: return MGX_F32;
    case shape::half_type: return MGX_F16;
    case shape::int8_type: return MGX_I8;
    case shape::uint8_type: return MGX_U8;
    case shape::int32_type: return MGX_I32;
    case shape::fp8e4m3fn_type: return MGX_FP8_E4M3FN;
    default: MIGRAPHX_THROW("cuda target: element type not supported by the kernels");
    }
}

struct rows_cols
{
    int64_t rows = 0, cols = 0, ld = 0;
};

// A data tensor seen as [rows, cols] with a row stride: the last axis is the column axis.
rows_cols as_matrix(const shape& s, const char* what)
{
    rows_cols r;
    if(s.ndim() == 0 or s.elements() == 0)
        return r;
    r.cols = static_cast<int64_t>(s.lens().back());
    r.rows = static_cast<int64_t>(s.elements()) / r.cols;
    if(s.standard())
    {
        r.ld = r.cols;
        return r;
    }
    if(s.ndim() == 2 and (s.strides()[1] == 1 or r.cols == 1) and
       static_cast<int64_t>(s.strides()[0]) >= r.cols)
    {
        r.ld = static_cast<int64_t>(s.strides()[0]);
        return r;
    }
    MIGRAPHX_THROW(std::string("cuda target: ") + what + " needs a standard or row-strided tensor");
}

// Strides (elements) with which a scale / zero-point view of the data tensor's dims is
// indexed as [rows, cols]: MIGraphX hands these operands over as broadcast views
// (stride 0 along broadcast axes; src/simplify_qdq.cpp:106-117).
void bcast_strides(const shape& s, const rows_cols& m, int64_t out[2], const char* what)
{
    const auto& st = s.strides();
    const auto& ln = s.lens();
    const auto n   = s.ndim();
    out[1]         = (n == 0 or ln.back() == 1) ? 0 : static_cast<int64_t>(st.back());
    bool lead_zero = true;
    for(std::size_t i = 0; i + 1 < n; ++i)
        if(ln[i] != 1 and st[i] != 0)
            lead_zero = false;
    if(lead_zero)
    {
        out[0] = 0;
        return;
    }
    if(s.standard())
    {
        out[0] = m.cols;
        out[1] = 1;
        return;
    }
    if(n == 2)
    {
        out[0] = static_cast<int64_t>(st[0]);
        return;
    }
    MIGRAPHX_THROW(std::string("cuda target: ") + what + " view cannot be indexed as [rows, cols]");
}

} // namespace

// ------------------------------------------------------------------ quantizelinear
shape op_quantizelinear::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(has_zp ? 4 : 3);
    return inputs.back();
}

argument op_quantizelinear::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& xs  = args[0].get_shape();
    const auto& out = args.back();
    const auto m    = as_matrix(xs, "quantizelinear input");
    const auto mo   = as_matrix(out.get_shape(), "quantizelinear output");
    int64_t ss[2] = {0, 0}, zs[2] = {0, 0};
    bcast_strides(args[1].get_shape(), m, ss, "quantizelinear scale");
    if(has_zp)
        bcast_strides(args[2].get_shape(), m, zs, "quantizelinear zero point");
    check_mgx(mgx_cuda_quantizelinear(args[0].data(), mgx_type(xs.type()), m.ld, args[1].data(), ss,
                                      has_zp ? args[2].data() : nullptr, zs, out.data(),
                                      mgx_type(out.get_shape().type()), mo.ld, m.rows, m.cols,
                                      ctx.stream()),
              "mgx_cuda_quantizelinear");
    return out;
}

// ------------------------------------------------------------------ dequantizelinear
shape op_dequantizelinear::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(has_zp ? 4 : 3);
    return inputs.back();
}

argument op_dequantizelinear::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& xs  = args[0].get_shape();
    const auto& out = args.back();
    const auto m    = as_matrix(xs, "dequantizelinear input");
    const auto mo   = as_matrix(out.get_shape(), "dequantizelinear output");
    int64_t ss[2] = {0, 0}, zs[2] = {0, 0};
    bcast_strides(args[1].get_shape(), m, ss, "dequantizelinear scale");
    if(has_zp)
        bcast_strides(args[2].get_shape(), m, zs, "dequantizelinear zero point");
    check_mgx(mgx_cuda_dequantizelinear(args[0].data(), mgx_type(xs.type()), m.ld, args[1].data(),
                                        mgx_type(args[1].get_shape().type()), ss,
                                        has_zp ? args[2].data() : nullptr, zs, out.data(), mo.ld,
                                        m.rows, m.cols, ctx.stream()),
              "mgx_cuda_dequantizelinear");
    return out;
}

// ------------------------------------------------------------------ int4 pack / unpack
shape op_unpack_int4::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(2).standard();
    return inputs.back();
}
argument op_unpack_int4::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto m = as_matrix(args[0].get_shape(), "unpack_int4 input");
    check_mgx(mgx_cuda_unpack_int4(args[0].data(), args[1].data(),
                                   mgx_type(args[0].get_shape().type()), m.rows, m.cols, ctx.stream()),
              "mgx_cuda_unpack_int4");
    return args[1];
}

shape op_pack_int4::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(2).standard();
    return inputs.back();
}
argument op_pack_int4::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto m = as_matrix(args[1].get_shape(), "pack_int4 output");
    check_mgx(mgx_cuda_pack_int4(args[0].data(), args[1].data(), mgx_type(args[0].get_shape().type()),
                                 m.rows, m.cols, ctx.stream()),
              "mgx_cuda_pack_int4");
    return args[1];
}

// ------------------------------------------------------------------ quant_dot (+ epilogue)
shape op_qgemm::compute_shape(const std::vector<shape>& inputs) const
{
    const bool dual          = q_type != 0 and write_d;
    const std::size_t expect = 3 + (scale_mode != MGX_SCALE_NONE) + has_bias + has_residual + has_lut + has_workspace + dual;
    check_shapes{inputs, *this}.has(expect);
    const auto& a = inputs[0];
    const auto& b = inputs[1];
    if(a.ndim() < 2 or b.ndim() != a.ndim())
        MIGRAPHX_THROW("cuda::qgemm: operands must have the same rank >= 2");
    if(a.type() != b.type())
        MIGRAPHX_THROW("cuda::qgemm: operand types differ");
    if(a.type() == shape::half_type and (scale_mode != MGX_SCALE_NONE or q_type != 0))
        MIGRAPHX_THROW("cuda::qgemm: an fp16 dot takes no scale and no fused quantizelinear");
    const auto k  = a.lens().back();
    const auto kb = b_nk ? b.lens().back() : b.lens()[b.ndim() - 2];
    if(k != kb)
        MIGRAPHX_THROW("cuda::qgemm: inner dimensions differ");
    auto lens   = a.lens();
    lens.back() = b_nk ? b.lens()[b.ndim() - 2] : b.lens().back();
    const bool only_q = q_type != 0 and not write_d;
    const shape expected{static_cast<shape::type_t>(only_q ? q_type : out_type), lens};
    if(inputs.back().lens() != expected.lens() or inputs.back().type() != expected.type())
        MIGRAPHX_THROW("cuda::qgemm: output buffer does not match the result shape");
    if(dual)
    {
        const auto& qb = inputs[inputs.size() - 2];
        if(qb.lens() != lens or qb.type() != static_cast<shape::type_t>(q_type) or not qb.standard())
            MIGRAPHX_THROW("cuda::qgemm: quantised output buffer does not match");
    }
    return inputs.back();
}

argument op_qgemm::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    std::size_t i          = 2;
    const argument* scale  = scale_mode != MGX_SCALE_NONE ? &args[i++] : nullptr;
    const argument* bias   = has_bias ? &args[i++] : nullptr;
    const argument* resid  = has_residual ? &args[i++] : nullptr;
    const argument* lut    = has_lut ? &args[i++] : nullptr;
    const argument* wspace = has_workspace ? &args[i++] : nullptr;
    const bool dual        = q_type != 0 and write_d;
    const bool only_q      = q_type != 0 and not write_d;
    const argument* qbuf   = dual ? &args[i++] : (only_q ? &args.back() : nullptr);
    const argument& out    = args.back();
    const auto& as         = args[0].get_shape();
    const auto& bs         = args[1].get_shape();
    const auto& ds         = out.get_shape();
    const auto nd          = as.ndim();
    if(not ds.standard())
        MIGRAPHX_THROW("cuda::qgemm: output must be a standard tensor");
    if(resid != nullptr and resid->get_shape().lens() != ds.lens())
        MIGRAPHX_THROW("cuda::qgemm: residual must have the output's shape");

    mgx_qgemm_desc d{};
    d.M = static_cast<int64_t>(as.lens()[nd - 2]);
    d.K = static_cast<int64_t>(as.lens()[nd - 1]);
    d.N = static_cast<int64_t>(ds.lens()[nd - 1]);
    int64_t batch = 1;
    for(std::size_t j = 0; j + 2 < nd; ++j)
        batch *= static_cast<int64_t>(as.lens()[j]);
    if(as.strides()[nd - 1] != 1 and d.K != 1)
        MIGRAPHX_THROW("cuda::qgemm: A must be K-contiguous");
    d.lda = static_cast<int64_t>(as.strides()[nd - 2]);
    d.ldb = static_cast<int64_t>(bs.strides()[nd - 2]);
    d.ldd = d.N;
    // a [K,N] operand that is the transpose view of a K-contiguous [N,K] tensor (Q . K^T of
    // attention) is already in the layout the kernel reads
    bool view_nk = false;
    if(not b_nk and bs.strides()[nd - 1] != 1 and bs.strides()[nd - 2] == 1)
    {
        view_nk = true;
        d.ldb   = static_cast<int64_t>(bs.strides()[nd - 1]);
    }
    else if(bs.strides()[nd - 1] != 1)
        MIGRAPHX_THROW("cuda::qgemm: B must be contiguous along its last axis");
    bool b_shared = true; // B is the same matrix for every batch entry (broadcast view)
    for(std::size_t j = 0; j + 2 < nd; ++j)
        if(bs.lens()[j] != 1 and bs.strides()[j] != 0)
            b_shared = false;
    if(batch > 1)
    {
        // batch entries must be evenly spaced: the leading dimensions step like a standard
        // tensor's (one stride serves every entry)
        for(std::size_t j = 0; j + 3 < nd; ++j)
        {
            if(as.lens()[j] != 1 and as.strides()[j] != as.strides()[j + 1] * as.lens()[j + 1])
                MIGRAPHX_THROW("cuda::qgemm: the batch entries of A are not evenly spaced");
            if(not b_shared and bs.lens()[j] != 1 and
               bs.strides()[j] != bs.strides()[j + 1] * bs.lens()[j + 1])
                MIGRAPHX_THROW("cuda::qgemm: the batch entries of B are not evenly spaced");
        }
        const auto rows_a = static_cast<int64_t>(as.strides()[nd - 3]);
        d.stride_a        = rows_a;
        d.stride_d        = d.M * d.N;
        if(b_shared and rows_a == d.M * d.lda)
        {
            // one weight matrix for all entries: fold the batch into the rows
            d.M *= batch;
            batch = 1;
        }
        else
            d.stride_b = static_cast<int64_t>(bs.strides()[nd - 3]);
    }
    d.batch      = batch;
    d.ab_type    = mgx_type(as.type());
    d.out_type   = mgx_type(static_cast<shape::type_t>(out_type));
    d.b_layout   = (b_nk or view_nk) ? MGX_B_NK : MGX_B_KN;
    d.scale_mode = scale_mode;
    d.act        = act;
    d.flags      = half_math ? MGX_QGEMM_HALF_MATH : 0;
    mgx_qgemm_qout qo{};
    if(qbuf != nullptr)
    {
        qo.q          = qbuf->data();
        qo.ldq        = d.N;
        qo.stride_q   = d.M * d.N;
        qo.q_type     = mgx_type(static_cast<shape::type_t>(q_type));
        qo.scale      = q_scale;
        qo.zero_point = q_zp;
        if(lut != nullptr)
        {
            if(lut->get_shape().bytes() != 65536)
                MIGRAPHX_THROW("cuda::qgemm: the activation / quantizelinear table must hold 65536 bytes");
            qo.flags = MGX_QOUT_LUT;
            qo.lut   = lut->data();
        }
    }
    check_mgx(mgx_cuda_qgemm_ex(&d, args[0].data(), args[1].data(), only_q ? nullptr : out.data(),
                                scale != nullptr ? reinterpret_cast<const float*>(scale->data()) : nullptr,
                                bias != nullptr ? reinterpret_cast<const float*>(bias->data()) : nullptr,
                                resid != nullptr ? resid->data() : nullptr,
                                qbuf != nullptr ? &qo : nullptr,
                                wspace != nullptr ? wspace->data() : nullptr,
                                wspace != nullptr ? wspace->get_shape().bytes() : 0, ctx.stream()),
              "mgx_cuda_qgemm");
    return out;
}

// ------------------------------------------------------------------ weight-only int4 linear
shape op_w4a16::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(4 + has_zp + has_workspace);
    const auto& a  = inputs[0];
    const auto& bp = inputs[1];
    if(a.type() != shape::half_type or bp.type() != shape::uint8_type or bp.ndim() != 2)
        MIGRAPHX_THROW("cuda::w4a16: expects fp16 activations and 2-D uint8 packed weights");
    if(a.lens().back() != 2 * bp.lens()[1])
        MIGRAPHX_THROW("cuda::w4a16: K of the activations and of the packed weights differ");
    return inputs.back();
}

argument op_w4a16::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    std::size_t i          = 3;
    const argument* zp     = has_zp ? &args[i++] : nullptr;
    const argument* wspace = has_workspace ? &args[i++] : nullptr;
    const argument& out    = args.back();
    const auto m           = as_matrix(args[0].get_shape(), "w4a16 activations");
    mgx_w4_desc d{};
    d.M        = m.rows;
    d.K        = m.cols;
    d.N        = static_cast<int64_t>(args[1].get_shape().lens()[0]);
    d.lda      = m.ld;
    d.ldd      = d.N;
    d.group    = group;
    d.zp_const = zp_const;
    d.act      = MGX_ACT_NONE;
    check_mgx(mgx_cuda_w4a16(&d, args[0].data(), args[1].data(), args[2].data(),
                             zp != nullptr ? zp->data() : nullptr, out.data(),
                             wspace != nullptr ? wspace->data() : nullptr,
                             wspace != nullptr ? wspace->get_shape().bytes() : 0, ctx.stream()),
              "mgx_cuda_w4a16");
    return out;
}

// ------------------------------------------------------------------ all_reduce
shape op_all_reduce::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(1).standard();
    return inputs.front();
}

argument op_all_reduce::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& s = args[0].get_shape();
    check_mgx(mgx_cuda_all_reduce(args[0].data(), s.elements(), mgx_type(s.type()), nullptr, ctx.stream()),
              "mgx_cuda_all_reduce");
    return args[0];
}

shape op_second_output::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(2);
    return inputs.at(1);
}
argument op_second_output::compute(context&, const shape&, const std::vector<argument>& args) const
{
    return args.at(1);
}

// ------------------------------------------------------------------ element-wise
static int pw_type(shape::type_t t, bool byte_copy = false)
{
    // a bool is a byte holding 0 or 1; a pure copy moves 8-bit elements of any type as bytes
    if(byte_copy and shape{t}.type_size() == 1)
        return MGX_U8;
    return t == shape::bool_type ? MGX_I8 : mgx_type(t);
}

shape op_pointwise::compute_shape(const std::vector<shape>& inputs) const
{
    if(inputs.empty() or ops.empty() or types.size() != ops.size() or srcs.size() != 3 * ops.size() or
       imms.size() != ops.size())
        MIGRAPHX_THROW("cuda::pointwise: malformed instruction list");
    if(inputs.size() - 1 > MGX_PW_MAXIN or ops.size() > MGX_PW_MAXINSN)
        MIGRAPHX_THROW("cuda::pointwise: too many inputs or instructions");
    const auto& out = inputs.back();
    for(std::size_t i = 0; i + 1 < inputs.size(); ++i)
        if(inputs[i].lens() != out.lens())
            MIGRAPHX_THROW("cuda::pointwise: every operand must have the output's dimensions");
    if(not out.standard())
        MIGRAPHX_THROW("cuda::pointwise: output must be a standard tensor");
    return out;
}

argument op_pointwise::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& out = args.back();
    const auto& os = out.get_shape();
    mgx_pw_desc d{};
    // more dimensions than the kernel indexes: fold the leading ones when every operand is packed
    std::vector<std::size_t> lens = os.lens();
    bool flat = lens.size() > MGX_PW_MAXDIMS;
    if(flat)
    {
        for(std::size_t i = 0; i + 1 < args.size(); ++i)
            if(not args[i].get_shape().standard())
                MIGRAPHX_THROW("cuda::pointwise: more than 5 dimensions need packed operands");
        lens = {os.elements()};
    }
    d.ndim    = static_cast<int32_t>(lens.size());
    d.ninputs = static_cast<int32_t>(args.size() - 1);
    d.ninsns  = static_cast<int32_t>(ops.size());
    for(std::size_t k = 0; k < lens.size(); ++k)
        d.lens[k] = static_cast<int64_t>(lens[k]);
    // a packed copy of a strided view (one identity instruction, same type in and out)
    const bool byte_copy = ops.size() == 1 and ops[0] == MGX_PW_IDENTITY and args.size() == 2 and
                           args[0].get_shape().type() == os.type();
    const void* ptrs[MGX_PW_MAXIN] = {};
    for(std::size_t i = 0; i + 1 < args.size(); ++i)
    {
        const auto& s = args[i].get_shape();
        d.in_type[i]  = pw_type(s.type(), byte_copy);
        ptrs[i]       = args[i].data();
        if(flat)
            d.in_strides[i][0] = 1;
        else
            for(std::size_t k = 0; k < lens.size(); ++k)
                d.in_strides[i][k] = static_cast<int64_t>(s.strides()[k]);
    }
    for(std::size_t n = 0; n < ops.size(); ++n)
    {
        d.insn[n].op   = ops[n];
        d.insn[n].type = pw_type(static_cast<shape::type_t>(types[n]), byte_copy);
        d.insn[n].imm  = imms[n];
        for(int j = 0; j < 3; ++j)
            d.insn[n].src[j] = srcs[3 * n + j];
    }
    check_mgx(mgx_cuda_pointwise(&d, ptrs, out.data(), ctx.stream()), "mgx_cuda_pointwise");
    return out;
}

// ------------------------------------------------------------------ reductions, softmax
static void check_rows(const std::string& name, const shape& x)
{
    if(not x.standard() or x.ndim() == 0)
        MIGRAPHX_THROW(name + ": input must be a standard tensor");
    if(x.type() != shape::float_type and x.type() != shape::half_type)
        MIGRAPHX_THROW(name + ": float and half only");
}

shape op_reduce::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(2);
    check_rows(name(), inputs[0]);
    // the output is the packed input with its trailing dimensions (at least the last) set to 1
    const auto& xl = inputs[0].lens();
    const auto& ol = inputs[1].lens();
    bool ok        = ol.size() == xl.size() and ol.back() == 1 and inputs[1].type() == inputs[0].type() and
              inputs[1].standard();
    bool tail = true; // still inside the reduced trailing dimensions
    for(std::size_t i = xl.size(); ok and i-- > 0;)
    {
        if(tail and ol[i] == 1)
            continue;
        tail = false;
        ok   = ol[i] == xl[i];
    }
    if(not ok)
        MIGRAPHX_THROW("cuda::reduce: output must be the packed input with trailing dimensions of 1");
    return inputs[1];
}

argument op_reduce::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& out = args.back();
    const auto& xs     = args[0].get_shape();
    const int64_t rows = static_cast<int64_t>(out.get_shape().elements());
    const int64_t cols = static_cast<int64_t>(xs.elements()) / rows;
    check_mgx(mgx_cuda_reduce(args[0].data(), mgx_type(xs.type()), cols, rows, cols, mode, out.data(), ctx.stream()),
              "mgx_cuda_reduce");
    return out;
}

// ------------------------------------------------------------------ layernorm
shape op_layernorm::compute_shape(const std::vector<shape>& inputs) const
{
    const std::size_t n = 1 + has_gamma + has_beta + has_dq + (q_type != 0 ? 1 : 0) + (write_y ? 1 : 0);
    check_shapes{inputs, *this}.has(n);
    const auto& x = inputs[0];
    if(x.type() != shape::float_type and x.type() != shape::half_type)
        MIGRAPHX_THROW("cuda::layernorm: float and half only");
    if(not mgx_cuda_layernorm_supported(mgx_type(x.type()), static_cast<int64_t>(x.lens().back())))
        MIGRAPHX_THROW("cuda::layernorm: row length not supported");
    for(std::size_t i = 1; i < inputs.size(); ++i)
        if(i > static_cast<std::size_t>(has_gamma + has_beta) and inputs[i].lens() != x.lens())
            MIGRAPHX_THROW("cuda::layernorm: buffers must have the input's dimensions");
    return inputs.back();
}

argument op_layernorm::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    std::size_t i         = 1;
    const argument* gamma = has_gamma ? &args[i++] : nullptr;
    const argument* beta  = has_beta ? &args[i++] : nullptr;
    const argument* dqbuf = has_dq ? &args[i++] : nullptr;
    const argument* qbuf  = q_type != 0 ? &args[i++] : nullptr;
    const argument* ybuf  = write_y ? &args[i++] : nullptr;
    const auto m          = as_matrix(args[0].get_shape(), "layernorm input");
    mgx_layernorm_desc d{};
    d.rows = m.rows;
    d.cols = m.cols;
    d.ldx  = m.ld;
    d.ldy  = ybuf != nullptr ? as_matrix(ybuf->get_shape(), "layernorm output").ld : 0;
    d.ldq  = qbuf != nullptr ? as_matrix(qbuf->get_shape(), "layernorm quantised output").ld : 0;
    d.type = mgx_type(args[0].get_shape().type());
    d.eps  = eps;
    d.flags = rms ? MGX_LAYERNORM_RMS : 0;
    if(qbuf != nullptr)
    {
        d.q_type       = mgx_type(static_cast<shape::type_t>(q_type));
        d.q_scale      = q_scale;
        d.q_zero_point = q_zp;
    }
    check_mgx(mgx_cuda_layernorm_ex(&d, args[0].data(), gamma != nullptr ? gamma->data() : nullptr,
                                    beta != nullptr ? beta->data() : nullptr, ybuf != nullptr ? ybuf->data() : nullptr,
                                    qbuf != nullptr ? qbuf->data() : nullptr,
                                    dqbuf != nullptr ? dqbuf->data() : nullptr,
                                    dqbuf != nullptr ? as_matrix(dqbuf->get_shape(), "layernorm dequantised output").ld : 0,
                                    dq_scale, ctx.stream()),
              "mgx_cuda_layernorm");
    return args.back();
}

// ------------------------------------------------------------------ attention
shape op_attention::compute_shape(const std::vector<shape>& inputs) const
{
    const std::size_t n = 3 + (q_type != 0 ? 1 : 0) + (write_o ? 1 : 0);
    check_shapes{inputs, *this}.has(n);
    const std::size_t rows = batch * seq, width = heads * head_dim;
    for(std::size_t i = 0; i < 3; ++i)
    {
        const auto& s = inputs[i];
        if(s.type() != shape::half_type or s.elements() != rows * width or s.lens().back() != width or
           s.strides().back() != 1)
            MIGRAPHX_THROW("cuda::attention: Q, K and V must be fp16 [batch * seq, heads * head_dim] matrices");
    }
    for(std::size_t i = 3; i < inputs.size(); ++i)
        if(inputs[i].elements() != rows * width or not inputs[i].standard())
            MIGRAPHX_THROW("cuda::attention: result buffers must be packed [batch * seq, heads * head_dim]");
    return inputs.back();
}

argument op_attention::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    std::size_t i        = 3;
    const argument* qbuf = q_type != 0 ? &args[i++] : nullptr;
    const argument* obuf = write_o ? &args[i++] : nullptr;
    // row stride of a [.., width] tensor whose leading dimensions step like a packed matrix's rows
    auto row_stride = [&](const shape& s) {
        const auto nd = s.ndim();
        return static_cast<int64_t>(nd >= 2 ? s.strides()[nd - 2] : s.lens().back());
    };
    mgx_attention_desc d{};
    d.batch    = static_cast<int64_t>(batch);
    d.seq      = static_cast<int64_t>(seq);
    d.heads    = static_cast<int64_t>(heads);
    d.head_dim = static_cast<int64_t>(head_dim);
    d.ldq      = row_stride(args[0].get_shape());
    d.ldk      = row_stride(args[1].get_shape());
    d.ldv      = row_stride(args[2].get_shape());
    d.ldo      = static_cast<int64_t>(heads * head_dim);
    d.ldoq     = d.ldo;
    d.scale    = scale;
    d.q_scale  = q_scale;
    d.q_zero_point = q_zp;
    d.flags        = fp32_softmax ? MGX_ATTENTION_FP32_SOFTMAX : 0;
    check_mgx(mgx_cuda_attention(&d, args[0].data(), args[1].data(), args[2].data(),
                                 obuf != nullptr ? obuf->data() : nullptr, qbuf != nullptr ? qbuf->data() : nullptr,
                                 ctx.stream()),
              "mgx_cuda_attention");
    return args.back();
}

// ------------------------------------------------------------------ KV cache, rotary embedding
static int index_type(shape::type_t t)
{
    if(t == shape::int32_type)
        return MGX_I32;
    if(t == shape::int64_type)
        return MGX_I64;
    MIGRAPHX_THROW("cuda target: sequence lengths must be int32 or int64");
}

shape op_concat_past_present::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(3);
    const auto& pr = inputs[0];
    const auto& pa = inputs[2];
    if(pr.ndim() != 4 or pa.ndim() != 4 or pr.type() != pa.type() or not pa.standard() or
       pr.strides().back() != 1 or pr.lens()[0] != pa.lens()[0] or pr.lens()[1] != pa.lens()[1] or
       pr.lens()[3] != pa.lens()[3])
        MIGRAPHX_THROW("cuda::concat_past_present: expects present [B, H, L, D] with contiguous rows and a packed "
                       "cache [B, H, T, D] of the same type");
    return pa;
}

argument op_concat_past_present::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& pr = args[0].get_shape();
    const auto& pa = args[2].get_shape();
    const auto es  = static_cast<int64_t>(pr.type_size());
    const int64_t strides[3] = {static_cast<int64_t>(pr.strides()[0]) * es, static_cast<int64_t>(pr.strides()[1]) * es,
                                static_cast<int64_t>(pr.strides()[2]) * es};
    check_mgx(mgx_cuda_concat_past_present(args[0].data(), strides, static_cast<int64_t>(pr.lens()[0]),
                                           static_cast<int64_t>(pr.lens()[1]), static_cast<int64_t>(pr.lens()[2]),
                                           static_cast<int64_t>(pr.lens()[3]) * es, args[1].data(),
                                           index_type(args[1].get_shape().type()), args[2].data(),
                                           static_cast<int64_t>(pa.lens()[2]), ctx.stream()),
              "mgx_cuda_concat_past_present");
    return args[2];
}

shape op_gqa_rotary_embedding::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(5);
    const auto& x = inputs[0];
    if(x.ndim() != 4 or not x.standard() or x.lens()[1] != num_heads + 2 * kv_num_heads or
       (x.type() != shape::half_type and x.type() != shape::float_type) or inputs[2].type() != x.type() or
       inputs[3].type() != x.type() or inputs[2].ndim() != 2 or not inputs[2].standard() or
       not inputs[3].standard() or inputs[4].lens() != x.lens() or not inputs[4].standard())
        MIGRAPHX_THROW("cuda::gqa_rotary_embedding: expects packed QKV [B, heads + 2 kv_heads, S, D], 2-D caches of "
                       "the same type and a packed output");
    return inputs[4];
}

argument op_gqa_rotary_embedding::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& out = args.back();
    const auto& x = args[0].get_shape();
    const auto& c = args[2].get_shape();
    check_mgx(mgx_cuda_gqa_rotary_embedding(
                  args[0].data(), mgx_type(x.type()), static_cast<int64_t>(x.lens()[0]), static_cast<int64_t>(num_heads),
                  static_cast<int64_t>(kv_num_heads), static_cast<int64_t>(x.lens()[2]), static_cast<int64_t>(x.lens()[3]),
                  args[2].data(), args[3].data(), static_cast<int64_t>(c.lens()[0]), static_cast<int64_t>(c.lens()[1]) * 2,
                  args[1].data(), index_type(args[1].get_shape().type()), interleaved ? 1 : 0, out.data(), ctx.stream()),
              "mgx_cuda_gqa_rotary_embedding");
    return out;
}

shape op_rotary_embedding::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(5);
    const auto& x = inputs[0];
    if(x.ndim() != 4 or x.strides().back() != 1 or x.lens()[3] % 2 != 0 or
       (x.type() != shape::half_type and x.type() != shape::float_type))
        MIGRAPHX_THROW("cuda::rotary_embedding: expects fp16 / fp32 [B, heads, S, D] with contiguous rows");
    if(inputs[1].elements() != x.lens()[0] * x.lens()[2] or not inputs[1].standard() or
       (inputs[1].type() != shape::int32_type and inputs[1].type() != shape::int64_type))
        MIGRAPHX_THROW("cuda::rotary_embedding: expects one int32 / int64 position per (batch entry, row)");
    for(int i : {2, 3})
        if(inputs[i].type() != x.type() or inputs[i].ndim() != 2 or not inputs[i].standard() or
           inputs[i].lens()[1] * 2 != x.lens()[3] or inputs[i].lens() != inputs[2].lens())
            MIGRAPHX_THROW("cuda::rotary_embedding: expects packed [max_pos, D / 2] caches of x's type");
    if(inputs[4].lens() != x.lens() or inputs[4].type() != x.type() or not inputs[4].standard())
        MIGRAPHX_THROW("cuda::rotary_embedding: output must be a packed tensor of x's shape");
    return inputs[4];
}

argument op_rotary_embedding::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& out = args.back();
    const auto& x = args[0].get_shape();
    const int64_t strides[3] = {static_cast<int64_t>(x.strides()[0]), static_cast<int64_t>(x.strides()[1]),
                                static_cast<int64_t>(x.strides()[2])};
    check_mgx(mgx_cuda_rotary_embedding(args[0].data(), mgx_type(x.type()), strides, static_cast<int64_t>(x.lens()[0]),
                                        static_cast<int64_t>(x.lens()[1]), static_cast<int64_t>(x.lens()[2]),
                                        static_cast<int64_t>(x.lens()[3]), args[1].data(),
                                        index_type(args[1].get_shape().type()), args[2].data(), args[3].data(),
                                        static_cast<int64_t>(args[2].get_shape().lens()[0]), out.data(), ctx.stream()),
              "mgx_cuda_rotary_embedding");
    return out;
}

shape op_gqa_decode_attention::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(5);
    const auto& q = inputs[0];
    const auto& k = inputs[1];
    if(q.ndim() != 4 or q.type() != shape::half_type or q.lens()[1] != num_heads or q.lens()[2] != 1 or
       q.strides().back() != 1)
        MIGRAPHX_THROW("cuda::gqa_decode_attention: expects fp16 queries [B, heads, 1, D] with contiguous rows");
    if(k.ndim() != 4 or not k.standard() or k.type() != shape::half_type or k.lens()[0] != q.lens()[0] or
       k.lens()[1] != kv_num_heads or k.lens()[3] != q.lens()[3] or inputs[2] != k)
        MIGRAPHX_THROW("cuda::gqa_decode_attention: expects packed fp16 caches [B, kv_heads, T, D]");
    if(inputs[3].elements() != q.lens()[0] or not inputs[3].standard() or
       (inputs[3].type() != shape::int32_type and inputs[3].type() != shape::int64_type))
        MIGRAPHX_THROW("cuda::gqa_decode_attention: expects one int32 / int64 past length per batch entry");
    if(inputs[4].lens() != q.lens() or not inputs[4].standard() or inputs[4].type() != shape::half_type)
        MIGRAPHX_THROW("cuda::gqa_decode_attention: output must be a packed fp16 tensor of the queries' shape");
    return inputs[4];
}

argument op_gqa_decode_attention::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& out = args.back();
    const auto& q = args[0].get_shape();
    const auto& k = args[1].get_shape();
    mgx_gqa_decode_desc d{};
    d.batch          = static_cast<int64_t>(q.lens()[0]);
    d.heads          = static_cast<int64_t>(num_heads);
    d.kv_heads       = static_cast<int64_t>(kv_num_heads);
    d.head           = static_cast<int64_t>(q.lens()[3]);
    d.cache_seq      = static_cast<int64_t>(k.lens()[2]);
    d.q_batch_stride = static_cast<int64_t>(q.strides()[0]);
    d.q_head_stride  = static_cast<int64_t>(q.strides()[1]);
    d.scale          = scale;
    d.seqlens_type   = index_type(args[3].get_shape().type());
    check_mgx(mgx_cuda_gqa_decode_attention(&d, args[0].data(), args[1].data(), args[2].data(), args[3].data(),
                                            out.data(), ctx.stream()),
              "mgx_cuda_gqa_decode_attention");
    return out;
}

shape op_softmax::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(2);
    check_rows(name(), inputs[0]);
    if(inputs[1].lens() != inputs[0].lens() or inputs[1].type() != inputs[0].type() or not inputs[1].standard())
        MIGRAPHX_THROW("cuda::softmax: output must be a packed tensor of the input's shape");
    return inputs[1];
}

argument op_softmax::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& out = args.back();
    const auto& xs     = args[0].get_shape();
    const int64_t cols = static_cast<int64_t>(xs.lens().back());
    const int64_t rows = static_cast<int64_t>(xs.elements()) / cols;
    check_mgx(mgx_cuda_softmax(args[0].data(), mgx_type(xs.type()), cols, out.data(), cols, rows, cols, ctx.stream()),
              "mgx_cuda_softmax");
    return out;
}

// ------------------------------------------------------------------ gather, concat
shape op_gather::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(3);
    if(not inputs[0].standard() or not inputs[1].standard() or not inputs[2].standard())
        MIGRAPHX_THROW("cuda::gather: operands must be standard tensors");
    if(inputs[1].type() != shape::int32_type and inputs[1].type() != shape::int64_type)
        MIGRAPHX_THROW("cuda::gather: indices must be int32 or int64");
    if(axis < 0 or axis >= static_cast<int64_t>(inputs[0].ndim()) or inputs[2].type() != inputs[0].type())
        MIGRAPHX_THROW("cuda::gather: bad axis or output type");
    return inputs[2];
}

argument op_gather::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& out = args.back();
    const auto& ds = args[0].get_shape();
    int64_t outer = 1, inner = static_cast<int64_t>(ds.type_size());
    for(int64_t i = 0; i < axis; ++i)
        outer *= static_cast<int64_t>(ds.lens()[i]);
    for(std::size_t i = axis + 1; i < ds.ndim(); ++i)
        inner *= static_cast<int64_t>(ds.lens()[i]);
    const auto& is = args[1].get_shape();
    check_mgx(mgx_cuda_gather(args[0].data(), outer, static_cast<int64_t>(ds.lens()[axis]), inner, args[1].data(),
                              is.type() == shape::int32_type ? MGX_I32 : MGX_I64,
                              static_cast<int64_t>(is.elements()), out.data(), ctx.stream()),
              "mgx_cuda_gather");
    return out;
}

shape op_concat::compute_shape(const std::vector<shape>& inputs) const
{
    if(inputs.size() < 2)
        MIGRAPHX_THROW("cuda::concat: needs at least one tensor and the output buffer");
    const auto& out = inputs.back();
    if(axis < 0 or axis >= static_cast<int64_t>(out.ndim()) or not out.standard())
        MIGRAPHX_THROW("cuda::concat: bad axis or output layout");
    std::size_t along = 0;
    for(std::size_t i = 0; i + 1 < inputs.size(); ++i)
    {
        const auto& s = inputs[i];
        if(not s.standard() or s.type() != out.type() or s.ndim() != out.ndim())
            MIGRAPHX_THROW("cuda::concat: inputs must be standard tensors of the output's type and rank");
        for(std::size_t d = 0; d < s.ndim(); ++d)
            if(static_cast<int64_t>(d) != axis and s.lens()[d] != out.lens()[d])
                MIGRAPHX_THROW("cuda::concat: dimensions other than the axis must match");
        along += s.lens()[axis];
    }
    if(along != out.lens()[axis])
        MIGRAPHX_THROW("cuda::concat: the inputs do not fill the output");
    return out;
}

argument op_concat::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& out = args.back();
    const auto& os = out.get_shape();
    int64_t outer = 1, inner = static_cast<int64_t>(os.type_size());
    for(int64_t i = 0; i < axis; ++i)
        outer *= static_cast<int64_t>(os.lens()[i]);
    for(std::size_t i = axis + 1; i < os.ndim(); ++i)
        inner *= static_cast<int64_t>(os.lens()[i]);
    const int64_t dst_pitch = static_cast<int64_t>(os.lens()[axis]) * inner;
    int64_t off             = 0;
    for(std::size_t i = 0; i + 1 < args.size(); ++i)
    {
        const int64_t row_bytes = static_cast<int64_t>(args[i].get_shape().lens()[axis]) * inner;
        check_mgx(mgx_cuda_copy_rows(args[i].data(), row_bytes, out.data() + off, dst_pitch, outer, row_bytes,
                                     ctx.stream()),
                  "mgx_cuda_copy_rows");
        off += row_bytes;
    }
    return out;
}

shape op_pad_rows::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(2);
    const auto& x = inputs[0];
    const auto& o = inputs[1];
    if(not x.standard() or x.ndim() < 1 or o.lens() != x.lens() or o.type() != x.type() or
       o.strides().back() != 1)
        MIGRAPHX_THROW("cuda::pad_rows: expects a standard input and an output of the same dimensions");
    return o;
}

argument op_pad_rows::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& out = args.back();
    const auto& xs      = args[0].get_shape();
    const auto& os      = out.get_shape();
    const int64_t es    = static_cast<int64_t>(xs.type_size());
    const int64_t cols  = static_cast<int64_t>(xs.lens().back());
    const int64_t rows  = static_cast<int64_t>(xs.elements()) / cols;
    const int64_t pitch = xs.ndim() > 1 ? static_cast<int64_t>(os.strides()[xs.ndim() - 2]) : cols;
    check_mgx(mgx_cuda_copy_rows(args[0].data(), cols * es, out.data(), pitch * es, rows, cols * es, ctx.stream()),
              "mgx_cuda_copy_rows");
    return out;
}

MIGRAPHX_REGISTER_OP(op_pad_rows)
MIGRAPHX_REGISTER_OP(op_gather)
MIGRAPHX_REGISTER_OP(op_concat)
MIGRAPHX_REGISTER_OP(op_reduce)
MIGRAPHX_REGISTER_OP(op_softmax)
MIGRAPHX_REGISTER_OP(op_layernorm)
MIGRAPHX_REGISTER_OP(op_attention)
MIGRAPHX_REGISTER_OP(op_concat_past_present)
MIGRAPHX_REGISTER_OP(op_gqa_rotary_embedding)
MIGRAPHX_REGISTER_OP(op_gqa_decode_attention)
MIGRAPHX_REGISTER_OP(op_rotary_embedding)
MIGRAPHX_REGISTER_OP(op_pointwise)
MIGRAPHX_REGISTER_OP(op_second_output)
MIGRAPHX_REGISTER_OP(op_align_anchor)
MIGRAPHX_REGISTER_OP(op_all_reduce)
MIGRAPHX_REGISTER_OP(op_quantizelinear)
MIGRAPHX_REGISTER_OP(op_dequantizelinear)
MIGRAPHX_REGISTER_OP(op_unpack_int4)
MIGRAPHX_REGISTER_OP(op_pack_int4)
MIGRAPHX_REGISTER_OP(op_qgemm)
MIGRAPHX_REGISTER_OP(op_w4a16)

} // namespace cuda
} // namespace MIGRAPHX_INLINE_NS
} // namespace migraphx
