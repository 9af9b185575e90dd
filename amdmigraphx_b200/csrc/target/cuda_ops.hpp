// Operators of the `cuda` target.  Every compute operator follows the convention of
// MIGraphX's device targets (src/targets/gpu/include/migraphx/gpu/gemm.hpp:109-127): the
// output buffer is the LAST input and is what compute() returns (output_alias), so that the
// generic replace_allocate / memory_coloring passes can plan all buffers into one arena.
#ifndef MGX_CUDA_OPS_HPP
#define MGX_CUDA_OPS_HPP

#include "cuda_target.hpp"
#include <migraphx/literal.hpp>
#include <migraphx/reflect.hpp>
#include <migraphx/functional.hpp>

namespace migraphx {
inline namespace MIGRAPHX_INLINE_NS {
namespace cuda {

// ---- memory ---------------------------------------------------------------------------
struct op_allocate
{
    shape s{};
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.s, "shape"));
    }
    std::string name() const { return "cuda::allocate"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
};

// Arena / parameter replacement created by preallocate_param: allocated once at finalize.
struct op_preallocate
{
    shape s{};
    std::string id{};
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.s, "shape"), f(self.id, "id"));
    }
    std::string name() const { return "cuda::preallocate"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    void finalize(context& ctx, const shape&, const std::vector<shape>&) const;
};

// A constant uploaded to the device once, at finalize.
struct op_literal
{
    literal l{};
    std::string id{};
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.l, "literal"), f(self.id, "id"));
    }
    std::string name() const { return "cuda::literal"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    void finalize(context& ctx, const shape&, const std::vector<shape>&) const;
    friend std::ostream& operator<<(std::ostream& os, const op_literal& x)
    {
        os << x.name() << "[id=" << x.id << "]";
        return os;
    }
};

struct op_copy_to // (host, device_out) -> device_out
{
    std::string name() const { return "cuda::copy_to"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>&) const { return {1}; }
};

struct op_copy_from // (device) -> new host buffer; synchronises the stream
{
    std::string name() const { return "cuda::copy_from"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
};

struct op_copy // (device_src, device_out) -> device_out
{
    std::string name() const { return "cuda::copy"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>&) const { return {1}; }
};

struct op_sync_stream
{
    std::string name() const { return "cuda::sync_stream"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& args) const
    {
        if(args.empty())
            return {};
        return {0};
    }
};

// Evaluates its submodule (see insert_graph_ops): instruction by instruction at first, as one
// recorded CUDA graph afterwards.  Inputs: the submodule's parameters in the order of `params`.
// Result: the tuple of the submodule's results.
struct op_graph_run
{
    std::vector<std::string> params;
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.params, "params"));
    }
    std::string name() const { return "cuda::graph_run"; }
    shape compute_shape(const std::vector<shape>& inputs, std::vector<module_ref> mods) const;
    argument compute(context& ctx,
                     const shape& out,
                     const std::vector<argument>& args,
                     const std::vector<module_ref>& mods,
                     const std::function<std::vector<argument>(
                         module_ref&, const std::unordered_map<std::string, argument>&)>& run) const;
};

// ---- stream scheduling (inserted by the generic schedule pass through schedule_model) ----
struct op_set_stream
{
    std::size_t stream = 0;
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.stream, "stream"));
    }
    std::string name() const { return "cuda::set_stream"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    void finalize(context& ctx, const shape&, const std::vector<shape>&) const;
};

struct op_record_event
{
    std::size_t event = 0;
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.event, "event"));
    }
    std::string name() const { return "cuda::record_event"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    void finalize(context& ctx, const shape&, const std::vector<shape>&) const;
};

struct op_wait_event
{
    std::size_t event = 0;
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.event, "event"));
    }
    std::string name() const { return "cuda::wait_event"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
};

// ---- quantized path ---------------------------------------------------------------------
// quantizelinear: inputs (x, scale view, [zero-point view], out).  Replaces
// op::quantizelinear (src/include/migraphx/op/quantizelinear.hpp).
struct op_quantizelinear
{
    bool has_zp = false;
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.has_zp, "has_zp"));
    }
    std::string name() const { return "cuda::quantizelinear"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& s) const { return {s.size() - 1}; }
};

// dequantizelinear: inputs (x, scale view, [zero-point view], out).
struct op_dequantizelinear
{
    bool has_zp = false;
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.has_zp, "has_zp"));
    }
    std::string name() const { return "cuda::dequantizelinear"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& s) const { return {s.size() - 1}; }
};

// unpack_int4 / pack_int4 along the last axis: inputs (x, out).
struct op_unpack_int4
{
    std::string name() const { return "cuda::unpack_int4"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& s) const { return {s.size() - 1}; }
};
struct op_pack_int4
{
    std::string name() const { return "cuda::pack_int4"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& s) const { return {s.size() - 1}; }
};

// quant_dot with the fused epilogue dequantizelinear -> add(bias) -> activation ->
// add(residual) -> convert.  Inputs, in order:
//   A [..,M,K], B ([..,K,N] or, when b_nk, [..,N,K]), [scale (fp32 vector or scalar)],
//   [bias (fp32 [N])], [residual (out's shape and type)], [workspace], out.
struct op_qgemm
{
    int scale_mode    = 0; // mgx_scale_mode
    int act           = 0; // mgx_act
    bool has_bias     = false;
    bool has_residual = false;
    bool b_nk         = false; // B was re-laid out [N,K] at compile time
    bool has_workspace = false;
    int out_type       = static_cast<int>(shape::int32_type); // shape::type_t of the (un-quantised) result
    // fused trailing quantizelinear (per-tensor): q_type = 0 (none) or the shape::type_t of the
    // quantised tensor.  write_d = false: the quantised tensor is the only result (it is the
    // last input); write_d = true: it is an extra input just before the output buffer and is
    // read back through cuda::second_output.
    int q_type    = 0;
    float q_scale = 1.0f;
    float q_zp    = 0.0f;
    bool write_d  = true;
    // fp16 result whose epilogue operators (bias add, activation, residual add) are half operators
    // in the program (the convert to half directly follows dequantizelinear): each is rounded to half
    bool half_math = false;
    // an extra input after the residual: 65536 bytes, activation + quantizelinear of every half
    // (half_math with the quantised tensor as the only result; see MGX_QOUT_LUT)
    bool has_lut = false;
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.half_math, "half_math"), f(self.has_lut, "has_lut"), f(self.scale_mode, "scale_mode"), f(self.act, "act"),
                    f(self.has_bias, "has_bias"), f(self.has_residual, "has_residual"),
                    f(self.b_nk, "b_nk"), f(self.has_workspace, "has_workspace"),
                    f(self.out_type, "out_type"), f(self.q_type, "q_type"),
                    f(self.q_scale, "q_scale"), f(self.q_zp, "q_zp"), f(self.write_d, "write_d"));
    }
    std::string name() const { return "cuda::qgemm"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& s) const { return {s.size() - 1}; }
};

// (x, a 64-byte double buffer) -> x.  memory_coloring places every buffer of the arena at a
// multiple of ONE alignment, the largest any allocation asks for by its element type and count
// (src/memory_coloring.cpp:158-172, 290-300); programs of int8 / fp16 tensors alone would get 4 or
// 8 bytes.  The double[8] allocation this operator keeps alive asks for 32, which is what the
// kernels' 16-byte vector and tensor-map accesses need.
struct op_align_anchor
{
    std::string name() const { return "cuda::align_anchor"; }
    shape compute_shape(const std::vector<shape>& inputs) const { return inputs.at(0); }
    argument compute(const shape&, const std::vector<argument>& args) const { return args.at(0); }
    std::vector<std::size_t> output_alias(const std::vector<shape>&) const { return {0}; }
};

// (producer result, buffer the producer also wrote) -> that buffer: gives the second result
// of an operator with two outputs its own instruction, ordered after the producer.
struct op_second_output
{
    std::string name() const { return "cuda::second_output"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>&) const { return {1}; }
};

// Element-wise instructions evaluated per output element (mgx_cuda_pointwise): value i is input i
// for i < n inputs, then the instructions' results; the last result is the output.  Inputs: the
// operands (strided / broadcast views of the output's index space), then the output buffer.
struct op_pointwise
{
    std::vector<int> ops;    // mgx_pw_op per instruction
    std::vector<int> types;  // shape::type_t of every result
    std::vector<int> srcs;   // three operand indices per instruction
    std::vector<float> imms; // one immediate per instruction
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.ops, "ops"), f(self.types, "types"), f(self.srcs, "srcs"), f(self.imms, "imms"));
    }
    std::string name() const { return "cuda::pointwise"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& args) const { return {args.size() - 1}; }
};

// reduce_sum / reduce_mean / reduce_max / reduce_min over the innermost axis
// (src/include/migraphx/op/reduce_op.hpp).  Inputs: x (standard), out (x's lens, last = 1).
struct op_reduce
{
    int mode = 0; // mgx_reduce_op
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.mode, "mode"));
    }
    std::string name() const { return "cuda::reduce"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& args) const { return {args.size() - 1}; }
};

// LayerNorm over the innermost axis in one launch (mgx_cuda_layernorm), the fusion of the chain
// reduce_mean, sub, mul, reduce_mean, add(eps), rsqrt, mul, [mul(gamma)], [add(beta)] the ONNX
// parser emits (src/onnx/parse_layernorm.cpp:100-140), optionally with the per-tensor
// quantizelinear that reads its result and the dequantizelinear of that quantised tensor (has_dq:
// the dequantised copy simplify_qdq makes other readers use).  Inputs: x, [gamma [cols]],
// [beta [cols]], [dequantised buffer], then - as for cuda::qgemm - the quantised buffer
// (q_type != 0) and / or the output buffer; the last input is what compute() returns.
struct op_layernorm
{
    float eps      = 1e-5f;
    bool has_gamma = false;
    bool has_beta  = false;
    int q_type     = 0; // shape::type_t of the fused quantizelinear's result, 0 = none
    float q_scale  = 1.0f;
    float q_zp     = 0.0f;
    bool write_y   = true;
    bool has_dq    = false;
    float dq_scale = 1.0f;
    bool rms       = false; // RMS normalisation (MGX_LAYERNORM_RMS): no mean, no beta
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.rms, "rms"), f(self.eps, "eps"), f(self.has_gamma, "has_gamma"), f(self.has_beta, "has_beta"),
                    f(self.q_type, "q_type"), f(self.q_scale, "q_scale"), f(self.q_zp, "q_zp"),
                    f(self.write_y, "write_y"), f(self.has_dq, "has_dq"), f(self.dq_scale, "dq_scale"));
    }
    std::string name() const { return "cuda::layernorm"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& s) const { return {s.size() - 1}; }
};

// Multi-head attention without a mask in one launch (mgx_cuda_attention): softmax(scale * Q K^T) V
// per batch entry and head, heads split from and merged into [batch * seq, heads * head_dim]
// matrices in place.  Inputs: Q, K, V (2-D fp16, unit column stride), then - as for cuda::qgemm - the
// quantised buffer (q_type != 0) and / or the output buffer; the last input is what compute() returns.
struct op_attention
{
    std::size_t batch = 1, seq = 1, heads = 1, head_dim = 64;
    float scale   = 1.0f;
    int q_type    = 0; // shape::type_t of the fused quantizelinear's result, 0 = none
    float q_scale = 1.0f;
    float q_zp    = 0.0f;
    bool write_o  = true;
    bool fp32_softmax = false; // MGX_ATTENTION_FP32_SOFTMAX (MIGRAPHX_CUDA_ATTENTION=fp32 at compile time)
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.batch, "batch"), f(self.seq, "seq"), f(self.heads, "heads"), f(self.head_dim, "head_dim"),
                    f(self.scale, "scale"), f(self.q_type, "q_type"), f(self.q_scale, "q_scale"),
                    f(self.q_zp, "q_zp"), f(self.write_o, "write_o"), f(self.fp32_softmax, "fp32_softmax"));
    }
    std::string name() const { return "cuda::attention"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& s) const { return {s.size() - 1}; }
};

// softmax over the innermost axis (src/include/migraphx/op/softmax.hpp).  Inputs: x, out.
struct op_softmax
{
    std::string name() const { return "cuda::softmax"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& args) const { return {args.size() - 1}; }
};

// Copy of a standard tensor into a buffer whose rows (innermost dimension) are padded to a
// multiple of 16 bytes, the row pitch the tensor maps of the GEMM kernels need.  The padding is
// never read (the maps are bounded by the logical row length).  Inputs: x, out (padded strides).
struct op_pad_rows
{
    std::string name() const { return "cuda::pad_rows"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& args) const { return {args.size() - 1}; }
};

// gather along `axis` of a standard tensor (src/include/migraphx/op/gather.hpp).
// Inputs: data, indices (int32 / int64), out.
struct op_gather
{
    int64_t axis = 0;
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.axis, "axis"));
    }
    std::string name() const { return "cuda::gather"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& args) const { return {args.size() - 1}; }
};

// concat of standard tensors along `axis` (src/include/migraphx/op/concat.hpp): one strided
// row copy per input.  Inputs: the tensors, out.
struct op_concat
{
    int64_t axis = 0;
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.axis, "axis"));
    }
    std::string name() const { return "cuda::concat"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& args) const { return {args.size() - 1}; }
};

// op::concat_past_present on the device (src/include/migraphx/op/concat_past_present.hpp): inputs
// present [B, kv_heads, L, D] (any strides with contiguous rows), seqlens_k [B] (int32 / int64),
// the cache [B, kv_heads, T, D] (packed), which is updated in place and returned.
struct op_concat_past_present
{
    std::size_t kv_num_heads = 0;
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.kv_num_heads, "kv_num_heads"));
    }
    std::string name() const { return "cuda::concat_past_present"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>&) const { return {2}; }
};

// op::gqa_rotary_embedding on the device (src/include/migraphx/op/gqa_rotary_embedding.hpp): inputs
// packed QKV [B, heads + 2 kv_heads, S, D] (packed), seqlens_k [B], cos cache, sin cache, out.
struct op_gqa_rotary_embedding
{
    std::size_t num_heads    = 0;
    std::size_t kv_num_heads = 0;
    bool interleaved         = false;
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.num_heads, "num_heads"), f(self.kv_num_heads, "kv_num_heads"),
                    f(self.interleaved, "interleaved"));
    }
    std::string name() const { return "cuda::gqa_rotary_embedding"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& s) const { return {s.size() - 1}; }
};

// The rotation the rotary_embedding builder emits (src/op/builder/rotary_embedding.cpp:60-230,
// non-interleaved: gathernd of the cos / sin rows, concat, rotate-half, mul, mul, mul, add) as one
// launch.  Inputs: x [B, heads, S, D] (rows contiguous), positions [B, S, 1], cos cache, sin cache
// [max_pos, D / 2], out [B, heads, S, D] (packed).
struct op_rotary_embedding
{
    std::string name() const { return "cuda::rotary_embedding"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& s) const { return {s.size() - 1}; }
};

// Decode-step attention against the KV cache: the chain dot(Q, K^T), mul, where(mask), softmax,
// dot(P, V) of a GroupQueryAttention node with one query row per head
// (src/onnx/parse_group_query_attention.cpp:184-262) as one launch.  Inputs: Q [B, heads, 1, D]
// (rows contiguous, any batch / head strides), K cache and V cache [B, kv_heads, T, D] (packed),
// seqlens_k [B, 1] or [B], out [B, heads, 1, D] (packed).
struct op_gqa_decode_attention
{
    std::size_t num_heads    = 0;
    std::size_t kv_num_heads = 0;
    float scale              = 1.0f;
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.num_heads, "num_heads"), f(self.kv_num_heads, "kv_num_heads"), f(self.scale, "scale"));
    }
    std::string name() const { return "cuda::gqa_decode_attention"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& s) const { return {s.size() - 1}; }
};

// Weight-only int4 linear (unpack_int4 + dequantizelinear + transpose + dot fused).
// Inputs: A fp16 [M,K], packed weights uint8 [N,K/2], scales fp16 [N,K/group],
// [zero points uint8 [N,K/group]], [workspace], out fp16 [M,N].
struct op_w4a16
{
    int group          = 128;
    int zp_const       = 8;
    bool has_zp        = false;
    bool has_workspace = false;
    template <class Self, class F>
    static auto reflect(Self& self, F f)
    {
        return pack(f(self.group, "group"), f(self.zp_const, "zp_const"), f(self.has_zp, "has_zp"),
                    f(self.has_workspace, "has_workspace"));
    }
    std::string name() const { return "cuda::w4a16"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>& s) const { return {s.size() - 1}; }
};

// In-place sum all-reduce across the tensor-parallel ranks (one process per GPU) over the
// process's default NCCL communicator (mgx_cuda_comm_set_default).  Input: the partial result
// of a row-split linear; output: the same buffer holding the sum.  New: the reference has no
// collective operator.
struct op_all_reduce
{
    std::string name() const { return "cuda::all_reduce"; }
    shape compute_shape(const std::vector<shape>& inputs) const;
    argument compute(context& ctx, const shape& out, const std::vector<argument>& args) const;
    std::vector<std::size_t> output_alias(const std::vector<shape>&) const { return {0}; }
};

} // namespace cuda
} // namespace MIGRAPHX_INLINE_NS
} // namespace migraphx
#endif
