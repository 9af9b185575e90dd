// Generic element-wise operator: a tiny register machine evaluated per output element.
// Stands in for op::pointwise::compute (src/include/migraphx/op/pointwise.hpp:81-114) and for the
// single element-wise operators (src/include/migraphx/op/{unary,binary}.hpp apply() lambdas).
// Values are held as fp32; after every instruction the value is converted to the instruction's
// type and back, so fp16 chains round (truncate) exactly where the reference's migraphx::half
// arithmetic does, and integer results wrap / saturate the way a cast to that type does.
#include "common.cuh"
#include "qgemm_math.cuh"
#include <cuda_fp16.h>

namespace mgx {

struct pw_args
{
    mgx_pw_desc d;
    const void* in[MGX_PW_MAXIN];
    void* out;
    int64_t total;
};

__device__ __forceinline__ float pw_load(const void* p, int type, int64_t i)
{
    switch(type)
    {
    case MGX_F32: return static_cast<const float*>(p)[i];
    case MGX_F16: return __half2float(static_cast<const __half*>(p)[i]);
    case MGX_I8: return static_cast<float>(static_cast<const int8_t*>(p)[i]);
    case MGX_U8: return static_cast<float>(static_cast<const uint8_t*>(p)[i]);
    default: return static_cast<float>(static_cast<const int32_t*>(p)[i]);
    }
}

// the value as the given type holds it
__device__ __forceinline__ float pw_as_type(float v, int type)
{
    switch(type)
    {
    case MGX_F32: return v;
    case MGX_F16: return truncate_to_half_precision(v);
    case MGX_I8: return static_cast<float>(static_cast<int8_t>(static_cast<int>(v)));
    case MGX_U8: return static_cast<float>(static_cast<uint8_t>(static_cast<int>(v)));
    default: return static_cast<float>(static_cast<int32_t>(v));
    }
}

__device__ __forceinline__ void pw_store(void* p, int type, int64_t i, float v)
{
    switch(type)
    {
    case MGX_F32: static_cast<float*>(p)[i] = v; break;
    case MGX_F16: static_cast<__half*>(p)[i] = __float2half_rz(v); break;
    case MGX_I8: static_cast<int8_t*>(p)[i] = static_cast<int8_t>(static_cast<int>(v)); break;
    case MGX_U8: static_cast<uint8_t*>(p)[i] = static_cast<uint8_t>(static_cast<int>(v)); break;
    default: static_cast<int32_t*>(p)[i] = static_cast<int32_t>(v); break;
    }
}

__global__ void __launch_bounds__(256) pointwise_kernel(const __grid_constant__ pw_args a)
{
    const mgx_pw_desc& d = a.d;
    float r[MGX_PW_MAXIN + MGX_PW_MAXINSN];
    for(int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < a.total;
        idx += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        // multi-index of the output element -> offset into every (strided, broadcast) input
        int64_t off[MGX_PW_MAXIN];
        for(int i = 0; i < d.ninputs; ++i)
            off[i] = 0;
        int64_t rem = idx;
        for(int k = d.ndim - 1; k >= 0; --k)
        {
            const int64_t c = rem % d.lens[k];
            rem /= d.lens[k];
            for(int i = 0; i < d.ninputs; ++i)
                off[i] += c * d.in_strides[i][k];
        }
        for(int i = 0; i < d.ninputs; ++i)
            r[i] = pw_load(a.in[i], d.in_type[i], off[i]);
        for(int n = 0; n < d.ninsns; ++n)
        {
            const mgx_pw_insn& ins = d.insn[n];
            const float x = r[ins.src[0]], y = r[ins.src[1]], z = r[ins.src[2]];
            float v;
            switch(ins.op)
            {
            case MGX_PW_ADD: v = __fadd_rn(x, y); break;
            case MGX_PW_SUB: v = __fsub_rn(x, y); break;
            case MGX_PW_MUL: v = __fmul_rn(x, y); break;
            case MGX_PW_DIV: v = __fdiv_rn(x, y); break;
            case MGX_PW_MIN: v = y < x ? y : x; break; // std::min
            case MGX_PW_MAX: v = x < y ? y : x; break; // std::max
            case MGX_PW_POW: v = powf(x, y); break;
            case MGX_PW_NEG: v = -x; break;
            case MGX_PW_ABS: v = fabsf(x); break;
            case MGX_PW_EXP: v = expf(x); break;
            case MGX_PW_LOG: v = logf(x); break;
            case MGX_PW_SQRT: v = __fsqrt_rn(x); break;
            case MGX_PW_RSQRT: v = __fdiv_rn(1.0f, __fsqrt_rn(x)); break;
            case MGX_PW_RECIP: v = __fdiv_rn(1.0f, x); break;
            case MGX_PW_TANH: v = tanhf(x); break;
            case MGX_PW_SIGMOID: v = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); break;
            case MGX_PW_ERF: v = erff(x); break;
            case MGX_PW_RELU: v = x < 0.0f ? 0.0f : x; break; // std::max(0, x)
            case MGX_PW_SIN: v = sinf(x); break;
            case MGX_PW_COS: v = cosf(x); break;
            case MGX_PW_FLOOR: v = floorf(x); break;
            case MGX_PW_CEIL: v = ceilf(x); break;
            case MGX_PW_ROUND: v = roundf(x); break;
            case MGX_PW_NEARBYINT: v = nearbyintf(x); break;
            case MGX_PW_CONVERT: v = x; break;
            case MGX_PW_WHERE: v = x != 0.0f ? y : z; break;
            case MGX_PW_CLIP: v = fminf(fmaxf(x, y), z); break;
            case MGX_PW_EQUAL: v = x == y ? 1.0f : 0.0f; break;
            case MGX_PW_GREATER: v = x > y ? 1.0f : 0.0f; break;
            case MGX_PW_LESS: v = x < y ? 1.0f : 0.0f; break;
            case MGX_PW_LEAKY_RELU: v = x > 0.0f ? x : __fmul_rn(x, ins.imm); break;
            case MGX_PW_CONST: v = ins.imm; break;
            default: v = x; break;
            }
            r[d.ninputs + n] = pw_as_type(v, ins.type);
        }
        pw_store(a.out, d.insn[d.ninsns - 1].type, idx, r[d.ninputs + d.ninsns - 1]);
    }
}

} // namespace mgx

using namespace mgx;

extern "C" int mgx_cuda_pointwise(const mgx_pw_desc* d, const void* const* inputs, void* out, void* stream_)
{
    if(d == nullptr or out == nullptr or (d->ninputs > 0 and inputs == nullptr))
        return MGX_E_INVALID_ARG;
    if(d->ndim < 1 or d->ndim > MGX_PW_MAXDIMS or d->ninputs < 0 or d->ninputs > MGX_PW_MAXIN or
       d->ninsns < 1 or d->ninsns > MGX_PW_MAXINSN)
        return MGX_E_UNSUPPORTED;
    pw_args a{};
    a.d     = *d;
    a.out   = out;
    a.total = 1;
    for(int k = 0; k < d->ndim; ++k)
    {
        if(d->lens[k] < 0)
            return MGX_E_INVALID_ARG;
        a.total *= d->lens[k];
    }
    for(int i = 0; i < d->ninputs; ++i)
    {
        if(inputs[i] == nullptr or d->in_type[i] < MGX_F32 or d->in_type[i] > MGX_I32)
            return MGX_E_INVALID_ARG;
        a.in[i] = inputs[i];
    }
    for(int n = 0; n < d->ninsns; ++n)
    {
        const auto& ins = d->insn[n];
        if(ins.op < 0 or ins.op >= MGX_PW_OP_COUNT or ins.type < MGX_F32 or ins.type > MGX_I32)
            return MGX_E_UNSUPPORTED;
        for(int s : ins.src)
            if(s < 0 or s >= d->ninputs + n)
                if(not(s == 0 and d->ninputs + n == 0)) // constants have no operands
                    return MGX_E_INVALID_ARG;
    }
    if(a.total == 0)
        return MGX_OK;
    const int64_t blocks = ceil_div(a.total, 256);
    const int grid       = static_cast<int>(blocks < 148 * 8 ? blocks : 148 * 8);
    pointwise_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_)>>>(a);
    return static_cast<int>(cudaGetLastError());
}
