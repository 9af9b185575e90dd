// Generic element-wise operator: a tiny register machine evaluated per output element.
// Stands in for op::pointwise::compute (src/include/migraphx/op/pointwise.hpp:81-114) and for the
// single element-wise operators (src/include/migraphx/op/{unary,binary}.hpp apply() lambdas).
// Values are held as fp32; after every instruction the value is converted to the instruction's
// type and back, so fp16 chains round (truncate) exactly where the reference's migraphx::half
// arithmetic does, and integer results wrap / saturate the way a cast to that type does.
#include "common.cuh"
#include "ptx.cuh"
#include "qgemm_math.cuh"
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace mgx {

struct pw_args
{
    mgx_pw_desc d;
    const void* in[MGX_PW_MAXIN];
    void* out;
    int64_t total;
    // division by lens[k] for indices below 2^31: q = (n * magic[k]) >> shift[k]
    uint64_t magic[MGX_PW_MAXDIMS];
    int shift[MGX_PW_MAXDIMS];
    // bit n: the result of instruction n is read by an instruction other than n + 1 (it must be
    // kept in r[]; the result of the previous instruction is always at hand in registers)
    uint32_t keep;
};

// fp8 e4m3fn as the reference's float8 class converts (src/include/migraphx/float8_impl.hpp:
// round to nearest even, clipped to the largest finite value; NaN stays NaN)
__device__ __forceinline__ float fp8_e4m3fn_value(uint8_t b)
{
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3)));
}
__device__ __forceinline__ uint8_t fp8_e4m3fn_bits(float v)
{
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float pw_load(const void* p, int type, int64_t i)
{
    switch(type)
    {
    case MGX_F32: return static_cast<const float*>(p)[i];
    case MGX_F16: return __half2float(static_cast<const __half*>(p)[i]);
    case MGX_I8: return static_cast<float>(static_cast<const int8_t*>(p)[i]);
    case MGX_U8: return static_cast<float>(static_cast<const uint8_t*>(p)[i]);
    case MGX_FP8_E4M3FN: return fp8_e4m3fn_value(static_cast<const uint8_t*>(p)[i]);
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
    case MGX_FP8_E4M3FN: return fp8_e4m3fn_value(fp8_e4m3fn_bits(v));
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
    case MGX_FP8_E4M3FN: static_cast<uint8_t*>(p)[i] = fp8_e4m3fn_bits(v); break;
    default: static_cast<int32_t*>(p)[i] = static_cast<int32_t>(v); break;
    }
}

// V consecutive elements of the innermost dimension per thread: the multi-index is decomposed
// once per V elements, contiguous operands are read and the result written as 16-byte vectors,
// and every instruction is dispatched once per V elements.  Operands that are inputs are read
// from global memory where they are used and the last result goes straight to the store, so only
// the intermediate results of a chain pass through r[slot][v], which the program indexes and
// which therefore lives in (L1-resident) local memory.
// operands an operator reads
__device__ __forceinline__ int pw_arity(int op)
{
    switch(op)
    {
    case MGX_PW_CONST: return 0;
    case MGX_PW_ADD:
    case MGX_PW_SUB:
    case MGX_PW_MUL:
    case MGX_PW_DIV:
    case MGX_PW_MIN:
    case MGX_PW_MAX:
    case MGX_PW_POW:
    case MGX_PW_EQUAL:
    case MGX_PW_GREATER:
    case MGX_PW_LESS: return 2;
    case MGX_PW_WHERE:
    case MGX_PW_CLIP: return 3;
    default: return 1;
    }
}

template <int V>
__device__ __forceinline__ void pw_load_vec(const void* p, int type, int64_t off, int64_t stride, float (&r)[V])
{
    if(stride == 0)
    {
        const float x = pw_load(p, type, off);
#pragma unroll
        for(int v = 0; v < V; ++v)
            r[v] = x;
        return;
    }
    if constexpr(V == 8)
    {
        if(stride == 1 and type == MGX_F16 and ((reinterpret_cast<uintptr_t>(p) + 2 * off) & 15u) == 0)
        {
            const uint4 w     = *reinterpret_cast<const uint4*>(static_cast<const __half*>(p) + off);
            const __half2* h2 = reinterpret_cast<const __half2*>(&w);
#pragma unroll
            for(int v = 0; v < 4; ++v)
            {
                const float2 f = __half22float2(h2[v]);
                r[2 * v]       = f.x;
                r[2 * v + 1]   = f.y;
            }
            return;
        }
        if(stride == 1 and type == MGX_F32 and ((reinterpret_cast<uintptr_t>(p) + 4 * off) & 15u) == 0)
        {
            const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + off);
            const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + off + 4);
            r[0] = a.x, r[1] = a.y, r[2] = a.z, r[3] = a.w, r[4] = b.x, r[5] = b.y, r[6] = b.z, r[7] = b.w;
            return;
        }
    }
#pragma unroll
    for(int v = 0; v < V; ++v)
        r[v] = pw_load(p, type, off + v * stride);
}

template <int V>
__device__ __forceinline__ void pw_store_vec(void* p, int type, int64_t i, const float (&r)[V])
{
    if constexpr(V == 8)
    {
        if(type == MGX_F16 and ((reinterpret_cast<uintptr_t>(p) + 2 * i) & 15u) == 0)
        {
            uint4 w;
            w.x = cvt_rz_f16x2(r[0], r[1]);
            w.y = cvt_rz_f16x2(r[2], r[3]);
            w.z = cvt_rz_f16x2(r[4], r[5]);
            w.w = cvt_rz_f16x2(r[6], r[7]);
            *reinterpret_cast<uint4*>(static_cast<__half*>(p) + i) = w;
            return;
        }
        if(type == MGX_F32 and ((reinterpret_cast<uintptr_t>(p) + 4 * i) & 15u) == 0)
        {
            float* o                         = static_cast<float*>(p) + i;
            *reinterpret_cast<float4*>(o)     = make_float4(r[0], r[1], r[2], r[3]);
            *reinterpret_cast<float4*>(o + 4) = make_float4(r[4], r[5], r[6], r[7]);
            return;
        }
    }
#pragma unroll
    for(int v = 0; v < V; ++v)
        pw_store(p, type, i + v, r[v]);
}

#define MGX_PW_EACH1(expr)                       \
    _Pragma("unroll") for(int v = 0; v < V; ++v) \
    {                                            \
        const float x = rx[v];                   \
        ro[v]         = (expr);                  \
    }                                            \
    break
#define MGX_PW_EACH2(expr)                       \
    _Pragma("unroll") for(int v = 0; v < V; ++v) \
    {                                            \
        const float x = rx[v], y = ry[v];        \
        ro[v]         = (expr);                  \
    }                                            \
    break

template <int V, class IndexT>
__global__ void __launch_bounds__(256) pointwise_kernel(const __grid_constant__ pw_args a)
{
    const mgx_pw_desc& d = a.d;
    float r[MGX_PW_MAXINSN][V];
    const int last       = d.ndim - 1;
    const IndexT nvec    = static_cast<IndexT>(a.total / V);
    for(IndexT vec = blockIdx.x * static_cast<IndexT>(256) + threadIdx.x; vec < nvec;
        vec += static_cast<IndexT>(gridDim.x) * 256)
    {
        // multi-index of the first element -> offset into every (strided, broadcast) input
        const IndexT idx = vec * V;
        int64_t off[MGX_PW_MAXIN];
        for(int i = 0; i < d.ninputs; ++i)
            off[i] = 0;
        IndexT rem = idx;
        for(int k = last; k > 0; --k)
        {
            const IndexT len = static_cast<IndexT>(d.lens[k]);
            IndexT q;
            if constexpr(sizeof(IndexT) == 4)
                q = static_cast<IndexT>((static_cast<uint64_t>(rem) * a.magic[k]) >> a.shift[k]);
            else
                q = rem / len;
            const IndexT c = rem - q * len;
            rem            = q;
            for(int i = 0; i < d.ninputs; ++i)
                off[i] += static_cast<int64_t>(c) * d.in_strides[i][k];
        }
        // the outermost index needs no division
        for(int i = 0; i < d.ninputs; ++i)
            off[i] += static_cast<int64_t>(rem) * d.in_strides[i][0];
        float prev[V];
#pragma unroll
        for(int v = 0; v < V; ++v)
            prev[v] = 0.0f;
        int prev_slot = -1;
        auto fetch = [&](int src, float(&dst)[V]) {
            if(src < d.ninputs)
                pw_load_vec<V>(a.in[src], d.in_type[src], off[src], d.in_strides[src][last], dst);
            else if(src == prev_slot)
            {
#pragma unroll
                for(int v = 0; v < V; ++v)
                    dst[v] = prev[v];
            }
            else
            {
#pragma unroll
                for(int v = 0; v < V; ++v)
                    dst[v] = r[src - d.ninputs][v];
            }
        };
        for(int n = 0; n < d.ninsns; ++n)
        {
            const mgx_pw_insn& ins = d.insn[n];
            float ro[V];
            const float imm = ins.imm;
            const int arity = pw_arity(ins.op);
            // one dispatch per arity: only the operands an operator reads are fetched
            if(arity == 2)
            {
                float rx[V], ry[V];
                fetch(ins.src[0], rx);
                fetch(ins.src[1], ry);
                switch(ins.op)
                {
                case MGX_PW_ADD: MGX_PW_EACH2(__fadd_rn(x, y));
                case MGX_PW_SUB: MGX_PW_EACH2(__fsub_rn(x, y));
                case MGX_PW_MUL: MGX_PW_EACH2(__fmul_rn(x, y));
                case MGX_PW_DIV: MGX_PW_EACH2(__fdiv_rn(x, y));
                case MGX_PW_MIN: MGX_PW_EACH2(y < x ? y : x); // std::min
                case MGX_PW_MAX: MGX_PW_EACH2(x < y ? y : x); // std::max
                case MGX_PW_POW: MGX_PW_EACH2(powf(x, y));
                case MGX_PW_EQUAL: MGX_PW_EACH2(x == y ? 1.0f : 0.0f);
                case MGX_PW_GREATER: MGX_PW_EACH2(x > y ? 1.0f : 0.0f);
                default: MGX_PW_EACH2(x < y ? 1.0f : 0.0f); // less
                }
            }
            else if(arity == 1)
            {
                float rx[V];
                fetch(ins.src[0], rx);
                switch(ins.op)
                {
                case MGX_PW_NEG: MGX_PW_EACH1(-x);
                case MGX_PW_ABS: MGX_PW_EACH1(fabsf(x));
                case MGX_PW_EXP: MGX_PW_EACH1(expf(x));
                case MGX_PW_LOG: MGX_PW_EACH1(logf(x));
                case MGX_PW_SQRT: MGX_PW_EACH1(__fsqrt_rn(x));
                case MGX_PW_RSQRT: MGX_PW_EACH1(__fdiv_rn(1.0f, __fsqrt_rn(x)));
                case MGX_PW_RECIP: MGX_PW_EACH1(__fdiv_rn(1.0f, x));
                case MGX_PW_TANH: MGX_PW_EACH1(tanhf(x));
                case MGX_PW_SIGMOID: MGX_PW_EACH1(__fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))));
                case MGX_PW_ERF: MGX_PW_EACH1(erff(x));
                case MGX_PW_RELU: MGX_PW_EACH1(x < 0.0f ? 0.0f : x); // std::max(0, x)
                case MGX_PW_SIN: MGX_PW_EACH1(sinf(x));
                case MGX_PW_COS: MGX_PW_EACH1(cosf(x));
                case MGX_PW_FLOOR: MGX_PW_EACH1(floorf(x));
                case MGX_PW_CEIL: MGX_PW_EACH1(ceilf(x));
                case MGX_PW_ROUND: MGX_PW_EACH1(roundf(x));
                case MGX_PW_NEARBYINT: MGX_PW_EACH1(nearbyintf(x));
                case MGX_PW_LEAKY_RELU: MGX_PW_EACH1(x > 0.0f ? x : __fmul_rn(x, imm));
                default: MGX_PW_EACH1(x); // convert, identity
                }
            }
            else if(arity == 3)
            {
                float rx[V], ry[V], rz[V];
                fetch(ins.src[0], rx);
                fetch(ins.src[1], ry);
                fetch(ins.src[2], rz);
#pragma unroll
                for(int v = 0; v < V; ++v)
                    ro[v] = ins.op == MGX_PW_WHERE ? (rx[v] != 0.0f ? ry[v] : rz[v])
                                                   : fminf(fmaxf(rx[v], ry[v]), rz[v]); // clip
            }
            else
            {
#pragma unroll
                for(int v = 0; v < V; ++v)
                    ro[v] = imm;
            }
            if(n == d.ninsns - 1)
            {
                // the store converts (fp16: truncates) by itself
                pw_store_vec<V>(a.out, ins.type, static_cast<int64_t>(idx), ro);
                break;
            }
            if(ins.type == MGX_F16)
            {
                // all values normal halves (the common case): cut the mantissas
                float hi = 0.0f, lo = 65536.0f;
#pragma unroll
                for(int v = 0; v < V; ++v)
                {
                    hi = fmaxf(hi, fabsf(ro[v]));
                    lo = fminf(lo, fabsf(ro[v]));
                }
                if(hi < 65536.0f and lo >= 6.103515625e-5f)
                {
#pragma unroll
                    for(int v = 0; v < V; ++v)
                        ro[v] = __uint_as_float(__float_as_uint(ro[v]) & 0xFFFFE000u);
                }
                else
                {
#pragma unroll
                    for(int v = 0; v < V; ++v)
                        ro[v] = truncate_to_half_precision(ro[v]);
                }
            }
            else if(ins.type != MGX_F32)
            {
#pragma unroll
                for(int v = 0; v < V; ++v)
                    ro[v] = pw_as_type(ro[v], ins.type);
            }
            prev_slot = d.ninputs + n;
#pragma unroll
            for(int v = 0; v < V; ++v)
                prev[v] = ro[v];
            if((a.keep >> n) & 1u)
            {
#pragma unroll
                for(int v = 0; v < V; ++v)
                    r[n][v] = ro[v];
            }
        }
    }
}
#undef MGX_PW_EACH1
#undef MGX_PW_EACH2

template <int V>
static int launch_pointwise(const pw_args& a, cudaStream_t stream)
{
    const int64_t nvec   = a.total / V;
    const int64_t blocks = ceil_div(nvec, 256);
    // one wave of resident blocks: a grid-stride loop over more blocks than fit at once would
    // leave a partial second wave
    static const int resident = [] {
        int n = 0;
        if(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, pointwise_kernel<V, uint32_t>, 256, 0) != cudaSuccess or n < 1)
            n = 4;
        return n;
    }();
    const int64_t cap = static_cast<int64_t>(device_sm_count()) * resident;
    const int grid    = static_cast<int>(blocks < cap ? blocks : cap);
    if(a.total < (int64_t{1} << 31))
        pointwise_kernel<V, uint32_t><<<grid, 256, 0, stream>>>(a);
    else
        pointwise_kernel<V, int64_t><<<grid, 256, 0, stream>>>(a);
    return static_cast<int>(cudaGetLastError());
}

// ---- fixed-function forms of the two programs a decoder layer evaluates once per token -------
// The register machine above costs several microseconds per launch whatever the size (program
// decoding, a large instruction footprint); a residual add and the SwiGLU gate are evaluated here
// with the same operations and the same roundings, 8 halves per thread.
struct pw_f16_args
{
    const __half* in0;
    const __half* in1;
    __half* out;
    int64_t stride0, stride1; // elements between rows of the two operands
    uint32_t rows, row_vecs;  // 16-byte vectors per row
    int op;                   // PW_FORM_BINARY: MGX_PW_ADD | MGX_PW_SUB | MGX_PW_MUL
};
enum { PW_FORM_BINARY, PW_FORM_SWIGLU };

template <int FORM>
__global__ void __launch_bounds__(256) pointwise_f16_kernel(const pw_f16_args a)
{
    const uint32_t nvec = a.rows * a.row_vecs;
    for(uint32_t vec = blockIdx.x * 256u + threadIdx.x; vec < nvec; vec += gridDim.x * 256u)
    {
        const uint32_t row = vec / a.row_vecs, col = vec - row * a.row_vecs;
        float x[8], y[8], r[8];
        pw_load_vec<8>(a.in0, MGX_F16, row * a.stride0 + col * 8, 1, x);
        pw_load_vec<8>(a.in1, MGX_F16, row * a.stride1 + col * 8, 1, y);
        if constexpr(FORM == PW_FORM_BINARY)
        {
#pragma unroll
            for(int v = 0; v < 8; ++v)
                r[v] = a.op == MGX_PW_ADD ? __fadd_rn(x[v], y[v])
                                          : (a.op == MGX_PW_SUB ? __fsub_rn(x[v], y[v]) : __fmul_rn(x[v], y[v]));
        }
        else
        {
            // sigmoid(x), x * sigmoid(x), (x * sigmoid(x)) * y: a half after every operator
#pragma unroll
            for(int v = 0; v < 8; ++v)
            {
                const float s = truncate_to_half_precision(__fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x[v]))));
                const float t = truncate_to_half_precision(__fmul_rn(x[v], s));
                r[v]          = __fmul_rn(t, y[v]);
            }
        }
        pw_store_vec<8>(a.out, MGX_F16, static_cast<int64_t>(vec) * 8, r);
    }
}

// true (and the launch done, its status in `status`) when the program is one of the fixed forms
// over fp16 operands whose rows are contiguous and 16-byte aligned
static bool launch_pointwise_f16_form(const pw_args& a, cudaStream_t stream, int& status)
{
    const mgx_pw_desc& d = a.d;
    if(d.ninputs != 2 or d.ndim > 2 or a.total >= (int64_t{1} << 31))
        return false;
    const int last      = d.ndim - 1;
    const int64_t inner = d.lens[last];
    if(inner % 8 != 0 or reinterpret_cast<uintptr_t>(a.out) % 16 != 0)
        return false;
    for(int i = 0; i < 2; ++i)
    {
        if(d.in_type[i] != MGX_F16 or d.in_strides[i][last] != 1 or reinterpret_cast<uintptr_t>(a.in[i]) % 16 != 0)
            return false;
        if(d.ndim == 2 and (d.in_strides[i][0] % 8 != 0 or d.in_strides[i][0] < 0))
            return false;
    }
    for(int n = 0; n < d.ninsns; ++n)
        if(d.insn[n].type != MGX_F16)
            return false;
    auto reads = [&](int n, int p, int q) {
        const auto& s = d.insn[n].src;
        return (s[0] == p and s[1] == q) or (s[0] == q and s[1] == p);
    };
    int form = -1, first = 0; // first: the input that is x (the gate) of the SwiGLU form
    if(d.ninsns == 1 and (d.insn[0].op == MGX_PW_ADD or d.insn[0].op == MGX_PW_MUL) and reads(0, 0, 1))
        form = PW_FORM_BINARY;
    else if(d.ninsns == 1 and d.insn[0].op == MGX_PW_SUB and d.insn[0].src[0] == 0 and d.insn[0].src[1] == 1)
        form = PW_FORM_BINARY;
    else if(d.ninsns == 3 and d.insn[0].op == MGX_PW_SIGMOID and d.insn[0].src[0] < 2 and
            d.insn[1].op == MGX_PW_MUL and d.insn[2].op == MGX_PW_MUL)
    {
        first = d.insn[0].src[0];
        if(reads(1, first, 2) and reads(2, 3, 1 - first))
            form = PW_FORM_SWIGLU;
    }
    if(form < 0)
        return false;
    pw_f16_args f{};
    f.in0      = static_cast<const __half*>(a.in[first]);
    f.in1      = static_cast<const __half*>(a.in[1 - first]);
    f.out      = static_cast<__half*>(a.out);
    f.rows     = d.ndim == 2 ? static_cast<uint32_t>(d.lens[0]) : 1u;
    f.row_vecs = static_cast<uint32_t>(inner / 8);
    f.stride0  = d.ndim == 2 ? d.in_strides[first][0] : 0;
    f.stride1  = d.ndim == 2 ? d.in_strides[1 - first][0] : 0;
    f.op       = d.insn[0].op;
    const int64_t blocks = ceil_div(a.total / 8, 256);
    const int64_t cap    = static_cast<int64_t>(device_sm_count()) * 8;
    const int grid       = static_cast<int>(blocks < cap ? blocks : cap);
    if(form == PW_FORM_BINARY)
        pointwise_f16_kernel<PW_FORM_BINARY><<<grid, 256, 0, stream>>>(f);
    else
        pointwise_f16_kernel<PW_FORM_SWIGLU><<<grid, 256, 0, stream>>>(f);
    status = static_cast<int>(cudaGetLastError());
    return true;
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
        if(inputs[i] == nullptr or d->in_type[i] < MGX_F32 or d->in_type[i] > MGX_FP8_E4M3FN)
            return MGX_E_INVALID_ARG;
        a.in[i] = inputs[i];
    }
    for(int n = 0; n < d->ninsns; ++n)
    {
        const auto& ins = d->insn[n];
        if(ins.op < 0 or ins.op >= MGX_PW_OP_COUNT or ins.type < MGX_F32 or ins.type > MGX_FP8_E4M3FN)
            return MGX_E_UNSUPPORTED;
        for(int s : ins.src)
            if(s < 0 or s >= d->ninputs + n)
                if(not(s == 0 and d->ninputs + n == 0)) // constants have no operands
                    return MGX_E_INVALID_ARG;
    }
    for(int n = 0; n < d->ninsns; ++n)
        for(int m = n + 2; m < d->ninsns; ++m)
            for(int sidx : d->insn[m].src)
                if(sidx == d->ninputs + n)
                    a.keep |= 1u << n;
    if(a.total == 0)
        return MGX_OK;
    // fewer dimensions, fewer divisions per element: drop dimensions of length 1 and merge a
    // dimension into its inner neighbour where every operand steps through both as through one
    {
        mgx_pw_desc& c = a.d;
        int nd         = 0;
        for(int k = 0; k < d->ndim; ++k)
        {
            if(d->lens[k] == 1)
                continue;
            bool merge = nd > 0;
            for(int i = 0; merge and i < d->ninputs; ++i)
                if(c.in_strides[i][nd - 1] != d->in_strides[i][k] * d->lens[k])
                    merge = false;
            if(merge)
            {
                c.lens[nd - 1] *= d->lens[k];
                for(int i = 0; i < d->ninputs; ++i)
                    c.in_strides[i][nd - 1] = d->in_strides[i][k];
            }
            else
            {
                c.lens[nd] = d->lens[k];
                for(int i = 0; i < d->ninputs; ++i)
                    c.in_strides[i][nd] = d->in_strides[i][k];
                ++nd;
            }
        }
        if(nd == 0)
        {
            // a single element
            c.lens[0] = 1;
            for(int i = 0; i < d->ninputs; ++i)
                c.in_strides[i][0] = 0;
            nd = 1;
        }
        c.ndim = nd;
        for(int k = 0; k < nd; ++k)
        {
            const uint64_t len = static_cast<uint64_t>(c.lens[k]);
            int l              = 0;
            while((uint64_t{1} << l) < len)
                ++l;
            a.shift[k] = 31 + l;
            a.magic[k] = ((uint64_t{1} << a.shift[k]) + len - 1) / len;
        }
    }
    // vectors never straddle a row: V divides the innermost length
    const int64_t inner = a.d.lens[a.d.ndim - 1];
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int status          = MGX_OK;
    if(launch_pointwise_f16_form(a, stream, status))
        return status;
    if(inner % 8 == 0)
        return launch_pointwise<8>(a, stream);
    if(inner % 2 == 0)
        return launch_pointwise<2>(a, stream);
    return launch_pointwise<1>(a, stream);
}
