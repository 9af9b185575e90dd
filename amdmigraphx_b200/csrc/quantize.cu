// HBM-bound element-wise kernels of the quantized path: quantizelinear,
// dequantizelinear, unpack_int4 / pack_int4 and the 8-bit transpose used to make
// quant_dot's [K,N] operand K-contiguous.
//
// Arithmetic follows the MIGraphX operators exactly:
//   quantizelinear   src/include/migraphx/op/quantizelinear.hpp:71-108
//   dequantizelinear src/include/migraphx/op/dequantizelinear.hpp:60-82
//   unpack_int4      src/include/migraphx/op/unpack_int4.hpp:75-120
//   pack_int4        src/include/migraphx/op/pack_int4.hpp:79-123
#include "common.cuh"
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace mgx {

// ------------------------------------------------------------------ helpers
template <class T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v)
{
    return v;
}
template <>
__device__ __forceinline__ float to_f32<__half>(__half v)
{
    return __half2float(v);
}

// x / s evaluated in the input type (the reference divides `input[i] / scales[i]`
// in the tensor's own type for integer targets).  migraphx::half divides in fp32 and
// converts the quotient back by shifting the mantissa, i.e. rounding toward zero
// (src/include/migraphx/generic_float.hpp:180-230, 321-329).
template <class T>
__device__ __forceinline__ float div_in_type(float x, float s);
template <>
__device__ __forceinline__ float div_in_type<float>(float x, float s)
{
    return __fdiv_rn(x, s);
}
template <>
__device__ __forceinline__ float div_in_type<__half>(float x, float s)
{
    return __half2float(__float2half_rz(__fdiv_rn(x, s)));
}

struct q_i8
{
    using type = int8_t;
    static __device__ __forceinline__ float zp(int8_t z) { return static_cast<float>(z); }
    template <class In>
    static __device__ __forceinline__ int8_t quant(float x, float s, float z)
    {
        // nearbyint (round-half-even) of the quotient, + zero point, saturate.
        // fminf/fmaxf drop a NaN operand, as std::min/std::max do in the reference's
        // argument order, so NaN saturates to the maximum.
        float q = rintf(div_in_type<In>(x, s)) + z;
        q       = fmaxf(-128.0f, fminf(127.0f, q));
        return static_cast<int8_t>(static_cast<int>(q));
    }
};
struct q_u8
{
    using type = uint8_t;
    static __device__ __forceinline__ float zp(uint8_t z) { return static_cast<float>(z); }
    template <class In>
    static __device__ __forceinline__ uint8_t quant(float x, float s, float z)
    {
        float q = rintf(div_in_type<In>(x, s)) + z;
        q       = fmaxf(0.0f, fminf(255.0f, q));
        return static_cast<uint8_t>(static_cast<int>(q));
    }
};
struct q_fp8
{
    using type = uint8_t; // e4m3fn bit pattern
    static __device__ __forceinline__ float zp(uint8_t z)
    {
        return __half2float(__half(__nv_cvt_fp8_to_halfraw(z, __NV_E4M3)));
    }
    template <class In>
    static __device__ __forceinline__ uint8_t quant(float x, float s, float z)
    {
        // no nearbyint for floating targets: x/s + zp in double, clamp to +-448, then
        // one round-to-nearest-even cast.  fp32 division of fp32 operands equals the
        // double quotient rounded to fp32; the sum with a non-zero zp is done in double.
        float q;
        if(z == 0.0f)
            q = __fdiv_rn(x, s);
        else
            q = static_cast<float>(static_cast<double>(x) / static_cast<double>(s) +
                                   static_cast<double>(z));
        q = fmaxf(-448.0f, fminf(448.0f, q));
        return static_cast<uint8_t>(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3));
    }
};

struct view2
{
    int64_t s0, s1;
};

// One work item = 16 bytes of one input row (4 fp32 or 8 fp16 columns) -> 4 or 8 output
// bytes.  Index arithmetic is done in IdxT (32-bit whenever the tensor allows it: a 64-bit
// division per item would make the kernel ALU-bound).  UNIFORM: scale and zero point are
// per-tensor (all strides 0) and are read once per thread.
template <class In, class Q, class IdxT, bool UNIFORM>
__global__ void __launch_bounds__(256)
    quantize_vec_kernel(const In* __restrict__ x, int64_t ldx, const In* __restrict__ scale,
                        view2 ss, const typename Q::type* __restrict__ zp, view2 zs,
                        typename Q::type* __restrict__ y, int64_t ldy, IdxT rows, IdxT colsv)
{
    constexpr int VEC = 16 / sizeof(In);
    const IdxT total  = rows * colsv;
    const IdxT stride = static_cast<IdxT>(gridDim.x) * blockDim.x;
    float s0 = 1.0f, z0 = 0.0f;
    if(UNIFORM)
    {
        s0 = to_f32<In>(scale[0]);
        z0 = zp == nullptr ? 0.0f : Q::zp(zp[0]);
    }
    for(IdxT i = static_cast<IdxT>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
    {
        const IdxT r = i / colsv;
        const IdxT c = (i - r * colsv) * VEC;
        const uint4 raw = *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(r) * ldx + c);
        float xv[VEC];
        if constexpr(std::is_same<In, float>::value)
        {
            xv[0] = __uint_as_float(raw.x), xv[1] = __uint_as_float(raw.y);
            xv[2] = __uint_as_float(raw.z), xv[3] = __uint_as_float(raw.w);
        }
        else
        {
            const __half* vh = reinterpret_cast<const __half*>(&raw);
#pragma unroll
            for(int j = 0; j < VEC; ++j)
                xv[j] = __half2float(vh[j]);
        }
        uint32_t packed[VEC / 4];
#pragma unroll
        for(int w = 0; w < VEC / 4; ++w)
            packed[w] = 0;
#pragma unroll
        for(int j = 0; j < VEC; ++j)
        {
            float sv = s0, zv = z0;
            if(not UNIFORM)
            {
                sv = to_f32<In>(scale[static_cast<int64_t>(r) * ss.s0 + (c + j) * ss.s1]);
                zv = zp == nullptr ? 0.0f
                                   : Q::zp(zp[static_cast<int64_t>(r) * zs.s0 + (c + j) * zs.s1]);
            }
            const uint32_t q = static_cast<uint8_t>(Q::template quant<In>(xv[j], sv, zv));
            packed[j / 4] |= q << (8 * (j % 4));
        }
        typename Q::type* dst = y + static_cast<int64_t>(r) * ldy + c;
        if constexpr(VEC == 4)
            *reinterpret_cast<uint32_t*>(dst) = packed[0];
        else
            *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[1]);
    }
}

// Per-tensor int8 quantizelinear without conversion instructions (int <-> float, float <-> half
// and round-to-integer issue at an eighth of the fp32 rate on this GPU and would bound the
// kernel well below the HBM rate).  Bit-identical to Q::quant for q_i8:
//  * fp16 -> fp32: the half's exponent and mantissa bits are moved to the fp32 position and the
//    value is rescaled by 2^112 (exact, also for subnormal halves);
//  * x / s: quotient from the reciprocal computed once, refined with the remainder;
//  * fp16 input: the quotient is cut to 10 mantissa bits (migraphx::half's truncating conversion);
//  * round half to even and float -> int by adding 1.5 * 2^23 after saturating.
template <class In, class IdxT>
__global__ void __launch_bounds__(256)
    quantize_i8_uniform_kernel(const In* __restrict__ x, int64_t ldx, const In* __restrict__ scale,
                               const int8_t* __restrict__ zp, int8_t* __restrict__ y, int64_t ldy,
                               IdxT rows, IdxT colsv)
{
    constexpr int VEC = 16 / sizeof(In);
    // chained launches: the next kernel of the stream may set itself up now; this one reads
    // the previous kernel's output only after that kernel has completed
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const IdxT total  = rows * colsv;
    const IdxT stride = static_cast<IdxT>(gridDim.x) * blockDim.x;
    const float s     = to_f32<In>(scale[0]);
    const float rcp   = static_cast<float>(1.0 / static_cast<double>(s));
    const int z       = zp == nullptr ? 0 : static_cast<int>(zp[0]);
    const bool plain  = s > 0.0f and isfinite(rcp);
    for(IdxT i = static_cast<IdxT>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
    {
        const IdxT r = i / colsv;
        const IdxT c = (i - r * colsv) * VEC;
        const uint4 raw = *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(r) * ldx + c);
        float xv[VEC];
        if constexpr(std::is_same<In, float>::value)
        {
            xv[0] = __uint_as_float(raw.x), xv[1] = __uint_as_float(raw.y);
            xv[2] = __uint_as_float(raw.z), xv[3] = __uint_as_float(raw.w);
        }
        else
        {
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for(int k = 0; k < 4; ++k)
            {
                const uint32_t lo = ((w[k] & 0x7FFFu) << 13) | ((w[k] & 0x8000u) << 16);
                const uint32_t hi = ((w[k] >> 3) & 0x0FFFE000u) | (w[k] & 0x80000000u);
                xv[2 * k]     = __uint_as_float(lo) * 5.192296858534828e33f; // 2^112
                xv[2 * k + 1] = __uint_as_float(hi) * 5.192296858534828e33f;
            }
        }
        uint32_t packed[VEC / 4];
#pragma unroll
        for(int w = 0; w < VEC / 4; ++w)
            packed[w] = 0;
#pragma unroll
        for(int j = 0; j < VEC; ++j)
        {
            uint32_t b;
            if(plain)
            {
                float q         = __fmul_rn(xv[j], rcp);
                const float rem = __fmaf_rn(-s, q, xv[j]);
                q               = __fmaf_rn(rem, rcp, q);
                if constexpr(not std::is_same<In, float>::value)
                    q = __uint_as_float(__float_as_uint(q) & 0xFFFFE000u);
                q             = fmaxf(-300.0f, fminf(300.0f, q));
                const float t = __fadd_rn(q, 12582912.0f);
                int qi        = __float_as_int(t) - 0x4B400000 + z;
                qi            = max(-128, min(127, qi));
                b             = static_cast<uint32_t>(qi) & 0xFFu;
            }
            else
                b = static_cast<uint8_t>(q_i8::quant<In>(xv[j], s, static_cast<float>(z)));
            packed[j / 4] |= b << (8 * (j % 4));
        }
        int8_t* dst = y + static_cast<int64_t>(r) * ldy + c;
        if constexpr(VEC == 4)
            *reinterpret_cast<uint32_t*>(dst) = packed[0];
        else
            *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[1]);
    }
}

template <class In, class Q>
__global__ void __launch_bounds__(256)
    quantize_scalar_kernel(const In* __restrict__ x, int64_t ldx, const In* __restrict__ scale,
                           view2 ss, const typename Q::type* __restrict__ zp, view2 zs,
                           typename Q::type* __restrict__ y, int64_t ldy, int64_t rows,
                           int64_t cols)
{
    const int64_t total = rows * cols;
    for(int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
        i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        const int64_t r = i / cols;
        const int64_t c = i - r * cols;
        const float s   = to_f32<In>(scale[r * ss.s0 + c * ss.s1]);
        const float z   = zp == nullptr ? 0.0f : Q::zp(zp[r * zs.s0 + c * zs.s1]);
        y[r * ldy + c]  = Q::template quant<In>(to_f32<In>(x[r * ldx + c]), s, z);
    }
}

static int grid_for(int64_t work_items, int threads)
{
    const int64_t blocks = ceil_div(work_items, threads);
    const int64_t cap    = static_cast<int64_t>(device_sm_count()) * 8;
    return static_cast<int>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

template <class In, class Q>
static int launch_quantize(const void* x, int64_t ldx, const void* scale, view2 ss, const void* zp,
                           view2 zs, void* y, int64_t ldy, int64_t rows, int64_t cols,
                           cudaStream_t stream)
{
    using Out         = typename Q::type;
    constexpr int VEC = 16 / sizeof(In);
    const bool vec    = cols % VEC == 0 and ldx % VEC == 0 and ldy % VEC == 0 and
                     (reinterpret_cast<uintptr_t>(x) % 16) == 0 and
                     (reinterpret_cast<uintptr_t>(y) % VEC) == 0;
    if(vec)
    {
        const int64_t n    = rows * (cols / VEC);
        const bool uniform = ss.s0 == 0 and ss.s1 == 0 and (zp == nullptr or (zs.s0 == 0 and zs.s1 == 0));
        const bool small   = n < (int64_t{1} << 31) and rows * ldx < (int64_t{1} << 31);
        const int grid     = grid_for(n, 256);
#define MGX_LAUNCH_QV(IDX, UNI)                                                                  \
    quantize_vec_kernel<In, Q, IDX, UNI><<<grid, 256, 0, stream>>>(                              \
        static_cast<const In*>(x), ldx, static_cast<const In*>(scale), ss,                       \
        static_cast<const Out*>(zp), zs, static_cast<Out*>(y), ldy, static_cast<IDX>(rows),      \
        static_cast<IDX>(cols / VEC))
        if constexpr(std::is_same<Q, q_i8>::value)
        {
            if(small and uniform)
            {
                cudaLaunchConfig_t cfg{};
                cfg.gridDim          = dim3(static_cast<unsigned>(grid));
                cfg.blockDim         = dim3(256);
                cfg.dynamicSmemBytes = 0;
                cfg.stream           = stream;
                cudaLaunchAttribute attr[1];
                attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
                attr[0].val.programmaticStreamSerializationAllowed = 1;
                cfg.attrs    = attr;
                cfg.numAttrs = 1;
                return static_cast<int>(cudaLaunchKernelEx(
                    &cfg, quantize_i8_uniform_kernel<In, uint32_t>, static_cast<const In*>(x), ldx,
                    static_cast<const In*>(scale), static_cast<const int8_t*>(zp),
                    static_cast<int8_t*>(y), ldy, static_cast<uint32_t>(rows),
                    static_cast<uint32_t>(cols / VEC)));
            }
        }
        if(small and uniform)
            MGX_LAUNCH_QV(uint32_t, true);
        else if(small)
            MGX_LAUNCH_QV(uint32_t, false);
        else if(uniform)
            MGX_LAUNCH_QV(int64_t, true);
        else
            MGX_LAUNCH_QV(int64_t, false);
#undef MGX_LAUNCH_QV
    }
    else
    {
        const int64_t n = rows * cols;
        quantize_scalar_kernel<In, Q><<<grid_for(n, 256), 256, 0, stream>>>(
            static_cast<const In*>(x), ldx, static_cast<const In*>(scale), ss,
            static_cast<const Out*>(zp), zs, static_cast<Out*>(y), ldy, rows, cols);
    }
    return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------ dequantize
template <class X>
__device__ __forceinline__ double x_to_double(X v)
{
    return static_cast<double>(v);
}
struct fp8_bits
{
    uint8_t b;
};
template <>
__device__ __forceinline__ double x_to_double<fp8_bits>(fp8_bits v)
{
    return static_cast<double>(__half2float(__half(__nv_cvt_fp8_to_halfraw(v.b, __NV_E4M3))));
}

template <class X, class S>
__global__ void __launch_bounds__(256)
    dequantize_kernel(const X* __restrict__ x, int64_t ldx, const S* __restrict__ scale, view2 ss,
                      const X* __restrict__ zp, view2 zs, S* __restrict__ y, int64_t ldy,
                      int64_t rows, int64_t cols)
{
    const int64_t total = rows * cols;
    for(int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
        i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        const int64_t r = i / cols;
        const int64_t c = i - r * cols;
        const double xv = x_to_double<X>(x[r * ldx + c]);
        const double zv = zp == nullptr ? 0.0 : x_to_double<X>(zp[r * zs.s0 + c * zs.s1]);
        const double sv = static_cast<double>(to_f32<S>(scale[r * ss.s0 + c * ss.s1]));
        const double d  = (xv - zv) * sv;
        if constexpr(std::is_same<S, float>::value)
            y[r * ldy + c] = static_cast<float>(d);
        else
            // double -> float (nearest) -> half (toward zero), as migraphx::half converts
            y[r * ldy + c] = __float2half_rz(static_cast<float>(d));
    }
}

template <class X>
static int launch_dequantize(const void* x, int64_t ldx, const void* scale, int scale_type,
                             view2 ss, const void* zp, view2 zs, void* y, int64_t ldy,
                             int64_t rows, int64_t cols, cudaStream_t stream)
{
    const int64_t n = rows * cols;
    if(scale_type == MGX_F32)
        dequantize_kernel<X, float><<<grid_for(n, 256), 256, 0, stream>>>(
            static_cast<const X*>(x), ldx, static_cast<const float*>(scale), ss,
            static_cast<const X*>(zp), zs, static_cast<float*>(y), ldy, rows, cols);
    else if(scale_type == MGX_F16)
        dequantize_kernel<X, __half><<<grid_for(n, 256), 256, 0, stream>>>(
            static_cast<const X*>(x), ldx, static_cast<const __half*>(scale), ss,
            static_cast<const X*>(zp), zs, static_cast<__half*>(y), ldy, rows, cols);
    else
        return MGX_E_UNSUPPORTED;
    return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------ int4 pack/unpack
template <bool SIGNED>
__global__ void __launch_bounds__(256)
    unpack_int4_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int64_t n)
{
    for(int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
        i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        const uint8_t b = in[i];
        uint8_t lo = b & 0xF, hi = b >> 4;
        if(SIGNED)
        {
            lo = static_cast<uint8_t>(static_cast<int8_t>(b << 4) >> 4);
            hi = static_cast<uint8_t>(static_cast<int8_t>(b) >> 4);
        }
        *reinterpret_cast<uchar2*>(out + 2 * i) = make_uchar2(lo, hi);
    }
}

template <bool SIGNED>
__global__ void __launch_bounds__(256)
    pack_int4_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int64_t n)
{
    for(int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
        i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        const uchar2 v = *reinterpret_cast<const uchar2*>(in + 2 * i);
        uint8_t a, b;
        if(SIGNED)
        {
            const int x0 = max(-8, min(7, static_cast<int>(static_cast<int8_t>(v.x))));
            const int x1 = max(-8, min(7, static_cast<int>(static_cast<int8_t>(v.y))));
            a = static_cast<uint8_t>(x0), b = static_cast<uint8_t>(x1);
        }
        else
        {
            a = min(v.x, static_cast<uint8_t>(15));
            b = min(v.y, static_cast<uint8_t>(15));
        }
        out[i] = static_cast<uint8_t>((b << 4) | (a & 0xF));
    }
}

// ------------------------------------------------------------ 8-bit transpose
// 64 x 64 byte tile through shared memory; both the global reads (rows of src)
// and the global writes (rows of dst) are 4-byte per thread, 64 B per 16 lanes.
__global__ void __launch_bounds__(256)
    transpose_8bit_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows,
                          int64_t cols, int64_t ld_dst)
{
    __shared__ uint8_t tile[64][64 + 4];
    const int64_t b  = blockIdx.z;
    const uint8_t* s = src + b * rows * cols;
    uint8_t* d       = dst + b * cols * ld_dst;
    const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 64;
    const int64_t c0 = static_cast<int64_t>(blockIdx.x) * 64;
    const int tx     = threadIdx.x & 15; // 16 threads x 4 bytes = 64 columns
    const int ty     = threadIdx.x >> 4; // 16 row slots
    const bool fast_in = (cols % 4 == 0) and ((reinterpret_cast<uintptr_t>(s) & 3u) == 0);
#pragma unroll
    for(int i = 0; i < 4; ++i)
    {
        const int rr    = ty + i * 16;
        const int64_t r = r0 + rr;
        const int64_t c = c0 + tx * 4;
        uint32_t v      = 0;
        if(r < rows)
        {
            if(fast_in and c + 4 <= cols)
                v = *reinterpret_cast<const uint32_t*>(s + r * cols + c);
            else
                for(int j = 0; j < 4; ++j)
                    if(c + j < cols)
                        v |= static_cast<uint32_t>(s[r * cols + c + j]) << (8 * j);
        }
#pragma unroll
        for(int j = 0; j < 4; ++j)
            tile[rr][tx * 4 + j] = static_cast<uint8_t>(v >> (8 * j));
    }
    __syncthreads();
    const bool fast_out = (ld_dst % 4 == 0) and ((reinterpret_cast<uintptr_t>(d) & 3u) == 0);
#pragma unroll
    for(int i = 0; i < 4; ++i)
    {
        const int cc    = ty + i * 16; // column of src = row of dst
        const int64_t c = c0 + cc;
        const int64_t r = r0 + tx * 4;
        if(c >= cols)
            continue;
        uint32_t v = 0;
#pragma unroll
        for(int j = 0; j < 4; ++j)
            v |= static_cast<uint32_t>(tile[tx * 4 + j][cc]) << (8 * j);
        if(fast_out and r + 4 <= rows)
            *reinterpret_cast<uint32_t*>(d + c * ld_dst + r) = v;
        else
            for(int j = 0; j < 4; ++j)
                if(r + j < rows)
                    d[c * ld_dst + r + j] = static_cast<uint8_t>(v >> (8 * j));
    }
}

int transpose_8bit_ld(const void* src, void* dst, int64_t rows, int64_t cols, int64_t batch,
                      int64_t ld_dst, cudaStream_t stream)
{
    if(src == nullptr or dst == nullptr or rows <= 0 or cols <= 0 or batch <= 0 or ld_dst < rows)
        return MGX_E_INVALID_ARG;
    const int64_t gx = ceil_div(cols, 64), gy = ceil_div(rows, 64);
    if(gy > 65535 or batch > 65535)
        return MGX_E_TOO_LARGE;
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(batch));
    transpose_8bit_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(src),
                                                    static_cast<uint8_t*>(dst), rows, cols, ld_dst);
    return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------ 16-bit transpose
// 32 x 32 tile of 16-bit elements through shared memory (the [K,N] operand of an fp16 dot
// re-laid out K-contiguous); rows of dst beyond `rows` up to ld_dst are not written.
__global__ void __launch_bounds__(256)
    transpose_16bit_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, int64_t rows,
                           int64_t cols, int64_t ld_dst)
{
    __shared__ uint16_t tile[32][32 + 2];
    const int64_t b   = blockIdx.z;
    const uint16_t* s = src + b * rows * cols;
    uint16_t* d       = dst + b * cols * ld_dst;
    const int64_t r0  = static_cast<int64_t>(blockIdx.y) * 32;
    const int64_t c0  = static_cast<int64_t>(blockIdx.x) * 32;
    const int tx      = threadIdx.x & 31;
    const int ty      = threadIdx.x >> 5; // 8 row slots
#pragma unroll
    for(int i = 0; i < 4; ++i)
    {
        const int rr    = ty + i * 8;
        const int64_t r = r0 + rr, c = c0 + tx;
        tile[rr][tx]    = (r < rows and c < cols) ? s[r * cols + c] : uint16_t{0};
    }
    __syncthreads();
#pragma unroll
    for(int i = 0; i < 4; ++i)
    {
        const int cc    = ty + i * 8; // column of src = row of dst
        const int64_t c = c0 + cc, r = r0 + tx;
        if(c < cols and r < rows)
            d[c * ld_dst + r] = tile[tx][cc];
    }
}

int transpose_16bit_ld(const void* src, void* dst, int64_t rows, int64_t cols, int64_t batch,
                       int64_t ld_dst, cudaStream_t stream)
{
    if(src == nullptr or dst == nullptr or rows <= 0 or cols <= 0 or batch <= 0 or ld_dst < rows)
        return MGX_E_INVALID_ARG;
    const int64_t gx = ceil_div(cols, 32), gy = ceil_div(rows, 32);
    if(gy > 65535 or batch > 65535)
        return MGX_E_TOO_LARGE;
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(batch));
    transpose_16bit_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(src),
                                                     static_cast<uint16_t*>(dst), rows, cols, ld_dst);
    return static_cast<int>(cudaGetLastError());
}

} // namespace mgx

using namespace mgx;

extern "C" int mgx_cuda_quantizelinear(const void* x, int x_type, int64_t ldx, const void* scale,
                                       const int64_t scale_strides[2], const void* zp,
                                       const int64_t zp_strides[2], void* y, int y_type,
                                       int64_t ldy, int64_t rows, int64_t cols, void* stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if(rows < 0 or cols < 0)
        return MGX_E_INVALID_ARG;
    if(rows == 0 or cols == 0)
        return MGX_OK; // empty tensors may come with null pointers
    if(x == nullptr or scale == nullptr or y == nullptr or scale_strides == nullptr)
        return MGX_E_INVALID_ARG;
    if(ldx < cols or ldy < cols)
        return MGX_E_INVALID_ARG;
    if(zp != nullptr and zp_strides == nullptr)
        return MGX_E_INVALID_ARG;
    const view2 ss{scale_strides[0], scale_strides[1]};
    const view2 zs = zp != nullptr ? view2{zp_strides[0], zp_strides[1]} : view2{0, 0};
#define MGX_Q_CASE(IN, Q) return launch_quantize<IN, Q>(x, ldx, scale, ss, zp, zs, y, ldy, rows, cols, stream)
    if(x_type == MGX_F32)
    {
        if(y_type == MGX_I8)
            MGX_Q_CASE(float, q_i8);
        if(y_type == MGX_U8)
            MGX_Q_CASE(float, q_u8);
        if(y_type == MGX_FP8_E4M3FN)
            MGX_Q_CASE(float, q_fp8);
    }
    else if(x_type == MGX_F16)
    {
        if(y_type == MGX_I8)
            MGX_Q_CASE(__half, q_i8);
        if(y_type == MGX_U8)
            MGX_Q_CASE(__half, q_u8);
        if(y_type == MGX_FP8_E4M3FN)
            MGX_Q_CASE(__half, q_fp8);
    }
#undef MGX_Q_CASE
    return MGX_E_UNSUPPORTED;
}

extern "C" int mgx_cuda_dequantizelinear(const void* x, int x_type, int64_t ldx, const void* scale,
                                         int scale_type, const int64_t scale_strides[2],
                                         const void* zp, const int64_t zp_strides[2], void* y,
                                         int64_t ldy, int64_t rows, int64_t cols, void* stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if(rows < 0 or cols < 0)
        return MGX_E_INVALID_ARG;
    if(rows == 0 or cols == 0)
        return MGX_OK; // empty tensors may come with null pointers
    if(x == nullptr or scale == nullptr or y == nullptr or scale_strides == nullptr)
        return MGX_E_INVALID_ARG;
    if(ldx < cols or ldy < cols)
        return MGX_E_INVALID_ARG;
    if(zp != nullptr and zp_strides == nullptr)
        return MGX_E_INVALID_ARG;
    const view2 ss{scale_strides[0], scale_strides[1]};
    const view2 zs = zp != nullptr ? view2{zp_strides[0], zp_strides[1]} : view2{0, 0};
    switch(x_type)
    {
    case MGX_I8:
        return launch_dequantize<int8_t>(x, ldx, scale, scale_type, ss, zp, zs, y, ldy, rows, cols, stream);
    case MGX_U8:
        return launch_dequantize<uint8_t>(x, ldx, scale, scale_type, ss, zp, zs, y, ldy, rows, cols, stream);
    case MGX_I32:
        return launch_dequantize<int32_t>(x, ldx, scale, scale_type, ss, zp, zs, y, ldy, rows, cols, stream);
    case MGX_FP8_E4M3FN:
        return launch_dequantize<fp8_bits>(x, ldx, scale, scale_type, ss, zp, zs, y, ldy, rows, cols, stream);
    default: return MGX_E_UNSUPPORTED;
    }
}

extern "C" int mgx_cuda_unpack_int4(const void* in, void* out, int type, int64_t rows,
                                    int64_t packed_cols, void* stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if(in == nullptr or out == nullptr or rows < 0 or packed_cols < 0)
        return MGX_E_INVALID_ARG;
    const int64_t n = rows * packed_cols;
    if(n == 0)
        return MGX_OK;
    if(reinterpret_cast<uintptr_t>(out) & 1u)
        return MGX_E_ALIGNMENT;
    if(type == MGX_U8)
        unpack_int4_kernel<false><<<grid_for(n, 256), 256, 0, stream>>>(
            static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), n);
    else if(type == MGX_I8)
        unpack_int4_kernel<true><<<grid_for(n, 256), 256, 0, stream>>>(
            static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), n);
    else
        return MGX_E_UNSUPPORTED;
    return static_cast<int>(cudaGetLastError());
}

extern "C" int mgx_cuda_pack_int4(const void* in, void* out, int type, int64_t rows,
                                  int64_t packed_cols, void* stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if(in == nullptr or out == nullptr or rows < 0 or packed_cols < 0)
        return MGX_E_INVALID_ARG;
    const int64_t n = rows * packed_cols;
    if(n == 0)
        return MGX_OK;
    if(reinterpret_cast<uintptr_t>(in) & 1u)
        return MGX_E_ALIGNMENT;
    if(type == MGX_U8)
        pack_int4_kernel<false><<<grid_for(n, 256), 256, 0, stream>>>(
            static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), n);
    else if(type == MGX_I8)
        pack_int4_kernel<true><<<grid_for(n, 256), 256, 0, stream>>>(
            static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), n);
    else
        return MGX_E_UNSUPPORTED;
    return static_cast<int>(cudaGetLastError());
}

extern "C" int mgx_cuda_transpose_8bit(const void* src, void* dst, int64_t rows, int64_t cols,
                                       int64_t batch, void* stream_)
{
    return transpose_8bit_ld(src, dst, rows, cols, batch, rows, static_cast<cudaStream_t>(stream_));
}
