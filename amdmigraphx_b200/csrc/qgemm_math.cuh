// Element-wise arithmetic of the quant_dot epilogues (shared by the tiled GEMM and the
// skinny-M kernel): exact dequantisation of int32 accumulators, activations, the truncating
// float -> half conversion of the reference, all without the conversion pipe where possible.
#pragma once
#include "common.cuh"
#include <cuda_fp16.h>

namespace mgx {

// erf by Abramowitz & Stegun 7.1.26 (|error| <= 1.5e-7 + fp32 rounding): one reciprocal,
// one exponential, five fused multiply-adds.  GELU uses erf only through 1 + erf(.), so
// an absolute error of this size is below fp32 resolution of the result.
__device__ __forceinline__ float fast_erf(float x)
{
    const float ax = fabsf(x);
    // the reciprocal's operand is >= 1 and an exponential below 2^-126 may flush to zero (the
    // result is then exactly 1, as it rounds to anyway): the flush-to-zero forms are single
    // instructions, the default forms carry extra range handling
    float t;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, ax, 1.0f)));
    float y        = fmaf(1.061405429f, t, -1.453152027f);
    y              = fmaf(y, t, 1.421413741f);
    y              = fmaf(y, t, -0.284496736f);
    y              = fmaf(y, t, 0.254829592f);
    y *= t;
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(ax * ax * -1.4426950408889634f));
    const float r = fmaf(-y, e, 1.0f);
    return copysignf(r, x);
}

template <int ACT>
__device__ __forceinline__ float apply_act(float v)
{
    if constexpr(ACT == MGX_ACT_RELU)
        return fmaxf(v, 0.0f);
    else if constexpr(ACT == MGX_ACT_GELU_ERF)
        // (x*0.5) * (erf(x / sqrt(2)) + 1): operation order of src/op/builder/gelu.cpp:58-74
        return __fmul_rn(__fmul_rn(v, 0.5f), __fadd_rn(fast_erf(v * 0.70710678118654752440f), 1.0f));
    else if constexpr(ACT == MGX_ACT_GELU_TANH)
    {
        float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
        return 0.5f * v * (1.0f + tanhf(u));
    }
    else if constexpr(ACT == MGX_ACT_SILU)
        return v / (1.0f + __expf(-v));
    else
        return v;
}

// Conversions (int <-> float, float <-> half, rounding to integer) issue on a pipe with an
// eighth of the fp32 rate on this GPU; the epilogue handles 32 K values per tile, so they are
// replaced by exact integer / fp32-add tricks wherever the value range allows.
//
// float(acc), exact, for |acc| < 2^22: 0x4B400000 is 1.5 * 2^23, whose ulp is 1.
__device__ __forceinline__ float int_to_float_small(int32_t acc)
{
    return __int_as_float(0x4B400000 + acc) - 12582912.0f;
}

__device__ __forceinline__ bool fits_small(int32_t a)
{
    return static_cast<uint32_t>(a + (1 << 22)) < (1u << 23);
}

// float(double(acc) * double(s)) without fp64 instructions.  For |acc| < 2^24 the
// conversion is exact and one fp32 multiply rounds exactly like the reference's
// double product.  Larger accumulators are split into an exactly representable high
// part and a small remainder, and the product is summed with error compensation.
__device__ __forceinline__ float dequant_i32(int32_t acc, float s)
{
    if(fits_small(acc))
        return __fmul_rn(int_to_float_small(acc), s);
    const float a = __int2float_rn(acc);
    float x       = __fmul_rn(a, s);
    if(acc >= (1 << 24) or acc <= -(1 << 24))
    {
        const float lo = __int2float_rn(acc - __float2int_rn(a));
        const float e  = __fmaf_rn(a, s, -x);
        x              = __fadd_rn(x, __fmaf_rn(lo, s, e));
    }
    return x;
}

// float(half_rz(v)): fp32 value with the mantissa cut to fp16's 10 bits.  Exact for
// 2^-14 <= |v| < 65536 and for zero; the rare values in fp16's subnormal range (or beyond
// its maximum) take the real conversion.
__device__ __forceinline__ float truncate_to_half_precision(float v)
{
    const float av = fabsf(v);
    if(v == 0.0f or (av >= 6.103515625e-5f and av < 65536.0f))
        return __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    return __half2float(__float2half_rz(v));
}

} // namespace mgx
