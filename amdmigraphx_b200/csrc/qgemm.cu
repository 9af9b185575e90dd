// quant_dot for sm_100a: int8 x int8 -> int32 and fp8(e4m3fn) x fp8 -> fp32 as a
// persistent, warp-specialised, TMA-fed tcgen05 GEMM with the accumulator in
// tensor memory and dequantizelinear / bias / activation / residual fused into
// the epilogue.
//
// Arithmetic contract (MIGraphX `ref` target): src/targets/ref/lowering.cpp:205-249
// -> gemm_naive (src/gemm.cpp:43-63): int8 products summed exactly, stored as
// int32; fp8 products summed in (at least) fp32, stored as fp32.  The fused
// epilogue reproduces dequantizelinear (src/include/migraphx/op/dequantizelinear.hpp:74-77:
// double(x) * scale, one rounding to fp32), then add, then the activation, each
// as a separate fp32 operation like the un-fused instructions.
//
// CTA = 576 threads: warp 0 = TMA producer (one lane), warp 1 = tensor-memory
// owner + MMA issuer (one lane), warps 2..17 = epilogue (each owns the TMEM lane
// quarter warp_id % 4 and a quarter of the tile's columns).  Two accumulator buffers of BN columns let the epilogue
// of tile i overlap the main loop of tile i+1.
#include "common.cuh"
#include <cstdlib>
#include "ptx.cuh"
#include "qgemm_math.cuh"
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <mutex>

namespace mgx {

constexpr int BM        = 128; // rows of D per tile (UMMA M, one TMEM lane per row)
constexpr int BK        = 128; // bytes (= 8-bit elements) of K per pipeline stage
constexpr int UMMA_K    = 32;  // K per tcgen05.mma for 8-bit operands
constexpr int EPI_WARPS = 16;  // four per TMEM lane quarter, each takes a quarter of the columns
constexpr int NTHREADS  = 64 + 32 * EPI_WARPS;
constexpr int EPI_COLS  = 16;  // columns per epilogue chunk (one tcgen05.ld.32x32b.x16)

struct qgemm_params
{
    int64_t M, N, K, batch;
    int64_t ldd, stride_d;
    void* D;
    const float* scale;
    const float* bias;
    const void* residual;
    int tiles_m, tiles_n;
    int64_t num_tiles;
    int num_kb;
    int scale_mode;
    int act;
    void* Dq;          // optional second output: quantizelinear(D) as int8 / fp8 (may be the only one)
    int64_t ldq, stride_q;
    float q_scale;     // per-tensor scale of that quantizelinear, already in D's type
    float q_zp;
    float q_rcp;       // 1 / q_scale refined to full precision
    int q_fp8;         // 0: int8, 1: fp8 e4m3fn
    int write_d;       // D itself is wanted
    int vec_sb; // scale / bias vectors are 16-byte aligned (float4 loads allowed)
    int fast;   // the whole problem takes the epilogue's check-free path (see epi_store_chunk_fast)
    int acc24;  // every accumulator is below 2^24 in magnitude (int8 operands, K < 1024)
    int q_mask; // the fused quantizelinear may take the mantissa-cut value (see launch_qgemm)
    int vec_io; // D (and residual) rows can be accessed with 16-byte (fp32/int32) / 8-byte (fp16) vectors
    // fp16 results whose epilogue operators run in half (MGX_QGEMM_HALF_MATH): 0xFFFFE000, the
    // mantissa cut that truncates an fp32 value in the normal half range to half; else all ones
    uint32_t hmask;
    const uint8_t* lut; // activation + quantizelinear of every half as a table (MGX_QOUT_LUT), or null
    float act_rcp; // erf-GELU: 1 / the constant x is divided by (sqrt 2, or its half value)
};

// v with the mantissa cut by mask (see qgemm_params::hmask); values in the half subnormal range
// keep up to 2^-24 too much, which no later step can see
__device__ __forceinline__ float hcut(float v, uint32_t mask)
{
    return __uint_as_float(__float_as_uint(v) & mask);
}

// the activation with every step rounded by hcut (all ones: the fp32 operator chain)
template <int ACT>
__device__ __forceinline__ float apply_act_cut(float v, uint32_t mask, float act_rcp)
{
    if constexpr(ACT == MGX_ACT_GELU_ERF)
    {
        // (x * 0.5) * (erf(x / c) + 1), operation order of src/op/builder/gelu.cpp:58-74; x * 0.5 is exact
        const float dv = hcut(v * act_rcp, mask);
        const float e1 = hcut(__fadd_rn(hcut(fast_erf(dv), mask), 1.0f), mask);
        return hcut(__fmul_rn(__fmul_rn(v, 0.5f), e1), mask);
    }
    else
        return apply_act<ACT>(v);
}

template <int BN>
struct qgemm_smem
{
    static constexpr int a_bytes     = BM * BK;
    static constexpr int b_bytes     = BN * BK;
    static constexpr int stage_bytes = a_bytes + b_bytes;
    static constexpr int stages      = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 8);
    static constexpr int epi_bytes   = EPI_WARPS * 32 * EPI_COLS * 4; // 32 rows x 16 words per warp
    static constexpr int bar_bytes   = 256;
    static constexpr int total = stages * stage_bytes + epi_bytes + bar_bytes + 1024; // + alignment slack
};

struct epi_ctx
{
    const qgemm_params* p;
    uint8_t* box;      // this warp's 32 x 64-byte staging area (16-byte pieces XOR-swizzled by row)
    int lane;
    int64_t row0;      // global row of staging row 0
    int64_t batch_off; // b * stride_d
    int64_t batch_off_q; // b * stride_q
};

// Second half of the epilogue for one 16-column chunk: read the raw accumulators back
// from shared memory so that 4 consecutive lanes cover one 64-byte row segment, apply
// dequantizelinear / bias / activation / residual, convert and store coalesced.
template <bool IS_INT, class OutT, int ACT>
__device__ __forceinline__ void epi_store_chunk(const epi_ctx& e, int64_t col, float4 sc4, float4 bi4)
{
    const qgemm_params& p = *e.p;
    const int pc          = e.lane & 3;  // which 4-column piece of the chunk this lane owns
    const int rsub        = e.lane >> 2; // row within a group of 8
    const int64_t c4      = col + pc * 4;
    const float sc[4]     = {sc4.x, sc4.y, sc4.z, sc4.w};
    const float bi[4]     = {bi4.x, bi4.y, bi4.z, bi4.w};
    const bool full       = p.vec_io and c4 + 4 <= p.N;
    const bool has_bias   = p.bias != nullptr;
#pragma unroll 1
    for(int it = 0; it < 4; ++it)
    {
        const int r       = it * 8 + rsub;
        const int64_t row = e.row0 + r;
        const uint4 w =
            *reinterpret_cast<const uint4*>(e.box + r * 64 + ((pc ^ ((r >> 1) & 3)) * 16));
        if(row >= p.M or c4 >= p.N)
            continue;
        const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
        OutT* dst = static_cast<OutT*>(p.D) + e.batch_off + row * p.ldd + c4;
        if constexpr(std::is_same<OutT, int32_t>::value)
        {
            if(full)
                *reinterpret_cast<uint4*>(dst) = w;
            else
                for(int j = 0; j < 4 and c4 + j < p.N; ++j)
                    dst[j] = static_cast<int32_t>(wv[j]);
        }
        else
        {
            float v[4];
            float rs = 1.0f;
            if(p.scale_mode == MGX_SCALE_PER_ROW)
                rs = __ldg(p.scale + row);
#pragma unroll
            for(int j = 0; j < 4; ++j)
            {
                float x;
                const float s = p.scale_mode == MGX_SCALE_PER_ROW ? rs : sc[j];
                if constexpr(IS_INT)
                {
                    const int32_t a = static_cast<int32_t>(wv[j]);
                    x = p.scale_mode == MGX_SCALE_NONE ? (fits_small(a) ? int_to_float_small(a) : __int2float_rn(a)) : dequant_i32(a, s);
                }
                else
                {
                    x = __uint_as_float(wv[j]);
                    if(p.scale_mode != MGX_SCALE_NONE)
                        x = __fmul_rn(x, s);
                }
                if constexpr(std::is_same<OutT, __half>::value)
                {
                    x = hcut(x, p.hmask);
                    if(has_bias)
                        x = hcut(__fadd_rn(x, bi[j]), p.hmask);
                    v[j] = apply_act_cut<ACT>(x, p.hmask, p.act_rcp);
                }
                else
                {
                    if(has_bias)
                        x = __fadd_rn(x, bi[j]);
                    v[j] = apply_act<ACT>(x);
                }
            }
            if(p.residual != nullptr)
            {
                const OutT* res =
                    static_cast<const OutT*>(p.residual) + e.batch_off + row * p.ldd + c4;
                float q[4] = {0.f, 0.f, 0.f, 0.f};
                if(full)
                {
                    if constexpr(std::is_same<OutT, float>::value)
                    {
                        const float4 t = *reinterpret_cast<const float4*>(res);
                        q[0] = t.x, q[1] = t.y, q[2] = t.z, q[3] = t.w;
                    }
                    else
                    {
                        const uint2 t    = *reinterpret_cast<const uint2*>(res);
                        const __half* th = reinterpret_cast<const __half*>(&t);
#pragma unroll
                        for(int j = 0; j < 4; ++j)
                            q[j] = __half2float(th[j]);
                    }
                }
                else
                {
                    for(int j = 0; j < 4 and c4 + j < p.N; ++j)
                    {
                        if constexpr(std::is_same<OutT, float>::value)
                            q[j] = res[j];
                        else
                            q[j] = __half2float(res[j]);
                    }
                }
#pragma unroll
                for(int j = 0; j < 4; ++j)
                {
                    // fp16 model: the reference converts to half by truncating the mantissa
                    // (src/include/migraphx/generic_float.hpp:180-230) before the half add
                    if constexpr(std::is_same<OutT, __half>::value)
                        v[j] = truncate_to_half_precision(v[j]);
                    v[j] = __fadd_rn(v[j], q[j]);
                }
            }
            if constexpr(std::is_same<OutT, __half>::value)
            {
                // the stored value is the truncated half; a fused quantizelinear sees that value
                if(p.Dq != nullptr)
                {
#pragma unroll
                    for(int j = 0; j < 4; ++j)
                        v[j] = truncate_to_half_precision(v[j]);
                }
            }
            if(p.write_d)
            {
                if constexpr(std::is_same<OutT, float>::value)
                {
                    if(full)
                        *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                    else
                        for(int j = 0; j < 4 and c4 + j < p.N; ++j)
                            dst[j] = v[j];
                }
                else
                {
                    if(full)
                        *reinterpret_cast<uint2*>(dst) =
                            make_uint2(cvt_rz_f16x2(v[0], v[1]), cvt_rz_f16x2(v[2], v[3]));
                    else
                        for(int j = 0; j < 4 and c4 + j < p.N; ++j)
                            dst[j] = __float2half_rz(v[j]);
                }
            }
            if(p.Dq != nullptr)
            {
                // quantizelinear of the value just produced (per-tensor scale and zero point):
                // x / s in D's type (fp16: fp32 quotient truncated to half, as migraphx::half
                // divides), round half to even, + zero point, saturate
                uint32_t packed = 0;
#pragma unroll
                for(int j = 0; j < 4; ++j)
                {
                    // correctly rounded v / s from the reciprocal computed once per kernel
                    // (one refinement of the quotient, as the division routine does)
                    float qv        = __fmul_rn(v[j], p.q_rcp);
                    const float rem = __fmaf_rn(-p.q_scale, qv, v[j]);
                    qv              = __fmaf_rn(rem, p.q_rcp, qv);
                    uint32_t b;
                    if(p.q_fp8)
                    {
                        qv = fmaxf(-448.0f, fminf(448.0f, qv + p.q_zp));
                        b  = static_cast<uint32_t>(__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3));
                    }
                    else
                    {
                        if constexpr(std::is_same<OutT, __half>::value)
                            qv = __uint_as_float(__float_as_uint(qv) & 0xFFFFE000u); // half quotient, truncated
                        // saturate first (keeps the magic-number rounding in range), then round
                        // half to even by adding 1.5 * 2^23; the low mantissa bits are the integer
                        qv = fmaxf(-300.0f, fminf(300.0f, qv));
                        const float r = __fadd_rn(qv, 12582912.0f);
                        int qi        = __float_as_int(r) - 0x4B400000 + static_cast<int>(p.q_zp);
                        qi            = max(-128, min(127, qi));
                        b             = static_cast<uint32_t>(qi) & 0xFFu;
                    }
                    packed |= b << (8 * j);
                }
                uint8_t* qdst = static_cast<uint8_t*>(p.Dq) + e.batch_off_q + row * p.ldq + c4;
                if(c4 + 4 <= p.N and ((reinterpret_cast<uintptr_t>(qdst) & 3u) == 0))
                    *reinterpret_cast<uint32_t*>(qdst) = packed;
                else
                    for(int j = 0; j < 4 and c4 + j < p.N; ++j)
                        qdst[j] = static_cast<uint8_t>(packed >> (8 * j));
            }
        }
    }
}

// float(half_rz(v)) for |v| < 65536 without a conversion and without a branch: normal halves
// keep the top 10 mantissa bits; below 2^-14 a half is a multiple of 2^-24, and |v| + 0.5 rounded
// toward zero keeps exactly those bits (the spacing of fp32 in [0.5, 1) is 2^-24).
__device__ __forceinline__ float half_rz_in_range(float v)
{
    const float av    = fabsf(v);
    const float big   = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    const float small = copysignf(__fsub_rn(__fadd_rz(av, 0.5f), 0.5f), v);
    return av < 6.103515625e-5f ? small : big;
}

// Four values at once; the real conversion only when one of them is beyond the half range
// (or not a number).
__device__ __forceinline__ void truncate4_to_half_precision(float (&v)[4])
{
    const float hi = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    const float lo = fminf(fminf(fabsf(v[0]), fabsf(v[1])), fminf(fabsf(v[2]), fabsf(v[3])));
    if(hi < 65536.0f and lo >= 6.103515625e-5f)
    {
        // all four are normal halves (the common case): cut the mantissa
#pragma unroll
        for(int j = 0; j < 4; ++j)
            v[j] = __uint_as_float(__float_as_uint(v[j]) & 0xFFFFE000u);
    }
    else if(hi < 65536.0f)
    {
#pragma unroll
        for(int j = 0; j < 4; ++j)
            v[j] = half_rz_in_range(v[j]);
    }
    else
    {
#pragma unroll
        for(int j = 0; j < 4; ++j)
            v[j] = truncate_to_half_precision(v[j]);
    }
}

// The chunk's store phase when nothing needs checking: every row and column of every tile is in
// range, all accesses are vectors, the scale is per column or per tensor (already in sc4; 1.0 when
// there is none), bi4 is -0.0 without a bias (x + -0.0 == x for every x), an optional
// quantizelinear output is int8 with 4-byte aligned rows.  Same arithmetic as epi_store_chunk.
// MODE 1: residual / quantizelinear / D chosen by the launch's parameters; 2: D only;
// 3: residual, D and quantizelinear; 4: quantizelinear only; 8: residual and D (the combinations
// of an encoder layer's four GEMMs get branch-free loops of their own); 7: the table look-up.
template <bool IS_INT, class OutT, int ACT, int MODE>
__device__ __forceinline__ void epi_store_chunk_fast(const epi_ctx& e, int64_t col, float4 sc4, float4 bi4)
{
    const qgemm_params& p = *e.p;
    const int pc          = e.lane & 3;
    const int rsub        = e.lane >> 2;
    const float sc[4]     = {sc4.x, sc4.y, sc4.z, sc4.w};
    const float bi[4]     = {bi4.x, bi4.y, bi4.z, bi4.w};
    const int64_t off     = e.batch_off + (e.row0 + rsub) * p.ldd + col + pc * 4;
    OutT* dst             = static_cast<OutT*>(p.D) + off;
    const OutT* res       = static_cast<const OutT*>(p.residual) + off;
    uint8_t* qdst = static_cast<uint8_t*>(p.Dq) + e.batch_off_q + (e.row0 + rsub) * p.ldq + col + pc * 4;
    const int64_t dstep = 8 * p.ldd, qstep = 8 * p.ldq;
    // 5 = 2 and 6 = 4 with accumulators below 2^24 (and the mantissa-cut quantizelinear input)
    const bool has_res = MODE == 1 ? p.residual != nullptr : (MODE == 3 or MODE == 8);
    const bool has_q   = MODE == 1 ? p.Dq != nullptr : (MODE == 3 or MODE == 4 or MODE == 6 or MODE == 7);
    const bool wr      = MODE == 1 ? p.write_d != 0 : (MODE != 4 and MODE != 6 and MODE != 7);
    const bool acc24   = (MODE == 5 or MODE == 6) ? true : p.acc24 != 0;
    const bool q_mask  = MODE == 6 ? true : (has_q and p.q_mask != 0);
    // saturation before rounding: bounds are integers, so round-to-nearest stays inside
    const float q_lo = -128.0f - p.q_zp, q_hi = 127.0f - p.q_zp;
    const int q_bias = static_cast<int>(p.q_zp) - 0x4B400000;
    const uint32_t hmask = p.hmask;
    const uint8_t* box = e.box + rsub * 64;
#pragma unroll 2
    for(int it = 0; it < 4; ++it)
    {
        const int r   = it * 8 + rsub;
        const uint4 w = *reinterpret_cast<const uint4*>(box + it * 512 + ((pc ^ ((r >> 1) & 3)) * 16));
        const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
        float v[4];
        if constexpr(IS_INT)
        {
            // one uniform branch around all four values, so that only one variant is issued
            if(acc24)
            {
                // |acc| < 2^24: the conversion is exact and the one fp32 multiply rounds like the
                // reference's double product; no range test, no large-accumulator path
#pragma unroll
                for(int j = 0; j < 4; ++j)
                    v[j] = __fmul_rn(__int2float_rn(static_cast<int32_t>(wv[j])), sc[j]);
            }
            else
            {
#pragma unroll
                for(int j = 0; j < 4; ++j)
                    v[j] = dequant_i32(static_cast<int32_t>(wv[j]), sc[j]);
            }
        }
        else
        {
#pragma unroll
            for(int j = 0; j < 4; ++j)
                v[j] = __fmul_rn(__uint_as_float(wv[j]), sc[j]);
        }
        if constexpr(MODE == 7)
        {
            // the half the chain holds after dequantizelinear and bias (the packing conversion
            // truncates, subnormal halves included) indexes the table of activation + quantizelinear
            const uint32_t i01 = cvt_rz_f16x2(__fadd_rn(hcut(v[0], hmask), bi[0]), __fadd_rn(hcut(v[1], hmask), bi[1]));
            const uint32_t i23 = cvt_rz_f16x2(__fadd_rn(hcut(v[2], hmask), bi[2]), __fadd_rn(hcut(v[3], hmask), bi[3]));
            const uint32_t b0 = __ldg(p.lut + (i01 & 0xFFFFu)), b1 = __ldg(p.lut + (i01 >> 16));
            const uint32_t b2 = __ldg(p.lut + (i23 & 0xFFFFu)), b3 = __ldg(p.lut + (i23 >> 16));
            *reinterpret_cast<uint32_t*>(qdst) = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
            qdst += qstep;
            continue;
        }
        if constexpr(std::is_same<OutT, __half>::value)
        {
            // fp16 model: dequantised value, bias sum and the activation's steps each rounded to half
            // when the launch asks for it (hmask), plain fp32 operators otherwise
#pragma unroll
            for(int j = 0; j < 4; ++j)
                v[j] = apply_act_cut<ACT>(hcut(__fadd_rn(hcut(v[j], hmask), bi[j]), hmask), hmask, p.act_rcp);
        }
        else
        {
#pragma unroll
            for(int j = 0; j < 4; ++j)
                v[j] = apply_act<ACT>(__fadd_rn(v[j], bi[j]));
        }
        if(has_res)
        {
            float q[4];
            if constexpr(std::is_same<OutT, float>::value)
            {
                const float4 t = *reinterpret_cast<const float4*>(res);
                q[0] = t.x, q[1] = t.y, q[2] = t.z, q[3] = t.w;
            }
            else
            {
                const uint2 t    = *reinterpret_cast<const uint2*>(res);
                const __half* th = reinterpret_cast<const __half*>(&t);
#pragma unroll
                for(int j = 0; j < 4; ++j)
                    q[j] = __half2float(th[j]);
                truncate4_to_half_precision(v); // the half add works on the truncated half
            }
#pragma unroll
            for(int j = 0; j < 4; ++j)
                v[j] = __fadd_rn(v[j], q[j]);
        }
        if constexpr(std::is_same<OutT, __half>::value)
        {
            // quantizelinear sees the stored half
            if(q_mask)
            {
                // cutting the mantissa is enough: values in the half subnormal range quantise to
                // zero either way, values beyond the half range saturate either way, and the
                // store below truncates by itself
#pragma unroll
                for(int j = 0; j < 4; ++j)
                    v[j] = __uint_as_float(__float_as_uint(v[j]) & 0xFFFFE000u);
            }
            else if(has_q)
                truncate4_to_half_precision(v);
        }
        if(wr)
        {
            if constexpr(std::is_same<OutT, float>::value)
                *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            else
                *reinterpret_cast<uint2*>(dst) =
                    make_uint2(cvt_rz_f16x2(v[0], v[1]), cvt_rz_f16x2(v[2], v[3]));
        }
        if(has_q)
        {
            uint32_t b[4];
#pragma unroll
            for(int j = 0; j < 4; ++j)
            {
                float qv        = __fmul_rn(v[j], p.q_rcp);
                const float rem = __fmaf_rn(-p.q_scale, qv, v[j]);
                qv              = __fmaf_rn(rem, p.q_rcp, qv);
                if constexpr(std::is_same<OutT, __half>::value)
                    qv = __uint_as_float(__float_as_uint(qv) & 0xFFFFE000u); // half quotient, truncated
                qv   = fmaxf(q_lo, fminf(q_hi, qv));
                b[j] = static_cast<uint32_t>(__float_as_int(__fadd_rn(qv, 12582912.0f)) + q_bias);
            }
            *reinterpret_cast<uint32_t*>(qdst) =
                __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
        }
        dst += dstep;
        res += dstep;
        qdst += qstep;
    }
}

// The epilogue role, one instantiation per activation so that the code a warp executes is
// one contiguous region (the activation is chosen once per kernel, not per element).
// Each warp owns TMEM lane quarter (warp % 4) = 32 rows of the tile, and a quarter of the
// tile's columns.  Per 16-column chunk: tcgen05.ld (one row per thread) -> swizzled shared
// memory -> read back with 4 lanes per 64-byte row segment -> dequantizelinear / bias /
// activation / residual -> coalesced global stores.
template <int BN, bool IS_INT, class OutT, int ACT, int MODE>
__device__ __forceinline__ void epilogue_role(const qgemm_params& p, uint8_t* epi_base,
                                              uint64_t* accf_bar, uint64_t* acce_bar,
                                              volatile uint32_t* abort_flag, uint32_t tmem_base,
                                              int warp, int lane, int64_t first_tile,
                                              int64_t tile_step, int64_t tiles_mn)
{
    const int ew      = warp - 2;
    const int quarter = warp & 3;
    const int slice   = ew >> 2;
    constexpr int COLS_PER_WARP = BN / 4;
    constexpr int NCHUNK        = COLS_PER_WARP / EPI_COLS;
    epi_ctx e;
    e.p    = &p;
    e.box  = epi_base + ew * (32 * EPI_COLS * 4);
    e.lane = lane;
    uint8_t* my_row    = e.box + lane * 64;
    const int my_swz   = (lane >> 1) & 3;
    const bool per_col = p.scale_mode == MGX_SCALE_PER_COL;
    const float tensor_scale = p.scale_mode == MGX_SCALE_PER_TENSOR ? __ldg(p.scale) : 1.0f;
    uint32_t lt = 0;
    for(int64_t t = first_tile; t < p.num_tiles; t += tile_step, ++lt)
    {
        const int b     = static_cast<int>(t / tiles_mn);
        const int r     = static_cast<int>(t % tiles_mn);
        const int m_blk = r % p.tiles_m;
        const int n_blk = r / p.tiles_m;
        const uint32_t buf = lt & 1u;
        const int64_t col0 = static_cast<int64_t>(n_blk) * BN + slice * COLS_PER_WARP;
        e.row0      = static_cast<int64_t>(m_blk) * BM + quarter * 32;
        e.batch_off = b * p.stride_d;
        e.batch_off_q = b * p.stride_q;

        // this lane's 4 columns of a chunk: scale and bias.  The first chunk's are fetched
        // before the wait for the accumulator (latency hidden behind the main loop), the
        // next chunk's while the current one is processed.  The loops below are deliberately
        // not unrolled: a tile's epilogue runs only a few times per launch, so straight-line
        // code would be bound by instruction fetch.
        auto load_sb = [&](int ch, float4& sc, float4& bi) {
            sc = make_float4(tensor_scale, tensor_scale, tensor_scale, tensor_scale);
            bi = MODE != 0 ? make_float4(-0.f, -0.f, -0.f, -0.f) : make_float4(0.f, 0.f, 0.f, 0.f);
            if constexpr(not std::is_same<OutT, int32_t>::value)
            {
                const int64_t c4 = col0 + ch * EPI_COLS + (lane & 3) * 4;
                if(c4 + 4 <= p.N and p.vec_sb)
                {
                    if(per_col)
                        sc = __ldg(reinterpret_cast<const float4*>(p.scale + c4));
                    if(p.bias != nullptr)
                        bi = __ldg(reinterpret_cast<const float4*>(p.bias + c4));
                }
                else
                {
                    float* sp = reinterpret_cast<float*>(&sc);
                    float* bp = reinterpret_cast<float*>(&bi);
                    for(int j = 0; j < 4; ++j)
                    {
                        if(c4 + j < p.N)
                        {
                            if(per_col)
                                sp[j] = __ldg(p.scale + c4 + j);
                            if(p.bias != nullptr)
                                bp[j] = __ldg(p.bias + c4 + j);
                        }
                    }
                }
            }
        };
        // The residual is read inside the store loop; asking for its lines a chunk ahead turns
        // those reads into L1 hits (the loop is not unrolled, so their latency would be exposed).
        auto prefetch_res = [&](int ch) {
            if constexpr(not std::is_same<OutT, int32_t>::value)
            {
                const int64_t c4 = col0 + ch * EPI_COLS + (lane & 3) * 4;
                if(p.residual == nullptr or c4 >= p.N)
                    return;
#pragma unroll
                for(int it = 0; it < 4; ++it)
                {
                    const int64_t row = e.row0 + it * 8 + (lane >> 2);
                    if(row < p.M)
                        asm volatile("prefetch.global.L1 [%0];" ::"l"(
                            static_cast<const OutT*>(p.residual) + e.batch_off + row * p.ldd + c4));
                }
            }
        };
        float4 sc_next, bi_next;
        load_sb(0, sc_next, bi_next);
        prefetch_res(0);

        if(not mbar_wait_bounded(&accf_bar[buf], (lt >> 1) & 1u, abort_flag, 3))
            break;
        tc_fence_after_sync();

#pragma unroll 1
        for(int ch = 0; ch < NCHUNK; ++ch)
        {
            const int64_t col = col0 + ch * EPI_COLS;
            const float4 sc_cur = sc_next, bi_cur = bi_next;
            if(ch + 1 < NCHUNK)
            {
                load_sb(ch + 1, sc_next, bi_next);
                prefetch_res(ch + 1);
            }
            uint32_t acc[EPI_COLS];
            __syncwarp(); // tcgen05.ld is warp-collective; also orders reuse of the box
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   buf * BN + slice * COLS_PER_WARP + ch * EPI_COLS;
            tmem_ld_32x32b_x16(taddr, acc);
            tmem_ld_wait();
            if(col < p.N)
            {
#pragma unroll
                for(int q = 0; q < 4; ++q)
                    *reinterpret_cast<uint4*>(my_row + ((q ^ my_swz) * 16)) =
                        make_uint4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
                __syncwarp();
                if constexpr(MODE != 0 and not std::is_same<OutT, int32_t>::value)
                    epi_store_chunk_fast<IS_INT, OutT, ACT, MODE>(e, col, sc_cur, bi_cur);
                else
                    epi_store_chunk<IS_INT, OutT, ACT>(e, col, sc_cur, bi_cur);
            }
        }
        // all TMEM reads of this buffer are complete (wait::ld above)
        tc_fence_before_sync();
        __syncwarp();
        if(lane == 0)
            mbar_arrive(&acce_bar[buf]);
    }
}

// IS_INT: accumulator registers hold int32 (kind::i8) else fp32 bit patterns.
// OutT: int32_t (raw accumulator), float or __half.
// F16: the operands are fp16 (kind::f16, 64 elements of K per 128-byte stage row); the byte
// layout of the pipeline is the one of the 8-bit kinds.
template <int BN, bool IS_INT, class OutT, bool F16 = false>
__global__ void __launch_bounds__(NTHREADS, 1)
    qgemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b,
                 const qgemm_params p)
{
    using S = qgemm_smem<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem           = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);

    uint8_t* epi_base   = smem + S::stages * S::stage_bytes;
    uint8_t* bar_base   = epi_base + S::epi_bytes;
    uint64_t* full_bar  = reinterpret_cast<uint64_t*>(bar_base);
    uint64_t* empty_bar = full_bar + S::stages;
    uint64_t* accf_bar  = empty_bar + S::stages; // [2] accumulator ready
    uint64_t* acce_bar  = accf_bar + 2;          // [2] accumulator drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acce_bar + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    constexpr uint32_t TMEM_COLS = 2 * BN; // 128, 256 or 512: a power of two >= 32

    // the next kernel of the stream may set itself up while this one runs
    grid_launch_dependents();

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < S::stages; ++s)
        {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for(int b = 0; b < 2; ++b)
        {
            mbar_init(&accf_bar[b], 1);
            mbar_init(&acce_bar[b], EPI_WARPS); // one arrival per epilogue warp
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
    }
    if(warp == 1)
    {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t first_tile = blockIdx.x;
    const int64_t tile_step  = gridDim.x;
    const int64_t tiles_mn   = static_cast<int64_t>(p.tiles_m) * p.tiles_n;

    if(warp == 0)
    {
        // ---------------------------------------------------- TMA producer
        if(lane == 0)
        {
            // everything up to here overlapped the previous kernel of the stream; its results
            // (this kernel's operands) are complete after the wait
            grid_dependency_wait();
            uint32_t it = 0;
            bool ok     = true;
            for(int64_t t = first_tile; ok and t < p.num_tiles; t += tile_step)
            {
                const int b     = static_cast<int>(t / tiles_mn);
                const int r     = static_cast<int>(t % tiles_mn);
                const int m_blk = r % p.tiles_m;
                const int n_blk = r / p.tiles_m;
                for(int kb = 0; kb < p.num_kb; ++kb, ++it)
                {
                    const uint32_t s  = it % S::stages;
                    const uint32_t ph = (it / S::stages) & 1u;
                    if(not mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, 2))
                    {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + s * S::stage_bytes;
                    uint8_t* sb = sa + S::a_bytes;
                    mbar_expect_tx(&full_bar[s], S::stage_bytes);
                    tma_load_3d(sa, &tmap_a, &full_bar[s], kb * BK, m_blk * BM, b);
                    tma_load_3d(sb, &tmap_b, &full_bar[s], kb * BK, n_blk * BN, b);
                }
            }
        }
    }
    else if(warp == 1)
    {
        // ---------------------------------------------------- MMA issuer
        if(lane == 0)
        {
            constexpr uint32_t idesc = IS_INT ? make_idesc(2u, 1u, 1u, BM, BN)  // s32 += s8*s8
                                              : make_idesc(1u, 0u, 0u, BM, BN); // f32 += e4m3*e4m3 (f16*f16)
            // the operands arrive only after the previous kernel of the stream is done: the
            // bounded waits below must not count that time
            grid_dependency_wait();
            uint32_t it = 0;
            uint32_t lt = 0; // local tile counter
            bool ok     = true;
            for(int64_t t = first_tile; ok and t < p.num_tiles; t += tile_step, ++lt)
            {
                const uint32_t buf = lt & 1u;
                if(not mbar_wait_bounded(&acce_bar[buf], ((lt >> 1) & 1u) ^ 1u, abort_flag, 4))
                    break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for(int kb = 0; kb < p.num_kb; ++kb, ++it)
                {
                    const uint32_t s  = it % S::stages;
                    const uint32_t ph = (it / S::stages) & 1u;
                    if(not mbar_wait_bounded(&full_bar[s], ph, abort_flag, 1))
                    {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t sa    = smem_u32(smem + s * S::stage_bytes);
                    const uint64_t adesc = make_smem_desc_sw128(sa);
                    const uint64_t bdesc = make_smem_desc_sw128(sa + S::a_bytes);
#pragma unroll
                    for(int k = 0; k < BK / UMMA_K; ++k)
                    {
                        // advancing K inside the 128-byte swizzle row: +32 B on the start address
                        const uint64_t koff = static_cast<uint64_t>((k * UMMA_K) >> 4);
                        if constexpr(IS_INT)
                            mma_i8(d_tmem, adesc + koff, bdesc + koff, idesc, (kb | k) != 0);
                        else if constexpr(F16)
                            mma_f16(d_tmem, adesc + koff, bdesc + koff, idesc, (kb | k) != 0);
                        else
                            mma_f8(d_tmem, adesc + koff, bdesc + koff, idesc, (kb | k) != 0);
                    }
                    tc_commit(&empty_bar[s]); // stage reusable once these MMAs have read it
                }
                if(ok)
                    tc_commit(&accf_bar[buf]); // accumulator complete
            }
        }
    }
    else
    {
        // ---------------------------------------------------- epilogue
        // (reads residual / scale / bias and writes D: only after the previous kernel is done)
        grid_dependency_wait();
        // the check-free variant is chosen once per launch: the tile loop a warp runs holds
        // only the store path it takes
#define MGX_EPI_MODE(ACT, MODE)                                                                           \
    epilogue_role<BN, IS_INT, OutT, ACT, MODE>(p, epi_base, accf_bar, acce_bar, abort_flag, tmem_base, warp, \
                                               lane, first_tile, tile_step, tiles_mn)
#define MGX_EPILOGUE(ACT)                    \
    switch(mode)                             \
    {                                        \
    case 0: MGX_EPI_MODE(ACT, 0); break;     \
    case 2: MGX_EPI_MODE(ACT, 2); break;     \
    case 3: MGX_EPI_MODE(ACT, 3); break;     \
    case 4: MGX_EPI_MODE(ACT, 4); break;     \
    case 5: MGX_EPI_MODE(ACT, 5); break;     \
    case 6: MGX_EPI_MODE(ACT, 6); break;     \
    case 8: MGX_EPI_MODE(ACT, 8); break;     \
    default: MGX_EPI_MODE(ACT, 1); break;    \
    }
        const bool m_res = p.residual != nullptr, m_q = p.Dq != nullptr, m_wr = p.write_d != 0;
        const bool m_24  = IS_INT and p.acc24 != 0;
        const int mode   = p.fast == 0 ? 0
                           : (not m_res and not m_q and m_wr) ? (m_24 ? 5 : 2)
                           : (m_res and m_q and m_wr)         ? 3
                           : (m_res and not m_q and m_wr)     ? 8
                           : (not m_res and m_q and not m_wr) ? ((m_24 and p.q_mask != 0) ? 6 : 4)
                                                              : 1;
        if(std::is_same<OutT, __half>::value and p.lut != nullptr and p.fast != 0 and not m_res and m_q and not m_wr)
        {
            if constexpr(std::is_same<OutT, __half>::value)
                MGX_EPI_MODE(MGX_ACT_NONE, 7);
        }
        else
        switch(std::is_same<OutT, int32_t>::value ? MGX_ACT_NONE : p.act)
        {
        case MGX_ACT_RELU: MGX_EPILOGUE(MGX_ACT_RELU); break;
        case MGX_ACT_GELU_ERF: MGX_EPILOGUE(MGX_ACT_GELU_ERF); break;
        case MGX_ACT_GELU_TANH: MGX_EPILOGUE(MGX_ACT_GELU_TANH); break;
        case MGX_ACT_SILU: MGX_EPILOGUE(MGX_ACT_SILU); break;
        default: MGX_EPILOGUE(MGX_ACT_NONE); break;
        }
#undef MGX_EPILOGUE
#undef MGX_EPI_MODE
    }

    // ---------------------------------------------------------- teardown
    if(*abort_flag != 0)
    {
        // give copies that may still be in flight time to land before the CTA's
        // shared memory is released
        for(int i = 0; i < 1000; ++i)
            __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if(warp == 1)
    {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------ host
struct qout_args
{
    void* Dq        = nullptr;
    int64_t ldq     = 0;
    int64_t stride_q = 0;
    float scale     = 1.0f;
    float zp        = 0.0f;
    int fp8         = 0;
    int write_d     = 1;
    const void* lut = nullptr;
};

static int encode_operand_map(CUtensorMap* map, const void* base, int64_t k, int64_t rows,
                              int64_t batch, int64_t ld, int64_t batch_stride, int box_rows)
{
    cuTensorMapEncodeTiled_t encode = get_tensor_map_encoder();
    if(encode == nullptr)
        return MGX_E_DRIVER;
    cuuint64_t dims[3]    = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows),
                             static_cast<cuuint64_t>(batch)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld),
                             static_cast<cuuint64_t>(batch > 1 ? batch_stride : ld * rows)};
    cuuint32_t box[3]     = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows), 1u};
    cuuint32_t estr[3]    = {1u, 1u, 1u};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MGX_OK : MGX_E_INVALID_ARG;
}

template <int BN, bool IS_INT, class OutT, bool F16 = false>
static int launch_qgemm(const mgx_qgemm_desc& d, const void* A, const void* B, void* D,
                        const float* scale, const float* bias, const void* residual,
                        int64_t ldb, int64_t stride_b, const qout_args& qo, cudaStream_t stream)
{
    using S = qgemm_smem<BN>;
    CUtensorMap ta, tb;
    constexpr int64_t ab = F16 ? 2 : 1; // bytes per operand element: the maps address bytes
    int rc = encode_operand_map(&ta, A, d.K * ab, d.M, d.batch, d.lda * ab, d.stride_a * ab, BM);
    if(rc != MGX_OK)
        return rc;
    rc = encode_operand_map(&tb, B, d.K * ab, d.N, d.batch, ldb * ab, stride_b * ab, BN);
    if(rc != MGX_OK)
        return rc;
    qgemm_params p{};
    constexpr int es = sizeof(OutT);
    p.vec_sb = ((reinterpret_cast<uintptr_t>(scale) & 15u) == 0 and (reinterpret_cast<uintptr_t>(bias) & 15u) == 0) ? 1 : 0;
    const int64_t valign = es == 4 ? 16 : 8; // bytes per lane in the coalesced store
    p.vec_io = ((reinterpret_cast<uintptr_t>(D) % valign) == 0 and (d.ldd * es) % valign == 0 and
                (d.batch == 1 or (d.stride_d * es) % valign == 0) and
                (residual == nullptr or (reinterpret_cast<uintptr_t>(residual) % valign) == 0))
                   ? 1
                   : 0;
    p.M          = d.M;
    p.N          = d.N;
    p.K          = d.K;
    p.batch      = d.batch;
    p.ldd        = d.ldd;
    p.stride_d   = d.stride_d;
    p.D          = D;
    p.scale      = scale;
    p.bias       = bias;
    p.residual   = residual;
    p.tiles_m    = static_cast<int>((d.M + BM - 1) / BM);
    p.tiles_n    = static_cast<int>((d.N + BN - 1) / BN);
    p.num_tiles  = static_cast<int64_t>(p.tiles_m) * p.tiles_n * d.batch;
    p.num_kb     = static_cast<int>((d.K * ab + BK - 1) / BK);
    p.scale_mode = d.scale_mode;
    p.act        = d.act;
    p.Dq         = qo.Dq;
    p.ldq        = qo.ldq;
    p.stride_q   = qo.stride_q;
    p.q_scale    = qo.scale;
    p.q_rcp      = static_cast<float>(1.0 / static_cast<double>(qo.scale));
    p.q_zp       = qo.zp;
    p.q_fp8      = qo.fp8;
    p.write_d    = qo.write_d;
    // the epilogue's check-free path: whole tiles in M, whole 16-column chunks in N, vector
    // access everywhere, no per-row scale, quantizelinear output (if any) int8 in aligned words.
    // The residual shares D's leading dimension and must allow the same vector width.
    {
        const size_t es     = std::is_same<OutT, __half>::value ? 2 : 4;
        const size_t valign = es * 4;
        const bool res_ok   = residual == nullptr or (reinterpret_cast<uintptr_t>(residual) % valign) == 0;
        const bool q_ok     = qo.Dq == nullptr or
                          (qo.fp8 == 0 and (reinterpret_cast<uintptr_t>(qo.Dq) & 3u) == 0 and
                           qo.ldq % 4 == 0 and qo.stride_q % 4 == 0);
        p.fast = (not std::is_same<OutT, int32_t>::value and p.vec_io and p.vec_sb and res_ok and q_ok and
                  d.scale_mode != MGX_SCALE_PER_ROW and d.M % BM == 0 and d.N % EPI_COLS == 0)
                     ? 1
                     : 0;
    }
    p.hmask      = (std::is_same<OutT, __half>::value and (d.flags & MGX_QGEMM_HALF_MATH) != 0) ? 0xFFFFE000u
                                                                                                 : 0xFFFFFFFFu;
    p.act_rcp    = p.hmask != 0xFFFFFFFFu ? 1.0f / 1.4140625f : 0.70710678118654752440f;
    // the table stands for activation + quantizelinear of a half: only where the chain holds one
    p.lut        = (p.hmask != 0xFFFFFFFFu and qo.fp8 == 0) ? static_cast<const uint8_t*>(qo.lut) : nullptr;
    p.acc24      = (IS_INT and d.K < 1024) ? 1 : 0; // |a b| <= 2^14 for int8 operands
    // |v| < 2^-14 (half subnormals) divided by a scale >= 2^-12 stays below 1/4: quantises to zero
    // whatever its low bits; no zero point may shift the rounding boundary
    p.q_mask     = (qo.Dq != nullptr and qo.fp8 == 0 and qo.scale >= 0.000244140625f and
                    qo.zp == static_cast<float>(static_cast<int>(qo.zp))) ? 1 : 0;
    auto kernel  = qgemm_kernel<BN, IS_INT, OutT, F16>;
    int rc2 = ensure_smem_optin(reinterpret_cast<const void*>(kernel), S::total);
    if(rc2 != MGX_OK)
        return rc2;
    const int sms = device_sm_count();
    const int grid = static_cast<int>(p.num_tiles < sms ? p.num_tiles : sms);
    // programmatic dependent launch: set-up (tensor-memory allocation, barriers, descriptor
    // prefetch) overlaps the tail of the previous kernel of the stream
    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = dim3(static_cast<unsigned>(grid));
    cfg.blockDim         = dim3(NTHREADS);
    cfg.dynamicSmemBytes = S::total;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs                                          = attr;
    cfg.numAttrs                                       = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, ta, tb, p));
}

template <int BN, bool IS_INT, bool F16 = false>
static int dispatch_out(const mgx_qgemm_desc& d, const void* A, const void* B, void* D,
                        const float* scale, const float* bias, const void* residual, int64_t ldb,
                        int64_t stride_b, const qout_args& qo, cudaStream_t stream)
{
    switch(d.out_type)
    {
    case MGX_I32:
        if constexpr(IS_INT)
            return launch_qgemm<BN, true, int32_t>(d, A, B, D, scale, bias, residual, ldb, stride_b, qo, stream);
        else
            return MGX_E_UNSUPPORTED;
    case MGX_F32:
        return launch_qgemm<BN, IS_INT, float, F16>(d, A, B, D, scale, bias, residual, ldb, stride_b, qo, stream);
    case MGX_F16:
        return launch_qgemm<BN, IS_INT, __half, F16>(d, A, B, D, scale, bias, residual, ldb, stride_b, qo, stream);
    default: return MGX_E_UNSUPPORTED;
    }
}

// Tile width: the BN in {256, 128, 64} with the smallest estimated time
//   waves x (k-blocks x cycles per k-block + epilogue cycles) + launch.
// A k-block (128 bytes of K) moves 128 x (128 + BN) operand bytes from L2 into the SM;
// measured on B200 that stream sustains about 64 B/clk per SM with every SM loading, which
// - not the tensor pipe (4 MMAs x BN/2 cycles) - bounds the main loop: 2 x (128 + BN) cycles.
// The epilogue costs about 12 cycles per output column of the tile.
static int pick_bn(const mgx_qgemm_desc& d)
{
    // tuning knob: MGX_CUDA_QGEMM_BN = 64 | 128 | 256 forces the tile width
    static const int forced = [] {
        const char* e = std::getenv("MGX_CUDA_QGEMM_BN");
        const int v   = e != nullptr ? std::atoi(e) : 0;
        return (v == 64 or v == 128 or v == 256) ? v : 0;
    }();
    if(forced != 0)
        return forced;
    const int64_t sms = device_sm_count();
    const int64_t tm  = (d.M + BM - 1) / BM;
    const int64_t kb  = (d.K * (d.ab_type == MGX_F16 ? 2 : 1) + BK - 1) / BK;
    int best          = 64;
    int64_t best_cost = INT64_MAX;
    for(int bn : {256, 128, 64})
    {
        const int64_t tiles = tm * ((d.N + bn - 1) / bn) * d.batch;
        const int64_t waves = (tiles + sms - 1) / sms;
        const int64_t mma   = 2 * (128 + bn);
        const int64_t cost  = waves * (kb * mma + 12 * bn) + 1500;
        if(cost < best_cost)
        {
            best_cost = cost;
            best      = bn;
        }
    }
    return best;
}

} // namespace mgx

using namespace mgx;

extern "C" size_t mgx_cuda_qgemm_workspace(const mgx_qgemm_desc* d)
{
    if(d == nullptr)
        return 0;
    if(d->b_layout != MGX_B_KN)
    {
        // optional: with it, launches of at most 16 rows take the weight-streaming kernel
        // (partial sums of tiles shared between thread blocks); without it they run as tiles
        if(d->M > 0 and d->N > 0 and d->K > 0 and d->ab_type != MGX_F16 and qgemv_applicable(*d, false, false))
            return qgemv_workspace(*d);
        return 0;
    }
    if(d->ab_type == MGX_F16)
        return static_cast<size_t>(d->batch) * d->N * ((d->K + 7) / 8 * 8) * 2;
    const int64_t kpad = (d->K + 15) / 16 * 16;
    return static_cast<size_t>(d->batch) * d->N * kpad;
}

extern "C" int mgx_cuda_qgemm(const mgx_qgemm_desc* d, const void* A, const void* B, void* D,
                              const float* scale, const float* bias, const void* residual,
                              void* workspace, size_t workspace_bytes, void* stream_)
{
    if(D == nullptr)
        return MGX_E_INVALID_ARG;
    return mgx_cuda_qgemm_ex(d, A, B, D, scale, bias, residual, nullptr, workspace, workspace_bytes,
                             stream_);
}

extern "C" int mgx_cuda_qgemm_ex(const mgx_qgemm_desc* d, const void* A, const void* B, void* D,
                                 const float* scale, const float* bias, const void* residual,
                                 const mgx_qgemm_qout* q, void* workspace, size_t workspace_bytes,
                                 void* stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if(d == nullptr or A == nullptr or B == nullptr)
        return MGX_E_INVALID_ARG;
    qout_args qo;
    if(q != nullptr and q->q != nullptr)
    {
        if(q->q_type != MGX_I8 and q->q_type != MGX_FP8_E4M3FN)
            return MGX_E_UNSUPPORTED;
        if(d->out_type == MGX_I32 or q->ldq < d->N or not(q->scale > 0.0f))
            return MGX_E_INVALID_ARG;
        qo.Dq       = q->q;
        qo.ldq      = q->ldq;
        qo.stride_q = q->stride_q;
        qo.scale    = q->scale;
        qo.zp       = q->zero_point;
        qo.fp8      = q->q_type == MGX_FP8_E4M3FN ? 1 : 0;
        qo.write_d  = D != nullptr ? 1 : 0;
        qo.lut      = (q->flags & MGX_QOUT_LUT) != 0 ? q->lut : nullptr;
    }
    else if(D == nullptr)
        return MGX_E_INVALID_ARG;
    if(D == nullptr)
        D = qo.Dq; // never written (write_d = 0); keeps the pointer checks below uniform
    if(d->M <= 0 or d->N <= 0 or d->K <= 0 or d->batch <= 0)
        return MGX_E_INVALID_ARG;
    if(d->ab_type != MGX_I8 and d->ab_type != MGX_FP8_E4M3FN and d->ab_type != MGX_F16)
        return MGX_E_UNSUPPORTED;
    const bool f16       = d->ab_type == MGX_F16;
    const int64_t ealign = f16 ? 8 : 16; // elements per 16 bytes
    if(f16 and qo.Dq != nullptr)
        return MGX_E_UNSUPPORTED;
    if(d->scale_mode < MGX_SCALE_NONE or d->scale_mode > MGX_SCALE_PER_ROW)
        return MGX_E_INVALID_ARG;
    if(d->scale_mode != MGX_SCALE_NONE and scale == nullptr)
        return MGX_E_INVALID_ARG;
    if(d->act < MGX_ACT_NONE or d->act > MGX_ACT_SILU)
        return MGX_E_INVALID_ARG;
    if(d->out_type == MGX_I32 and
       (d->ab_type != MGX_I8 or d->scale_mode != MGX_SCALE_NONE or bias != nullptr or
        residual != nullptr or d->act != MGX_ACT_NONE))
        return MGX_E_UNSUPPORTED;
    if(d->M > INT32_MAX or d->N > INT32_MAX or d->K > INT32_MAX)
        return MGX_E_TOO_LARGE;
    if(d->lda < d->K or d->ldd < d->N)
        return MGX_E_INVALID_ARG;
    if((reinterpret_cast<uintptr_t>(A) & 15u) or (d->lda % ealign) or
       (d->batch > 1 and (d->stride_a % ealign)))
        return MGX_E_ALIGNMENT;

    const void* Bk   = B;
    int64_t ldb      = d->ldb;
    int64_t stride_b = d->stride_b;
    if(d->b_layout == MGX_B_KN)
    {
        // quant_dot's [K,N] operand is re-laid out K-contiguous into the workspace
        if(d->ldb != d->N or (d->batch > 1 and d->stride_b != d->K * d->N))
            return MGX_E_UNSUPPORTED;
        const size_t need = mgx_cuda_qgemm_workspace(d);
        if(workspace == nullptr or workspace_bytes < need)
            return MGX_E_WORKSPACE;
        if(reinterpret_cast<uintptr_t>(workspace) & 15u)
            return MGX_E_ALIGNMENT;
        const int64_t kpad = (d->K + ealign - 1) / ealign * ealign;
        int rc = f16 ? transpose_16bit_ld(B, workspace, d->K, d->N, d->batch, kpad, stream)
                     : transpose_8bit_ld(B, workspace, d->K, d->N, d->batch, kpad, stream);
        if(rc != MGX_OK)
            return rc;
        Bk       = workspace;
        ldb      = kpad;
        stride_b = d->N * kpad;
    }
    else if(d->b_layout != MGX_B_NK)
        return MGX_E_INVALID_ARG;
    if(ldb < d->K)
        return MGX_E_INVALID_ARG;
    if((reinterpret_cast<uintptr_t>(Bk) & 15u) or (ldb % ealign) or
       (d->batch > 1 and (stride_b % ealign)))
        return MGX_E_ALIGNMENT;

    // at most 16 rows: stream the weights once, if the caller lent the workspace for it
    if(not f16 and qgemv_applicable(*d, residual != nullptr, qo.Dq != nullptr) and workspace != nullptr and
       workspace_bytes >= qgemv_workspace(*d))
        return qgemv_launch(*d, A, Bk, D, scale, bias, ldb, workspace, workspace_bytes, stream);
    const bool is_int = d->ab_type == MGX_I8;
    if(f16)
    {
        switch(pick_bn(*d))
        {
        case 256: return dispatch_out<256, false, true>(*d, A, Bk, D, scale, bias, residual, ldb, stride_b, qo, stream);
        case 128: return dispatch_out<128, false, true>(*d, A, Bk, D, scale, bias, residual, ldb, stride_b, qo, stream);
        default: return dispatch_out<64, false, true>(*d, A, Bk, D, scale, bias, residual, ldb, stride_b, qo, stream);
        }
    }
    switch(pick_bn(*d))
    {
    case 256:
        return is_int ? dispatch_out<256, true>(*d, A, Bk, D, scale, bias, residual, ldb, stride_b, qo, stream)
                      : dispatch_out<256, false>(*d, A, Bk, D, scale, bias, residual, ldb, stride_b, qo, stream);
    case 128:
        return is_int ? dispatch_out<128, true>(*d, A, Bk, D, scale, bias, residual, ldb, stride_b, qo, stream)
                      : dispatch_out<128, false>(*d, A, Bk, D, scale, bias, residual, ldb, stride_b, qo, stream);
    default:
        return is_int ? dispatch_out<64, true>(*d, A, Bk, D, scale, bias, residual, ldb, stride_b, qo, stream)
                      : dispatch_out<64, false>(*d, A, Bk, D, scale, bias, residual, ldb, stride_b, qo, stream);
    }
}

int mgx::qgemm_status(unsigned int* out) { return read_and_clear_status(out); }

// ------------------------------------------------------------------ allocation-free variant
// Scratch for mgx_cuda_qgemm_static_scratch(): lives in the library's device image, one copy
// per GPU that loads the library, held until the process exits.
namespace {
constexpr size_t static_scratch_bytes = size_t{16} << 20; // 16 MiB
static __device__ __align__(256) uint8_t g_static_scratch[static_scratch_bytes];

// Device address of g_static_scratch on the current device.  In host code the array's name
// is only a handle for the runtime, not a device pointer, so the address is looked up once
// per device (with that device current) and cached.
int static_scratch_address(void** out)
{
    constexpr int max_devices = 64;
    static std::mutex m;
    static void* cached[max_devices] = {};
    int dev       = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if(e != cudaSuccess)
        return static_cast<int>(e);
    if(dev < 0 or dev >= max_devices)
        return MGX_E_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(m);
    if(cached[dev] == nullptr)
    {
        void* p = nullptr;
        e       = cudaGetSymbolAddress(&p, g_static_scratch);
        if(e != cudaSuccess)
            return static_cast<int>(e);
        cached[dev] = p;
    }
    *out = cached[dev];
    return MGX_OK;
}
} // namespace

extern "C" size_t mgx_cuda_qgemm_static_scratch_limit(void) { return static_scratch_bytes; }

extern "C" int mgx_cuda_qgemm_static_scratch(const mgx_qgemm_desc* d, const void* A, const void* B,
                                             void* D, const float* scale, const float* bias,
                                             const void* residual, void* stream)
{
    if(d == nullptr)
        return MGX_E_INVALID_ARG;
    if(d->M <= 0 or d->N <= 0 or d->K <= 0 or d->batch <= 0)
        return MGX_E_INVALID_ARG;
    size_t need = mgx_cuda_qgemm_workspace(d);
    if(need > static_scratch_bytes)
    {
        // a [K,N] operand has to be re-laid out into the scratch: no way around the limit.
        // For [N,K] operands the scratch only enables the weight-streaming kernel for at most
        // 16 rows; beyond the limit the tiled kernel runs, which needs none.
        if(d->b_layout == MGX_B_KN)
            return MGX_E_TOO_LARGE;
        need = 0;
    }
    void* scratch = nullptr;
    if(need > 0)
    {
        const int rc = static_scratch_address(&scratch);
        if(rc != MGX_OK)
            return rc;
    }
    return mgx_cuda_qgemm(d, A, B, D, scale, bias, residual, scratch, need, stream);
}
