// LayerNorm over the innermost axis as one kernel, with an optional fused per-tensor
// quantizelinear of the result.  It stands in for the instruction chain MIGraphX's ONNX parser
// emits for LayerNormalization (src/onnx/parse_layernorm.cpp:100-140):
//   mean = reduce_mean(x); d = x - mean; var = reduce_mean(d * d); y = d * rsqrt(var + eps) * gamma + beta
// and reproduces the roundings those separate operators make: with fp16 tensors every
// intermediate result (mean, d, d*d, var, var + eps, rsqrt, each product, the sum) is truncated to
// half, as migraphx::half arithmetic does (src/include/migraphx/generic_float.hpp:180-230); fp32
// tensors take plain fp32 operations in the same order.  The reference sums in double; the kernel
// sums fp32 partials as a tree (within 1e-6 relative).
//
// One warp per row, the row held in registers (x is read once): HBM-bound, bytes in + out.
#include "common.cuh"
#include "qgemm_math.cuh"
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include "ptx.cuh"

namespace mgx {

// A result stored in T.  half: the mantissa cut, which is migraphx::half's truncation for every
// value in the normal half range; a value below 2^-14 keeps up to 2^-24 too much (the deviations
// from the mean and their squares can be that small), far below what the next rounding resolves.
// One instruction instead of a range test per rounding: with eight roundings per element the
// kernel is bound by instruction issue otherwise.
template <class T>
__device__ __forceinline__ float ln_round(float v)
{
    if constexpr(std::is_same<T, float>::value)
        return v;
    else
        return __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
}

struct ln_params
{
    const void* x;
    const void* gamma;
    const void* beta;
    void* y;
    void* q;
    void* dq; // dequantizelinear(q) in x's type, or null
    int64_t rows, ldx, ldy, ldq, lddq;
    int cols;
    float eps;
    float inv_n;
    float q_scale, q_rcp, q_zp;
    float dq_scale;
    int q_fp8;
    int rms; // RMS normalisation: no mean, squares and their mean in fp32 (see mgx_layernorm_desc::flags)
};

// T: float or __half.  NV: 16-byte vectors per thread.  WPR: warps per row - 1 (a warp per row, a
// thread owns vectors lane, lane + 32, ...) or 8 (a block per row: few, long rows, e.g. the single
// token of a decode step, where one warp per row would leave a 4096-element row to 32 threads).
template <class T, int NV, int WPR>
__global__ void __launch_bounds__(256) layernorm_kernel(const ln_params p)
{
    constexpr int VE  = 16 / sizeof(T); // elements per vector
    constexpr int TPR = 32 * WPR;       // threads per row
    __shared__ float red[2][8];
    const int lane    = WPR == 1 ? (threadIdx.x & 31) : threadIdx.x;
    const int64_t row = WPR == 1 ? static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)
                                 : static_cast<int64_t>(blockIdx.x);
    if(row >= p.rows)
        return; // (a whole block when WPR > 1: nobody is left waiting at a barrier)
    // sum over the row's threads
    auto row_sum = [&](float v, int slot) {
#pragma unroll
        for(int o = 16; o > 0; o >>= 1)
            v += __shfl_xor_sync(0xffffffffu, v, o);
        if constexpr(WPR > 1)
        {
            if((threadIdx.x & 31) == 0)
                red[slot][threadIdx.x >> 5] = v;
            __syncthreads();
            v = 0.0f;
#pragma unroll
            for(int w = 0; w < WPR; ++w)
                v += red[slot][w];
        }
        return v;
    };
    const int nvec = p.cols / VE; // vectors in a row
    const T* xr    = static_cast<const T*>(p.x) + row * p.ldx;
    float v[NV][VE];
    float sum = 0.0f;
#pragma unroll
    for(int i = 0; i < NV; ++i)
    {
        const int vi = lane + TPR * i;
        if(vi < nvec)
        {
            const uint4 w = *reinterpret_cast<const uint4*>(xr + vi * VE);
            if constexpr(std::is_same<T, float>::value)
            {
                v[i][0] = __uint_as_float(w.x), v[i][1] = __uint_as_float(w.y);
                v[i][2] = __uint_as_float(w.z), v[i][3] = __uint_as_float(w.w);
            }
            else
            {
                const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
                for(int j = 0; j < 4; ++j)
                {
                    const float2 f  = __half22float2(h[j]);
                    v[i][2 * j]     = f.x;
                    v[i][2 * j + 1] = f.y;
                }
            }
#pragma unroll
            for(int j = 0; j < VE; ++j)
                sum += v[i][j];
        }
        else
        {
#pragma unroll
            for(int j = 0; j < VE; ++j)
                v[i][j] = 0.0f;
        }
    }
    sum = row_sum(sum, 0);
    const float mean = ln_round<T>(sum * p.inv_n);
    float sq = 0.0f;
    if(p.rms)
    {
        // SimplifiedLayerNormalization (src/onnx/parse_simplified_layer_normalization.cpp:91-106): x is
        // converted to float, squared and averaged in fp32; only the mean is stored in T again
#pragma unroll
        for(int i = 0; i < NV; ++i)
            if(lane + TPR * i < nvec)
            {
#pragma unroll
                for(int j = 0; j < VE; ++j)
                    sq += __fmul_rn(v[i][j], v[i][j]);
            }
    }
    else
    {
#pragma unroll
        for(int i = 0; i < NV; ++i)
        {
            if(lane + TPR * i < nvec)
            {
#pragma unroll
                for(int j = 0; j < VE; ++j)
                {
                    v[i][j] = ln_round<T>(v[i][j] - mean);
                    sq += ln_round<T>(v[i][j] * v[i][j]);
                }
            }
        }
    }
    sq = row_sum(sq, 1);
    const float var = ln_round<T>(sq * p.inv_n);
    const float ve  = ln_round<T>(var + p.eps);
    // rsqrt as the reference computes it: 1 / sqrt(x), both correctly rounded in fp32
    const float rs  = ln_round<T>(__fdiv_rn(1.0f, __fsqrt_rn(ve)));
    const T* g = static_cast<const T*>(p.gamma);
    const T* b = static_cast<const T*>(p.beta);
    const float q_lo = -128.0f - p.q_zp, q_hi = 127.0f - p.q_zp;
#pragma unroll
    for(int i = 0; i < NV; ++i)
    {
        const int vi = lane + TPR * i;
        if(vi >= nvec)
            continue;
        float gv[VE], bv[VE];
        if(g != nullptr)
        {
            const uint4 w = __ldg(reinterpret_cast<const uint4*>(g + vi * VE));
            if constexpr(std::is_same<T, float>::value)
                gv[0] = __uint_as_float(w.x), gv[1] = __uint_as_float(w.y), gv[2] = __uint_as_float(w.z),
                gv[3] = __uint_as_float(w.w);
            else
            {
                const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
                for(int j = 0; j < 4; ++j)
                {
                    const float2 f = __half22float2(h[j]);
                    gv[2 * j] = f.x, gv[2 * j + 1] = f.y;
                }
            }
        }
        if(b != nullptr)
        {
            const uint4 w = __ldg(reinterpret_cast<const uint4*>(b + vi * VE));
            if constexpr(std::is_same<T, float>::value)
                bv[0] = __uint_as_float(w.x), bv[1] = __uint_as_float(w.y), bv[2] = __uint_as_float(w.z),
                bv[3] = __uint_as_float(w.w);
            else
            {
                const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
                for(int j = 0; j < 4; ++j)
                {
                    const float2 f = __half22float2(h[j]);
                    bv[2 * j] = f.x, bv[2 * j + 1] = f.y;
                }
            }
        }
        float o[VE];
#pragma unroll
        for(int j = 0; j < VE; ++j)
        {
            float t = ln_round<T>(v[i][j] * rs);
            if(g != nullptr)
                t = ln_round<T>(t * gv[j]);
            if(b != nullptr)
                t = ln_round<T>(t + bv[j]);
            o[j] = t;
        }
        if(p.y != nullptr)
        {
            T* yr = static_cast<T*>(p.y) + row * p.ldy + vi * VE;
            if constexpr(std::is_same<T, float>::value)
                *reinterpret_cast<float4*>(yr) = make_float4(o[0], o[1], o[2], o[3]);
            else
                *reinterpret_cast<uint4*>(yr) = make_uint4(cvt_rz_f16x2(o[0], o[1]), cvt_rz_f16x2(o[2], o[3]),
                                                           cvt_rz_f16x2(o[4], o[5]), cvt_rz_f16x2(o[6], o[7]));
        }
        if(p.q != nullptr)
        {
            // quantizelinear(y, scale, zero point): y / scale in y's type (fp16: the fp32 quotient
            // truncated to half), round half to even, + zero point, saturate
            // (src/include/migraphx/op/quantizelinear.hpp:89-103)
            uint8_t qb[VE];
            float dqv[VE]; // (q - zero point) * scale, the dequantised copy some programs read next
#pragma unroll
            for(int j = 0; j < VE; ++j)
            {
                float qv        = __fmul_rn(o[j], p.q_rcp);
                const float rem = __fmaf_rn(-p.q_scale, qv, o[j]);
                qv              = ln_round<T>(__fmaf_rn(rem, p.q_rcp, qv)); // correctly rounded quotient
                if(p.q_fp8)
                {
                    qv     = fmaxf(-448.0f, fminf(448.0f, qv + p.q_zp));
                    qb[j]  = static_cast<uint8_t>(__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3));
                    dqv[j] = 0.0f; // not offered for fp8 (rejected on the host)
                }
                else
                {
                    qv           = fmaxf(q_lo, fminf(q_hi, qv));
                    const int qr = __float_as_int(__fadd_rn(qv, 12582912.0f)) - 0x4B400000; // q - zero point
                    qb[j]        = static_cast<uint8_t>(qr + static_cast<int>(p.q_zp));
                    dqv[j]       = ln_round<T>(static_cast<float>(qr) * p.dq_scale);
                }
            }
            if(p.dq != nullptr)
            {
                T* dr = static_cast<T*>(p.dq) + row * p.lddq + vi * VE;
                if constexpr(std::is_same<T, float>::value)
                    *reinterpret_cast<float4*>(dr) = make_float4(dqv[0], dqv[1], dqv[2], dqv[3]);
                else
                    *reinterpret_cast<uint4*>(dr) =
                        make_uint4(cvt_rz_f16x2(dqv[0], dqv[1]), cvt_rz_f16x2(dqv[2], dqv[3]),
                                   cvt_rz_f16x2(dqv[4], dqv[5]), cvt_rz_f16x2(dqv[6], dqv[7]));
            }
            uint8_t* qr = static_cast<uint8_t*>(p.q) + row * p.ldq + vi * VE;
            if constexpr(VE == 8)
                *reinterpret_cast<uint2*>(qr) = *reinterpret_cast<const uint2*>(qb);
            else
                *reinterpret_cast<uint32_t*>(qr) = *reinterpret_cast<const uint32_t*>(qb);
        }
    }
}

template <class T>
static int launch_layernorm(const ln_params& p, cudaStream_t stream)
{
    constexpr int VE = 16 / sizeof(T);
    const int nvec   = p.cols / VE;
    // few rows: a block per row (each thread at most 8 vectors), so that a launch of a few hundred rows
    // is spread over all SMs with one vector or two per thread; otherwise a warp per row, for rows of
    // up to 16 vectors per lane (measured on 768-wide fp16 rows inside the encoder program: the block form
    // wins at 384 and 768 rows, the warp form at 3072)
    const bool block_per_row = p.rows <= 8 * device_sm_count() or nvec > 32 * 16;
    if(block_per_row)
    {
        const int nv = (nvec + 255) / 256;
        const dim3 grid(static_cast<unsigned>(p.rows));
        if(nv <= 1)
            layernorm_kernel<T, 1, 8><<<grid, 256, 0, stream>>>(p);
        else if(nv <= 2)
            layernorm_kernel<T, 2, 8><<<grid, 256, 0, stream>>>(p);
        else if(nv <= 4)
            layernorm_kernel<T, 4, 8><<<grid, 256, 0, stream>>>(p);
        else if(nv <= 8)
            layernorm_kernel<T, 8, 8><<<grid, 256, 0, stream>>>(p);
        else
            return MGX_E_UNSUPPORTED;
        return static_cast<int>(cudaGetLastError());
    }
    const int nv    = (nvec + 31) / 32;
    const int warps = 8;
    const dim3 grid(static_cast<unsigned>((p.rows + warps - 1) / warps));
    const dim3 block(32 * warps);
    if(nv <= 1)
        layernorm_kernel<T, 1, 1><<<grid, block, 0, stream>>>(p);
    else if(nv <= 2)
        layernorm_kernel<T, 2, 1><<<grid, block, 0, stream>>>(p);
    else if(nv <= 3)
        layernorm_kernel<T, 3, 1><<<grid, block, 0, stream>>>(p);
    else if(nv <= 4)
        layernorm_kernel<T, 4, 1><<<grid, block, 0, stream>>>(p);
    else if(nv <= 6)
        layernorm_kernel<T, 6, 1><<<grid, block, 0, stream>>>(p);
    else if(nv <= 8)
        layernorm_kernel<T, 8, 1><<<grid, block, 0, stream>>>(p);
    else if(nv <= 16)
        layernorm_kernel<T, 16, 1><<<grid, block, 0, stream>>>(p);
    else
        return MGX_E_UNSUPPORTED;
    return static_cast<int>(cudaGetLastError());
}

} // namespace mgx

extern "C" int mgx_cuda_layernorm_supported(int type, int64_t cols)
{
    // (a block per row: 256 threads x 8 vectors)
    if(type == MGX_F16)
        return cols > 0 and cols % 8 == 0 and cols <= 8 * 256 * 8;
    if(type == MGX_F32)
        return cols > 0 and cols % 4 == 0 and cols <= 4 * 256 * 8;
    return 0;
}

extern "C" int mgx_cuda_layernorm(const mgx_layernorm_desc* d, const void* x, const void* gamma, const void* beta,
                                  void* y, void* q, void* stream_)
{
    return mgx_cuda_layernorm_ex(d, x, gamma, beta, y, q, nullptr, 0, 0.0f, stream_);
}

extern "C" int mgx_cuda_layernorm_ex(const mgx_layernorm_desc* d, const void* x, const void* gamma, const void* beta,
                                     void* y, void* q, void* dq, int64_t lddq, float dq_scale, void* stream_)
{
    using namespace mgx;
    if(d == nullptr or x == nullptr or (y == nullptr and q == nullptr))
        return MGX_E_INVALID_ARG;
    if(d->rows <= 0 or d->cols <= 0 or d->ldx < d->cols)
        return MGX_E_INVALID_ARG;
    if(not mgx_cuda_layernorm_supported(d->type, d->cols))
        return MGX_E_UNSUPPORTED;
    const int es = d->type == MGX_F16 ? 2 : 4;
    auto misaligned = [&](const void* ptr, int64_t ld, int bytes) {
        return ptr != nullptr and ((reinterpret_cast<uintptr_t>(ptr) % bytes) != 0 or (ld * es) % bytes != 0);
    };
    if(misaligned(x, d->ldx, 16) or misaligned(y, d->ldy, 16) or misaligned(gamma, 0, 16) or misaligned(beta, 0, 16))
        return MGX_E_ALIGNMENT;
    if(q != nullptr)
    {
        if(d->q_type != MGX_I8 and d->q_type != MGX_FP8_E4M3FN)
            return MGX_E_UNSUPPORTED;
        const int qa = d->type == MGX_F16 ? 8 : 4;
        if((reinterpret_cast<uintptr_t>(q) % qa) != 0 or d->ldq % qa != 0 or d->ldq < d->cols or not(d->q_scale > 0.0f))
            return MGX_E_ALIGNMENT;
    }
    if(y != nullptr and d->ldy < d->cols)
        return MGX_E_INVALID_ARG;
    if(dq != nullptr)
    {
        if(q == nullptr or d->q_type != MGX_I8)
            return MGX_E_UNSUPPORTED;
        if(lddq < d->cols)
            return MGX_E_INVALID_ARG;
        if(misaligned(dq, lddq, 16))
            return MGX_E_ALIGNMENT;
    }
    ln_params p{};
    p.x       = x;
    p.gamma   = gamma;
    p.beta    = beta;
    p.y       = y;
    p.q       = q;
    p.dq      = dq;
    p.lddq    = lddq;
    p.dq_scale = dq_scale;
    p.rows    = d->rows;
    p.cols    = static_cast<int>(d->cols);
    p.ldx     = d->ldx;
    p.ldy     = d->ldy;
    p.ldq     = d->ldq;
    p.eps     = d->eps;
    p.inv_n   = 1.0f / static_cast<float>(d->cols);
    p.q_scale = d->q_scale;
    p.q_rcp   = q != nullptr ? static_cast<float>(1.0 / static_cast<double>(d->q_scale)) : 0.0f;
    p.q_zp    = d->q_zero_point;
    p.q_fp8   = d->q_type == MGX_FP8_E4M3FN ? 1 : 0;
    p.rms     = (d->flags & MGX_LAYERNORM_RMS) != 0 ? 1 : 0;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    return d->type == MGX_F16 ? launch_layernorm<__half>(p, stream) : launch_layernorm<float>(p, stream);
}
