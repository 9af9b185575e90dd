// Weight-only int4 linear: D[M,N] = A[M,K] (fp16) . W^T with
// W[n,k] = fp16((q[n,k] - zp) * s[n, k/group]); unpack_int4 and the group-wise
// dequantizelinear are fused into the weight load, the dequantised matrix is never
// written to memory.
//
// Arithmetic contract: the IR src/onnx/parse_matmulnbits.cpp:85-158 builds is
//   unpack_int4 (low nibble = even k; src/include/migraphx/op/unpack_int4.hpp:108-115)
//   -> dequantizelinear to fp16 ((double(q) - double(zp)) * scale, one rounding to
//      fp16; src/include/migraphx/op/dequantizelinear.hpp:74-77)
//   -> dot (fp16 operands, wide accumulate, one rounding to fp16; src/gemm.cpp:55-61).
// Here: q - zp is exact in fp16, the product with the fp16 scale is rounded once to
// fp16 (__hmul2), products with A are accumulated in fp32 and rounded once to fp16.
#include "common.cuh"
#include "ptx.cuh"
#include <cuda_fp16.h>

namespace mgx {

struct w4_params
{
    const __half* A;
    const uint8_t* Bp;
    const __half* scales;
    const uint8_t* zp; // may be null
    __half* D;
    float* partial; // [splits][M][N] when splits > 1
    int64_t M, N, K, lda, ldd;
    int group;
    int groups_per_row;
    int zp_const;
    int act;
    int splits;
    int64_t k_per_split; // multiple of 32
};

__device__ __forceinline__ float w4_act(float v, int act)
{
    switch(act)
    {
    case MGX_ACT_RELU: return fmaxf(v, 0.0f);
    case MGX_ACT_SILU: return v / (1.0f + expf(-v));
    case MGX_ACT_GELU_ERF: return (v * 0.5f) * (erff(v / 1.41421356237309504880f) + 1.0f);
    case MGX_ACT_GELU_TANH: {
        float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
        return 0.5f * v * (1.0f + tanhf(u));
    }
    default: return v;
    }
}

// Eight nibbles of `w` -> eight exactly dequantised fp16 weights, as four half2
// pairs (k+e, k+e+4), e = 0..3.  (0x6400 | q) is the fp16 number 1024 + q, so
// subtracting 1024 + zp gives q - zp exactly; the multiply by the scale rounds once.
__device__ __forceinline__ void dequant8(uint32_t w, __half2 zp1024, __half2 s2, __half2 (&out)[4])
{
#pragma unroll
    for(int e = 0; e < 4; ++e)
    {
        uint32_t bits = ((w >> (4 * e)) & 0x000F000Fu) | 0x64006400u;
        __half2 q     = *reinterpret_cast<__half2*>(&bits);
        out[e]        = __hmul2(__hsub2(q, zp1024), s2);
    }
}

// General kernel: one warp per (output column n, K split); each lane walks units of
// 32 consecutive k (16 packed bytes).  Works for any K % 32 == 0, group % 32 == 0.
template <int MT>
__global__ void __launch_bounds__(256) w4a16_gemv_simple_kernel(const w4_params p)
{
    const int warps_per_block = blockDim.x >> 5;
    const int64_t n = static_cast<int64_t>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
    const int lane  = threadIdx.x & 31;
    const int split = blockIdx.y;
    if(n >= p.N)
        return;
    const int64_t k_begin = split * p.k_per_split;
    const int64_t k_end   = min(p.K, k_begin + p.k_per_split);
    float acc[MT];
#pragma unroll
    for(int m = 0; m < MT; ++m)
        acc[m] = 0.0f;
    const uint8_t* brow = p.Bp + n * (p.K / 2);
    const __half* srow  = p.scales + n * p.groups_per_row;
    const uint8_t* zrow = p.zp == nullptr ? nullptr : p.zp + n * p.groups_per_row;

    for(int64_t k = k_begin + lane * 32; k < k_end; k += 32 * 32)
    {
        const uint4 packed = *reinterpret_cast<const uint4*>(brow + k / 2);
        const int g        = static_cast<int>(k / p.group);
        const __half s     = srow[g];
        const int z        = zrow == nullptr ? p.zp_const : static_cast<int>(zrow[g]);
        const __half2 s2   = __half2half2(s);
        const __half2 z2   = __half2half2(__int2half_rn(1024 + z));
        const uint32_t w[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
        for(int j = 0; j < 4; ++j)
        {
            __half2 d[4];
            dequant8(w[j], z2, s2, d);
            float wf[8];
#pragma unroll
            for(int e = 0; e < 4; ++e)
            {
                wf[e]     = __low2float(d[e]);
                wf[e + 4] = __high2float(d[e]);
            }
#pragma unroll
            for(int m = 0; m < MT; ++m)
            {
                if(m < p.M)
                {
                    const uint4 av =
                        *reinterpret_cast<const uint4*>(p.A + m * p.lda + k + j * 8);
                    const __half* ah = reinterpret_cast<const __half*>(&av);
#pragma unroll
                    for(int e = 0; e < 8; ++e)
                        acc[m] = fmaf(wf[e], __half2float(ah[e]), acc[m]);
                }
            }
        }
    }
#pragma unroll
    for(int m = 0; m < MT; ++m)
    {
        float v = acc[m];
#pragma unroll
        for(int o = 16; o > 0; o >>= 1)
            v += __shfl_xor_sync(0xffffffffu, v, o);
        if(lane == 0 and m < p.M)
        {
            if(p.splits > 1)
                p.partial[(static_cast<int64_t>(split) * p.M + m) * p.N + n] = v;
            else
                p.D[m * p.ldd + n] = __float2half_rn(w4_act(v, p.act));
        }
    }
}

__global__ void __launch_bounds__(256) w4a16_splitk_reduce_kernel(const w4_params p)
{
    const int64_t total = p.M * p.N;
    for(int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
        i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        float v = 0.0f;
        for(int s = 0; s < p.splits; ++s)
            v += p.partial[s * total + i];
        const int64_t m = i / p.N, n = i - m * p.N;
        p.D[m * p.ldd + n] = __float2half_rn(w4_act(v, p.act));
    }
}

static int validate_w4(const mgx_w4_desc* d, const void* A, const void* Bp, const void* scales,
                       void* D)
{
    if(d == nullptr or A == nullptr or Bp == nullptr or scales == nullptr or D == nullptr)
        return MGX_E_INVALID_ARG;
    if(d->M <= 0 or d->N <= 0 or d->K <= 0 or d->group <= 0)
        return MGX_E_INVALID_ARG;
    if(d->lda < d->K or d->ldd < d->N)
        return MGX_E_INVALID_ARG;
    if(d->K % 32 != 0 or d->group % 32 != 0 or d->K % d->group != 0)
        return MGX_E_UNSUPPORTED;
    if(d->zp_const < 0 or d->zp_const > 15)
        return MGX_E_INVALID_ARG;
    if((reinterpret_cast<uintptr_t>(A) & 15u) or (reinterpret_cast<uintptr_t>(Bp) & 15u) or
       (d->lda % 8))
        return MGX_E_ALIGNMENT;
    if(d->act < MGX_ACT_NONE or d->act > MGX_ACT_SILU)
        return MGX_E_INVALID_ARG;
    return MGX_OK;
}

// Split K only when the columns alone cannot fill the machine.
static int pick_splits(const mgx_w4_desc& d)
{
    const int64_t warps_wanted = static_cast<int64_t>(device_sm_count()) * 16;
    if(d.N >= warps_wanted)
        return 1;
    int64_t s       = ceil_div(warps_wanted, d.N);
    const int64_t mx = d.K / 1024 > 0 ? d.K / 1024 : 1;
    if(s > mx)
        s = mx;
    if(s > 16)
        s = 16;
    return static_cast<int>(s < 1 ? 1 : s);
}

} // namespace mgx

using namespace mgx;

int mgx::w4a16_status(unsigned int* out) { return read_and_clear_status(out); }

extern "C" size_t mgx_cuda_w4a16_workspace(const mgx_w4_desc* d)
{
    if(d == nullptr or d->M <= 0 or d->N <= 0 or d->K <= 0)
        return 0;
    if(d->M > 16)
        return 0;
    const int s = pick_splits(*d);
    return s > 1 ? static_cast<size_t>(s) * d->M * d->N * sizeof(float) : 0;
}

extern "C" int mgx_cuda_w4a16_gemv(const mgx_w4_desc* d, const void* A, const void* Bp,
                                   const void* scales, const void* zp, void* D, void* workspace,
                                   size_t workspace_bytes, void* stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc = validate_w4(d, A, Bp, scales, D);
    if(rc != MGX_OK)
        return rc;
    if(d->M > 16)
        return MGX_E_UNSUPPORTED;
    w4_params p{};
    p.A              = static_cast<const __half*>(A);
    p.Bp             = static_cast<const uint8_t*>(Bp);
    p.scales         = static_cast<const __half*>(scales);
    p.zp             = static_cast<const uint8_t*>(zp);
    p.D              = static_cast<__half*>(D);
    p.M              = d->M;
    p.N              = d->N;
    p.K              = d->K;
    p.lda            = d->lda;
    p.ldd            = d->ldd;
    p.group          = d->group;
    p.groups_per_row = static_cast<int>(d->K / d->group);
    p.zp_const       = d->zp_const;
    p.act            = d->act;
    p.splits         = pick_splits(*d);
    p.k_per_split    = ceil_div(ceil_div(d->K, p.splits), 32) * 32;
    if(p.splits > 1)
    {
        const size_t need = static_cast<size_t>(p.splits) * d->M * d->N * sizeof(float);
        if(workspace == nullptr or workspace_bytes < need)
            return MGX_E_WORKSPACE;
        if(reinterpret_cast<uintptr_t>(workspace) & 3u)
            return MGX_E_ALIGNMENT;
        p.partial = static_cast<float*>(workspace);
    }
    const int warps = 8;
    dim3 grid(static_cast<unsigned>(ceil_div(d->N, warps)), static_cast<unsigned>(p.splits));
    if(d->M == 1)
        w4a16_gemv_simple_kernel<1><<<grid, warps * 32, 0, stream>>>(p);
    else if(d->M <= 4)
        w4a16_gemv_simple_kernel<4><<<grid, warps * 32, 0, stream>>>(p);
    else
        w4a16_gemv_simple_kernel<16><<<grid, warps * 32, 0, stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if(e != cudaSuccess)
        return static_cast<int>(e);
    if(p.splits > 1)
    {
        const int64_t total = d->M * d->N;
        const int blocks    = static_cast<int>(ceil_div(total, 256) < 1184 ? ceil_div(total, 256) : 1184);
        w4a16_splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(p);
        e = cudaGetLastError();
    }
    return static_cast<int>(e);
}

extern "C" int mgx_cuda_w4a16_gemm(const mgx_w4_desc* d, const void* A, const void* Bp,
                                   const void* scales, const void* zp, void* D, void* workspace,
                                   size_t workspace_bytes, void* stream_)
{
    (void)workspace;
    (void)workspace_bytes;
    (void)zp;
    (void)stream_;
    int rc = validate_w4(d, A, Bp, scales, D);
    if(rc != MGX_OK)
        return rc;
    return MGX_E_UNSUPPORTED;
}

extern "C" int mgx_cuda_w4a16(const mgx_w4_desc* d, const void* A, const void* Bp,
                              const void* scales, const void* zp, void* D, void* workspace,
                              size_t workspace_bytes, void* stream)
{
    if(d != nullptr and d->M <= 16)
        return mgx_cuda_w4a16_gemv(d, A, Bp, scales, zp, D, workspace, workspace_bytes, stream);
    return mgx_cuda_w4a16_gemm(d, A, Bp, scales, zp, D, workspace, workspace_bytes, stream);
}
