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
#include <cstdlib>
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

// ------------------------------------------------------------------ tensor-core decode kernel
// M <= 16 rows of activations against packed int4 weights, HBM-bound by design: the weights
// are read once, 16 bytes per thread, straight into registers, dequantised there and fed to
// mma.sync.m16n8k16 (the register-operand tensor-core path: the B fragment is produced in
// registers, which tcgen05 - operands in shared / tensor memory - cannot take).
//
// Work split: a block owns ROWS_PER_BLOCK = 128 output columns (4 warps x 4 n-tiles of 8) and
// one K slice; every warp walks the whole slice in chunks of 128 k.  Within a warp, lane
// (g = lane / 4, t = lane % 4) loads, for each of its 4 n-tiles, the 16 bytes holding
// k = chunk + 32 t .. + 31 of weight row (tile * 8 + g): four lanes cover 64 contiguous bytes.
// The reduction index of an MMA may be permuted freely as long as A and B agree: word w
// (8 nibbles, k = 8 w .. 8 w + 7) yields the half2 pairs (k0,k4) (k1,k5) (k2,k6) (k3,k7) by
// mask-and-or, which are the B registers of two MMAs; A is staged in shared memory already
// permuted to the same order, so one 16-byte shared load gives the matching A registers.
constexpr int W4_ROWS_PER_BLOCK = 128;
constexpr int W4_TILES          = 4;   // n-tiles of 8 columns per warp
constexpr int W4_CHUNK          = 128; // k per loop trip
constexpr int W4_MAX_SLICE      = 512;
constexpr int W4_STAGES         = 4;   // chunks of packed weights in flight per warp (cp.async ring)
constexpr int W4_RING_BYTES     = W4_STAGES * W4_TILES * 32 * 16; // per warp

__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
                 "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// HI: activations have more than 8 rows (the upper half of the MMA's M = 16 is used).
template <bool HI>
__global__ void __launch_bounds__(128, 4) w4a16_gemv_mma_kernel(const w4_params p)
{
    extern __shared__ __align__(16) uint8_t smem_a[];
    const int warp  = threadIdx.x >> 5;
    const int lane  = threadIdx.x & 31;
    const int g     = lane >> 2;
    const int t     = lane & 3;
    const int split = blockIdx.y;
    const int64_t k_lo    = split * p.k_per_split;
    const int64_t k_hi    = min(p.K, k_lo + p.k_per_split);
    const int64_t m_base  = static_cast<int64_t>(blockIdx.z) * 16; // slab of activations rows
    const int rows_a      = HI ? 16 : 8;
    constexpr int pitch   = W4_MAX_SLICE * 2 + 64; // bytes; = 64 mod 128 keeps the 16-byte loads conflict free

    const int64_t n_base = static_cast<int64_t>(blockIdx.x) * W4_ROWS_PER_BLOCK + warp * (W4_TILES * 8);
    const bool active    = n_base < p.N;

    // weight rows of this lane (clamped: rows past N are loaded from the last row and dropped)
    const uint8_t* brow[W4_TILES];
#pragma unroll
    for(int j = 0; j < W4_TILES; ++j)
    {
        int64_t n = n_base + j * 8 + g;
        n         = n < p.N ? n : p.N - 1;
        brow[j]   = p.Bp + n * (p.K / 2) + (t * 32) / 2;
    }

    // Arithmetic without fp16 or conversion instructions (both run at a fraction of the
    // fp32 rate on this GPU and would bound the kernel): the MMA's B operand is the bit
    // pattern 0x6400 | q, i.e. the fp16 number 1024 + q, produced by one shift and one
    // logic operation per two weights.  Per group of 128 k the tensor core accumulates
    //   P[m,n] = sum_k a[m,k] * (1024 + q[n,k])   and, with a B operand of ones,   S[m] = sum_k a[m,k];
    // the group's contribution is then  s[n] * (P[m,n] - (1024 + zp[n]) * S[m])  in fp32.
    // (Products are exact in the tensor core; the reference rounds every dequantised weight
    // to fp16 first, so this is the more accurate of the two, well inside the tolerance.)
    float acc[W4_TILES][4];
#pragma unroll
    for(int j = 0; j < W4_TILES; ++j)
#pragma unroll
        for(int q = 0; q < 4; ++q)
            acc[j][q] = 0.0f;

    // scale / zero-point rows of the two output columns (2t, 2t+1) this lane owns per tile
    const __half* scol[W4_TILES][2];
    const uint8_t* zcol[W4_TILES][2];
#pragma unroll
    for(int j = 0; j < W4_TILES; ++j)
#pragma unroll
        for(int e = 0; e < 2; ++e)
        {
            int64_t n  = n_base + j * 8 + 2 * t + e;
            n          = n < p.N ? n : p.N - 1;
            scol[j][e] = p.scales + n * p.groups_per_row;
            zcol[j][e] = p.zp == nullptr ? nullptr : p.zp + n * p.groups_per_row;
        }

    // the block's K range is walked in slices of at most W4_MAX_SLICE (the shared-memory copy
    // of the activations), each slice in chunks of 128 k
#pragma unroll 1
    for(int64_t k_begin = k_lo; k_begin < k_hi; k_begin += W4_MAX_SLICE)
    {
    const int slice   = static_cast<int>(min(static_cast<int64_t>(W4_MAX_SLICE), k_hi - k_begin));
    const int nchunks = slice / W4_CHUNK;
    if(k_begin != k_lo)
        __syncthreads(); // everyone is done with the previous slice's activations
    // ---- packed weights stream through a per-warp ring in shared memory: W4_STAGES chunks
    //      (2 KB each) are in flight per warp, which is what hides the HBM latency; every
    //      lane later reads back exactly the 16 bytes it copied
    uint8_t* ring = smem_a + rows_a * pitch + warp * W4_RING_BYTES + lane * 16;
    auto issue = [&](int c) {
        if(active and c < nchunks)
        {
            const uint32_t dst = smem_u32(ring + (c % W4_STAGES) * (W4_TILES * 512));
#pragma unroll
            for(int j = 0; j < W4_TILES; ++j)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + j * 512),
                             "l"(brow[j] + (k_begin + static_cast<int64_t>(c) * W4_CHUNK) / 2)
                             : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for(int c = 0; c < W4_STAGES - 1; ++c)
        issue(c);

    // ---- stage A[0..rows_a) x [k_begin, k_end) in shared memory, permuted per 8 k:
    //      position (chunk, w, t) holds halves of k = chunk*128 + t*32 + w*8 + {0,4,1,5,2,6,3,7}
    const int units = rows_a * (slice / 8);
    for(int u = threadIdx.x; u < units; u += blockDim.x)
    {
        const int m  = u / (slice / 8);
        const int k8 = u - m * (slice / 8); // which group of 8 k inside the slice
        uint4 v      = make_uint4(0u, 0u, 0u, 0u);
        if(m_base + m < p.M)
            v = *reinterpret_cast<const uint4*>(p.A + (m_base + m) * p.lda + k_begin + k8 * 8);
        // v = halves h0..h7 ; wanted order h0 h4 h1 h5 h2 h6 h3 h7
        uint4 o;
        o.x = __byte_perm(v.x, v.z, 0x5410); // h0 | h4
        o.y = __byte_perm(v.x, v.z, 0x7632); // h1 | h5
        o.z = __byte_perm(v.y, v.w, 0x5410); // h2 | h6
        o.w = __byte_perm(v.y, v.w, 0x7632); // h3 | h7
        const int chunk = k8 >> 4;       // 16 groups of 8 per 128-k chunk
        const int tt    = (k8 >> 2) & 3; // k offset / 32 inside the chunk
        const int w     = k8 & 3;        // word inside the lane's 32 k
        *reinterpret_cast<uint4*>(smem_a + m * pitch + chunk * 256 + (w * 4 + tt) * 16) = o;
    }
    __syncthreads();

    {
        const uint8_t* a_lo = smem_a + g * pitch + t * 16;
        const uint8_t* a_hi = smem_a + (g + 8) * pitch + t * 16;
        constexpr uint32_t ones = 0x3C003C00u; // half2(1, 1)
#pragma unroll 1
        for(int c = 0; c < nchunks; ++c)
        {
            issue(c + W4_STAGES - 1);
            asm volatile("cp.async.wait_group %0;" ::"n"(W4_STAGES - 1) : "memory");
            if(not active)
                continue;
            uint4 wcur[W4_TILES];
#pragma unroll
            for(int j = 0; j < W4_TILES; ++j)
                wcur[j] = *reinterpret_cast<const uint4*>(ring + (c % W4_STAGES) * (W4_TILES * 512) + j * 512);
            // this group's scales and zero points (loads overlap the MMAs below)
            const int gi = static_cast<int>((k_begin + static_cast<int64_t>(c) * W4_CHUNK) / p.group);
            float sc[W4_TILES][2], zc[W4_TILES][2];
#pragma unroll
            for(int j = 0; j < W4_TILES; ++j)
#pragma unroll
                for(int e = 0; e < 2; ++e)
                {
                    sc[j][e] = __half2float(scol[j][e][gi]);
                    zc[j][e] = static_cast<float>(1024 + (zcol[j][e] == nullptr ? p.zp_const : static_cast<int>(zcol[j][e][gi])));
                }
            float pg[W4_TILES][4];
            float sg[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for(int j = 0; j < W4_TILES; ++j)
#pragma unroll
                for(int q = 0; q < 4; ++q)
                    pg[j][q] = 0.0f;
#pragma unroll
            for(int w = 0; w < 4; ++w)
            {
                const uint4 alo = *reinterpret_cast<const uint4*>(a_lo + c * 256 + w * 64);
                uint4 ahi       = make_uint4(0u, 0u, 0u, 0u);
                if(HI)
                    ahi = *reinterpret_cast<const uint4*>(a_hi + c * 256 + w * 64);
                mma_m16n8k16(sg, alo.x, ahi.x, alo.y, ahi.y, ones, ones);
                mma_m16n8k16(sg, alo.z, ahi.z, alo.w, ahi.w, ones, ones);
#pragma unroll
                for(int j = 0; j < W4_TILES; ++j)
                {
                    const uint32_t word = w == 0 ? wcur[j].x : (w == 1 ? wcur[j].y : (w == 2 ? wcur[j].z : wcur[j].w));
                    const uint32_t b0 = (word & 0x000F000Fu) | 0x64006400u;         // (k0, k4)
                    const uint32_t b1 = ((word >> 4) & 0x000F000Fu) | 0x64006400u;  // (k1, k5)
                    const uint32_t b2 = ((word >> 8) & 0x000F000Fu) | 0x64006400u;  // (k2, k6)
                    const uint32_t b3 = ((word >> 12) & 0x000F000Fu) | 0x64006400u; // (k3, k7)
                    mma_m16n8k16(pg[j], alo.x, ahi.x, alo.y, ahi.y, b0, b1);
                    mma_m16n8k16(pg[j], alo.z, ahi.z, alo.w, ahi.w, b2, b3);
                }
            }
            // sg[0] = S[row g], sg[2] = S[row g + 8] (every column of the ones tile is the same)
#pragma unroll
            for(int j = 0; j < W4_TILES; ++j)
            {
                acc[j][0] = fmaf(sc[j][0], fmaf(-zc[j][0], sg[0], pg[j][0]), acc[j][0]);
                acc[j][1] = fmaf(sc[j][1], fmaf(-zc[j][1], sg[0], pg[j][1]), acc[j][1]);
                acc[j][2] = fmaf(sc[j][0], fmaf(-zc[j][0], sg[2], pg[j][2]), acc[j][2]);
                acc[j][3] = fmaf(sc[j][1], fmaf(-zc[j][1], sg[2], pg[j][3]), acc[j][3]);
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    } // slices
    // ---- results: c0,c1 = row g, columns 2t, 2t+1 of the tile; c2,c3 = row g + 8
#pragma unroll
    for(int j = 0; j < W4_TILES; ++j)
    {
        const int64_t n = n_base + j * 8 + 2 * t;
#pragma unroll
        for(int half_idx = 0; half_idx < (HI ? 2 : 1); ++half_idx)
        {
            const int64_t m = m_base + g + half_idx * 8;
            if(m >= p.M)
                continue;
#pragma unroll
            for(int e = 0; e < 2; ++e)
            {
                if(n + e >= p.N)
                    continue;
                const float v = acc[j][half_idx * 2 + e];
                if(p.splits > 1)
                    p.partial[(static_cast<int64_t>(split) * p.M + m) * p.N + n + e] = v;
                else
                    p.D[m * p.ldd + n + e] = __float2half_rn(w4_act(v, p.act));
            }
        }
    }
}

// ------------------------------------------------------------------ batch-1 / batch-2 decode kernel
// One or two activation rows: the tensor core has nothing to amortise, so this kernel runs
// on the fp32 pipe and is built around instruction count (about three per weight):
//  * a block of 8 warps owns 64 output columns and one K range; a warp owns 8 of them and
//    walks K in chunks of 1024: lane l reads the 16 bytes holding k = chunk + 32 l .. + 31 of
//    each of its 8 weight rows (a warp reads 512 contiguous bytes per row);
//  * the nibble at bit 4j of a word, OR-ed into the mantissa of 2^23, is the fp32 number
//    2^23 + q * 2^(4j): one logic instruction per weight, no shifts (the upper three nibbles
//    come from the word shifted right by 12).  Subtracting 2^23 + zp * 2^(4j) leaves
//    (q - zp) * 2^(4j) exactly, and the activations are pre-multiplied by 2^(-4j) when the
//    block stages them (as fp32) in shared memory, so one subtract and one FMA finish a weight;
//  * the group's scale is applied once per lane and chunk (a lane's 32 k lie in one group),
//    i.e. products are accumulated exactly and scaled afterwards - more accurate than the
//    reference's per-weight fp16 rounding, well inside the tolerance.
constexpr int W1_ROWS_PER_WARP = 8;
constexpr int W1_WARPS         = 8;
constexpr int W1_CHUNK         = 1024;

template <int MT>
__global__ void __launch_bounds__(W1_WARPS * 32) w4a16_gemv_fp32_kernel(const w4_params p)
{
    __shared__ __align__(16) float a_s[MT][W1_CHUNK];
    const int warp  = threadIdx.x >> 5;
    const int lane  = threadIdx.x & 31;
    const int split = blockIdx.y;
    const int64_t k_lo = split * p.k_per_split;
    const int64_t k_hi = min(p.K, k_lo + p.k_per_split);
    const int64_t n0   = (static_cast<int64_t>(blockIdx.x) * W1_WARPS + warp) * W1_ROWS_PER_WARP;

    const uint8_t* brow[W1_ROWS_PER_WARP];
    const __half* srow[W1_ROWS_PER_WARP];
    const uint8_t* zrow[W1_ROWS_PER_WARP];
#pragma unroll
    for(int r = 0; r < W1_ROWS_PER_WARP; ++r)
    {
        int64_t n = n0 + r;
        n         = n < p.N ? n : p.N - 1;
        brow[r]   = p.Bp + n * (p.K / 2) + lane * 16;
        srow[r]   = p.scales + n * p.groups_per_row;
        zrow[r]   = p.zp == nullptr ? nullptr : p.zp + n * p.groups_per_row;
    }
    float acc[MT][W1_ROWS_PER_WARP];
#pragma unroll
    for(int m = 0; m < MT; ++m)
#pragma unroll
        for(int r = 0; r < W1_ROWS_PER_WARP; ++r)
            acc[m][r] = 0.0f;

    // position of nibble e (k = 8 w + e) after the extraction below: e < 5 stays at bit 4e,
    // e = 5, 6, 7 come from (word >> 12) at bits 8, 12, 16
#define MGX_W1_POS(e) ((e) < 5 ? (e) : (e) - 3)

#pragma unroll 1
    for(int64_t kc = k_lo; kc < k_hi; kc += W1_CHUNK)
    {
        const int len = static_cast<int>(min(static_cast<int64_t>(W1_CHUNK), k_hi - kc)); // multiple of 32
        // this lane's weights of the chunk, all rows in flight before anything is consumed
        uint4 wv[W1_ROWS_PER_WARP];
        const bool lane_on = lane * 32 < len;
#pragma unroll
        for(int r = 0; r < W1_ROWS_PER_WARP; ++r)
            wv[r] = lane_on ? __ldg(reinterpret_cast<const uint4*>(brow[r] + kc / 2)) : make_uint4(0u, 0u, 0u, 0u);
        __syncthreads(); // previous chunk's activations are no longer read
        for(int i = threadIdx.x; i < MT * W1_CHUNK; i += blockDim.x)
        {
            const int m = i / W1_CHUNK, k = i - m * W1_CHUNK;
            float v     = 0.0f;
            if(k < len and m < p.M)
                v = __half2float(p.A[m * p.lda + kc + k]);
            // 2^(-4 pos): exact scaling by a power of two
            a_s[m][k] = v * __uint_as_float(static_cast<uint32_t>(127 - 4 * MGX_W1_POS(k & 7)) << 23);
        }
        __syncthreads();
        if(not lane_on or n0 >= p.N)
            continue;
        const int gi = static_cast<int>((kc + lane * 32) / p.group);
        float part[MT][W1_ROWS_PER_WARP];
        float asum[MT]; // sum of this lane's 32 activations (for the zero-point term)
#pragma unroll
        for(int m = 0; m < MT; ++m)
        {
            asum[m] = 0.0f;
#pragma unroll
            for(int r = 0; r < W1_ROWS_PER_WARP; ++r)
                part[m][r] = 0.0f;
        }
#pragma unroll
        for(int w = 0; w < 4; ++w)
        {
            float a[MT][8];
#pragma unroll
            for(int m = 0; m < MT; ++m)
            {
                const float4 lo = *reinterpret_cast<const float4*>(&a_s[m][lane * 32 + w * 8]);
                const float4 hi = *reinterpret_cast<const float4*>(&a_s[m][lane * 32 + w * 8 + 4]);
                a[m][0] = lo.x, a[m][1] = lo.y, a[m][2] = lo.z, a[m][3] = lo.w;
                a[m][4] = hi.x, a[m][5] = hi.y, a[m][6] = hi.z, a[m][7] = hi.w;
#pragma unroll
                for(int e = 0; e < 8; ++e) // undo the 2^(-4 pos) pre-scaling: exact
                    asum[m] = fmaf(a[m][e], static_cast<float>(1 << (4 * MGX_W1_POS(e))), asum[m]);
            }
#pragma unroll
            for(int r = 0; r < W1_ROWS_PER_WARP; ++r)
            {
                const uint32_t word = w == 0 ? wv[r].x : (w == 1 ? wv[r].y : (w == 2 ? wv[r].z : wv[r].w));
                const uint32_t hi12 = word >> 12;
#pragma unroll
                for(int e = 0; e < 8; ++e)
                {
                    const uint32_t src  = e < 5 ? word : hi12;
                    const uint32_t bits = (src & (0xFu << (4 * MGX_W1_POS(e)))) | 0x4B000000u;
                    const float v       = __uint_as_float(bits) - 8388608.0f; // q * 2^(4 pos), exact
#pragma unroll
                    for(int m = 0; m < MT; ++m)
                        part[m][r] = fmaf(v, a[m][e], part[m][r]);
                }
            }
        }
#pragma unroll
        for(int r = 0; r < W1_ROWS_PER_WARP; ++r)
        {
            const float sc = __half2float(__ldg(srow[r] + gi));
            const float z  = static_cast<float>(zrow[r] == nullptr ? p.zp_const : static_cast<int>(__ldg(zrow[r] + gi)));
#pragma unroll
            for(int m = 0; m < MT; ++m)
                acc[m][r] = fmaf(sc, fmaf(-z, asum[m], part[m][r]), acc[m][r]);
        }
    }
#undef MGX_W1_POS
    // ---- reduce over the lanes (each holds a different part of K) and store
#pragma unroll
    for(int m = 0; m < MT; ++m)
#pragma unroll
        for(int r = 0; r < W1_ROWS_PER_WARP; ++r)
        {
            float v = acc[m][r];
#pragma unroll
            for(int o = 16; o > 0; o >>= 1)
                v += __shfl_xor_sync(0xffffffffu, v, o);
            acc[m][r] = v;
        }
    if(lane == 0)
    {
#pragma unroll
        for(int m = 0; m < MT; ++m)
        {
            if(m >= p.M)
                continue;
#pragma unroll
            for(int r = 0; r < W1_ROWS_PER_WARP; ++r)
            {
                const int64_t n = n0 + r;
                if(n >= p.N)
                    continue;
                if(p.splits > 1)
                    p.partial[(static_cast<int64_t>(split) * p.M + m) * p.N + n] = acc[m][r];
                else
                    p.D[m * p.ldd + n] = __float2half_rn(w4_act(acc[m][r], p.act));
            }
        }
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

// one or two activation rows: the fp32-pipe kernel
static bool use_fp32_path(const mgx_w4_desc& d) { return d.M <= 2 and d.group % 32 == 0 and d.K % 32 == 0; }

static bool use_mma_path(const mgx_w4_desc& d)
{
    if(use_fp32_path(d))
        return false;
    // a group must cover whole 128-k chunks: the per-group scale is applied after the MMAs
    return d.K % W4_CHUNK == 0 and d.group % W4_CHUNK == 0;
}

// K is split so that about three 128-column blocks per SM are in flight and no slice is
// longer than W4_MAX_SLICE (shared-memory copy of the activations); slices are multiples of
// 128 k.  The simple kernel splits K only when the columns alone cannot fill the machine.
static int pick_splits(const mgx_w4_desc& d)
{
    if(use_fp32_path(d))
    {
        // blocks of 64 columns; split K (in whole 1024-k chunks) until ~4 blocks sit on every SM
        const int64_t nblocks = ceil_div(d.N, W1_WARPS * W1_ROWS_PER_WARP);
        const int64_t chunks  = ceil_div(d.K, W1_CHUNK);
        int64_t s             = ceil_div(static_cast<int64_t>(device_sm_count()) * 4, nblocks);
        if(s > chunks)
            s = chunks;
        return static_cast<int>(s < 1 ? 1 : s);
    }
    if(use_mma_path(d))
    {
        // blocks = column blocks x 16-row slabs of the activations; K is split only as far
        // as needed to put about three blocks on every SM
        const int64_t nblocks = ceil_div(d.N, W4_ROWS_PER_BLOCK) * ceil_div(d.M, 16);
        const int64_t chunks  = d.K / W4_CHUNK;
        int64_t s             = ceil_div(static_cast<int64_t>(device_sm_count()) * 3, nblocks);
        if(s > chunks)
            s = chunks;
        if(s > 32)
            s = 32;
        return static_cast<int>(s < 1 ? 1 : s);
    }
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

// MGX_CUDA_W4_TC=0 keeps decode on the CUDA-core / mma.sync kernels (for comparisons).
static bool tc_enabled()
{
    static const bool on = [] {
        const char* e = std::getenv("MGX_CUDA_W4_TC");
        return e == nullptr or e[0] != '0';
    }();
    return on;
}

extern "C" size_t mgx_cuda_w4a16_workspace(const mgx_w4_desc* d)
{
    if(d == nullptr or d->M <= 0 or d->N <= 0 or d->K <= 0)
        return 0;
    // enough for either decode path: the tensor-core one is taken only when the
    // pointers it is later given are 16-byte aligned
    const size_t tc = tc_enabled() and w4a16_tc_applicable(*d) ? w4a16_tc_workspace(*d) + 256 : 0;
    if(d->M > 16 and not use_mma_path(*d))
        return tc;
    int s            = pick_splits(*d);
    const int64_t kq = use_fp32_path(*d) ? W1_CHUNK : (use_mma_path(*d) ? W4_CHUNK : 32);
    const int64_t kp = ceil_div(ceil_div(d->K, s), kq) * kq;
    s                = static_cast<int>(ceil_div(d->K, kp));
    const size_t cc  = s > 1 ? static_cast<size_t>(s) * d->M * d->N * sizeof(float) : 0;
    return tc > cc ? tc : cc;
}

extern "C" int mgx_cuda_w4a16_gemv(const mgx_w4_desc* d, const void* A, const void* Bp,
                                   const void* scales, const void* zp, void* D, void* workspace,
                                   size_t workspace_bytes, void* stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc = validate_w4(d, A, Bp, scales, D);
    if(rc != MGX_OK)
        return rc;
    if(tc_enabled() and w4a16_tc_applicable(*d) and w4a16_tc_pointers_ok(*d, A, Bp, scales, zp))
    {
        // 256-byte aligned view of the caller's workspace
        auto addr          = reinterpret_cast<uintptr_t>(workspace);
        const size_t shift = workspace == nullptr ? 0 : (256 - (addr & 255u)) & 255u;
        if(workspace == nullptr or workspace_bytes < shift)
            return MGX_E_WORKSPACE;
        return w4a16_tc_launch(*d, A, Bp, scales, zp, D, static_cast<uint8_t*>(workspace) + shift,
                               workspace_bytes - shift, stream);
    }
    if(d->M > 16 and not use_mma_path(*d))
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
    const bool mma   = use_mma_path(*d);
    const bool fp32p = use_fp32_path(*d);
    p.splits         = pick_splits(*d);
    const int64_t kq = fp32p ? W1_CHUNK : (mma ? W4_CHUNK : 32);
    p.k_per_split    = ceil_div(ceil_div(d->K, p.splits), kq) * kq;
    p.splits         = static_cast<int>(ceil_div(d->K, p.k_per_split));
    if(p.splits > 1)
    {
        const size_t need = static_cast<size_t>(p.splits) * d->M * d->N * sizeof(float);
        if(workspace == nullptr or workspace_bytes < need)
            return MGX_E_WORKSPACE;
        if(reinterpret_cast<uintptr_t>(workspace) & 3u)
            return MGX_E_ALIGNMENT;
        p.partial = static_cast<float*>(workspace);
    }
    if(fp32p)
    {
        dim3 grid(static_cast<unsigned>(ceil_div(d->N, W1_WARPS * W1_ROWS_PER_WARP)), static_cast<unsigned>(p.splits));
        if(d->M == 1)
            w4a16_gemv_fp32_kernel<1><<<grid, W1_WARPS * 32, 0, stream>>>(p);
        else
            w4a16_gemv_fp32_kernel<2><<<grid, W1_WARPS * 32, 0, stream>>>(p);
    }
    else if(mma)
    {
        const bool hi     = d->M > 8;
        const int smem    = (hi ? 16 : 8) * (W4_MAX_SLICE * 2 + 64) + 4 * W4_RING_BYTES;
        // the opt-in is made once per kernel with the largest size any launch can ask for
        constexpr int smem_max = 16 * (W4_MAX_SLICE * 2 + 64) + 4 * W4_RING_BYTES;
        const int64_t slabs = ceil_div(d->M, 16);
        if(slabs > 65535)
            return MGX_E_TOO_LARGE;
        dim3 grid(static_cast<unsigned>(ceil_div(d->N, W4_ROWS_PER_BLOCK)), static_cast<unsigned>(p.splits),
                  static_cast<unsigned>(slabs));
        if(hi)
        {
            int rc2 = ensure_smem_optin(reinterpret_cast<const void*>(w4a16_gemv_mma_kernel<true>), smem_max);
            if(rc2 != MGX_OK)
                return rc2;
            w4a16_gemv_mma_kernel<true><<<grid, 128, smem, stream>>>(p);
        }
        else
        {
            int rc2 = ensure_smem_optin(reinterpret_cast<const void*>(w4a16_gemv_mma_kernel<false>), smem_max);
            if(rc2 != MGX_OK)
                return rc2;
            w4a16_gemv_mma_kernel<false><<<grid, 128, smem, stream>>>(p);
        }
    }
    else
    {
        const int warps = 8;
        dim3 grid(static_cast<unsigned>(ceil_div(d->N, warps)), static_cast<unsigned>(p.splits));
        if(d->M == 1)
            w4a16_gemv_simple_kernel<1><<<grid, warps * 32, 0, stream>>>(p);
        else if(d->M <= 4)
            w4a16_gemv_simple_kernel<4><<<grid, warps * 32, 0, stream>>>(p);
        else
            w4a16_gemv_simple_kernel<16><<<grid, warps * 32, 0, stream>>>(p);
    }
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

// More than 16 rows of activations (prefill): the same tensor-core kernel over 16-row slabs
// of A (grid.z), every slab re-reading the packed weights through L2.
extern "C" int mgx_cuda_w4a16_gemm(const mgx_w4_desc* d, const void* A, const void* Bp,
                                   const void* scales, const void* zp, void* D, void* workspace,
                                   size_t workspace_bytes, void* stream_)
{
    int rc = validate_w4(d, A, Bp, scales, D);
    if(rc != MGX_OK)
        return rc;
    // more than 16 rows: dequantise-in-flight tcgen05 GEMM (MGX_CUDA_W4_TC=0 keeps the
    // mma.sync slabs, for comparisons)
    if(tc_enabled() and w4a16_prefill_applicable(*d, A, Bp))
        return w4a16_prefill_launch(*d, A, Bp, scales, zp, D, static_cast<cudaStream_t>(stream_));
    if(not use_mma_path(*d))
        return MGX_E_UNSUPPORTED;
    return mgx_cuda_w4a16_gemv(d, A, Bp, scales, zp, D, workspace, workspace_bytes, stream_);
}

extern "C" int mgx_cuda_w4a16(const mgx_w4_desc* d, const void* A, const void* Bp,
                              const void* scales, const void* zp, void* D, void* workspace,
                              size_t workspace_bytes, void* stream)
{
    if(d != nullptr and d->M <= 16)
        return mgx_cuda_w4a16_gemv(d, A, Bp, scales, zp, D, workspace, workspace_bytes, stream);
    return mgx_cuda_w4a16_gemm(d, A, Bp, scales, zp, D, workspace, workspace_bytes, stream);
}
