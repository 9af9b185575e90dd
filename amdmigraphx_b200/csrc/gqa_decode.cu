// Decode-step attention of a grouped-query decoder layer against the fp16 KV cache, one launch.
//
// Stands in for the operator chain the GroupQueryAttention parser emits after concat_past_present
// (src/onnx/parse_group_query_attention.cpp:184-262): the KV heads broadcast to the query heads,
// dot(Q, K^T) over the whole cache length, mul by the scale, where(position > seqlens_k, -inf),
// softmax, dot(P, V).  With one query row per head this is a stream over the valid part of the
// cache: HBM-bound, 2 * (seqlens_k + 1) * head * 2 bytes per (batch entry, KV head), read once for
// all the query heads that share the KV head.  Positions beyond seqlens_k are never read (their
// probabilities are exactly zero in the chain).
//
// Split-KV over a thread-block cluster: the cluster's CTAs take consecutive ranges of the valid
// positions; row maximum, sum of exponentials and the partial outputs are exchanged through
// distributed shared memory, so there is no second launch and no scratch in global memory.
//
// The chain's fp16 roundings are kept (migraphx::half truncates, src/include/migraphx/generic_float.hpp):
// the score is cut to half after the dot and after the scaling, exp(x - max) is cut to half, the
// sum runs over those halves in fp32, the quotient is cut to half before P V (ref_softmax,
// src/targets/ref/lowering.cpp:282-313).  Dots accumulate in fp32 (the reference: double).
#include "common.cuh"
#include "qgemm_math.cuh"
#include <cooperative_groups.h>
#include <cuda_fp16.h>

namespace cg = cooperative_groups;

namespace mgx {

struct gqa_decode_params
{
    const __half* q; // [batch][heads] rows of `head` contiguous halves
    int64_t q_sb, q_sh;
    const __half* k; // caches, packed [batch, kv_heads, cache_seq, head]
    const __half* v;
    const void* seqlens;
    int seqlens_i64;
    __half* out; // [batch, heads * head]
    float scale;
    int cache_seq, kv_heads, cap; // cap: score columns a CTA holds in shared memory
};

constexpr int GD_THREADS = 256;
constexpr int GD_WARPS   = GD_THREADS / 32;

__device__ __forceinline__ float gd_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// v >= 0 cut to half precision, subnormal halves included
__device__ __forceinline__ float gd_trunc_nonneg(float v)
{
    const float big   = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    const float small = __fsub_rn(__fadd_rz(v, 0.5f), 0.5f);
    return v < 6.103515625e-5f ? small : big;
}

__device__ __forceinline__ void gd_unpack8(const uint4& w, float (&f)[8])
{
    const __half2* h2 = reinterpret_cast<const __half2*>(&w);
#pragma unroll
    for(int i = 0; i < 4; ++i)
    {
        const float2 t = __half22float2(h2[i]);
        f[2 * i]       = t.x;
        f[2 * i + 1]   = t.y;
    }
}

__device__ __forceinline__ void gd_mma_16816(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1)
{
    // rows 8 .. 15 of A (fragments a1, a3) are zero: at most 8 query heads share a KV head
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
                 "{%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

// D: head size (64 or 128); FACT: query heads per KV head.
// MMA (FACT 4 or 8): the two products on the tensor cores (mma.sync m16n8k16, the query heads of the
// group as rows 0 .. FACT-1 of the 16-row operand), fragments loaded straight from global memory as
// 16-byte vectors.  The contraction index of Q K^T is the head dimension, whose order inside a
// fragment is free: lane (g, t) takes the 8 consecutive halves at 32 b + 8 t of key g (and of its
// query head g) for the two 16-wide steps of block b.  In P V the contraction index is the key and
// the free order is that of the output columns: lane (g, t) loads columns 8 g .. 8 g + 7 of its four
// keys and pairs them up with byte permutes; tile i of a 64-column half then holds column 8 n + i
// in its column n.  Without MMA the scalar loops need FACT x 8 FMAs per 16 cache bytes and are
// bound by FMA issue for FACT > 2.
template <int D, int FACT, bool MMA>
__global__ void __launch_bounds__(GD_THREADS) gqa_decode_kernel(const gqa_decode_params p)
{
    constexpr int LPR = D / 8;   // lanes per cache row (16 bytes each)
    constexpr int RPW = 32 / LPR; // rows per warp and iteration
    constexpr int RPI = RPW * GD_WARPS;
    constexpr int U   = FACT <= 2 ? 4 : 2; // 16-byte loads in flight per lane
    extern __shared__ __align__(16) uint8_t gd_smem[];
    __shared__ float red_m[FACT];           // this CTA's maxima / sums, read by the cluster
    __shared__ float red_s[FACT];
    __shared__ float wred[GD_WARPS][FACT];  // per-warp partials of a block reduction
    __shared__ float cta_out[FACT * D];     // this CTA's partial output, read by rank 0
    __half* sc  = reinterpret_cast<__half*>(gd_smem);                         // [FACT][cap]
    float* part = reinterpret_cast<float*>(gd_smem + sizeof(__half) * FACT * p.cap); // [warps][FACT][D]

    cg::cluster_group cluster = cg::this_cluster();
    const int rank    = static_cast<int>(cluster.block_rank());
    const int nsplit  = static_cast<int>(cluster.num_blocks());
    const int kvh     = blockIdx.y;
    const int b       = blockIdx.z;
    const int tid     = threadIdx.x;
    const int warp    = tid >> 5, lane = tid & 31;
    const int sub     = lane / LPR, li = lane % LPR;

    int64_t last = p.seqlens_i64 ? static_cast<const int64_t*>(p.seqlens)[b]
                                 : static_cast<int64_t>(static_cast<const int32_t*>(p.seqlens)[b]);
    // positions 0 .. seqlens_k take part; a length outside the cache is clamped (the chain would
    // mask nothing beyond the cache either)
    int len = last < 0 ? 1 : (last + 1 > p.cache_seq ? p.cache_seq : static_cast<int>(last + 1));
    int chunk = (len + nsplit - 1) / nsplit;
    if(chunk > p.cap)
        chunk = p.cap; // cannot happen for cap >= ceil(cache_seq / nsplit); keeps the indexing in bounds
    const int k0 = rank * chunk;
    const int k1 = min(len, k0 + chunk);
    const int n  = max(k1 - k0, 0);

    const int64_t head0 = static_cast<int64_t>(kvh) * FACT;
    const __half* kbase = p.k + (static_cast<int64_t>(b) * p.kv_heads + kvh) * p.cache_seq * D;
    const __half* vbase = p.v + (static_cast<int64_t>(b) * p.kv_heads + kvh) * p.cache_seq * D;

    const int g = lane >> 2, t = lane & 3; // fragment coordinates (MMA)
    constexpr int NB = D / 32;             // 32-wide blocks of the head dimension (MMA)
    // this lane's 8 columns of every query head of the group
    float qf[MMA ? 1 : FACT][8];
    uint4 qa[MMA ? NB : 1]; // MMA: query head g, halves 32 b + 8 t .. + 7
    if constexpr(MMA)
    {
#pragma unroll
        for(int blk = 0; blk < NB; ++blk)
        {
            qa[blk] = make_uint4(0, 0, 0, 0);
            if(g < FACT)
                qa[blk] = *reinterpret_cast<const uint4*>(p.q + b * p.q_sb + (head0 + g) * p.q_sh + blk * 32 + t * 8);
        }
    }
    else
    {
#pragma unroll
        for(int h = 0; h < FACT; ++h)
        {
            const __half* qp = p.q + b * p.q_sb + (head0 + h) * p.q_sh + li * 8;
#pragma unroll
            for(int c = 0; c < 8; ++c)
                qf[h][c] = __half2float(qp[c]);
        }
    }

    // ---- phase 1: scores of this CTA's positions, cut to half after the dot and after the scaling
    float mx[FACT];
#pragma unroll
    for(int h = 0; h < FACT; ++h)
        mx[h] = -INFINITY;
    if constexpr(MMA)
    {
        // 8 keys per warp and step, two steps per trip (their loads in flight together): lane (g, t)
        // loads key g of each step
        for(int j0 = warp * 8; j0 < n; j0 += 2 * GD_WARPS * 8)
        {
            uint4 kw[2][NB];
#pragma unroll
            for(int u = 0; u < 2; ++u)
            {
                const int key = j0 + u * GD_WARPS * 8 + g;
#pragma unroll
                for(int blk = 0; blk < NB; ++blk)
                {
                    kw[u][blk] = make_uint4(0, 0, 0, 0);
                    if(key < n)
                        kw[u][blk] = __ldg(reinterpret_cast<const uint4*>(kbase + static_cast<int64_t>(k0 + key) * D + blk * 32 + t * 8));
                }
            }
#pragma unroll
            for(int u = 0; u < 2; ++u)
            {
                const int jb = j0 + u * GD_WARPS * 8;
                float c[4]   = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for(int blk = 0; blk < NB; ++blk)
                {
                    gd_mma_16816(c, qa[blk].x, qa[blk].y, kw[u][blk].x, kw[u][blk].y);
                    gd_mma_16816(c, qa[blk].z, qa[blk].w, kw[u][blk].z, kw[u][blk].w);
                }
                // c[0], c[1]: head g, keys jb + 2 t and jb + 2 t + 1
                if(g < FACT)
                {
#pragma unroll
                    for(int e = 0; e < 2; ++e)
                    {
                        const int j = jb + 2 * t + e;
                        float sv    = truncate_to_half_precision(c[e]);
                        sv          = truncate_to_half_precision(__fmul_rn(sv, p.scale));
                        if(j < n)
                        {
                            mx[0]              = fmaxf(mx[0], sv);
                            sc[g * p.cap + j] = __float2half_rz(sv);
                        }
                    }
                }
            }
        }
        // this lane's maximum belongs to head g: over the four lanes of the head, then to slot h
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], 1));
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], 2));
        if(t == 0 and g < FACT)
            wred[warp][g] = mx[0];
    }
    else
    {
        for(int j0 = 0; j0 < n; j0 += U * RPI)
        {
            uint4 w[U];
#pragma unroll
            for(int u = 0; u < U; ++u)
            {
                const int j = j0 + u * RPI + warp * RPW + sub;
                w[u]        = make_uint4(0, 0, 0, 0);
                if(j < n)
                    w[u] = __ldg(reinterpret_cast<const uint4*>(kbase + static_cast<int64_t>(k0 + j) * D) + li);
            }
#pragma unroll
            for(int u = 0; u < U; ++u)
            {
                const int j = j0 + u * RPI + warp * RPW + sub;
                float kf[8];
                gd_unpack8(w[u], kf);
#pragma unroll
                for(int h = 0; h < FACT; ++h)
                {
                    float acc = 0.0f;
#pragma unroll
                    for(int c = 0; c < 8; ++c)
                        acc = fmaf(qf[h][c], kf[c], acc);
#pragma unroll
                    for(int o = LPR / 2; o > 0; o >>= 1)
                        acc += __shfl_xor_sync(0xffffffffu, acc, o);
                    float s = truncate_to_half_precision(acc);
                    s       = truncate_to_half_precision(__fmul_rn(s, p.scale));
                    if(j < n)
                    {
                        mx[h] = fmaxf(mx[h], s);
                        if(li == 0)
                            sc[h * p.cap + j] = __float2half_rz(s);
                    }
                }
            }
        }
#pragma unroll
        for(int h = 0; h < FACT; ++h)
        {
#pragma unroll
            for(int o = 16; o >= LPR; o >>= 1)
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], o));
            if(lane == 0)
                wred[warp][h] = mx[h];
        }
    }
    __syncthreads();
    if(tid < FACT)
    {
        float m = wred[0][tid];
#pragma unroll
        for(int w = 1; w < GD_WARPS; ++w)
            m = fmaxf(m, wred[w][tid]);
        red_m[tid] = m;
    }
    cluster.sync();
    float gm[FACT];
#pragma unroll
    for(int h = 0; h < FACT; ++h)
    {
        float m = -INFINITY;
        for(int r = 0; r < nsplit; ++r)
            m = fmaxf(m, cluster.map_shared_rank(red_m, r)[h]);
        gm[h] = m;
    }

    // ---- phase 2: e = half(exp(x - max)) in place, the sum over the stored halves in fp32
    constexpr float log2e = 1.4426950408889634f;
#pragma unroll
    for(int h = 0; h < FACT; ++h)
    {
        float s = 0.0f;
        for(int j = tid; j < n; j += GD_THREADS)
        {
            const float x = __half2float(sc[h * p.cap + j]);
            const float e = gd_trunc_nonneg(gd_exp2((x - gm[h]) * log2e));
            sc[h * p.cap + j] = __float2half_rz(e);
            s += e;
        }
#pragma unroll
        for(int o = 16; o > 0; o >>= 1)
            s += __shfl_xor_sync(0xffffffffu, s, o);
        if(lane == 0) // (the maxima in wred were read before the cluster barrier)
            wred[warp][h] = s;
    }
    __syncthreads();
    if(tid < FACT)
    {
        float s = 0.0f;
#pragma unroll
        for(int w = 0; w < GD_WARPS; ++w)
            s += wred[w][tid];
        red_s[tid] = s;
    }
    cluster.sync();
    float total[FACT], rcp[FACT];
#pragma unroll
    for(int h = 0; h < FACT; ++h)
    {
        float s = 0.0f;
        for(int r = 0; r < nsplit; ++r)
            s += cluster.map_shared_rank(red_s, r)[h];
        total[h] = s;
        rcp[h]   = __frcp_rn(s);
    }
    // p = half(e / sum): one reciprocal per row and a remainder correction
#pragma unroll
    for(int h = 0; h < FACT; ++h)
        for(int j = tid; j < n; j += GD_THREADS)
        {
            const float e = __half2float(sc[h * p.cap + j]);
            float a       = e * rcp[h];
            a             = __fmaf_rn(__fmaf_rn(-a, total[h], e), rcp[h], a);
            sc[h * p.cap + j] = __float2half_rz(gd_trunc_nonneg(a));
        }
    if constexpr(MMA)
    {
        // the P fragments are read in steps of 16 keys: zero probabilities up to the next multiple
        const int n16 = (n + 15) / 16 * 16;
        for(int i = tid; i < FACT * (n16 - n); i += GD_THREADS)
            sc[(i / (n16 - n)) * p.cap + n + i % (n16 - n)] = __float2half_rz(0.0f);
    }
    __syncthreads();

    // ---- phase 3: partial P V over this CTA's positions
    if constexpr(MMA)
    {
        // 16 keys per warp and step; lane (g, t): keys 2 t, 2 t + 1, 8 + 2 t, 9 + 2 t of the step
        float o[D / 8][4];
#pragma unroll
        for(int i = 0; i < D / 8; ++i)
            o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
        for(int j0 = warp * 16; j0 < n; j0 += GD_WARPS * 16)
        {
            const int ka = j0 + 2 * t, kc = j0 + 8 + 2 * t;
            uint32_t a0 = 0, a2 = 0;
            if(g < FACT)
            {
                a0 = *reinterpret_cast<const uint32_t*>(sc + g * p.cap + ka); // probabilities of keys ka, ka + 1
                a2 = *reinterpret_cast<const uint32_t*>(sc + g * p.cap + kc);
            }
            // all rows of the step first (8 or 16 loads in flight per lane), then the products
            uint4 vr[D / 64][4];
#pragma unroll
            for(int hd = 0; hd < D / 64; ++hd)
            {
                const __half* col = vbase + static_cast<int64_t>(k0) * D + hd * 64 + g * 8;
#pragma unroll
                for(int r = 0; r < 4; ++r)
                {
                    const int key = (r < 2 ? ka : kc) + (r & 1);
                    vr[hd][r]     = make_uint4(0, 0, 0, 0);
                    if(key < n)
                        vr[hd][r] = __ldg(reinterpret_cast<const uint4*>(col + static_cast<int64_t>(key) * D));
                }
            }
#pragma unroll
            for(int hd = 0; hd < D / 64; ++hd)
            {
                const uint32_t wa[4] = {vr[hd][0].x, vr[hd][0].y, vr[hd][0].z, vr[hd][0].w};
                const uint32_t wb[4] = {vr[hd][1].x, vr[hd][1].y, vr[hd][1].z, vr[hd][1].w};
                const uint32_t wc[4] = {vr[hd][2].x, vr[hd][2].y, vr[hd][2].z, vr[hd][2].w};
                const uint32_t wd[4] = {vr[hd][3].x, vr[hd][3].y, vr[hd][3].z, vr[hd][3].w};
#pragma unroll
                for(int i = 0; i < 8; ++i)
                {
                    // column 8 g + i of the four keys, paired along the key index
                    const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
                    const uint32_t b0  = __byte_perm(wa[i >> 1], wb[i >> 1], sel);
                    const uint32_t b1  = __byte_perm(wc[i >> 1], wd[i >> 1], sel);
                    gd_mma_16816(o[hd * 8 + i], a0, a2, b0, b1);
                }
            }
        }
        // o[8 hd + i][e]: head g, column 64 hd + 8 (2 t + e) + i
        if(g < FACT)
        {
#pragma unroll
            for(int hd = 0; hd < D / 64; ++hd)
#pragma unroll
                for(int i = 0; i < 8; ++i)
#pragma unroll
                    for(int e = 0; e < 2; ++e)
                        part[(warp * FACT + g) * D + hd * 64 + 8 * (2 * t + e) + i] = o[hd * 8 + i][e];
        }
    }
    else
    {
        float acc[FACT][8];
#pragma unroll
        for(int h = 0; h < FACT; ++h)
#pragma unroll
            for(int c = 0; c < 8; ++c)
                acc[h][c] = 0.0f;
        for(int j0 = 0; j0 < n; j0 += U * RPI)
        {
            uint4 w[U];
#pragma unroll
            for(int u = 0; u < U; ++u)
            {
                const int j = j0 + u * RPI + warp * RPW + sub;
                w[u]        = make_uint4(0, 0, 0, 0);
                if(j < n)
                    w[u] = __ldg(reinterpret_cast<const uint4*>(vbase + static_cast<int64_t>(k0 + j) * D) + li);
            }
#pragma unroll
            for(int u = 0; u < U; ++u)
            {
                const int j = j0 + u * RPI + warp * RPW + sub;
                if(j >= n)
                    continue;
                float vf[8];
                gd_unpack8(w[u], vf);
#pragma unroll
                for(int h = 0; h < FACT; ++h)
                {
                    const float pj = __half2float(sc[h * p.cap + j]);
#pragma unroll
                    for(int c = 0; c < 8; ++c)
                        acc[h][c] = fmaf(pj, vf[c], acc[h][c]);
                }
            }
        }
#pragma unroll
        for(int h = 0; h < FACT; ++h)
#pragma unroll
            for(int c = 0; c < 8; ++c)
            {
#pragma unroll
                for(int o = 16; o >= LPR; o >>= 1)
                    acc[h][c] += __shfl_xor_sync(0xffffffffu, acc[h][c], o);
                if(sub == 0)
                    part[(warp * FACT + h) * D + li * 8 + c] = acc[h][c];
            }
    }
    __syncthreads();
    for(int i = tid; i < FACT * D; i += GD_THREADS)
    {
        float s = 0.0f;
#pragma unroll
        for(int w = 0; w < GD_WARPS; ++w)
            s += part[w * FACT * D + i];
        cta_out[i] = s;
    }
    cluster.sync();
    if(rank == 0)
        for(int i = tid; i < FACT * D; i += GD_THREADS)
        {
            float s = 0.0f;
            for(int r = 0; r < nsplit; ++r)
                s += cluster.map_shared_rank(cta_out, r)[i];
            const int h = i / D, c = i - h * D;
            p.out[(static_cast<int64_t>(b) * p.kv_heads * FACT + head0 + h) * D + c] = __float2half_rz(s);
        }
    // no CTA leaves while rank 0 may still read its shared memory
    cluster.sync();
}

static size_t gqa_decode_smem(int64_t fact, int64_t head, int64_t cap);

template <int D, int FACT, bool MMA>
int launch_gqa_decode(const gqa_decode_params& p, int batch, int nsplit, cudaStream_t stream)
{
    const size_t smem = gqa_decode_smem(FACT, D, p.cap);
    if(smem > 200 * 1024)
        return MGX_E_TOO_LARGE;
    auto* kernel = gqa_decode_kernel<D, FACT, MMA>;
    static size_t opted = 0;
    if(opted == 0) // (the static arrays count toward the 48 KB a kernel gets without opting in)
    {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if(e != cudaSuccess)
            return static_cast<int>(e);
        opted = 200 * 1024;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = dim3(static_cast<unsigned>(nsplit), static_cast<unsigned>(p.kv_heads), static_cast<unsigned>(batch));
    cfg.blockDim         = dim3(GD_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(nsplit);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs    = attr;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, p));
}

} // namespace mgx

namespace mgx {
// splits: enough CTAs for the 148 SMs (measured: splitting further, 1024 CTAs in clusters of two
// instead of 512 single ones at batch 16 x 32 heads, is 7 % slower), at most the portable cluster
// size, at least 64 positions each
static int gqa_decode_splits(int64_t batch, int64_t kv_heads, int64_t cache_seq)
{
    int nsplit = 1;
    while(nsplit < 8 and batch * kv_heads * nsplit < 148 and cache_seq / (2 * nsplit) >= 64)
        nsplit *= 2;
    return nsplit;
}
static size_t gqa_decode_smem(int64_t fact, int64_t head, int64_t cap)
{
    return sizeof(__half) * fact * cap + sizeof(float) * GD_WARPS * fact * head;
}
} // namespace mgx

extern "C" int mgx_cuda_gqa_decode_supported(int64_t batch, int64_t heads, int64_t kv_heads, int64_t head,
                                             int64_t cache_seq)
{
    using namespace mgx;
    if(batch <= 0 or heads <= 0 or kv_heads <= 0 or cache_seq <= 0 or heads % kv_heads != 0)
        return 0;
    const int64_t fact = heads / kv_heads;
    if((head != 64 and head != 128) or (fact != 1 and fact != 2 and fact != 4 and fact != 8))
        return 0;
    if(batch > 65535 or kv_heads > 65535 or cache_seq > (int64_t{1} << 30))
        return 0;
    const int nsplit  = gqa_decode_splits(batch, kv_heads, cache_seq);
    const int64_t cap = ((cache_seq + nsplit - 1) / nsplit + 15) / 16 * 16;
    return gqa_decode_smem(fact, head, cap) <= 200 * 1024 ? 1 : 0;
}

extern "C" int mgx_cuda_gqa_decode_attention(const mgx_gqa_decode_desc* d, const void* q, const void* k_cache,
                                             const void* v_cache, const void* seqlens, void* out, void* stream_)
{
    using namespace mgx;
    if(d == nullptr or q == nullptr or k_cache == nullptr or v_cache == nullptr or seqlens == nullptr or out == nullptr)
        return MGX_E_INVALID_ARG;
    if(d->batch <= 0 or d->heads <= 0 or d->kv_heads <= 0 or d->cache_seq <= 0 or d->heads % d->kv_heads != 0)
        return MGX_E_INVALID_ARG;
    if(d->seqlens_type != MGX_I32 and d->seqlens_type != MGX_I64)
        return MGX_E_UNSUPPORTED;
    if(d->head != 64 and d->head != 128)
        return MGX_E_UNSUPPORTED;
    const int64_t fact = d->heads / d->kv_heads;
    if(fact != 1 and fact != 2 and fact != 4 and fact != 8)
        return MGX_E_UNSUPPORTED;
    if(d->batch > 65535 or d->kv_heads > 65535 or d->cache_seq > (int64_t{1} << 30))
        return MGX_E_TOO_LARGE;
    // rows are read as 16-byte vectors
    if((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) % 16 != 0 or
       reinterpret_cast<uintptr_t>(q) % 2 != 0 or reinterpret_cast<uintptr_t>(out) % 2 != 0)
        return MGX_E_ALIGNMENT;
    const int nsplit = gqa_decode_splits(d->batch, d->kv_heads, d->cache_seq);
    gqa_decode_params p{};
    p.q    = static_cast<const __half*>(q);
    p.q_sb = d->q_batch_stride, p.q_sh = d->q_head_stride;
    p.k = static_cast<const __half*>(k_cache), p.v = static_cast<const __half*>(v_cache);
    p.seqlens     = seqlens;
    p.seqlens_i64 = d->seqlens_type == MGX_I64 ? 1 : 0;
    p.out         = static_cast<__half*>(out);
    p.scale       = d->scale;
    p.cache_seq   = static_cast<int>(d->cache_seq);
    p.kv_heads    = static_cast<int>(d->kv_heads);
    p.cap         = static_cast<int>(((d->cache_seq + nsplit - 1) / nsplit + 15) / 16 * 16);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int batch     = static_cast<int>(d->batch);
    // four or eight query heads per KV head: the tensor-core form, which reads the query rows as
    // 16-byte vectors
    const bool mma = fact >= 4 and reinterpret_cast<uintptr_t>(q) % 16 == 0 and d->q_batch_stride % 8 == 0 and
                     d->q_head_stride % 8 == 0;
#define MGX_GD_CASE(DD, FF)                                                         \
    if(d->head == DD and fact == FF)                                                \
    {                                                                               \
        if(FF >= 4 and mma)                                                         \
            return launch_gqa_decode<DD, FF, (FF >= 4)>(p, batch, nsplit, stream);  \
        return launch_gqa_decode<DD, FF, false>(p, batch, nsplit, stream);          \
    }
    MGX_GD_CASE(128, 1)
    MGX_GD_CASE(128, 2)
    MGX_GD_CASE(128, 4)
    MGX_GD_CASE(128, 8)
    MGX_GD_CASE(64, 1)
    MGX_GD_CASE(64, 2)
    MGX_GD_CASE(64, 4)
    MGX_GD_CASE(64, 8)
#undef MGX_GD_CASE
    return MGX_E_UNSUPPORTED;
}
