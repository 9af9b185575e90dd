// Multi-head attention on fp16 tensors as one kernel: softmax(scale * Q K^T) V per (batch, head),
// the fusion of the instruction chain an encoder layer holds between its projections
//   reshape [B,S,H,D] -> transpose -> dot(Q, K^T) -> mul(scale) -> softmax -> dot(P, V) -> transpose
//   -> reshape [B*S, H*D]
// (what the reference's GPU target hands to its fused attention kernels,
// src/targets/gpu/fuse_mlir.cpp:1161-1234 / src/fuse_attention.cpp).  Q, K and V are read in place
// from row-strided [B*S, H*D] matrices (a head is a 64-column slice of a row), so the head split
// and merge need no copies; the result can additionally (or only) be written through a
// per-tensor quantizelinear as int8, the input of the quantized output projection.
//
// Two kernels.  attention_f16_chain_kernel (sequences of up to 1024 keys) makes every rounding of
// the operator chain it stands in for: the scores of a CTA's 64 query rows stay in shared memory as
// half (dot -> half, * scale -> half, truncating like migraphx::half), the softmax is ref_softmax's
// (src/targets/ref/lowering.cpp:253-320: exp(x - max) stored as half, summed in fp32, divided and
// stored as half), and the second product multiplies those half probabilities with V.  What
// differs from the reference is the order of the fp32 sums (its dot accumulates in double) and
// the last bit of exp: a result lands in the neighbouring half for about one element in a
// thousand.  That matters because a quantizelinear usually follows: a kernel that keeps more
// precision than the chain (the second kernel) moves values across its rounding boundaries.
// attention_f16_kernel (longer sequences) runs the softmax in fp32 over key blocks with a running
// maximum and sum (flash-attention style); against the chain it stays within the fp16 tolerance
// of the tests (rtol 2e-2 / atol 1e-2).
//
// One CTA = 4 warps = 64 query rows of one head; keys / values stream through shared memory in
// 64-row blocks (cp.async double buffering, 16-byte chunks XOR-swizzled against bank conflicts);
// mma.sync.m16n8k16 with ldmatrix fragments.  This is a "next"-row kernel off the quantized-GEMM
// path proper: it is sized by its 3.6 GFLOP per encoder layer, not by the tensor-core peak.
#include "common.cuh"
#include "qgemm_math.cuh"
#include "ptx.cuh"
#include <cuda_fp16.h>
#include <cfloat>

namespace mgx {

constexpr int AT_D  = 64; // head dimension
constexpr int AT_BM = 64; // query rows per CTA (16 per warp)
constexpr int AT_BN = 64; // keys per block

struct attention_params
{
    const __half* q;
    const __half* k;
    const __half* v;
    __half* o;
    int8_t* oq;
    int64_t ldq, ldk, ldv, ldo, ldoq;
    int seq, heads;
    float scale;
    float q_scale, q_rcp, q_zp;
};

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid)
{
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int bytes  = valid ? 16 : 0; // zero-fill when the row is outside the sequence
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem)
{
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem)
{
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
                 "{%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x for x <= 0 (and -inf-like arguments, which give 0): one instruction
__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// A [rows, 64] fp16 tile in shared memory: 128-byte rows, the 16-byte chunk index XOR-ed with the
// row's low three bits.
__device__ __forceinline__ __half* tile_ptr(__half* tile, int row, int chunk)
{
    return tile + row * AT_D + ((chunk ^ (row & 7)) << 3);
}

// 64 rows x 64 columns starting at g (row stride ld), rows at or beyond `rows_left` zero-filled
__device__ __forceinline__ void load_tile(__half* tile, const __half* g, int64_t ld, int rows_left, int tid)
{
#pragma unroll
    for(int i = 0; i < 4; ++i)
    {
        const int c   = tid + i * 128; // 512 chunks of 16 bytes
        const int row = c >> 3, chunk = c & 7;
        const bool ok = row < rows_left;
        cp_async_16(tile_ptr(tile, row, chunk), g + (ok ? row : 0) * ld + chunk * 8, ok);
    }
}

__global__ void __launch_bounds__(128) attention_f16_kernel(const attention_params p)
{
    __shared__ __align__(128) __half sq[AT_BM * AT_D];
    __shared__ __align__(128) __half sk[2][AT_BN * AT_D];
    __shared__ __align__(128) __half sv[2][AT_BN * AT_D];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int q0   = blockIdx.x * AT_BM;
    const int head = blockIdx.y;
    const int64_t row_base = static_cast<int64_t>(blockIdx.z) * p.seq; // first row of this sequence
    const __half* qg = p.q + (row_base + q0) * p.ldq + head * AT_D;
    const __half* kg = p.k + row_base * p.ldk + head * AT_D;
    const __half* vg = p.v + row_base * p.ldv + head * AT_D;
    const int nblocks = (p.seq + AT_BN - 1) / AT_BN;

    load_tile(sq, qg, p.ldq, p.seq - q0, tid);
    load_tile(sk[0], kg, p.ldk, p.seq, tid);
    load_tile(sv[0], vg, p.ldv, p.seq, tid);
    cp_async_commit();

    uint32_t qa[4][4]; // this warp's 16 query rows: A fragments of the four 16-wide k steps
    float o[8][4];     // output accumulators: 8 column tiles of 8
#pragma unroll
    for(int j = 0; j < 8; ++j)
        o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    float m_run[2] = {-FLT_MAX, -FLT_MAX}; // running maxima of rows g and g + 8
    float l_run[2] = {0.0f, 0.0f};         // running sums (this thread's share)
    constexpr float log2e = 1.4426950408889634f;

    for(int kb = 0; kb < nblocks; ++kb)
    {
        const int buf = kb & 1;
        if(kb + 1 < nblocks)
        {
            const int k1 = (kb + 1) * AT_BN;
            load_tile(sk[buf ^ 1], kg + static_cast<int64_t>(k1) * p.ldk, p.ldk, p.seq - k1, tid);
            load_tile(sv[buf ^ 1], vg + static_cast<int64_t>(k1) * p.ldv, p.ldv, p.seq - k1, tid);
            cp_async_commit();
            cp_async_wait<1>();
        }
        else
            cp_async_wait<0>();
        __syncthreads();
        if(kb == 0)
        {
#pragma unroll
            for(int ks = 0; ks < 4; ++ks)
                ldmatrix_x4(qa[ks], tile_ptr(sq, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * ks + (lane >> 4)));
        }
        // ---- S = Q K^T for this key block: 16 rows x 64 keys per warp
        float s[8][4];
#pragma unroll
        for(int j = 0; j < 8; ++j)
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
        for(int ks = 0; ks < 4; ++ks)
        {
#pragma unroll
            for(int jp = 0; jp < 4; ++jp) // two key tiles of 8 per ldmatrix.x4
            {
                uint32_t kf[4];
                ldmatrix_x4(kf, tile_ptr(sk[buf], jp * 16 + (lane & 7) + (lane >> 4) * 8, 2 * ks + ((lane >> 3) & 1)));
                mma_16816(s[2 * jp], qa[ks], kf[0], kf[1]);
                mma_16816(s[2 * jp + 1], qa[ks], kf[2], kf[3]);
            }
        }
        // ---- scores as the separate operators round them (dot -> half, * scale -> half; the mantissa
        // cut is the truncation for every value in the normal half range, and smaller ones vanish in
        // the softmax anyway), keys beyond the sequence masked (only the last block can hold any)
        const int kbase = kb * AT_BN;
        float mx[2] = {-FLT_MAX, -FLT_MAX};
        const bool tail = kbase + AT_BN > p.seq;
#pragma unroll
        for(int j = 0; j < 8; ++j)
        {
#pragma unroll
            for(int e = 0; e < 4; ++e)
            {
                float x = __uint_as_float(__float_as_uint(s[j][e]) & 0xFFFFE000u);
                x       = __uint_as_float(__float_as_uint(x * p.scale) & 0xFFFFE000u);
                if(tail)
                    x = kbase + j * 8 + 2 * t + (e & 1) < p.seq ? x : -FLT_MAX;
                s[j][e] = x;
                mx[e >> 1] = fmaxf(mx[e >> 1], x);
            }
        }
        float corr[2], mneg[2];
#pragma unroll
        for(int r = 0; r < 2; ++r)
        {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            corr[r]  = fast_exp2((m_run[r] - m_new) * log2e);
            m_run[r] = m_new;
            mneg[r]  = -m_new * log2e;
            l_run[r] *= corr[r];
        }
#pragma unroll
        for(int j = 0; j < 8; ++j)
        {
            o[j][0] *= corr[0], o[j][1] *= corr[0];
            o[j][2] *= corr[1], o[j][3] *= corr[1];
        }
        // ---- P = exp(s - max) as fp16 A fragments; O += P V
        uint32_t pa[4][4];
#pragma unroll
        for(int j = 0; j < 8; ++j)
        {
            float e[4];
#pragma unroll
            for(int i = 0; i < 4; ++i)
            {
                e[i] = fast_exp2(fmaf(s[j][i], log2e, mneg[i >> 1])); // exp(s - max)
                l_run[i >> 1] += e[i];
            }
            const __half2 lo = __floats2half2_rn(e[0], e[1]); // row g
            const __half2 hi = __floats2half2_rn(e[2], e[3]); // row g + 8
            // key tile j covers k columns 8j .. 8j+7 of the 16-wide step j / 2
            pa[j >> 1][(j & 1) * 2]     = *reinterpret_cast<const uint32_t*>(&lo);
            pa[j >> 1][(j & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&hi);
        }
#pragma unroll
        for(int ks = 0; ks < 4; ++ks) // 16 keys per step
        {
#pragma unroll
            for(int jp = 0; jp < 4; ++jp) // two output column tiles per ldmatrix.x4.trans
            {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, tile_ptr(sv[buf], ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * jp + (lane >> 4)));
                mma_16816(o[2 * jp], pa[ks], vf[0], vf[1]);
                mma_16816(o[2 * jp + 1], pa[ks], vf[2], vf[3]);
            }
        }
        __syncthreads(); // the other buffer is overwritten by the next iteration's loads
    }
    // ---- normalise and store rows g and g + 8 of this warp's 16
#pragma unroll
    for(int r = 0; r < 2; ++r)
    {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float q_lo = -128.0f - p.q_zp, q_hi = 127.0f - p.q_zp;
#pragma unroll
    for(int r = 0; r < 2; ++r)
    {
        const int row = q0 + warp * 16 + g + r * 8;
        if(row >= p.seq)
            continue;
        const float inv = 1.0f / l_run[r];
#pragma unroll
        for(int j = 0; j < 8; ++j)
        {
            const float a = truncate_to_half_precision(o[j][2 * r] * inv);
            const float b = truncate_to_half_precision(o[j][2 * r + 1] * inv);
            const int col = head * AT_D + j * 8 + 2 * t;
            if(p.o != nullptr)
                *reinterpret_cast<uint32_t*>(p.o + (row_base + row) * p.ldo + col) = cvt_rz_f16x2(a, b);
            if(p.oq != nullptr)
            {
                // quantizelinear of the half result: quotient in half (truncated), round half to even
                uint32_t qb[2];
                const float vals[2] = {a, b};
#pragma unroll
                for(int e = 0; e < 2; ++e)
                {
                    float qv        = __fmul_rn(vals[e], p.q_rcp);
                    const float rem = __fmaf_rn(-p.q_scale, qv, vals[e]);
                    qv              = truncate_to_half_precision(__fmaf_rn(rem, p.q_rcp, qv));
                    qv              = fmaxf(q_lo, fminf(q_hi, qv));
                    qb[e] = static_cast<uint32_t>(__float_as_int(__fadd_rn(qv, 12582912.0f)) - 0x4B400000 +
                                                  static_cast<int>(p.q_zp)) & 0xFFu;
                }
                *reinterpret_cast<uint16_t*>(p.oq + (row_base + row) * p.ldoq + col) =
                    static_cast<uint16_t>(qb[0] | (qb[1] << 8));
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The operator chain's own roundings (see the head of the file).  Dynamic shared memory:
// Q tile | two K / V tiles | scores [64][sp] half (sp = keys rounded up to 64, + 8 against bank
// conflicts) | row maxima.
constexpr int AT_CHAIN_MAX_SEQ = 1024;

// v >= 0 truncated to half precision, subnormal halves included (multiples of 2^-24 below 2^-14:
// v + 0.5 rounded toward zero keeps exactly those bits)
__device__ __forceinline__ float trunc_half_nonneg(float v)
{
    const float big   = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    const float small = __fsub_rn(__fadd_rz(v, 0.5f), 0.5f);
    return v < 6.103515625e-5f ? small : big;
}

constexpr int ATC_THREADS = 256;

// load_tile for a block of ATC_THREADS threads
__device__ __forceinline__ void load_tile_256(__half* tile, const __half* g, int64_t ld, int rows_left, int tid)
{
#pragma unroll
    for(int i = 0; i < 2; ++i)
    {
        const int c   = tid + i * ATC_THREADS; // 512 chunks of 16 bytes
        const int row = c >> 3, chunk = c & 7;
        const bool ok = row < rows_left;
        cp_async_16(tile_ptr(tile, row, chunk), g + (ok ? row : 0) * ld + chunk * 8, ok);
    }
}

// Eight warps per 64 query rows: in the two matrix phases warp (rg, kh) owns the 16 rows of row
// group rg and half kh of every 64-key tile (its scores / its share of P V, the two shares added
// through shared memory at the end); in the softmax phase every warp owns 8 whole rows.  Twice the
// warps of one-warp-per-16-rows at half the accumulator registers each: the kernel is bound by
// the latency of dependent instructions, which only more resident warps hide.
// NVMAX: half2 pairs per lane and row the softmax phase holds in registers (keys <= 64 NVMAX).
template <int NVMAX, int RG>
__global__ void __launch_bounds__(ATC_THREADS, 3) attention_f16_chain_kernel(const attention_params p, const int sp)
{
    constexpr int BMC = RG * 16;      // query rows per CTA
    constexpr int KS  = 8 / RG;       // warps that share a row group: each takes 64 / KS keys of a tile
    constexpr int JPW = 4 / KS;       // 16-key groups of a tile per warp
    constexpr int RPW = BMC / 8;      // whole rows per warp in the softmax phase
    extern __shared__ __align__(128) uint8_t at_smem[];
    __half* sq     = reinterpret_cast<__half*>(at_smem);
    __half* skv[2] = {sq + AT_BM * AT_D, sq + AT_BM * AT_D + AT_BN * AT_D};
    __half* sc     = sq + AT_BM * AT_D + 2 * AT_BN * AT_D; // [BMC][sp]
    float* rowmax  = reinterpret_cast<float*>(sc + BMC * sp); // [KS][BMC]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rg = warp % RG, kh = warp / RG;
    const int q0   = blockIdx.x * BMC;
    const int head = blockIdx.y;
    const int64_t row_base = static_cast<int64_t>(blockIdx.z) * p.seq;
    const __half* qg = p.q + (row_base + q0) * p.ldq + head * AT_D;
    const __half* kg = p.k + row_base * p.ldk + head * AT_D;
    const __half* vg = p.v + row_base * p.ldv + head * AT_D;
    const int nblocks = (p.seq + AT_BN - 1) / AT_BN;

    load_tile_256(sq, qg, p.ldq, p.seq - q0, tid);
    load_tile_256(skv[0], kg, p.ldk, p.seq, tid);
    cp_async_commit();

    // ---- phase 1: scores = half(half(Q K^T) * scale) into shared memory, row maxima
    {
        uint32_t qa[4][4];
        // running maxima of the stored halves, packed: mxh[r] = {max over even keys, max over odd
        // keys} of row g + 8 r
        const __half2 lowest = __floats2half2_rn(-65504.0f, -65504.0f);
        __half2 mxh[2]       = {lowest, lowest};
        for(int kb = 0; kb < nblocks; ++kb)
        {
            const int buf = kb & 1;
            if(kb + 1 < nblocks)
            {
                const int k1 = (kb + 1) * AT_BN;
                load_tile_256(skv[buf ^ 1], kg + static_cast<int64_t>(k1) * p.ldk, p.ldk, p.seq - k1, tid);
                cp_async_commit();
                cp_async_wait<1>();
            }
            else
                cp_async_wait<0>();
            __syncthreads();
            if(kb == 0)
            {
#pragma unroll
                for(int ks = 0; ks < 4; ++ks)
                    ldmatrix_x4(qa[ks], tile_ptr(sq, rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * ks + (lane >> 4)));
            }
            float s[2 * JPW][4];
#pragma unroll
            for(int j = 0; j < 2 * JPW; ++j)
                s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
            for(int ks = 0; ks < 4; ++ks)
            {
#pragma unroll
                for(int jp = 0; jp < JPW; ++jp)
                {
                    uint32_t kf[4];
                    ldmatrix_x4(kf, tile_ptr(skv[buf], (kh * JPW + jp) * 16 + (lane & 7) + (lane >> 4) * 8,
                                             2 * ks + ((lane >> 3) & 1)));
                    mma_16816(s[2 * jp], qa[ks], kf[0], kf[1]);
                    mma_16816(s[2 * jp + 1], qa[ks], kf[2], kf[3]);
                }
            }
            const int kbase = kb * AT_BN + kh * (16 * JPW);
            const bool tail = kbase + 16 * JPW > p.seq;
            // half(Q K^T): mantissa cut (a score in the half subnormal range keeps a few more bits:
            // below 2^-24 absolute, invisible after the exponential); half(score * scale): the
            // packing conversion itself rounds toward zero, subnormal halves included
#pragma unroll
            for(int j = 0; j < 2 * JPW; ++j)
            {
                float x[4];
#pragma unroll
                for(int e = 0; e < 4; ++e)
                    x[e] = __uint_as_float(__float_as_uint(s[j][e]) & 0xFFFFE000u) * p.scale;
                if(tail)
                {
                    // keys that do not exist: the lowest half, whose exponential is 0
#pragma unroll
                    for(int e = 0; e < 4; ++e)
                        if(kbase + j * 8 + 2 * t + (e & 1) >= p.seq)
                            x[e] = -65504.0f;
                }
                const uint32_t w0 = cvt_rz_f16x2(x[0], x[1]), w1 = cvt_rz_f16x2(x[2], x[3]);
                mxh[0]            = __hmax2(mxh[0], *reinterpret_cast<const __half2*>(&w0));
                mxh[1]            = __hmax2(mxh[1], *reinterpret_cast<const __half2*>(&w1));
                const int col     = kbase + j * 8 + 2 * t;
                *reinterpret_cast<uint32_t*>(sc + (rg * 16 + g) * sp + col)     = w0;
                *reinterpret_cast<uint32_t*>(sc + (rg * 16 + g + 8) * sp + col) = w1;
            }
            __syncthreads(); // the other tile is overwritten by the next iteration's load
        }
        // V's first tile travels while the softmax runs
        load_tile_256(skv[0], vg, p.ldv, p.seq, tid);
        cp_async_commit();
#pragma unroll
        for(int r = 0; r < 2; ++r)
        {
            const float2 m2 = __half22float2(mxh[r]);
            float mx        = fmaxf(m2.x, m2.y);
            mx              = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx              = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            if(t == 0)
                rowmax[kh * BMC + rg * 16 + g + r * 8] = mx;
        }
    }
    __syncthreads();

    // ---- phase 2: ref_softmax on this warp's 8 rows, in place: e = half(exp(x - max)), sum over
    // the stored halves in fp32, p = half(e / sum).  exp through ex2.approx (relative error ~1e-6
    // against the 5e-4 spacing of the halves it is truncated to), the quotient from one reciprocal
    // per row and a remainder correction (correctly rounded before the truncation).
    {
        const int nv = nblocks; // half2 pairs per lane and row: keys / 64
        constexpr float log2e = 1.4426950408889634f;
#pragma unroll 1
        for(int r = 0; r < RPW; ++r)
        {
            const int row = warp * RPW + r;
            __half* rowp  = sc + row * sp;
            float m       = rowmax[row];
#pragma unroll
            for(int h = 1; h < KS; ++h)
                m = fmaxf(m, rowmax[h * BMC + row]);
            // the packing conversion rounds toward zero (subnormal halves included); the sum runs
            // over the stored halves
            float2 e[NVMAX];
            float sum = 0.0f;
#pragma unroll
            for(int i = 0; i < NVMAX; ++i)
            {
                if(i < nv)
                {
                    const float2 x   = __half22float2(*reinterpret_cast<const __half2*>(rowp + i * 64 + lane * 2));
                    const uint32_t h = cvt_rz_f16x2(fast_exp2((x.x - m) * log2e), fast_exp2((x.y - m) * log2e));
                    e[i]             = __half22float2(*reinterpret_cast<const __half2*>(&h));
                    sum += e[i].x + e[i].y;
                }
            }
#pragma unroll
            for(int o = 16; o > 0; o >>= 1)
                sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const float rcp = __frcp_rn(sum);
#pragma unroll
            for(int i = 0; i < NVMAX; ++i)
            {
                if(i < nv)
                {
                    float a = e[i].x * rcp, b = e[i].y * rcp;
                    a       = __fmaf_rn(__fmaf_rn(-a, sum, e[i].x), rcp, a);
                    b       = __fmaf_rn(__fmaf_rn(-b, sum, e[i].y), rcp, b);
                    *reinterpret_cast<uint32_t*>(rowp + i * 64 + lane * 2) = cvt_rz_f16x2(a, b);
                }
            }
        }
    }
    __syncthreads();

    // ---- phase 3: O = P V with the half probabilities as A fragments straight from shared
    // memory; this warp's half of every tile's keys
    float o[8][4];
#pragma unroll
    for(int j = 0; j < 8; ++j)
        o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    for(int kb = 0; kb < nblocks; ++kb)
    {
        const int buf = kb & 1;
        if(kb + 1 < nblocks)
        {
            const int k1 = (kb + 1) * AT_BN;
            load_tile_256(skv[buf ^ 1], vg + static_cast<int64_t>(k1) * p.ldv, p.ldv, p.seq - k1, tid);
            cp_async_commit();
            cp_async_wait<1>();
        }
        else
            cp_async_wait<0>();
        __syncthreads();
#pragma unroll
        for(int k2 = 0; k2 < JPW; ++k2)
        {
            const int ks = kh * JPW + k2;
            uint32_t pa[4];
            ldmatrix_x4(pa, sc + (rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * sp + kb * AT_BN + ks * 16 +
                                (lane >> 4) * 8);
#pragma unroll
            for(int jp = 0; jp < 4; ++jp)
            {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, tile_ptr(skv[buf], ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * jp + (lane >> 4)));
                mma_16816(o[2 * jp], pa, vf[0], vf[1]);
                mma_16816(o[2 * jp + 1], pa, vf[2], vf[3]);
            }
        }
        __syncthreads();
    }
    // the key shares are added in a fixed order: the partial sums of shares 1 .. KS-1 go through
    // shared memory (tiles and scores are free now; (KS - 1) BMC x 64 floats = 16 or 24 KB from the start)
    float* red = reinterpret_cast<float*>(at_smem);
    if(kh != 0)
    {
#pragma unroll
        for(int j = 0; j < 8; ++j)
#pragma unroll
            for(int r = 0; r < 2; ++r)
                *reinterpret_cast<float2*>(red + ((kh - 1) * BMC + rg * 16 + g + r * 8) * AT_D + j * 8 + 2 * t) =
                    make_float2(o[j][2 * r], o[j][2 * r + 1]);
    }
    __syncthreads();
    if(kh != 0)
        return;
#pragma unroll
    for(int h = 1; h < KS; ++h)
#pragma unroll
        for(int j = 0; j < 8; ++j)
#pragma unroll
            for(int r = 0; r < 2; ++r)
            {
                const float2 u =
                    *reinterpret_cast<const float2*>(red + ((h - 1) * BMC + rg * 16 + g + r * 8) * AT_D + j * 8 + 2 * t);
                o[j][2 * r] += u.x;
                o[j][2 * r + 1] += u.y;
            }
    const float q_lo = -128.0f - p.q_zp, q_hi = 127.0f - p.q_zp;
#pragma unroll
    for(int r = 0; r < 2; ++r)
    {
        const int row = q0 + rg * 16 + g + r * 8;
        if(row >= p.seq)
            continue;
#pragma unroll
        for(int j = 0; j < 8; ++j)
        {
            const float a = truncate_to_half_precision(o[j][2 * r]);
            const float b = truncate_to_half_precision(o[j][2 * r + 1]);
            const int col = head * AT_D + j * 8 + 2 * t;
            if(p.o != nullptr)
                *reinterpret_cast<uint32_t*>(p.o + (row_base + row) * p.ldo + col) = cvt_rz_f16x2(a, b);
            if(p.oq != nullptr)
            {
                uint32_t qb[2];
                const float vals[2] = {a, b};
#pragma unroll
                for(int e = 0; e < 2; ++e)
                {
                    float qv        = __fmul_rn(vals[e], p.q_rcp);
                    const float rem = __fmaf_rn(-p.q_scale, qv, vals[e]);
                    qv              = truncate_to_half_precision(__fmaf_rn(rem, p.q_rcp, qv));
                    qv              = fmaxf(q_lo, fminf(q_hi, qv));
                    qb[e] = static_cast<uint32_t>(__float_as_int(__fadd_rn(qv, 12582912.0f)) - 0x4B400000 +
                                                  static_cast<int>(p.q_zp)) & 0xFFu;
                }
                *reinterpret_cast<uint16_t*>(p.oq + (row_base + row) * p.ldoq + col) =
                    static_cast<uint16_t>(qb[0] | (qb[1] << 8));
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The operator chain's roundings without a score buffer: three passes over the keys, each
// recomputing the 16 x 64 score tile on the tensor cores (the tensor pipe is nearly idle in this
// kernel, the instruction slots of the element-wise work are what it is short of):
//   pass 0: row maxima of the half scores;
//   pass 1: sum over e = half(exp(x - max));
//   pass 2: p = half(e / sum) straight into the A fragments of P V.
// Every value is rounded exactly as in attention_f16_chain_kernel; only the order of the fp32
// additions of the row sum differs.  40 KB of static shared memory (Q, two K and two V tiles) and
// no limit on the number of keys.
__global__ void __launch_bounds__(128, 4) attention_f16_chain3_kernel(const attention_params p)
{
    __shared__ __align__(128) __half sq[AT_BM * AT_D];
    __shared__ __align__(128) __half sk[2][AT_BN * AT_D];
    __shared__ __align__(128) __half sv[2][AT_BN * AT_D];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int q0   = blockIdx.x * AT_BM;
    const int head = blockIdx.y;
    const int64_t row_base = static_cast<int64_t>(blockIdx.z) * p.seq;
    const __half* qg = p.q + (row_base + q0) * p.ldq + head * AT_D;
    const __half* kg = p.k + row_base * p.ldk + head * AT_D;
    const __half* vg = p.v + row_base * p.ldv + head * AT_D;
    const int nblocks = (p.seq + AT_BN - 1) / AT_BN;
    const int total   = 3 * nblocks;

    load_tile(sq, qg, p.ldq, p.seq - q0, tid);
    load_tile(sk[0], kg, p.ldk, p.seq, tid);
    cp_async_commit();

    uint32_t qa[4][4];
    float o[8][4];
#pragma unroll
    for(int j = 0; j < 8; ++j)
        o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    const __half2 lowest = __floats2half2_rn(-65504.0f, -65504.0f);
    __half2 mxh[2]       = {lowest, lowest};
    float m[2] = {0.0f, 0.0f}, sum[2] = {0.0f, 0.0f}, rcp[2] = {0.0f, 0.0f};
    constexpr float log2e = 1.4426950408889634f;

    int pass = 0, kb = 0;
    for(int it = 0; it < total; ++it)
    {
        const int buf = it & 1;
        if(it + 1 < total)
        {
            const int kn    = kb + 1 == nblocks ? 0 : kb + 1;
            const int pn    = kb + 1 == nblocks ? pass + 1 : pass;
            const int k1    = kn * AT_BN;
            load_tile(sk[buf ^ 1], kg + static_cast<int64_t>(k1) * p.ldk, p.ldk, p.seq - k1, tid);
            if(pn == 2)
                load_tile(sv[buf ^ 1], vg + static_cast<int64_t>(k1) * p.ldv, p.ldv, p.seq - k1, tid);
            cp_async_commit();
            cp_async_wait<1>();
        }
        else
            cp_async_wait<0>();
        __syncthreads();
        if(it == 0)
        {
#pragma unroll
            for(int ks = 0; ks < 4; ++ks)
                ldmatrix_x4(qa[ks], tile_ptr(sq, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * ks + (lane >> 4)));
        }
        // ---- the tile's scores as halves: w[j][r] = keys 8 j + 2 t, + 1 of row g + 8 r
        uint32_t w[8][2];
        {
            float s[8][4];
#pragma unroll
            for(int j = 0; j < 8; ++j)
                s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
            for(int ks = 0; ks < 4; ++ks)
            {
#pragma unroll
                for(int jp = 0; jp < 4; ++jp)
                {
                    uint32_t kf[4];
                    ldmatrix_x4(kf, tile_ptr(sk[buf], jp * 16 + (lane & 7) + (lane >> 4) * 8, 2 * ks + ((lane >> 3) & 1)));
                    mma_16816(s[2 * jp], qa[ks], kf[0], kf[1]);
                    mma_16816(s[2 * jp + 1], qa[ks], kf[2], kf[3]);
                }
            }
            const int kbase = kb * AT_BN;
            const bool tail = kbase + AT_BN > p.seq;
            // half(Q K^T): mantissa cut; half(score * scale): the packing conversion rounds toward zero
#pragma unroll
            for(int j = 0; j < 8; ++j)
            {
                float x[4];
#pragma unroll
                for(int e = 0; e < 4; ++e)
                    x[e] = __uint_as_float(__float_as_uint(s[j][e]) & 0xFFFFE000u) * p.scale;
                if(tail)
                {
                    // keys that do not exist: the lowest half, whose exponential is 0
#pragma unroll
                    for(int e = 0; e < 4; ++e)
                        if(kbase + j * 8 + 2 * t + (e & 1) >= p.seq)
                            x[e] = -65504.0f;
                }
                w[j][0] = cvt_rz_f16x2(x[0], x[1]);
                w[j][1] = cvt_rz_f16x2(x[2], x[3]);
            }
        }
        if(pass == 0)
        {
#pragma unroll
            for(int j = 0; j < 8; ++j)
            {
                mxh[0] = __hmax2(mxh[0], *reinterpret_cast<const __half2*>(&w[j][0]));
                mxh[1] = __hmax2(mxh[1], *reinterpret_cast<const __half2*>(&w[j][1]));
            }
            if(kb + 1 == nblocks)
            {
#pragma unroll
                for(int r = 0; r < 2; ++r)
                {
                    const float2 m2 = __half22float2(mxh[r]);
                    float mx        = fmaxf(m2.x, m2.y);
                    mx              = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                    mx              = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                    m[r]            = mx;
                }
            }
        }
        else
        {
            // e = half(exp(x - max)) of both passes: the same instructions, the same bits
            uint32_t eh[8][2];
#pragma unroll
            for(int j = 0; j < 8; ++j)
#pragma unroll
                for(int r = 0; r < 2; ++r)
                {
                    const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&w[j][r]));
                    eh[j][r] = cvt_rz_f16x2(fast_exp2((x.x - m[r]) * log2e), fast_exp2((x.y - m[r]) * log2e));
                }
            if(pass == 1)
            {
#pragma unroll
                for(int j = 0; j < 8; ++j)
#pragma unroll
                    for(int r = 0; r < 2; ++r)
                    {
                        const float2 e = __half22float2(*reinterpret_cast<const __half2*>(&eh[j][r]));
                        sum[r] += e.x + e.y;
                    }
                if(kb + 1 == nblocks)
                {
#pragma unroll
                    for(int r = 0; r < 2; ++r)
                    {
                        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
                        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
                        rcp[r] = __frcp_rn(sum[r]);
                    }
                }
            }
            else
            {
                // p = half(e / sum): reciprocal and remainder correction, packed as the A fragments of
                // the four 16-key steps (tiles 2 ks and 2 ks + 1)
                uint32_t pa[4][4];
#pragma unroll
                for(int j = 0; j < 8; ++j)
#pragma unroll
                    for(int r = 0; r < 2; ++r)
                    {
                        const float2 e = __half22float2(*reinterpret_cast<const __half2*>(&eh[j][r]));
                        float a = e.x * rcp[r], b = e.y * rcp[r];
                        a       = __fmaf_rn(__fmaf_rn(-a, sum[r], e.x), rcp[r], a);
                        b       = __fmaf_rn(__fmaf_rn(-b, sum[r], e.y), rcp[r], b);
                        pa[j >> 1][(j & 1) * 2 + r] = cvt_rz_f16x2(a, b);
                    }
#pragma unroll
                for(int ks = 0; ks < 4; ++ks)
                {
#pragma unroll
                    for(int jp = 0; jp < 4; ++jp)
                    {
                        uint32_t vf[4];
                        ldmatrix_x4_trans(vf, tile_ptr(sv[buf], ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * jp + (lane >> 4)));
                        mma_16816(o[2 * jp], pa[ks], vf[0], vf[1]);
                        mma_16816(o[2 * jp + 1], pa[ks], vf[2], vf[3]);
                    }
                }
            }
        }
        __syncthreads(); // the other buffers are overwritten by the next iteration's loads
        if(++kb == nblocks)
        {
            kb = 0;
            ++pass;
        }
    }
    const float q_lo = -128.0f - p.q_zp, q_hi = 127.0f - p.q_zp;
#pragma unroll
    for(int r = 0; r < 2; ++r)
    {
        const int row = q0 + warp * 16 + g + r * 8;
        if(row >= p.seq)
            continue;
#pragma unroll
        for(int j = 0; j < 8; ++j)
        {
            const float a = truncate_to_half_precision(o[j][2 * r]);
            const float b = truncate_to_half_precision(o[j][2 * r + 1]);
            const int col = head * AT_D + j * 8 + 2 * t;
            if(p.o != nullptr)
                *reinterpret_cast<uint32_t*>(p.o + (row_base + row) * p.ldo + col) = cvt_rz_f16x2(a, b);
            if(p.oq != nullptr)
            {
                uint32_t qb[2];
                const float vals[2] = {a, b};
#pragma unroll
                for(int e = 0; e < 2; ++e)
                {
                    float qv        = __fmul_rn(vals[e], p.q_rcp);
                    const float rem = __fmaf_rn(-p.q_scale, qv, vals[e]);
                    qv              = truncate_to_half_precision(__fmaf_rn(rem, p.q_rcp, qv));
                    qv              = fmaxf(q_lo, fminf(q_hi, qv));
                    qb[e] = static_cast<uint32_t>(__float_as_int(__fadd_rn(qv, 12582912.0f)) - 0x4B400000 +
                                                  static_cast<int>(p.q_zp)) & 0xFFu;
                }
                *reinterpret_cast<uint16_t*>(p.oq + (row_base + row) * p.ldoq + col) =
                    static_cast<uint16_t>(qb[0] | (qb[1] << 8));
            }
        }
    }
}

} // namespace mgx

extern "C" int mgx_cuda_attention(const mgx_attention_desc* d, const void* q, const void* k, const void* v, void* o,
                                  void* oq, void* stream_)
{
    using namespace mgx;
    if(d == nullptr or q == nullptr or k == nullptr or v == nullptr or (o == nullptr and oq == nullptr))
        return MGX_E_INVALID_ARG;
    if(d->batch <= 0 or d->seq <= 0 or d->heads <= 0)
        return MGX_E_INVALID_ARG;
    if(d->head_dim != AT_D)
        return MGX_E_UNSUPPORTED;
    const int64_t width = d->heads * AT_D;
    if(d->ldq < width or d->ldk < width or d->ldv < width or (o != nullptr and d->ldo < width) or
       (oq != nullptr and d->ldoq < width))
        return MGX_E_INVALID_ARG;
    auto misaligned = [](const void* ptr, int64_t ld, int es, int bytes) {
        return (reinterpret_cast<uintptr_t>(ptr) % bytes) != 0 or (ld * es) % bytes != 0;
    };
    if(misaligned(q, d->ldq, 2, 16) or misaligned(k, d->ldk, 2, 16) or misaligned(v, d->ldv, 2, 16) or
       (o != nullptr and misaligned(o, d->ldo, 2, 4)) or (oq != nullptr and misaligned(oq, d->ldoq, 1, 2)))
        return MGX_E_ALIGNMENT;
    if(oq != nullptr and not(d->q_scale > 0.0f))
        return MGX_E_INVALID_ARG;
    if(d->heads > 65535 or d->batch > 65535 or d->seq > (1 << 24))
        return MGX_E_TOO_LARGE;
    attention_params p{};
    p.q = static_cast<const __half*>(q), p.k = static_cast<const __half*>(k), p.v = static_cast<const __half*>(v);
    p.o       = static_cast<__half*>(o);
    p.oq      = static_cast<int8_t*>(oq);
    p.ldq     = d->ldq, p.ldk = d->ldk, p.ldv = d->ldv, p.ldo = d->ldo, p.ldoq = d->ldoq;
    p.seq     = static_cast<int>(d->seq);
    p.heads   = static_cast<int>(d->heads);
    p.scale   = d->scale;
    p.q_scale = d->q_scale;
    p.q_rcp   = oq != nullptr ? static_cast<float>(1.0 / static_cast<double>(d->q_scale)) : 0.0f;
    p.q_zp    = d->q_zero_point;
    const dim3 grid(static_cast<unsigned>((d->seq + AT_BM - 1) / AT_BM), static_cast<unsigned>(d->heads),
                    static_cast<unsigned>(d->batch));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if((d->flags & MGX_ATTENTION_FP32_SOFTMAX) == 0 and
       ((d->flags & MGX_ATTENTION_THREE_PASS) != 0 or d->seq > AT_CHAIN_MAX_SEQ))
    {
        attention_f16_chain3_kernel<<<grid, 128, 0, stream>>>(p);
        return static_cast<int>(cudaGetLastError());
    }
    if(d->seq <= AT_CHAIN_MAX_SEQ and (d->flags & MGX_ATTENTION_FP32_SOFTMAX) == 0)
    {
        const int sp = static_cast<int>((d->seq + AT_BN - 1) / AT_BN * AT_BN) + 8;
        // 64 query rows per CTA, or 32 where that leaves SMs without a CTA (a single sequence per GPU)
        const bool narrow = static_cast<int64_t>(grid.x) * grid.y * grid.z < device_sm_count();
        const int rows    = narrow ? 32 : AT_BM;
        const dim3 cgrid(static_cast<unsigned>((d->seq + rows - 1) / rows), grid.y, grid.z);
        const int bytes = (AT_BM * AT_D + 2 * AT_BN * AT_D + rows * sp) * 2 + 2 * AT_BM * 4;
        // opted in once per instantiation, to the size its longest sequence needs
        auto launch = [&](auto kernel, int max_seq) {
            const int max_bytes = (AT_BM * AT_D + 2 * AT_BN * AT_D + AT_BM * (max_seq + 8)) * 2 + 2 * AT_BM * 4;
            const int rc        = ensure_smem_optin(reinterpret_cast<const void*>(kernel), max_bytes);
            if(rc != MGX_OK)
                return rc;
            kernel<<<cgrid, ATC_THREADS, bytes, stream>>>(p, sp);
            return static_cast<int>(cudaGetLastError());
        };
        if(narrow)
        {
            if(d->seq <= 384)
                return launch(attention_f16_chain_kernel<6, 2>, 384);
            if(d->seq <= 512)
                return launch(attention_f16_chain_kernel<8, 2>, 512);
            return launch(attention_f16_chain_kernel<AT_CHAIN_MAX_SEQ / 64, 2>, AT_CHAIN_MAX_SEQ);
        }
        if(d->seq <= 384)
            return launch(attention_f16_chain_kernel<6, 4>, 384);
        if(d->seq <= 512)
            return launch(attention_f16_chain_kernel<8, 4>, 512);
        return launch(attention_f16_chain_kernel<AT_CHAIN_MAX_SEQ / 64, 4>, AT_CHAIN_MAX_SEQ);
    }
    else
        attention_f16_kernel<<<grid, 128, 0, stream>>>(p);
    return static_cast<int>(cudaGetLastError());
}
