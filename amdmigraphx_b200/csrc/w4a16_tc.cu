// Weight-only int4 linear for decode (M <= 16 rows of activations) on the tcgen05 tensor core,
// built to be bound by the HBM stream of packed weights:
//
//   D[m,n] = sum_g  s[n,g] * sum_{k in g} (q[n,k] - zp[n,g]) * a[m,k]
//
// is evaluated with INTEGER tensor-core arithmetic.  A small pre-kernel writes every
// activation row as two int8 rows (a ~ sa[m] * (128 h + l), |error| <= sa/2, i.e. 15 bits of
// the row's range) and the per-group sums Sv[g,m] = sum_k (128 h + l).  The main kernel then
// computes, per group g of 128 k and per 128 output columns, with kind::i8 MMAs whose A operand
// is the UNSIGNED nibble q (unpacked to bytes: two logic operations per eight weights, nothing
// else touches a weight) and whose B operand are the h / l rows:
//   P_hi[n,m] = sum_k q h,   P_lo[n,m] = sum_k q l        (exact int32, one TMEM column each)
// and the epilogue folds   s[n,g] * (128 P_hi + P_lo - zp[n,g] * Sv[g,m])   into fp32 registers.
// The only inexact steps are the 15-bit activation rounding and the fp32 sum over groups; the
// reference (src/onnx/parse_matmulnbits.cpp:85-158 IR on the ref target) rounds every
// dequantised weight to fp16 instead, which is the coarser of the two.
//
// CTA = 384 threads, one CTA per SM:
//   warp 0      TMA producer of packed weights: 4 groups = two requests of 128 rows x 128 bytes
//   warp 10     TMA producer of the activation rows of the same 4 groups
//   warps 2..5  unpack: one thread per weight row, shared memory -> registers -> the row's lane
//               of TENSOR MEMORY (tcgen05.st); the MMA reads its A operand from there, so the
//               unpacked bytes never cross shared memory
//   warp 1      MMA issuer (A from tensor memory, B = activation rows in shared memory)
//   warp 11     loads and converts the epilogue's scales / zero points / group sums a pass ahead
//   warps 6..9  epilogue fold out of two accumulator buffers; the last CTA to finish a tile
//               that several CTAs share adds their partial sums in a fixed order
// Only plain TMA loads; every wait is bounded.
#include "common.cuh"
#include "ptx.cuh"
#include <cuda_fp16.h>

namespace mgx {

constexpr int TC_ROWS     = 128; // output columns (weight rows) per CTA tile = UMMA M
constexpr int TC_GROUP_K  = 128; // k per group
constexpr int TC_SUPER    = 4;   // groups per work item (each row gives 256 contiguous bytes)
constexpr int TC_PACKED   = TC_ROWS * TC_GROUP_K / 2; // 8192 bytes of packed weights per group
constexpr int TC_WSTAGE   = TC_SUPER * TC_PACKED;     // 32768
constexpr int TC_TSTAGES  = 2;   // A operand buffers in tensor memory
constexpr int TC_THREADS  = 384;
constexpr int TC_ACC_COLS = 128; // accumulator columns per buffer (two buffers)
constexpr int TC_A_COL0   = 256; // first tensor-memory column of the A operand buffers
constexpr int TC_A_COLS   = TC_GROUP_K / 4; // 32 columns per group
constexpr int TC_EPI      = 2 * (2 * 8 * 128 * 4 + 128 * 4) + 64; // two buffers of epilogue metadata

// ring depths by B-operand width: weights (32 KB each), activation tiles (4 NB x 128 bytes)
template <int NB>
struct tc_cfg
{
    static constexpr int wstages = NB == 16 ? 5 : 4;
    static constexpr int astages = NB == 16 ? 4 : 3;
    static constexpr int astage  = TC_SUPER * NB * TC_GROUP_K;
    static constexpr int ring    = wstages * TC_WSTAGE + astages * astage;
    static constexpr int smem    = ring + 512 + TC_EPI + 1024;
};

struct tc_params
{
    const __half* scales;
    const uint8_t* zp; // may be null
    const float* sa;   // [MB] per-row activation scale
    const float* sv;   // [K/128][MB] per-group sums of the quantised activations
    __half* D;
    float* partial;    // [slots][M][N]
    int* counters;     // [tiles] segments finished, zeroed by the pre-kernel
    int64_t M, N, K, ldd;
    int group, groups_per_row, zp_const, act;
    int items_total, items_per_cta; // (tile, 4-group block) work items, see the main kernel
};

__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void grid_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ------------------------------------------------------------------ activation pre-kernel
// grid = MB blocks (one per padded activation row), 1024 threads; a thread owns 8 consecutive k.
// Output: aq rows [0, MB) = h, rows [MB, 2 MB) = l, inside every 8 k the evens first, then the
// odds (the order the unpacked nibbles have); sv; sa; zeroed tile counters.
template <int MB>
__global__ void __launch_bounds__(1024)
    w4_prepare_acts_kernel(const __half* __restrict__ A, int64_t lda, int64_t M, int64_t K,
                           int8_t* __restrict__ aq, float* __restrict__ sa, float* __restrict__ sv,
                           int* __restrict__ counters, int ncounters)
{
    // the main kernel may start (and stream weights) right away; it waits for this grid's
    // completion before it touches anything written here
    grid_launch_dependents();
    __shared__ float red[32];
    __shared__ float s_scale;
    const int m   = blockIdx.x;
    const int tid = threadIdx.x;
    int8_t* hi    = aq + static_cast<int64_t>(m) * K;
    int8_t* lo    = aq + static_cast<int64_t>(MB + m) * K;
    for(int i = blockIdx.x * 1024 + tid; i < ncounters; i += gridDim.x * 1024)
        counters[i] = 0;
    if(m >= M)
    {
        for(int64_t k = tid * 16; k < K; k += 1024 * 16)
        {
            *reinterpret_cast<uint4*>(hi + k) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(lo + k) = make_uint4(0u, 0u, 0u, 0u);
        }
        for(int64_t g = tid; g < K / 128; g += 1024)
            sv[g * MB + m] = 0.0f;
        if(tid == 0)
            sa[m] = 0.0f;
        return;
    }
    const __half* row = A + m * lda;
    float mx          = 0.0f;
    uint4 first       = make_uint4(0u, 0u, 0u, 0u); // this thread's first octet stays in registers
    for(int64_t k = tid * 8; k < K; k += 1024 * 8)
    {
        const uint4 v = *reinterpret_cast<const uint4*>(row + k);
        if(k < 1024 * 8)
            first = v;
        const __half* vh = reinterpret_cast<const __half*>(&v);
#pragma unroll
        for(int e = 0; e < 8; ++e)
            mx = fmaxf(mx, fabsf(__half2float(vh[e])));
    }
#pragma unroll
    for(int o = 16; o > 0; o >>= 1)
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if((tid & 31) == 0)
        red[tid >> 5] = mx;
    __syncthreads();
    if(tid < 32)
    {
        float t = red[tid];
#pragma unroll
        for(int o = 16; o > 0; o >>= 1)
            t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
        if(tid == 0)
        {
            // 128 h + l spans [-16256, 16256] with h in [-127, 127], l in [-64, 63]
            s_scale = t > 0.0f ? t / 16256.0f : 1.0f;
            sa[m]   = s_scale;
        }
    }
    __syncthreads();
    const float inv = 1.0f / s_scale;
    for(int64_t kb = 0; kb < K; kb += 1024 * 8)
    {
        // every thread of a warp takes the same trips (the sums below are warp shuffles)
        const int64_t k  = kb + tid * 8;
        const bool valid = k < K;
        const uint4 v    = kb == 0 ? first
                                   : (valid ? *reinterpret_cast<const uint4*>(row + k)
                                            : make_uint4(0u, 0u, 0u, 0u));
        const __half* vh = reinterpret_cast<const __half*>(&v);
        int sum          = 0;
        uint32_t hw[2] = {0u, 0u}, lw[2] = {0u, 0u};
#pragma unroll
        for(int e = 0; e < 8; ++e)
        {
            int q = __float2int_rn(__half2float(vh[e]) * inv);
            q     = max(-16256, min(16256, q));
            const int h = (q + 64 + 128 * 256) / 128 - 256; // round(q / 128) for any sign
            const int l = q - 128 * h;
            sum += q;
            const int pos = (e & 1) * 4 + (e >> 1); // evens first, then odds
            hw[pos >> 2] |= static_cast<uint32_t>(h & 0xFF) << (8 * (pos & 3));
            lw[pos >> 2] |= static_cast<uint32_t>(l & 0xFF) << (8 * (pos & 3));
        }
        if(valid)
        {
            *reinterpret_cast<uint2*>(hi + k) = make_uint2(hw[0], hw[1]);
            *reinterpret_cast<uint2*>(lo + k) = make_uint2(lw[0], lw[1]);
        }
        // 16 consecutive threads hold one group of 128 k
#pragma unroll
        for(int o = 8; o > 0; o >>= 1)
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if(valid and (tid & 15) == 0)
            sv[(k >> 7) * MB + m] = static_cast<float>(sum);
    }
}

// ------------------------------------------------------------------ main kernel
// Work is the flat list of (tile, block) items, tile-major, a block being TC_SUPER consecutive
// groups (the last block of a tile may hold fewer): item F -> tile F / SG, block F % SG with
// SG = ceil(G / TC_SUPER), G = K / 128.  CTA c owns items [c U, (c + 1) U): every SM streams
// the same number of 32 KB weight blocks whatever N and K are.  A CTA's share of one tile is
// a "segment"; a segment that is the whole tile is written to D, any other goes to partial
// slot c - (tile SG) / U, and the CTA that finishes a shared tile last adds the slots in slot
// order, so the sum does not depend on timing.
struct tc_walk
{
    int F, F_hi, SG, G;
    int g; // group cursor inside the current tile
    __device__ tc_walk(int f_lo, int f_hi, int sg, int groups)
        : F(f_lo), F_hi(f_hi), SG(sg), G(groups), g((f_lo % sg) * TC_SUPER)
    {
    }
    // next pass: at most `cap` (a multiple of TC_SUPER) groups of one tile
    __device__ bool next(int cap, int& tile, int& g0, int& count, bool& seg_last)
    {
        if(F >= F_hi)
            return false;
        tile                 = F / SG;
        const int seg_end_sg = min(F_hi - tile * SG, SG);
        const int seg_end_g  = min(G, seg_end_sg * TC_SUPER);
        g0                   = g;
        count                = min(cap, seg_end_g - g);
        g += count;
        seg_last = g == seg_end_g;
        if(seg_last)
        {
            F = tile * SG + seg_end_sg;
            g = 0;
        }
        return true;
    }
};

// int32 known to lie in (-2^22, 2^22) -> float without the conversion pipe
__device__ __forceinline__ float small_int_to_float(uint32_t v)
{
    return __uint_as_float(v + 0x4B400000u) - 12582912.0f;
}

// NB: activation rows in the B operand (= UMMA N): 16 (M <= 8: 8 h rows + 8 l rows) or 32.
template <int NB>
__global__ void __launch_bounds__(TC_THREADS, 1)
    w4a16_tc_kernel(const __grid_constant__ CUtensorMap tmap_w,
                    const __grid_constant__ CUtensorMap tmap_a,
                    const tc_params p)
{
    using cfg            = tc_cfg<NB>;
    constexpr int MB     = NB / 2;           // padded activation rows
    constexpr int GPP    = TC_ACC_COLS / NB; // groups per pass (one accumulator buffer): 8 or 4
    constexpr int WST    = cfg::wstages;
    constexpr int AST    = cfg::astages;
    constexpr int ABYTES = NB * TC_GROUP_K;  // activation rows of one group
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem           = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint8_t* act_ring       = smem + WST * TC_WSTAGE;
    uint8_t* bar_base       = smem + cfg::ring;
    uint64_t* wfull_bar     = reinterpret_cast<uint64_t*>(bar_base); // weights landed
    uint64_t* wempty_bar    = wfull_bar + WST;                       // weights read by all rows
    uint64_t* afull_bar     = wempty_bar + WST;                      // activation tile landed
    uint64_t* afree_bar     = afull_bar + AST;                       // MMAs that read it retired
    uint64_t* unp_bar       = afree_bar + AST;                       // A operand in tensor memory
    uint64_t* tfree_bar     = unp_bar + TC_TSTAGES;                  // MMAs that read it retired
    uint64_t* accf_bar      = tfree_bar + TC_TSTAGES;
    uint64_t* acce_bar      = accf_bar + 2;
    uint64_t* epi_bar       = acce_bar + 2;
    uint64_t* mfull_bar     = epi_bar + 1; // metadata of a pass staged
    uint64_t* mempty_bar    = mfull_bar + 2;
    uint32_t* tmem_slot     = reinterpret_cast<uint32_t*>(mempty_bar + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    // epilogue metadata, two buffers: per output column and group of a pass the scale and
    // scale x zero point, GPP x MB activation group sums; one word for the tile-counter broadcast
    float* epi_sc = reinterpret_cast<float*>(bar_base + 512); // [2][8][128]
    float* epi_sz = epi_sc + 2 * 8 * 128;                     // [2][8][128]
    float* epi_sv = epi_sz + 2 * 8 * 128;                     // [2][128]
    int* epi_flag = reinterpret_cast<int*>(epi_sv + 2 * 128);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < WST; ++s)
        {
            mbar_init(&wfull_bar[s], 1);
            mbar_init(&wempty_bar[s], 128);
        }
        for(int s = 0; s < AST; ++s)
        {
            mbar_init(&afull_bar[s], 1);
            mbar_init(&afree_bar[s], 1);
        }
        for(int b = 0; b < 2; ++b)
        {
            mbar_init(&unp_bar[b], 128);
            mbar_init(&tfree_bar[b], 1);
            mbar_init(&accf_bar[b], 1);
            mbar_init(&acce_bar[b], 4);
            mbar_init(&mfull_bar[b], 32);
            mbar_init(&mempty_bar[b], 4);
        }
        mbar_init(epi_bar, 128);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmap_w);
        prefetch_tensormap(&tmap_a);
    }
    if(warp == 1)
    {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int G      = static_cast<int>(p.K / TC_GROUP_K);
    const int SG     = (G + TC_SUPER - 1) / TC_SUPER;
    const int f_lo   = min(p.items_total, static_cast<int>(blockIdx.x) * p.items_per_cta);
    const int f_hi   = min(p.items_total, f_lo + p.items_per_cta);
    const int nsuper = f_hi - f_lo;

    if(warp == 0)
    {
        // ---------------------------------------------------- TMA producer: packed weights
        // (constants of the model: no need to wait for the pre-kernel)
        if(lane == 0)
        {
            int tile = f_lo / SG, sg = f_lo - tile * SG;
            for(int j = 0; j < nsuper; ++j)
            {
                const uint32_t s  = j % WST;
                const uint32_t ph = (j / WST) & 1u;
                if(not mbar_wait_bounded(&wempty_bar[s], ph ^ 1u, abort_flag, 2))
                    break;
                // groups past the end of K are zero-filled and still counted
                mbar_expect_tx(&wfull_bar[s], TC_WSTAGE);
                tma_load_2d(smem + s * TC_WSTAGE, &tmap_w, &wfull_bar[s], sg * (TC_WSTAGE / TC_ROWS),
                            tile * TC_ROWS);
                tma_load_2d(smem + s * TC_WSTAGE + TC_WSTAGE / 2, &tmap_w, &wfull_bar[s],
                            sg * (TC_WSTAGE / TC_ROWS) + 128, tile * TC_ROWS);
                if(++sg == SG)
                {
                    sg = 0;
                    ++tile;
                }
            }
        }
    }
    else if(warp == 10)
    {
        // ---------------------------------------------------- TMA producer: activation rows
        if(lane == 0)
        {
            grid_dependency_wait(); // written by the pre-kernel
            int sg = f_lo % SG;
            for(int j = 0; j < nsuper; ++j)
            {
                const uint32_t s  = j % AST;
                const uint32_t ph = (j / AST) & 1u;
                if(not mbar_wait_bounded(&afree_bar[s], ph ^ 1u, abort_flag, 7))
                    break;
                mbar_expect_tx(&afull_bar[s], cfg::astage);
                tma_load_3d(act_ring + s * cfg::astage, &tmap_a, &afull_bar[s], 0, 0, sg * TC_SUPER);
                if(++sg == SG)
                    sg = 0;
            }
        }
    }
    else if(warp == 11)
    {
        // ---------------------------------------------------- epilogue metadata, a pass ahead
        // Global loads (scales, zero points, activation group sums) and their conversions
        // happen here, so that the epilogue warps never wait for global memory.  A lane
        // serves four output columns.
        grid_dependency_wait(); // sv comes from the pre-kernel
        const int ratio = p.group / TC_GROUP_K;
        tc_walk walk(f_lo, f_hi, SG, G);
        int tile, g0, count;
        bool seg_last;
        for(uint32_t pc = 0; walk.next(GPP, tile, g0, count, seg_last); ++pc)
        {
            const uint32_t b = pc & 1u;
            if(not __all_sync(0xffffffffu, mbar_wait_bounded(&mempty_bar[b], ((pc >> 1) & 1u) ^ 1u,
                                                             abort_flag, 9)))
                break;
            unsigned short rs[4][GPP];
            uint8_t rz[4][GPP];
#pragma unroll
            for(int c = 0; c < 4; ++c)
            {
                const int64_t n  = static_cast<int64_t>(tile) * TC_ROWS + c * 32 + lane;
                const int64_t nn = n < p.N ? n : p.N - 1;
                const unsigned short* srow =
                    reinterpret_cast<const unsigned short*>(p.scales) + nn * p.groups_per_row;
                const uint8_t* zrow = p.zp == nullptr ? nullptr : p.zp + nn * p.groups_per_row;
#pragma unroll
                for(int gl = 0; gl < GPP; ++gl)
                {
                    const int gi = (g0 + min(gl, count - 1)) / ratio;
                    rs[c][gl]    = __ldg(srow + gi);
                    rz[c][gl]    = zrow == nullptr ? static_cast<uint8_t>(p.zp_const) : __ldg(zrow + gi);
                }
            }
            // GPP x MB = 128 group sums: four per lane
            float4 sv4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if((lane * 4) / MB < count)
                sv4 = __ldg(reinterpret_cast<const float4*>(p.sv + static_cast<int64_t>(g0) * MB) + lane);
#pragma unroll
            for(int c = 0; c < 4; ++c)
            {
#pragma unroll
                for(int gl = 0; gl < GPP; ++gl)
                {
                    const float sc = __half2float(__ushort_as_half(rs[c][gl]));
                    epi_sc[(b * 8 + gl) * 128 + c * 32 + lane] = sc;
                    epi_sz[(b * 8 + gl) * 128 + c * 32 + lane] = sc * static_cast<float>(rz[c][gl]);
                }
            }
            *reinterpret_cast<float4*>(epi_sv + b * 128 + lane * 4) = sv4;
            mbar_arrive(&mfull_bar[b]);
        }
    }
    else if(warp == 1)
    {
        // ---------------------------------------------------- MMA issuer
        if(lane == 0)
        {
            // D s32 += A u8 (weights, tensor memory) * B s8 (activation rows, K-major shared
            // memory); M = 128, N = NB
            constexpr uint32_t idesc = make_idesc(2u, 0u, 1u, TC_ROWS, NB);
            tc_walk walk(f_lo, f_hi, SG, G);
            int tile, g0, count;
            bool seg_last;
            bool ok = true;
            int j   = 0;
            for(uint32_t pc = 0; ok and walk.next(GPP, tile, g0, count, seg_last); ++pc)
            {
                const uint32_t buf = pc & 1u;
                if(not mbar_wait_bounded(&acce_bar[buf], ((pc >> 1) & 1u) ^ 1u, abort_flag, 4))
                    break;
                tc_fence_after_sync();
                for(int gl = 0; gl < count; gl += TC_SUPER, ++j)
                {
                    const uint32_t a  = j % AST;
                    const uint32_t ap = (j / AST) & 1u;
                    const uint32_t t  = j & 1u;
                    const uint32_t tp = (j >> 1) & 1u;
                    if(not mbar_wait_bounded(&unp_bar[t], tp, abort_flag, 5) or
                       not mbar_wait_bounded(&afull_bar[a], ap, abort_flag, 1))
                    {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const int cnt = min(TC_SUPER, count - gl);
                    const uint32_t b_smem = smem_u32(act_ring + a * cfg::astage);
                    for(int q = 0; q < cnt; ++q)
                    {
                        const uint64_t bdesc  = make_smem_desc_sw128(b_smem + q * ABYTES);
                        const uint32_t a_tmem = tmem_base + TC_A_COL0 + (t * TC_SUPER + q) * TC_A_COLS;
                        const uint32_t d_tmem = tmem_base + buf * TC_ACC_COLS + (gl + q) * NB;
#pragma unroll
                        for(int k = 0; k < 4; ++k)
                        {
                            const uint64_t koff = static_cast<uint64_t>((k * 32) >> 4);
                            mma_i8_tmem_a(d_tmem, a_tmem + k * 8, bdesc + koff, idesc, k != 0);
                        }
                    }
                    tc_commit(&tfree_bar[t]);
                    tc_commit(&afree_bar[a]);
                }
                if(ok)
                    tc_commit(&accf_bar[buf]);
            }
        }
    }
    else if(warp < 6)
    {
        // ---------------------------------------------------- unpack: nibbles -> bytes
        // One thread per weight row: 64 packed bytes per group from shared memory (128-byte
        // swizzle, so a quarter warp's 16-byte reads fall in eight different bank groups), 32
        // words of bytes to this row's lane of tensor memory.  Inside every 8 k the evens come
        // first, then the odds; the activation rows are stored in the same order.
        const int row            = (warp & 3) * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const int sw             = row & 7;
        int sg                   = f_lo % SG;
        for(int j = 0; j < nsuper; ++j)
        {
            const uint32_t s  = j % WST;
            const uint32_t ph = (j / WST) & 1u;
            const uint32_t t  = j & 1u;
            const uint32_t tp = (j >> 1) & 1u;
            // the tensor-memory stores below are warp-wide: leave only as a whole warp
            if(not __all_sync(0xffffffffu, mbar_wait_bounded(&wfull_bar[s], ph, abort_flag, 1)))
                break;
            if(not __all_sync(0xffffffffu, mbar_wait_bounded(&tfree_bar[t], tp ^ 1u, abort_flag, 8)))
                break;
            tc_fence_after_sync();
            const int cnt = min(TC_SUPER, G - sg * TC_SUPER);
#pragma unroll
            for(int q = 0; q < TC_SUPER; ++q)
            {
                if(q < cnt)
                {
                    // [pair of groups][row][128 bytes], 16-byte chunks swizzled by the row
                    const uint8_t* pk = smem + s * TC_WSTAGE + (q >> 1) * (2 * TC_PACKED) + row * 128;
                    uint32_t u[32];
#pragma unroll
                    for(int c = 0; c < 4; ++c)
                    {
                        const uint4 w =
                            *reinterpret_cast<const uint4*>(pk + ((((q & 1) * 4 + c) ^ sw) << 4));
                        u[8 * c + 0] = w.x & 0x0F0F0F0Fu, u[8 * c + 1] = (w.x >> 4) & 0x0F0F0F0Fu;
                        u[8 * c + 2] = w.y & 0x0F0F0F0Fu, u[8 * c + 3] = (w.y >> 4) & 0x0F0F0F0Fu;
                        u[8 * c + 4] = w.z & 0x0F0F0F0Fu, u[8 * c + 5] = (w.z >> 4) & 0x0F0F0F0Fu;
                        u[8 * c + 6] = w.w & 0x0F0F0F0Fu, u[8 * c + 7] = (w.w >> 4) & 0x0F0F0F0Fu;
                    }
                    tmem_st_32x32b_x32(tmem_base + lane_addr + TC_A_COL0 +
                                           (t * TC_SUPER + q) * TC_A_COLS,
                                       u);
                }
            }
            mbar_arrive(&wempty_bar[s]); // the packed blocks are in registers
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive(&unp_bar[t]);
            if(++sg == SG)
                sg = 0;
        }
    }
    else
    {
        // ---------------------------------------------------- epilogue: fold the groups
        // Scales, zero points and activation group sums of the pass are already in shared
        // memory (metadata warp).  All arithmetic stays off the conversion pipe: |P_hi|,
        // |P_lo| < 2^18.
        grid_dependency_wait(); // sv, sa and the tile counters come from the pre-kernel
        const int quarter = warp & 3;
        const int te      = threadIdx.x - 192; // 0..127
        const int col     = quarter * 32 + lane; // output column inside the tile = TMEM lane
        float out[MB];
#pragma unroll
        for(int m = 0; m < MB; ++m)
            out[m] = 0.0f;
        tc_walk walk(f_lo, f_hi, SG, G);
        uint32_t epi_phase = 0;
        // all 128 epilogue threads meet here (bounded)
        auto epi_sync = [&]() {
            mbar_arrive(epi_bar);
            const bool r = mbar_wait_bounded(epi_bar, epi_phase & 1u, abort_flag, 6);
            ++epi_phase;
            return __all_sync(0xffffffffu, r);
        };
        // one group: out[m] += sc (128 P_hi + P_lo) - sc z Sv
        auto fold = [&](const uint32_t(&acc)[NB], int gl, const float* scb, const float* szb,
                        const float* svb) {
            const float sc = scb[gl * 128 + col];
            const float sz = szb[gl * 128 + col];
#pragma unroll
            for(int m = 0; m < MB; ++m)
            {
                const float fh = small_int_to_float(acc[m]);
                const float fl = small_int_to_float(acc[MB + m]);
                out[m]         = fmaf(sc, fmaf(fh, 128.0f, fl), out[m]);
                out[m]         = fmaf(-sz, svb[gl * MB + m], out[m]);
            }
        };
        int tile, g0, count;
        bool seg_last;
        bool ok = true;
        for(uint32_t pc = 0; ok and walk.next(GPP, tile, g0, count, seg_last); ++pc)
        {
            const uint32_t buf = pc & 1u;
            if(not __all_sync(0xffffffffu,
                              mbar_wait_bounded(&mfull_bar[buf], (pc >> 1) & 1u, abort_flag, 10)) or
               not __all_sync(0xffffffffu,
                              mbar_wait_bounded(&accf_bar[buf], (pc >> 1) & 1u, abort_flag, 3)))
                break;
            tc_fence_after_sync();
            const float* svb     = epi_sv + buf * 128;
            const float* scb     = epi_sc + buf * 8 * 128;
            const float* szb     = epi_sz + buf * 8 * 128;
            const uint32_t tbase = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   buf * TC_ACC_COLS;
            // two groups per trip: the second TMEM read is in flight while the first is folded
#pragma unroll 1
            for(int gl = 0; gl < count; gl += 2)
            {
                uint32_t acc0[NB], acc1[NB];
                const bool two = gl + 1 < count; // the same for the whole warp
                if constexpr(NB == 16)
                {
                    tmem_ld_32x32b_x16(tbase + gl * NB, acc0);
                    if(two)
                        tmem_ld_32x32b_x16(tbase + (gl + 1) * NB, acc1);
                }
                else
                {
                    tmem_ld_32x32b_x32(tbase + gl * NB, acc0);
                    if(two)
                        tmem_ld_32x32b_x32(tbase + (gl + 1) * NB, acc1);
                }
                tmem_ld_wait();
                fold(acc0, gl, scb, szb, svb);
                if(two)
                    fold(acc1, gl + 1, scb, szb, svb);
            }
            tc_fence_before_sync();
            __syncwarp();
            if(lane == 0)
            {
                mbar_arrive(&acce_bar[buf]);
                mbar_arrive(&mempty_bar[buf]);
            }
            if(seg_last)
            {
                // this CTA's share of the tile is complete
                const int64_t n  = static_cast<int64_t>(tile) * TC_ROWS + quarter * 32 + lane;
                const bool whole = f_lo <= tile * SG and f_hi >= (tile + 1) * SG;
                if(whole)
                {
#pragma unroll
                    for(int m = 0; m < MB; ++m)
                        if(m < p.M and n < p.N)
                            p.D[m * p.ldd + n] = __float2half_rn(out[m] * __ldg(p.sa + m));
                }
                else
                {
                    const int first = (tile * SG) / p.items_per_cta;
                    const int last  = ((tile + 1) * SG - 1) / p.items_per_cta;
                    const int slot  = static_cast<int>(blockIdx.x) - first;
#pragma unroll
                    for(int m = 0; m < MB; ++m)
                        if(m < p.M and n < p.N)
                            p.partial[(static_cast<int64_t>(slot) * p.M + m) * p.N + n] = out[m];
                    __threadfence();
                    ok = epi_sync();
                    if(ok and te == 0)
                        *epi_flag = atomicAdd(p.counters + tile, 1);
                    ok = ok and epi_sync();
                    if(ok and *epi_flag == last - first)
                    {
                        // every other segment of the tile is in memory: add them in slot order
                        __threadfence();
#pragma unroll
                        for(int m = 0; m < MB; ++m)
                        {
                            if(m < p.M and n < p.N)
                            {
                                float v = 0.0f;
                                for(int s = 0; s <= last - first; ++s)
                                    v += __ldcg(p.partial + (static_cast<int64_t>(s) * p.M + m) * p.N + n);
                                p.D[m * p.ldd + n] = __float2half_rn(v * __ldg(p.sa + m));
                            }
                        }
                    }
                }
#pragma unroll
                for(int m = 0; m < MB; ++m)
                    out[m] = 0.0f;
            }
        }
    }

    // ---------------------------------------------------------- teardown
    if(*abort_flag != 0)
    {
        for(int i = 0; i < 1000; ++i)
            __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if(warp == 1)
    {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

// ------------------------------------------------------------------ host
namespace {

struct tc_plan
{
    int nb, mb, tiles, groups, blocks, items_total, items_per_cta, grid, slots;
    size_t off_sa, off_sv, off_counters, off_partial, total;
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

tc_plan make_plan(const mgx_w4_desc& d)
{
    tc_plan pl{};
    pl.nb            = d.M <= 8 ? 16 : 32;
    pl.mb            = pl.nb / 2;
    pl.tiles         = static_cast<int>(ceil_div(d.N, TC_ROWS));
    pl.groups        = static_cast<int>(d.K / TC_GROUP_K);
    pl.blocks        = (pl.groups + TC_SUPER - 1) / TC_SUPER;
    pl.items_total   = pl.tiles * pl.blocks;
    // one CTA per SM, the same number of items (+-1) each
    pl.items_per_cta = static_cast<int>(ceil_div(pl.items_total, device_sm_count()));
    pl.grid          = static_cast<int>(ceil_div(pl.items_total, pl.items_per_cta));
    // CTAs that can share one tile
    pl.slots        = (pl.blocks - 1) / pl.items_per_cta + 2;
    pl.off_sa       = align_up(static_cast<size_t>(pl.nb) * d.K, 256);
    pl.off_sv       = pl.off_sa + 256;
    pl.off_counters = align_up(pl.off_sv + static_cast<size_t>(pl.groups) * pl.mb * sizeof(float), 256);
    pl.off_partial  = align_up(pl.off_counters + static_cast<size_t>(pl.tiles) * sizeof(int), 256);
    pl.total        = pl.off_partial + static_cast<size_t>(pl.slots) * d.M * d.N * sizeof(float);
    return pl;
}

// [group][row][inner bytes] view of a row-major byte matrix whose rows are `groups` runs of
// `inner` bytes: one request brings `box_groups` runs of `box_rows` rows.
int encode_grouped(CUtensorMap* map, const void* base, uint32_t inner, uint64_t rows, uint64_t pitch,
                   uint64_t groups, uint32_t box_rows, uint32_t box_groups, CUtensorMapSwizzle swz)
{
    cuTensorMapEncodeTiled_t encode = get_tensor_map_encoder();
    if(encode == nullptr)
        return MGX_E_DRIVER;
    cuuint64_t dims[3]    = {inner, rows, groups};
    cuuint64_t strides[2] = {pitch, inner};
    cuuint32_t box[3]     = {inner, box_rows, box_groups};
    cuuint32_t estr[3]    = {1u, 1u, 1u};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MGX_OK : MGX_E_INVALID_ARG;
}

template <int NB>
int launch_main(int grid, const CUtensorMap& tw, const CUtensorMap& ta, const tc_params& p,
                cudaStream_t stream)
{
    int rc = ensure_smem_optin(reinterpret_cast<const void*>(w4a16_tc_kernel<NB>), tc_cfg<NB>::smem);
    if(rc != MGX_OK)
        return rc;
    // programmatic dependent launch: the kernel may start while the pre-kernel still runs
    // and waits for it (griddepcontrol.wait) only where it reads what the pre-kernel wrote
    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = dim3(static_cast<unsigned>(grid));
    cfg.blockDim         = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = tc_cfg<NB>::smem;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs                                          = attr;
    cfg.numAttrs                                       = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, w4a16_tc_kernel<NB>, tw, ta, p));
}

} // namespace

bool w4a16_tc_applicable(const mgx_w4_desc& d)
{
    return d.M >= 1 and d.M <= 16 and d.K % TC_GROUP_K == 0 and d.group % TC_GROUP_K == 0 and
           d.act == MGX_ACT_NONE and d.lda % 8 == 0 and
           ceil_div(d.N, TC_ROWS) * (d.K / TC_GROUP_K) < (int64_t{1} << 30);
}

size_t w4a16_tc_workspace(const mgx_w4_desc& d) { return make_plan(d).total; }

int w4a16_tc_launch(const mgx_w4_desc& d, const void* A, const void* Bp, const void* scales,
                    const void* zp, void* D, void* workspace, size_t workspace_bytes,
                    cudaStream_t stream)
{
    const tc_plan pl = make_plan(d);
    if(workspace == nullptr or workspace_bytes < pl.total)
        return MGX_E_WORKSPACE;
    if((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 or
       ((reinterpret_cast<uintptr_t>(Bp) | reinterpret_cast<uintptr_t>(A)) & 15u) != 0)
        return MGX_E_ALIGNMENT;
    auto* ws       = static_cast<uint8_t*>(workspace);
    auto* aq       = reinterpret_cast<int8_t*>(ws);
    auto* sa       = reinterpret_cast<float*>(ws + pl.off_sa);
    auto* sv       = reinterpret_cast<float*>(ws + pl.off_sv);
    auto* counters = reinterpret_cast<int*>(ws + pl.off_counters);
    auto* part     = reinterpret_cast<float*>(ws + pl.off_partial);
    CUtensorMap tw, ta;
    // packed weights: rows of K / 2 bytes; one request = 128 rows x 128 bytes (two groups)
    int rc = MGX_OK;
    {
        cuTensorMapEncodeTiled_t encode = get_tensor_map_encoder();
        if(encode == nullptr)
            return MGX_E_DRIVER;
        cuuint64_t dims[2]    = {static_cast<cuuint64_t>(d.K / 2), static_cast<cuuint64_t>(d.N)};
        cuuint64_t strides[1] = {static_cast<cuuint64_t>(d.K / 2)};
        cuuint32_t box[2]     = {128u, TC_ROWS};
        cuuint32_t estr[2]    = {1u, 1u};
        if(encode(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(Bp), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            rc = MGX_E_INVALID_ARG;
    }
    if(rc != MGX_OK)
        return rc;
    rc = encode_grouped(&ta, aq, TC_GROUP_K, static_cast<uint64_t>(pl.nb), static_cast<uint64_t>(d.K),
                        static_cast<uint64_t>(pl.groups), static_cast<uint32_t>(pl.nb), TC_SUPER,
                        CU_TENSOR_MAP_SWIZZLE_128B);
    if(rc != MGX_OK)
        return rc;
    if(pl.nb == 16)
        w4_prepare_acts_kernel<8><<<8, 1024, 0, stream>>>(static_cast<const __half*>(A), d.lda, d.M,
                                                          d.K, aq, sa, sv, counters, pl.tiles);
    else
        w4_prepare_acts_kernel<16><<<16, 1024, 0, stream>>>(static_cast<const __half*>(A), d.lda, d.M,
                                                            d.K, aq, sa, sv, counters, pl.tiles);
    cudaError_t e = cudaGetLastError();
    if(e != cudaSuccess)
        return static_cast<int>(e);
    tc_params p{};
    p.scales         = static_cast<const __half*>(scales);
    p.zp             = static_cast<const uint8_t*>(zp);
    p.sa             = sa;
    p.sv             = sv;
    p.D              = static_cast<__half*>(D);
    p.partial        = part;
    p.counters       = counters;
    p.M              = d.M;
    p.N              = d.N;
    p.K              = d.K;
    p.ldd            = d.ldd;
    p.group          = d.group;
    p.groups_per_row = static_cast<int>(d.K / d.group);
    p.zp_const       = d.zp_const;
    p.act            = d.act;
    p.items_total    = pl.items_total;
    p.items_per_cta  = pl.items_per_cta;
    return pl.nb == 16 ? launch_main<16>(pl.grid, tw, ta, p, stream)
                       : launch_main<32>(pl.grid, tw, ta, p, stream);
}

int w4a16_tc_status(unsigned int* out) { return read_and_clear_status(out); }

} // namespace mgx
