// Weight-only int4 linear for decode (M <= 16 rows of activations) on the tcgen05 tensor core,
// built to be bound by the HBM stream of packed weights:
//
//   D[m,n] = sum_g  s[n,g] * sum_{k in g} (q[n,k] - zp[n,g]) * a[m,k]
//
// is evaluated with INTEGER tensor-core arithmetic.  A small pre-kernel writes every
// activation row as two int8 rows (a ~ sa[m] * (128 h + l), |error| <= sa/2, i.e. 15 bits of
// the row's range) and the per-group sums Sv[g,m] = sum_k (128 h + l).  The main kernel then
// computes, per group g of 128 k and per 128 output columns, with kind::i8 MMAs whose A operand
// is the UNSIGNED nibble q (unpacked to bytes in shared memory: two logic operations per eight
// weights, nothing else touches a weight) and whose B operand are the h / l rows:
//   P_hi[n,m] = sum_k q h,   P_lo[n,m] = sum_k q l        (exact int32, one TMEM column each)
// and the epilogue folds   s[n,g] * (128 P_hi + P_lo - zp[n,g] * Sv[g,m])   into fp32 registers.
// The only inexact steps are the 15-bit activation rounding and the fp32 sum over groups; the
// reference (src/onnx/parse_matmulnbits.cpp:85-158 IR on the ref target) rounds every
// dequantised weight to fp16 instead, which is the coarser of the two.
//
// CTA = 320 threads: warp 0 TMA producer, warp 1 TMEM owner + MMA issuer, warps 2..5 unpack
// nibbles -> bytes (UMMA K-major, 128-byte swizzle), warps 6..9 epilogue.  One pipeline stage
// = one group: 8 KB packed weights (TMA), 16 KB unpacked operand, up to 4 KB activation rows
// (TMA).  Two TMEM buffers of 256 columns hold a "pass" of 16 (NB = 16) or 8 (NB = 32) groups,
// so the fold of one pass overlaps the MMAs of the next.  Only plain TMA loads; every wait is
// bounded.
#include "common.cuh"
#include "ptx.cuh"
#include <cuda_fp16.h>

namespace mgx {

constexpr int TC_ROWS    = 128; // output columns (weight rows) per CTA tile = UMMA M
constexpr int TC_GROUP_K = 128; // k per stage
constexpr int TC_STAGES  = 7;
constexpr int TC_PACKED  = TC_ROWS * TC_GROUP_K / 2; // 8192
constexpr int TC_UNPACK  = TC_ROWS * TC_GROUP_K;     // 16384
constexpr int TC_ACT     = 32 * TC_GROUP_K;          // 4096 (room for NB = 32)
constexpr int TC_STAGE   = TC_PACKED + TC_UNPACK + TC_ACT;
constexpr int TC_EPI     = 16 * 128 * 4 + 2 * 128 * 4; // epilogue staging (scales, group sums)
constexpr int TC_SMEM    = TC_STAGES * TC_STAGE + 512 + TC_EPI + 1024;
constexpr int TC_THREADS = 320;
constexpr int TC_PASS_COLS = 256;

struct tc_params
{
    const __half* scales;
    const uint8_t* zp; // may be null
    const float* sa;   // [MB] per-row activation scale
    const int* sv;     // [K/128][MB] per-group sums of the quantised activations
    __half* D;
    float* partial;
    int64_t M, N, K, ldd;
    int group, groups_per_row, zp_const, act;
    int items_total, items_per_cta; // (tile, group) work items, see the main kernel
};

// ------------------------------------------------------------------ activation pre-kernel
// grid = MB blocks (one per padded activation row), 256 threads.
template <int MB>
__global__ void __launch_bounds__(256)
    w4_prepare_acts_kernel(const __half* __restrict__ A, int64_t lda, int64_t M, int64_t K,
                           int8_t* __restrict__ aq, float* __restrict__ sa, int* __restrict__ sv)
{
    __shared__ float red[8];
    __shared__ float s_scale;
    const int m   = blockIdx.x;
    const int tid = threadIdx.x;
    int8_t* hi    = aq + static_cast<int64_t>(m) * K;
    int8_t* lo    = aq + static_cast<int64_t>(MB + m) * K;
    if(m >= M)
    {
        for(int64_t k = tid * 16; k < K; k += 256 * 16)
        {
            *reinterpret_cast<uint4*>(hi + k) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(lo + k) = make_uint4(0u, 0u, 0u, 0u);
        }
        for(int64_t g = tid; g < K / 128; g += 256)
            sv[g * MB + m] = 0;
        if(tid == 0)
            sa[m] = 0.0f;
        return;
    }
    const __half* row = A + m * lda;
    float mx          = 0.0f;
    for(int64_t k = tid * 8; k < K; k += 256 * 8)
    {
        const uint4 v    = *reinterpret_cast<const uint4*>(row + k);
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
    if(tid == 0)
    {
        float t = 0.0f;
        for(int i = 0; i < 8; ++i)
            t = fmaxf(t, red[i]);
        // 128 h + l spans [-16256, 16256] with h in [-127, 127], l in [-64, 64]
        s_scale = t > 0.0f ? t / 16256.0f : 1.0f;
        sa[m]   = s_scale;
    }
    __syncthreads();
    const float inv = 1.0f / s_scale;
    // a warp handles one group of 128 k per trip: lane -> 4 consecutive k
    const int warp = tid >> 5, lane = tid & 31;
    for(int64_t g = warp; g < K / 128; g += 8)
    {
        const int64_t k0 = g * 128 + lane * 4;
        const uint2 v    = *reinterpret_cast<const uint2*>(row + k0);
        const __half* vh = reinterpret_cast<const __half*>(&v);
        int sum          = 0;
        int hq[4], lq[4];
#pragma unroll
        for(int e = 0; e < 4; ++e)
        {
            int q = __float2int_rn(__half2float(vh[e]) * inv);
            q     = max(-16256, min(16256, q));
            const int h = (q + 64 + 128 * 256) / 128 - 256; // round(q / 128) for any sign
            hq[e] = h;
            lq[e] = q - 128 * h;
            sum += q;
        }
#pragma unroll
        for(int o = 16; o > 0; o >>= 1)
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if(lane == 0)
            sv[g * MB + m] = sum;
        // k order inside every 8: evens first, then odds (the order the unpacked nibbles have):
        // position p of the octet goes to (p & 1) * 4 + p / 2
        const int64_t ob = k0 & ~int64_t{7};
#pragma unroll
        for(int e = 0; e < 4; ++e)
        {
            const int pp   = static_cast<int>(k0 & 7) + e;
            const int perm = (pp & 1) * 4 + (pp >> 1);
            hi[ob + perm]  = static_cast<int8_t>(hq[e]);
            lo[ob + perm]  = static_cast<int8_t>(lq[e]);
        }
    }
}

// ------------------------------------------------------------------ main kernel
// Work is the flat list of (tile, group) items, tile-major: item f -> tile f / G, group f % G
// (G = K / 128).  CTA c owns items [c U, (c + 1) U): every SM streams the same number of
// 8 KB weight blocks whatever N and K are.  A CTA's share of one tile is a "segment"; a
// segment that is the whole tile is written to D, any other goes to partial slot
// c - (tile G) / U and the reduce kernel adds the slots in a fixed order.
struct tc_walk
{
    int f, f_hi, G;
    // next pass: at most `cap` groups of one tile
    __device__ bool next(int cap, int& tile, int& g0, int& count, bool& seg_last)
    {
        if(f >= f_hi)
            return false;
        tile              = f / G;
        g0                = f - tile * G;
        const int seg_end = min(f_hi, (tile + 1) * G);
        count             = min(cap, seg_end - f);
        seg_last          = f + count == seg_end;
        f += count;
        return true;
    }
};

// NB: activation rows in the B operand (= UMMA N): 16 (M <= 8: 8 h rows + 8 l rows) or 32.
template <int NB>
__global__ void __launch_bounds__(TC_THREADS, 1)
    w4a16_tc_kernel(const __grid_constant__ CUtensorMap tmap_w,
                    const __grid_constant__ CUtensorMap tmap_a,
                    const tc_params p)
{
    constexpr int MB     = NB / 2;                // padded activation rows
    constexpr int GPP    = TC_PASS_COLS / NB;     // groups per pass (one TMEM buffer)
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem           = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint8_t* bar_base       = smem + TC_STAGES * TC_STAGE;
    uint64_t* full_bar      = reinterpret_cast<uint64_t*>(bar_base);
    uint64_t* unp_bar       = full_bar + TC_STAGES;
    uint64_t* empty_bar     = unp_bar + TC_STAGES;
    uint64_t* accf_bar      = empty_bar + TC_STAGES;
    uint64_t* acce_bar      = accf_bar + 2;
    uint64_t* epi_bar       = acce_bar + 2;
    uint32_t* tmem_slot     = reinterpret_cast<uint32_t*>(epi_bar + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    // epilogue staging: per thread GPP words (scale | zero point << 16), then two buffers of
    // GPP x MB activation group sums
    uint32_t* epi_sz = reinterpret_cast<uint32_t*>(bar_base + 512);
    int* epi_sv      = reinterpret_cast<int*>(epi_sz + GPP * 128);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < TC_STAGES; ++s)
        {
            mbar_init(&full_bar[s], 1);
            mbar_init(&unp_bar[s], 128);
            mbar_init(&empty_bar[s], 1);
        }
        for(int b = 0; b < 2; ++b)
        {
            mbar_init(&accf_bar[b], 1);
            mbar_init(&acce_bar[b], 4);
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
    const int f_lo   = min(p.items_total, static_cast<int>(blockIdx.x) * p.items_per_cta);
    const int f_hi   = min(p.items_total, f_lo + p.items_per_cta);
    const int nitems = f_hi - f_lo;

    if(warp == 0)
    {
        // ---------------------------------------------------- TMA producer
        if(lane == 0)
        {
            int tile = f_lo / G, g = f_lo - tile * G;
            for(int i = 0; i < nitems; ++i)
            {
                const uint32_t s  = i % TC_STAGES;
                const uint32_t ph = (i / TC_STAGES) & 1u;
                if(not mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, 2))
                    break;
                uint8_t* st = smem + s * TC_STAGE;
                mbar_expect_tx(&full_bar[s], TC_PACKED + NB * TC_GROUP_K);
                tma_load_2d(st, &tmap_w, &full_bar[s], g * (TC_GROUP_K / 2), tile * TC_ROWS);
                tma_load_2d(st + TC_PACKED + TC_UNPACK, &tmap_a, &full_bar[s], g * TC_GROUP_K, 0);
                if(++g == G)
                {
                    g = 0;
                    ++tile;
                }
            }
        }
    }
    else if(warp == 1)
    {
        // ---------------------------------------------------- MMA issuer
        if(lane == 0)
        {
            // D s32 += A u8 (weights, K-major) * B s8 (activation rows, K-major); M = 128, N = NB
            constexpr uint32_t idesc = make_idesc(2u, 0u, 1u, TC_ROWS, NB);
            tc_walk walk{f_lo, f_hi, G};
            int tile, g0, count;
            bool seg_last;
            bool ok = true;
            int i   = 0;
            for(uint32_t pc = 0; ok and walk.next(GPP, tile, g0, count, seg_last); ++pc)
            {
                const uint32_t buf = pc & 1u;
                if(not mbar_wait_bounded(&acce_bar[buf], ((pc >> 1) & 1u) ^ 1u, abort_flag, 4))
                    break;
                tc_fence_after_sync();
                for(int gl = 0; gl < count; ++gl, ++i)
                {
                    const uint32_t s  = i % TC_STAGES;
                    const uint32_t ph = (i / TC_STAGES) & 1u;
                    // unpacked weights ready (generic-proxy writes, fenced by the unpack
                    // threads) and activation rows landed (TMA)
                    if(not mbar_wait_bounded(&unp_bar[s], ph, abort_flag, 5) or
                       not mbar_wait_bounded(&full_bar[s], ph, abort_flag, 1))
                    {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t st     = smem_u32(smem + s * TC_STAGE);
                    const uint64_t adesc  = make_smem_desc_sw128(st + TC_PACKED);
                    const uint64_t bdesc  = make_smem_desc_sw128(st + TC_PACKED + TC_UNPACK);
                    const uint32_t d_tmem = tmem_base + buf * TC_PASS_COLS + gl * NB;
#pragma unroll
                    for(int k = 0; k < 4; ++k)
                    {
                        const uint64_t koff = static_cast<uint64_t>((k * 32) >> 4);
                        mma_i8(d_tmem, adesc + koff, bdesc + koff, idesc, k != 0);
                    }
                    tc_commit(&empty_bar[s]);
                }
                if(ok)
                    tc_commit(&accf_bar[buf]);
            }
        }
    }
    else if(warp < 6)
    {
        // ---------------------------------------------------- unpack: nibbles -> bytes
        // thread -> (row, 16 packed bytes = 32 k); 4 lanes cover a row's 64 packed bytes
        const int ut = threadIdx.x - 64; // 0..127
        for(int i = 0; i < nitems; ++i)
        {
            const uint32_t s  = i % TC_STAGES;
            const uint32_t ph = (i / TC_STAGES) & 1u;
            if(not mbar_wait_bounded(&full_bar[s], ph, abort_flag, 1))
                break;
            const uint8_t* pk = smem + s * TC_STAGE;
            uint8_t* up       = smem + s * TC_STAGE + TC_PACKED;
#pragma unroll
            for(int it = 0; it < 4; ++it)
            {
                const int idx = it * 128 + ut;
                const int row = idx >> 2;
                const int j   = idx & 3;
                const uint4 w = *reinterpret_cast<const uint4*>(pk + row * 64 + j * 16);
                uint4 c0, c1;
                c0.x = w.x & 0x0F0F0F0Fu, c0.y = (w.x >> 4) & 0x0F0F0F0Fu;
                c0.z = w.y & 0x0F0F0F0Fu, c0.w = (w.y >> 4) & 0x0F0F0F0Fu;
                c1.x = w.z & 0x0F0F0F0Fu, c1.y = (w.z >> 4) & 0x0F0F0F0Fu;
                c1.z = w.w & 0x0F0F0F0Fu, c1.w = (w.w >> 4) & 0x0F0F0F0Fu;
                uint8_t* dst = up + row * 128;
                *reinterpret_cast<uint4*>(dst + (((2 * j) ^ (row & 7)) * 16))     = c0;
                *reinterpret_cast<uint4*>(dst + (((2 * j + 1) ^ (row & 7)) * 16)) = c1;
            }
            fence_proxy_async_smem(); // make the generic-proxy stores visible to the tensor core
            mbar_arrive(&unp_bar[s]);
        }
    }
    else
    {
        // ---------------------------------------------------- epilogue: fold the groups
        // The per-group metadata of pass i + 1 (scale and zero point of this thread's output
        // column, the activation group sums) is fetched while pass i is folded, so that no
        // global load sits between two TMEM reads.
        const int quarter = warp & 3;
        const int te      = threadIdx.x - 192; // 0..127
        const int ratio   = p.group / TC_GROUP_K;
        float out[MB];
#pragma unroll
        for(int m = 0; m < MB; ++m)
            out[m] = 0.0f;
        tc_walk ahead{f_lo, f_hi, G};
        tc_walk walk{f_lo, f_hi, G};
        uint32_t nx[GPP];
        int nsv = 0;
        auto fetch = [&](int tile, int g0, int count) {
            const int64_t n  = static_cast<int64_t>(tile) * TC_ROWS + quarter * 32 + lane;
            const int64_t nn = n < p.N ? n : p.N - 1;
            const __half* srow  = p.scales + nn * p.groups_per_row;
            const uint8_t* zrow = p.zp == nullptr ? nullptr : p.zp + nn * p.groups_per_row;
#pragma unroll
            for(int gl = 0; gl < GPP; ++gl)
            {
                uint32_t w = 0;
                if(gl < count)
                {
                    const int gi = (g0 + gl) / ratio;
                    const uint32_t sc =
                        __ldg(reinterpret_cast<const unsigned short*>(srow) + gi);
                    const uint32_t z = zrow == nullptr ? static_cast<uint32_t>(p.zp_const)
                                                       : static_cast<uint32_t>(__ldg(zrow + gi));
                    w = sc | (z << 16);
                }
                nx[gl] = w;
            }
            const int ge = te / MB;
            nsv          = ge < count ? __ldg(p.sv + static_cast<int64_t>(g0) * MB + te) : 0;
        };
        auto stage = [&](uint32_t pc) {
#pragma unroll
            for(int gl = 0; gl < GPP; ++gl)
                epi_sz[gl * 128 + te] = nx[gl];
            epi_sv[(pc & 1u) * 128 + te] = nsv;
            mbar_arrive(epi_bar);
            return mbar_wait_bounded(epi_bar, pc & 1u, abort_flag, 6);
        };
        int tile, g0, count, a_tile, a_g0, a_count;
        bool seg_last, a_last;
        bool more = ahead.next(GPP, a_tile, a_g0, a_count, a_last);
        bool ok   = true;
        if(more)
        {
            fetch(a_tile, a_g0, a_count);
            ok = stage(0);
        }
        for(uint32_t pc = 0; ok and walk.next(GPP, tile, g0, count, seg_last); ++pc)
        {
            const uint32_t buf = pc & 1u;
            more = ahead.next(GPP, a_tile, a_g0, a_count, a_last);
            if(more)
                fetch(a_tile, a_g0, a_count);
            if(not mbar_wait_bounded(&accf_bar[buf], (pc >> 1) & 1u, abort_flag, 3))
                break;
            tc_fence_after_sync();
            const int* svb = epi_sv + buf * 128;
#pragma unroll 1
            for(int gl = 0; gl < count; ++gl)
            {
                const uint32_t w = epi_sz[gl * 128 + te];
                const float sc   = __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xFFFFu)));
                const int z      = static_cast<int>(w >> 16);
                uint32_t acc[NB];
                __syncwarp();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       buf * TC_PASS_COLS + gl * NB;
                if constexpr(NB == 16)
                    tmem_ld_32x32b_x16(taddr, acc);
                else
                    tmem_ld_32x32b_x32(taddr, acc);
                tmem_ld_wait();
#pragma unroll
                for(int m = 0; m < MB; ++m)
                {
                    const int v = (static_cast<int>(acc[m]) << 7) + static_cast<int>(acc[MB + m]) -
                                  z * svb[gl * MB + m];
                    out[m] = fmaf(sc, static_cast<float>(v), out[m]);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if(lane == 0)
                mbar_arrive(&acce_bar[buf]);
            if(seg_last)
            {
                // this CTA's share of the tile is complete
                const int64_t n   = static_cast<int64_t>(tile) * TC_ROWS + quarter * 32 + lane;
                const bool whole  = f_lo <= tile * G and f_hi >= (tile + 1) * G;
                const int slot    = static_cast<int>(blockIdx.x) - (tile * G) / p.items_per_cta;
#pragma unroll
                for(int m = 0; m < MB; ++m)
                {
                    if(m < p.M and n < p.N)
                    {
                        const float v = out[m] * __ldg(p.sa + m);
                        if(whole)
                            p.D[m * p.ldd + n] = __float2half_rn(v);
                        else
                            p.partial[(static_cast<int64_t>(slot) * p.M + m) * p.N + n] = v;
                    }
                    out[m] = 0.0f;
                }
            }
            if(more)
                ok = stage(pc + 1);
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

// Adds the partial slots of every tile that more than one CTA worked on (slot order = CTA
// order, so the sum is the same from run to run).
__global__ void __launch_bounds__(256)
    w4a16_tc_reduce_kernel(const float* __restrict__ partial, __half* __restrict__ D, int64_t M,
                           int64_t N, int64_t ldd, int G, int items_per_cta)
{
    const int64_t total = M * N;
    for(int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
        i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        const int64_t m = i / N, n = i - m * N;
        const int tile  = static_cast<int>(n / TC_ROWS);
        const int first = (tile * G) / items_per_cta;
        const int last  = ((tile + 1) * G - 1) / items_per_cta;
        if(first == last)
            continue; // written by the one CTA that owned the whole tile
        float v = 0.0f;
        for(int s = 0; s <= last - first; ++s)
            v += partial[s * total + i];
        D[m * ldd + n] = __float2half_rn(v);
    }
}

// ------------------------------------------------------------------ host
namespace {

struct tc_plan
{
    int nb, mb, tiles, groups, items_total, items_per_cta, grid, slots;
    size_t off_sa, off_sv, off_partial, total;
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

tc_plan make_plan(const mgx_w4_desc& d)
{
    tc_plan pl{};
    pl.nb            = d.M <= 8 ? 16 : 32;
    pl.mb            = pl.nb / 2;
    pl.tiles         = static_cast<int>(ceil_div(d.N, TC_ROWS));
    pl.groups        = static_cast<int>(d.K / TC_GROUP_K);
    pl.items_total   = pl.tiles * pl.groups;
    // one CTA per SM, the same number of items (+-1) each
    pl.items_per_cta = static_cast<int>(ceil_div(pl.items_total, device_sm_count()));
    pl.grid          = static_cast<int>(ceil_div(pl.items_total, pl.items_per_cta));
    // CTAs that can share one tile
    pl.slots       = (pl.groups - 1) / pl.items_per_cta + 2;
    pl.off_sa      = align_up(static_cast<size_t>(pl.nb) * d.K, 256);
    pl.off_sv      = pl.off_sa + 256;
    pl.off_partial = align_up(pl.off_sv + static_cast<size_t>(pl.groups) * pl.mb * sizeof(int), 256);
    pl.total       = pl.off_partial + static_cast<size_t>(pl.slots) * d.M * d.N * sizeof(float);
    return pl;
}

int encode_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint64_t pitch,
              uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swz)
{
    cuTensorMapEncodeTiled_t encode = get_tensor_map_encoder();
    if(encode == nullptr)
        return MGX_E_DRIVER;
    cuuint64_t dims[2]    = {inner, rows};
    cuuint64_t strides[1] = {pitch};
    cuuint32_t box[2]     = {box_inner, box_rows};
    cuuint32_t estr[2]    = {1u, 1u};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MGX_OK : MGX_E_INVALID_ARG;
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
    if((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 or (reinterpret_cast<uintptr_t>(Bp) & 15u) != 0)
        return MGX_E_ALIGNMENT;
    auto* ws   = static_cast<uint8_t*>(workspace);
    auto* aq   = reinterpret_cast<int8_t*>(ws);
    auto* sa   = reinterpret_cast<float*>(ws + pl.off_sa);
    auto* sv   = reinterpret_cast<int*>(ws + pl.off_sv);
    auto* part = reinterpret_cast<float*>(ws + pl.off_partial);
    if(pl.nb == 16)
        w4_prepare_acts_kernel<8><<<8, 256, 0, stream>>>(static_cast<const __half*>(A), d.lda, d.M, d.K, aq, sa, sv);
    else
        w4_prepare_acts_kernel<16><<<16, 256, 0, stream>>>(static_cast<const __half*>(A), d.lda, d.M, d.K, aq, sa, sv);
    cudaError_t e = cudaGetLastError();
    if(e != cudaSuccess)
        return static_cast<int>(e);
    CUtensorMap tw, ta;
    int rc = encode_2d(&tw, Bp, static_cast<uint64_t>(d.K / 2), static_cast<uint64_t>(d.N),
                       static_cast<uint64_t>(d.K / 2), TC_GROUP_K / 2, TC_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
    if(rc != MGX_OK)
        return rc;
    rc = encode_2d(&ta, aq, static_cast<uint64_t>(d.K), static_cast<uint64_t>(pl.nb),
                   static_cast<uint64_t>(d.K), TC_GROUP_K, static_cast<uint32_t>(pl.nb),
                   CU_TENSOR_MAP_SWIZZLE_128B);
    if(rc != MGX_OK)
        return rc;
    tc_params p{};
    p.scales           = static_cast<const __half*>(scales);
    p.zp               = static_cast<const uint8_t*>(zp);
    p.sa               = sa;
    p.sv               = sv;
    p.D                = static_cast<__half*>(D);
    p.partial          = part;
    p.M                = d.M;
    p.N                = d.N;
    p.K                = d.K;
    p.ldd              = d.ldd;
    p.group            = d.group;
    p.groups_per_row   = static_cast<int>(d.K / d.group);
    p.zp_const         = d.zp_const;
    p.act              = d.act;
    p.items_total      = pl.items_total;
    p.items_per_cta    = pl.items_per_cta;
    const int grid     = pl.grid;
    if(pl.nb == 16)
    {
        rc = ensure_smem_optin(reinterpret_cast<const void*>(w4a16_tc_kernel<16>), TC_SMEM);
        if(rc != MGX_OK)
            return rc;
        w4a16_tc_kernel<16><<<grid, TC_THREADS, TC_SMEM, stream>>>(tw, ta, p);
    }
    else
    {
        rc = ensure_smem_optin(reinterpret_cast<const void*>(w4a16_tc_kernel<32>), TC_SMEM);
        if(rc != MGX_OK)
            return rc;
        w4a16_tc_kernel<32><<<grid, TC_THREADS, TC_SMEM, stream>>>(tw, ta, p);
    }
    e = cudaGetLastError();
    if(e != cudaSuccess)
        return static_cast<int>(e);
    if(pl.items_per_cta % pl.groups != 0)
    {
        // some tile is shared between CTAs
        const int64_t total = d.M * d.N;
        const int blocks    = static_cast<int>(ceil_div(total, 256) < 592 ? ceil_div(total, 256) : 592);
        w4a16_tc_reduce_kernel<<<blocks, 256, 0, stream>>>(part, static_cast<__half*>(D), d.M, d.N,
                                                           d.ldd, pl.groups, pl.items_per_cta);
        e = cudaGetLastError();
    }
    return static_cast<int>(e);
}

int w4a16_tc_status(unsigned int* out) { return read_and_clear_status(out); }

} // namespace mgx
