// Weight-only int4 linear for decode (M <= 16 rows of activations) on the tcgen05 tensor core,
// built to be bound by the HBM stream of packed weights:
//
//   D[m,n] = sum_g  s[n,g] * sum_{k in g} (q[n,k] - zp[n,g]) * a[m,k]
//
// is evaluated with INTEGER tensor-core arithmetic.  A small pre-kernel writes every
// activation row as int8 rows (a ~ sa[g,m] * (128 h + l), |error| <= sa/2, i.e. 15 bits of the
// range of the row's own group g of 128 k: an outlier costs only the 127 other values of its
// group precision, not the whole row) and the per-group sums Sv[g,m] = sum_k (128 h + l).  The main kernel computes,
// per group g of 128 k and per 128 output columns, with kind::i8 MMAs whose A operand are the
// UNSIGNED weights and whose B operand are the activation rows, exact int32 sums
// Q[n,m] = sum_k q[n,k] a_int[m,k] (spread over 2 or 4 accumulator columns per activation row,
// see RAW below), and the epilogue folds  s[n,g] * sa[g,m] * (Q - zp[n,g] * Sv[g,m])  into fp32
// registers.
// The only inexact steps are the 15-bit activation rounding and the fp32 sum over groups; the
// reference (src/onnx/parse_matmulnbits.cpp:85-158 IR on the ref target) rounds every
// dequantised weight to fp16 instead, which is the coarser of the two.
//
// CTA = 480 threads (608 with a second set of epilogue warps), one CTA per SM:
//   warp 0        TMA producer: per work item (4 groups) two requests of 128 rows x 128 bytes of
//                 packed weights and one of the activation rows of the same groups
//   warps 2..5    unpack: one thread per weight row, shared memory -> registers -> the row's lane
//                 of TENSOR MEMORY (tcgen05.st); the MMA reads its A operand from there, so the
//                 unpacked bytes never cross shared memory
//   warps 1, 10..12  MMA issuers, one thread each: group i of every work item (an issue costs a
//                 thread about 80 cycles)
//   warps 13, 14  cp.async copies of the epilogue's scales / zero points / group sums, up to
//                 three passes ahead
//   warps 6..9 (and 15..18)  epilogue fold out of two accumulator buffers; the last warp to
//                 finish its 32 columns of a tile that several CTAs share adds the partial sums
//                 in a fixed order
// Launches are chained programmatically: the main kernel streams weights while the pre-kernel
// (and the tail of the previous kernel of the stream) still runs.
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
constexpr int TC_THREADS  = 480;
constexpr int TC_ISSUERS  = 4;   // MMA-issuing threads, one per group of a work item
constexpr int TC_ACC_COLS = 128; // accumulator columns per buffer (two buffers)
constexpr int TC_A_COL0   = 256; // first tensor-memory column of the A operand buffers
constexpr int TC_A_COLS   = TC_GROUP_K / 4; // 32 columns per group
constexpr int TC_EPI      = 3 * 128 * (5 + 3 + 2) * 4 + 64; // epilogue metadata

// ring depth by B-operand width; a stage = 32 KB of weights + 4 NB x 128 bytes of activations
template <int NB>
struct tc_cfg
{
    static constexpr int stages = NB == 16 ? 5 : 4;
    static constexpr int stage  = TC_WSTAGE + TC_SUPER * NB * TC_GROUP_K;
    static constexpr int ring   = stages * stage;
    static constexpr int smem   = ring + 512 + TC_EPI + 1024;
};

struct tc_params
{
    const __half* scales;
    const uint8_t* zp; // may be null
    const float* sa;   // [K/128][MB] activation scale of every (group, row)
    const int* sv;     // [K/128][MB] per-group sums of the quantised activations
    __half* D;
    float* partial;    // [slots][M][N]
    int* counters;     // [tiles][4] warps (by lane quarter) done with a shared tile, zeroed by the pre-kernel
    int64_t M, N, K, ldd;
    int group, groups_per_row, zp_const, act;
    int items_total, items_per_cta; // (tile, 4-group block) work items, see the main kernel
};

// ------------------------------------------------------------------ activation pre-kernel
// grid = MB blocks (one per padded activation row), 1024 threads; a thread owns 8 consecutive k.
// Every activation becomes q = round(a / sa) = 128 h + l.  Two layouts of the int8 rows the
// tensor core multiplies with the weights (K bytes per row, 128 per group):
//   RAW = false (2 rows per activation row m): row 2 m = h, row 2 m + 1 = l; inside every 8 k the
//         evens first, then the odds (the order of the nibbles unpacked to bytes);
//   RAW = true  (4 rows per m), for a weight operand whose first 64 bytes of a group are the LOW
//         nibbles L_j = q[2j] and whose last 64 bytes are the packed bytes B_j = 16 q[2j+1] + L_j
//         themselves: rows [e | 0] and [-o | o] for each of h and l, e_j = a[2j], o_j = a[2j+1], so
//         that  sum_j L_j e_j  and  sum_j (B_j - L_j) o_j = 16 sum_j q[2j+1] o_j  come out.
// Also written: sv (per-group sums of q), sa (per-group scales), zeroed tile counters.
template <int MB, bool RAW>
__global__ void __launch_bounds__(1024)
    w4_prepare_acts_kernel(const __half* __restrict__ A, int64_t lda, int64_t M, int64_t K,
                           int8_t* __restrict__ aq, float* __restrict__ sa, int* __restrict__ sv,
                           int* __restrict__ counters, int ncounters)
{
    // the main kernel may start (and stream weights) right away; it waits for this grid's
    // completion before it touches anything written here
    grid_launch_dependents();
    // this kernel itself may have been started before the previous kernel of the stream has
    // finished (which may still read the workspace, or be writing A)
    grid_dependency_wait();
    constexpr int RPM = RAW ? 4 : 2; // int8 rows per activation row
    const int m   = blockIdx.x;
    const int tid = threadIdx.x;
    int8_t* rows  = aq + static_cast<int64_t>(RPM * m) * K;
    for(int i = blockIdx.x * 1024 + tid; i < ncounters; i += gridDim.x * 1024)
        counters[i] = 0;
    if(m >= M)
    {
        for(int64_t k = tid * 16; k < RPM * K; k += 1024 * 16)
            *reinterpret_cast<uint4*>(rows + k) = make_uint4(0u, 0u, 0u, 0u);
        for(int64_t g = tid; g < K / 128; g += 1024)
        {
            sv[g * MB + m] = 0;
            sa[g * MB + m] = 0.0f;
        }
        return;
    }
    const __half* row = A + m * lda;
    for(int64_t kb = 0; kb < K; kb += 1024 * 8)
    {
        // every thread of a warp takes the same trips (the reductions below are warp shuffles);
        // 16 consecutive threads hold one group of 128 k
        const int64_t k  = kb + tid * 8;
        const bool valid = k < K;
        const uint4 v    = valid ? *reinterpret_cast<const uint4*>(row + k) : make_uint4(0u, 0u, 0u, 0u);
        const __half* vh = reinterpret_cast<const __half*>(&v);
        float mx         = 0.0f;
#pragma unroll
        for(int e = 0; e < 8; ++e)
            mx = fmaxf(mx, fabsf(__half2float(vh[e])));
#pragma unroll
        for(int o = 8; o > 0; o >>= 1)
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        // 128 h + l spans [-16256, 16256] with h in [-127, 127], l in [-64, 63]
        const float scale = mx > 0.0f ? mx / 16256.0f : 1.0f;
        const float inv   = 1.0f / scale;
        int sum           = 0;
        // bytes of the evens (e = 0, 2, 4, 6) and of the odds, for h and for l
        uint32_t he = 0u, ho = 0u, le = 0u, lo = 0u, nho = 0u, nlo = 0u;
#pragma unroll
        for(int e = 0; e < 8; ++e)
        {
            int q = __float2int_rn(__half2float(vh[e]) * inv);
            q     = max(-16256, min(16256, q));
            const int h = (q + 64 + 128 * 256) / 128 - 256; // round(q / 128) for any sign
            const int l = q - 128 * h;
            sum += q;
            const int sh = 8 * (e >> 1);
            if(e & 1)
            {
                ho |= static_cast<uint32_t>(h & 0xFF) << sh;
                lo |= static_cast<uint32_t>(l & 0xFF) << sh;
                nho |= static_cast<uint32_t>(-h & 0xFF) << sh;
                nlo |= static_cast<uint32_t>(-l & 0xFF) << sh;
            }
            else
            {
                he |= static_cast<uint32_t>(h & 0xFF) << sh;
                le |= static_cast<uint32_t>(l & 0xFF) << sh;
            }
        }
        if(valid)
        {
            if constexpr(RAW)
            {
                // byte j = k / 2 of the group's low half, 64 + j of its high half
                const int64_t o = (k & ~int64_t{127}) + ((k & 127) >> 1);
                *reinterpret_cast<uint32_t*>(rows + o)              = he;
                *reinterpret_cast<uint32_t*>(rows + o + 64)         = 0u;
                *reinterpret_cast<uint32_t*>(rows + K + o)          = nho;
                *reinterpret_cast<uint32_t*>(rows + K + o + 64)     = ho;
                *reinterpret_cast<uint32_t*>(rows + 2 * K + o)      = le;
                *reinterpret_cast<uint32_t*>(rows + 2 * K + o + 64) = 0u;
                *reinterpret_cast<uint32_t*>(rows + 3 * K + o)      = nlo;
                *reinterpret_cast<uint32_t*>(rows + 3 * K + o + 64) = lo;
            }
            else
            {
                *reinterpret_cast<uint2*>(rows + k)     = make_uint2(he, ho);
                *reinterpret_cast<uint2*>(rows + K + k) = make_uint2(le, lo);
            }
        }
#pragma unroll
        for(int o = 8; o > 0; o >>= 1)
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if(valid and (tid & 15) == 0)
        {
            sv[(k >> 7) * MB + m] = sum;
            sa[(k >> 7) * MB + m] = scale;
        }
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
    int tile, sg, left, SG, G; // cursor (tile, block), work items left
    __device__ tc_walk(int f_lo, int f_hi, int sg_per_tile, int groups)
        : tile(f_lo / sg_per_tile),
          sg(f_lo - (f_lo / sg_per_tile) * sg_per_tile),
          left(f_hi - f_lo),
          SG(sg_per_tile),
          G(groups)
    {
    }
    // next pass: at most `cap` (a multiple of TC_SUPER) groups of one tile
    __device__ bool next(int cap, int& tile_out, int& g0, int& count, bool& seg_last)
    {
        if(left <= 0)
            return false;
        tile_out       = tile;
        g0             = sg * TC_SUPER;
        const int nblk = min(cap / TC_SUPER, min(left, SG - sg));
        count          = min(G, (sg + nblk) * TC_SUPER) - g0;
        sg += nblk;
        left -= nblk;
        seg_last = sg == SG or left == 0;
        if(sg == SG)
        {
            sg = 0;
            ++tile;
        }
        return true;
    }
};

// MR: activation rows folded by the epilogue (M <= MR <= MB).
// RAW: the weight operand of a group is [64 bytes of low nibbles | the 64 packed bytes] and every
// activation row has 4 rows in the B operand (see the pre-kernel); otherwise it is the 128
// nibbles unpacked to bytes and 2 rows.  RAW costs one logic operation per eight weights
// instead of three, and twice the accumulator columns per activation row.
// ESETS: sets of four epilogue warps; with two, each set folds half of the MR rows (the second
// set is warps 15..18).
template <int NB, int MR, bool RAW, int ESETS>
__global__ void __launch_bounds__(TC_THREADS + (ESETS - 1) * 128, 1)
    w4a16_tc_kernel(const __grid_constant__ CUtensorMap tmap_w,
                    const __grid_constant__ CUtensorMap tmap_a,
                    const tc_params p)
{
    using cfg            = tc_cfg<NB>;
    constexpr int CPM    = RAW ? 4 : 2;      // accumulator columns per activation row
    constexpr int MB     = NB / CPM;         // padded activation rows
    constexpr int GPP    = TC_ACC_COLS / NB; // groups per pass (one accumulator buffer): 8 or 4
    constexpr int WST    = cfg::stages;
    constexpr int ABYTES = NB * TC_GROUP_K;  // activation rows of one group
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem           = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint8_t* bar_base       = smem + cfg::ring;
    uint64_t* full_bar      = reinterpret_cast<uint64_t*>(bar_base); // weights + activations landed
    uint64_t* empty_bar     = full_bar + WST;   // weights read by all rows, MMAs retired
    uint64_t* unp_bar       = empty_bar + WST;  // A operand in tensor memory
    uint64_t* tfree_bar     = unp_bar + TC_TSTAGES; // MMAs that read it retired
    uint64_t* accf_bar      = tfree_bar + TC_TSTAGES;
    uint64_t* acce_bar      = accf_bar + 2;
    uint64_t* meta_bar      = acce_bar + 2;     // [3] epilogue metadata of a pass staged
    uint64_t* mfree_bar     = meta_bar + 3;     // [3] ... and folded
    uint32_t* tmem_slot     = reinterpret_cast<uint32_t*>(mfree_bar + 3);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    // epilogue metadata, three buffers each: per output column the aligned 32-bit words that
    // hold the scales (at most 5) and zero points (at most 3) of a pass, GPP x MB activation
    // group sums and group scales
    uint32_t* epi_sw = reinterpret_cast<uint32_t*>(bar_base + 512);     // [3][128][5]
    uint32_t* epi_zw = epi_sw + 3 * 128 * 5;                            // [3][128][3]
    int* epi_sv      = reinterpret_cast<int*>(epi_zw + 3 * 128 * 3);    // [3][128]
    float* epi_sa    = reinterpret_cast<float*>(epi_sv + 3 * 128);      // [3][128]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // the next kernel of the stream may be started early if it asks for it (the pre-kernel of
    // the next linear does: it waits for this grid's completion before it reads or writes)
    grid_launch_dependents();
    if(threadIdx.x == 0)
    {
        for(int s = 0; s < WST; ++s)
        {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 128 + TC_ISSUERS);
        }
        for(int b = 0; b < 2; ++b)
        {
            mbar_init(&unp_bar[b], 128);
            mbar_init(&tfree_bar[b], TC_ISSUERS);
            mbar_init(&accf_bar[b], TC_ISSUERS);
            mbar_init(&acce_bar[b], 4 * ESETS);
        }
        for(int b = 0; b < 3; ++b)
        {
            mbar_init(&meta_bar[b], 64);
            mbar_init(&mfree_bar[b], 4 * ESETS);
        }
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
    // MMA issuers: warps 1, 10, 11, 12 -> group 0..3 of every work item
    const int issuer = warp == 1 ? 0 : (warp >= 10 and warp <= 12 ? warp - 9 : -1);

    if(warp == 0)
    {
        // ---------------------------------------------------- TMA producer
        // A stage = 4 groups of packed weights (two requests of 128 rows x 128 bytes) + the
        // activation rows of the same groups.  The weights are constants of the model and
        // are requested at once; the activation rows are written by the pre-kernel, whose
        // completion is awaited before their first request.
        if(lane == 0)
        {
            int tile = f_lo / SG, sg = f_lo - tile * SG;
            int a_sg = sg; // the activation requests trail the weight requests at the start
            const int head = min(nsuper, WST);
            for(int j = 0; j < nsuper; ++j)
            {
                const uint32_t s  = j % WST;
                const uint32_t ph = (j / WST) & 1u;
                if(not mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, 2))
                    break;
                uint8_t* st = smem + s * cfg::stage;
                // groups past the end of K are zero-filled and still counted
                mbar_expect_tx(&full_bar[s], cfg::stage);
                tma_load_2d(st, &tmap_w, &full_bar[s], sg * (TC_WSTAGE / TC_ROWS), tile * TC_ROWS);
                tma_load_2d(st + TC_WSTAGE / 2, &tmap_w, &full_bar[s],
                            sg * (TC_WSTAGE / TC_ROWS) + 128, tile * TC_ROWS);
                if(j >= head)
                    tma_load_3d(st + TC_WSTAGE, &tmap_a, &full_bar[s], 0, 0, sg * TC_SUPER);
                if(++sg == SG)
                {
                    sg = 0;
                    ++tile;
                }
                if(j == head - 1)
                {
                    grid_dependency_wait();
                    for(int i = 0; i < head; ++i)
                    {
                        tma_load_3d(smem + i * cfg::stage + TC_WSTAGE, &tmap_a, &full_bar[i], 0, 0,
                                    a_sg * TC_SUPER);
                        if(++a_sg == SG)
                            a_sg = 0;
                    }
                }
            }
        }
    }
    else if(issuer >= 0)
    {
        // ---------------------------------------------------- MMA issuers
        // One thread of each of four warps issues the four k-steps of "its" group of every
        // work item: an issue costs a thread some 80 cycles, so one thread alone could not
        // keep up with the weight stream.
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
            // the activation planes come from the previous kernel of the stream: the bounded
            // waits below must not count its run time
            grid_dependency_wait();
            for(uint32_t pc = 0; ok and walk.next(GPP, tile, g0, count, seg_last); ++pc)
            {
                const uint32_t buf = pc & 1u;
                if(not mbar_wait_bounded(&acce_bar[buf], ((pc >> 1) & 1u) ^ 1u, abort_flag, 4))
                    break;
                tc_fence_after_sync();
                for(int gl = 0; gl < count; gl += TC_SUPER, ++j)
                {
                    const uint32_t s  = j % WST;
                    const uint32_t t  = j & 1u;
                    const uint32_t tp = (j >> 1) & 1u;
                    // implies that the stage's TMA requests have landed
                    if(not mbar_wait_bounded(&unp_bar[t], tp, abort_flag, 5))
                    {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    if(gl + issuer < count)
                    {
                        const uint32_t b_smem = smem_u32(smem + s * cfg::stage + TC_WSTAGE + issuer * ABYTES);
                        const uint64_t bdesc  = make_smem_desc_sw128(b_smem);
                        const uint32_t a_tmem = tmem_base + TC_A_COL0 + (t * TC_SUPER + issuer) * TC_A_COLS;
                        const uint32_t d_tmem = tmem_base + buf * TC_ACC_COLS + (gl + issuer) * NB;
#pragma unroll
                        for(int k = 0; k < 4; ++k)
                            mma_i8_tmem_a(d_tmem, a_tmem + k * 8,
                                          bdesc + static_cast<uint64_t>((k * 32) >> 4), idesc, k != 0);
                    }
                    tc_commit(&tfree_bar[t]);
                    tc_commit(&empty_bar[s]);
                }
                if(ok)
                    tc_commit(&accf_bar[buf]);
            }
        }
    }
    else if(warp == 13 or warp == 14)
    {
        // ---------------------------------------------------- epilogue metadata, up to 3 passes ahead
        // cp.async copies of the aligned words around the scales and zero points of a pass
        // (consecutive lanes copy consecutive words of a column's run, so a request touches
        // few sectors) and of the activation group sums.  Each of the two warps serves 64
        // output columns.
        grid_dependency_wait(); // sv and sa come from the pre-kernel
        const int half  = warp - 13;
        const int rshift = 31 - __clz(p.group / TC_GROUP_K); // groups are powers of two
        const uint32_t sbase0 = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(p.scales) & 3u);
        const uint32_t zbase0 = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(p.zp) & 3u);
        const char* sptr = reinterpret_cast<const char*>(p.scales) - sbase0; // 4-byte aligned
        const char* zptr = reinterpret_cast<const char*>(p.zp) - zbase0;
        auto cp_async4 = [](const void* dst, const void* src) {
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src)
                         : "memory");
        };
        tc_walk walk(f_lo, f_hi, SG, G);
        int tile, g0, count;
        bool seg_last;
        for(uint32_t pc = 0; walk.next(GPP, tile, g0, count, seg_last); ++pc)
        {
            const uint32_t vb = pc % 3u;
            if(not mbar_wait_bounded(&mfree_bar[vb], ((pc / 3u) & 1u) ^ 1u, abort_flag, 9))
                break;
            const int gi0 = g0 >> rshift;
            const int ng  = ((g0 + count - 1) >> rshift) - gi0 + 1;
            const int n0  = tile * TC_ROWS + half * 64;
            // scales: up to 5 words per column
#pragma unroll 2
            for(int idx = lane; idx < 64 * 5; idx += 32)
            {
                const int r = idx / 5, w = idx - r * 5;
                const int n = min(n0 + r, static_cast<int>(p.N) - 1);
                // byte offsets from the aligned base: first scale, end of the run
                const uint32_t s = sbase0 + static_cast<uint32_t>(n * p.groups_per_row + gi0) * 2u;
                const uint32_t a = s & ~3u;
                const int nw     = static_cast<int>((((s + ng * 2 + 3u) & ~3u) - a) >> 2);
                if(w < nw)
                    cp_async4(epi_sw + (vb * 128 + half * 64 + r) * 5 + w, sptr + a + 4 * w);
            }
            if(p.zp != nullptr)
            {
#pragma unroll 2
                for(int idx = lane; idx < 64 * 3; idx += 32)
                {
                    const int r = idx / 3, w = idx - r * 3;
                    const int n = min(n0 + r, static_cast<int>(p.N) - 1);
                    const uint32_t z = zbase0 + static_cast<uint32_t>(n * p.groups_per_row + gi0);
                    const uint32_t a = z & ~3u;
                    const int nw     = static_cast<int>((((z + ng + 3u) & ~3u) - a) >> 2);
                    if(w < nw)
                        cp_async4(epi_zw + (vb * 128 + half * 64 + r) * 3 + w, zptr + a + 4 * w);
                }
            }
            // group sums and group scales: count x MB words each, half of them per warp
            for(int i = half * 64 + lane; i < count * MB; i += 32)
                if(i < half * 64 + 64)
                {
                    cp_async4(epi_sv + vb * 128 + i, p.sv + static_cast<int64_t>(g0) * MB + i);
                    cp_async4(epi_sa + vb * 128 + i, p.sa + static_cast<int64_t>(g0) * MB + i);
                }
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(
                             smem_u32(&meta_bar[vb]))
                         : "memory");
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    }
    else if(warp < 6)
    {
        // ---------------------------------------------------- unpack: nibbles -> bytes
        // One thread per weight row: 64 packed bytes per group from shared memory (128-byte
        // swizzle, so a quarter warp's 16-byte reads fall in eight different bank groups), 32
        // words to this row's lane of tensor memory: either the nibbles as bytes (inside every
        // 8 k the evens first, then the odds; the activation rows are stored in the same order)
        // or the low nibbles followed by the packed bytes as they are (RAW).
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
            if(not __all_sync(0xffffffffu, mbar_wait_bounded(&full_bar[s], ph, abort_flag, 1)))
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
                    const uint8_t* pk = smem + s * cfg::stage + (q >> 1) * (2 * TC_PACKED) + row * 128;
                    uint32_t u[32];
#pragma unroll
                    for(int c = 0; c < 4; ++c)
                    {
                        const uint4 w =
                            *reinterpret_cast<const uint4*>(pk + ((((q & 1) * 4 + c) ^ sw) << 4));
                        if constexpr(RAW)
                        {
                            u[4 * c + 0] = w.x & 0x0F0F0F0Fu, u[16 + 4 * c + 0] = w.x;
                            u[4 * c + 1] = w.y & 0x0F0F0F0Fu, u[16 + 4 * c + 1] = w.y;
                            u[4 * c + 2] = w.z & 0x0F0F0F0Fu, u[16 + 4 * c + 2] = w.z;
                            u[4 * c + 3] = w.w & 0x0F0F0F0Fu, u[16 + 4 * c + 3] = w.w;
                        }
                        else
                        {
                            u[8 * c + 0] = w.x & 0x0F0F0F0Fu, u[8 * c + 1] = (w.x >> 4) & 0x0F0F0F0Fu;
                            u[8 * c + 2] = w.y & 0x0F0F0F0Fu, u[8 * c + 3] = (w.y >> 4) & 0x0F0F0F0Fu;
                            u[8 * c + 4] = w.z & 0x0F0F0F0Fu, u[8 * c + 5] = (w.z >> 4) & 0x0F0F0F0Fu;
                            u[8 * c + 6] = w.w & 0x0F0F0F0Fu, u[8 * c + 7] = (w.w >> 4) & 0x0F0F0F0Fu;
                        }
                    }
                    tmem_st_32x32b_x32(tmem_base + lane_addr + TC_A_COL0 +
                                           (t * TC_SUPER + q) * TC_A_COLS,
                                       u);
                }
            }
            mbar_arrive(&empty_bar[s]); // the packed blocks are in registers
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
        // Scale, zero point and activation group sums of a pass are already in shared memory
        // (metadata warps).  Column 2 m of a group's accumulator is P_hi, column 2 m + 1 P_lo
        // of activation row m; only the MR rows in use are read.  All arithmetic stays off
        // the conversion pipe except one half -> float per group: |P_hi|, |P_lo| < 2^18.
        grid_dependency_wait(); // sa and the tile counters come from the pre-kernel
        constexpr int MRW = MR / ESETS;          // rows this warp folds ...
        const int eset    = warp >= 15 ? 1 : 0;
        const int m0      = eset * MRW;          // ... starting at this one
        const int quarter = warp & 3;
        const int col     = quarter * 32 + lane; // output column inside the tile = TMEM lane
        const int rshift  = 31 - __clz(p.group / TC_GROUP_K); // groups are powers of two
        const uint32_t sbase0 = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(p.scales) & 3u);
        const uint32_t zbase0 = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(p.zp) & 3u);
        float out[MRW];
#pragma unroll
        for(int m = 0; m < MRW; ++m)
            out[m] = 0.0f;
        tc_walk walk(f_lo, f_hi, SG, G);
        // one group: out[m] += sc sa[m] (Q[m] - z Sv[m]) with Q = sum_k q a_int, in exact integer
        // arithmetic up to the one conversion.  soff / zoff: byte offset of the group's scale /
        // zero point inside this column's staged words
        constexpr int C  = CPM * MRW; // accumulator columns read per group
        const bool has_zp = p.zp != nullptr;
        auto fold = [&](const uint32_t(&acc)[C], int gl, uint32_t vb, uint32_t soff, uint32_t zoff) {
            const uint32_t sw = epi_sw[(vb * 128 + col) * 5 + (soff >> 2)];
            const uint32_t sh = (soff & 2u) ? sw >> 16 : sw & 0xFFFFu;
            float sc          = __half2float(__ushort_as_half(static_cast<unsigned short>(sh)));
            // without zero points the staged word is not meaningful and not used
            const uint32_t zw = epi_zw[(vb * 128 + col) * 3 + (has_zp ? zoff >> 2 : 0u)];
            int z = has_zp ? static_cast<int>((zw >> (8u * (zoff & 3u))) & 0xFFu) : p.zp_const;
            if constexpr(RAW)
            {
                sc *= 0.0625f; // Q is computed times 16
                z *= 16;
            }
            const int* svb   = epi_sv + vb * 128 + gl * MB + m0;
            const float* sab = epi_sa + vb * 128 + gl * MB + m0;
#pragma unroll
            for(int m = 0; m < MRW; ++m)
            {
                int q;
                if constexpr(RAW)
                {
                    // columns: sum L e_h, 16 sum q_odd o_h, sum L e_l, 16 sum q_odd o_l;
                    // 16 Q = 2048 E_h + 128 O_h + 16 E_l + O_l
                    q = static_cast<int>(acc[4 * m]) * 2048 + static_cast<int>(acc[4 * m + 3]);
                    q = static_cast<int>(acc[4 * m + 1]) * 128 + q;
                    q = static_cast<int>(acc[4 * m + 2]) * 16 + q;
                }
                else
                    q = static_cast<int>(acc[2 * m]) * 128 + static_cast<int>(acc[2 * m + 1]);
                q      = q - z * svb[m];
                out[m] = fmaf(sc * sab[m], static_cast<float>(q), out[m]);
            }
        };
        // groups read from tensor memory per trip (all loads in flight before the first fold)
        constexpr int TR = C <= 4 ? 8 : (C <= 8 ? 4 : 2);
        int tile, g0, count;
        bool seg_last;
        bool ok = true;
        for(uint32_t pc = 0; ok and walk.next(GPP, tile, g0, count, seg_last); ++pc)
        {
            const uint32_t buf = pc & 1u;
            const uint32_t vb  = pc % 3u;
            if(not __all_sync(0xffffffffu,
                              mbar_wait_bounded(&meta_bar[vb], (pc / 3u) & 1u, abort_flag, 10)))
                break;
            if(not __all_sync(0xffffffffu,
                              mbar_wait_bounded(&accf_bar[buf], (pc >> 1) & 1u, abort_flag, 3)))
                break;
            tc_fence_after_sync();
            const int gi0 = g0 >> rshift;
            const int n   = min(tile * TC_ROWS + col, static_cast<int>(p.N) - 1);
            const uint32_t sbyte =
                (sbase0 + static_cast<uint32_t>(n * p.groups_per_row + gi0) * 2u) & 3u;
            const uint32_t zbyte = (zbase0 + static_cast<uint32_t>(n * p.groups_per_row + gi0)) & 3u;
            // quantisation group of group gl, relative to gi0
            auto grel = [&](int gl) { return static_cast<uint32_t>(((g0 + gl) >> rshift) - gi0); };
            const uint32_t tbase = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   buf * TC_ACC_COLS + CPM * m0;
#pragma unroll 1
            for(int gl = 0; gl < count; gl += TR)
            {
                uint32_t acc[TR][C];
                if(gl + TR <= count)
                {
                    // full trip: straight-line code, the folds interleave
#pragma unroll
                    for(int t = 0; t < TR; ++t)
                        tmem_ld_32x32b<C>(tbase + (gl + t) * NB, acc[t]);
                    tmem_ld_wait();
#pragma unroll
                    for(int t = 0; t < TR; ++t)
                        fold(acc[t], gl + t, vb, sbyte + 2u * grel(gl + t), zbyte + grel(gl + t));
                }
                else
                {
#pragma unroll
                    for(int t = 0; t < TR; ++t)
                        if(gl + t < count) // the same for the whole warp
                            tmem_ld_32x32b<C>(tbase + (gl + t) * NB, acc[t]);
                    tmem_ld_wait();
#pragma unroll
                    for(int t = 0; t < TR; ++t)
                        if(gl + t < count)
                            fold(acc[t], gl + t, vb, sbyte + 2u * grel(gl + t), zbyte + grel(gl + t));
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if(lane == 0)
            {
                mbar_arrive(&acce_bar[buf]);
                mbar_arrive(&mfree_bar[vb]);
            }
            if(seg_last)
            {
                // this CTA's share of the tile is complete
                const int64_t nc = static_cast<int64_t>(tile) * TC_ROWS + col;
                const bool whole = f_lo <= tile * SG and f_hi >= (tile + 1) * SG;
                if(whole)
                {
#pragma unroll
                    for(int m = 0; m < MRW; ++m)
                        if(m0 + m < p.M and nc < p.N)
                            p.D[(m0 + m) * p.ldd + nc] = __float2half_rn(out[m]);
                }
                else
                {
                    const int first = (tile * SG) / p.items_per_cta;
                    const int last  = ((tile + 1) * SG - 1) / p.items_per_cta;
                    const int slot  = static_cast<int>(blockIdx.x) - first;
#pragma unroll
                    for(int m = 0; m < MRW; ++m)
                        if(m0 + m < p.M and nc < p.N)
                            p.partial[(static_cast<int64_t>(slot) * p.M + m0 + m) * p.N + nc] = out[m];
                    // The tile's 32 columns of this warp are complete when the warps of the same
                    // lane quarter of all its CTAs have counted themselves in; the last one adds
                    // the slots.  The counting atomic releases this warp's stores (ordered before
                    // it by the warp barrier) and acquires the other warps'.
                    __syncwarp();
                    int old = 0;
                    if(lane == 0)
                        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;"
                                     : "=r"(old)
                                     : "l"(p.counters + (tile * 4 + quarter) * ESETS + eset)
                                     : "memory");
                    old = __shfl_sync(0xffffffffu, old, 0);
                    if(old == last - first)
                    {
                        // the MR loads of a slot are in flight together; slots add up in order
                        float v[MRW];
#pragma unroll
                        for(int m = 0; m < MRW; ++m)
                            v[m] = 0.0f;
#pragma unroll 4
                        for(int s = 0; s <= last - first; ++s)
                        {
                            float t[MRW];
#pragma unroll
                            for(int m = 0; m < MRW; ++m)
                                t[m] = m0 + m < p.M and nc < p.N
                                           ? __ldcg(p.partial + (static_cast<int64_t>(s) * p.M + m0 + m) * p.N + nc)
                                           : 0.0f;
#pragma unroll
                            for(int m = 0; m < MRW; ++m)
                                v[m] += t[m];
                        }
#pragma unroll
                        for(int m = 0; m < MRW; ++m)
                            if(m0 + m < p.M and nc < p.N)
                                p.D[(m0 + m) * p.ldd + nc] = __float2half_rn(v[m]);
                    }
                }
#pragma unroll
                for(int m = 0; m < MRW; ++m)
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
    // up to 8 rows: 4 int8 rows per activation row (RAW operand); up to 16: 2 rows
    pl.nb            = d.M <= 4 ? 16 : 32;
    pl.mb            = d.M <= 4 ? 4 : (d.M <= 8 ? 8 : 16);
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
    pl.off_sv       = align_up(pl.off_sa + static_cast<size_t>(pl.groups) * pl.mb * sizeof(float), 256);
    pl.off_counters = align_up(pl.off_sv + static_cast<size_t>(pl.groups) * pl.mb * sizeof(int), 256);
    pl.off_partial  = align_up(pl.off_counters + static_cast<size_t>(pl.tiles) * 8 * sizeof(int), 256);
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

template <int NB, int MR, bool RAW, int ESETS>
int launch_main(int grid, const CUtensorMap& tw, const CUtensorMap& ta, const tc_params& p,
                cudaStream_t stream)
{
    int rc = ensure_smem_optin(reinterpret_cast<const void*>(w4a16_tc_kernel<NB, MR, RAW, ESETS>), tc_cfg<NB>::smem);
    if(rc != MGX_OK)
        return rc;
    // programmatic dependent launch: the kernel may start while the pre-kernel still runs
    // and waits for it (griddepcontrol.wait) only where it reads what the pre-kernel wrote
    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = dim3(static_cast<unsigned>(grid));
    cfg.blockDim         = dim3(TC_THREADS + (ESETS - 1) * 128);
    cfg.dynamicSmemBytes = tc_cfg<NB>::smem;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs                                          = attr;
    cfg.numAttrs                                       = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, w4a16_tc_kernel<NB, MR, RAW, ESETS>, tw, ta, p));
}

} // namespace

bool w4a16_tc_applicable(const mgx_w4_desc& d)
{
    return d.M >= 1 and d.M <= 16 and d.K % TC_GROUP_K == 0 and d.group % TC_GROUP_K == 0 and
           ((d.group / TC_GROUP_K) & (d.group / TC_GROUP_K - 1)) == 0 and d.act == MGX_ACT_NONE and
           d.lda % 8 == 0 and
           ceil_div(d.N, TC_ROWS) * (d.K / TC_GROUP_K) < (int64_t{1} << 30) and
           (d.N + TC_ROWS) * (d.K / d.group) < (int64_t{1} << 30);
}

// The kernel copies the aligned 32-bit word around every scale and zero point, and fetches
// weights and activations in 16-byte units.
bool w4a16_tc_pointers_ok(const mgx_w4_desc& d, const void* A, const void* Bp, const void* scales,
                          const void* zp)
{
    const int64_t nmeta = d.N * (d.K / d.group);
    return ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(Bp)) & 15u) == 0 and
           (reinterpret_cast<uintptr_t>(scales) & 3u) == 0 and nmeta % 2 == 0 and
           (zp == nullptr or ((reinterpret_cast<uintptr_t>(zp) & 3u) == 0 and nmeta % 4 == 0));
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
       not w4a16_tc_pointers_ok(d, A, Bp, scales, zp))
        return MGX_E_ALIGNMENT;
    auto* ws       = static_cast<uint8_t*>(workspace);
    auto* aq       = reinterpret_cast<int8_t*>(ws);
    auto* sa       = reinterpret_cast<float*>(ws + pl.off_sa);
    auto* sv       = reinterpret_cast<int*>(ws + pl.off_sv);
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
    const auto* a16 = static_cast<const __half*>(A);
    {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim          = dim3(static_cast<unsigned>(pl.mb));
        cfg.blockDim         = dim3(1024);
        cfg.dynamicSmemBytes = 0;
        cfg.stream           = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs    = attr;
        cfg.numAttrs = 1;
        const int64_t lda = d.lda, M = d.M, K = d.K;
        const int ntiles  = pl.tiles * 8; // one counter per tile, lane quarter and epilogue warp set
        cudaError_t e     = cudaSuccess;
        if(pl.mb == 4)
            e = cudaLaunchKernelEx(&cfg, w4_prepare_acts_kernel<4, true>, a16, lda, M, K, aq, sa, sv,
                                   counters, ntiles);
        else if(pl.mb == 8)
            e = cudaLaunchKernelEx(&cfg, w4_prepare_acts_kernel<8, true>, a16, lda, M, K, aq, sa, sv,
                                   counters, ntiles);
        else
            e = cudaLaunchKernelEx(&cfg, w4_prepare_acts_kernel<16, false>, a16, lda, M, K, aq, sa,
                                   sv, counters, ntiles);
        if(e != cudaSuccess)
            return static_cast<int>(e);
    }
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
    if(d.M == 1)
        return launch_main<16, 1, true, 1>(pl.grid, tw, ta, p, stream);
    if(d.M == 2)
        return launch_main<16, 2, true, 1>(pl.grid, tw, ta, p, stream);
    if(d.M <= 4)
        return launch_main<16, 4, true, 1>(pl.grid, tw, ta, p, stream);
    if(d.M <= 8)
        return launch_main<32, 8, true, 2>(pl.grid, tw, ta, p, stream);
    return launch_main<32, 16, false, 2>(pl.grid, tw, ta, p, stream);
}

int w4a16_tc_status(unsigned int* out) { return read_and_clear_status(out); }

} // namespace mgx
