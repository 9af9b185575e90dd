// Weight-only int4 linear for prefill (M > 16 activation rows) on the tcgen05 tensor core:
//
//   D[m,n] = sum_k a[m,k] * (q[n,k] - zp[n,k/group]) * s[n,k/group]
//
// as an fp16 x fp16 -> fp32 GEMM whose A operand is dequantised on the fly: the packed weights
// of 128 output columns x 128 k arrive by TMA, four warps (one thread per weight row) turn them
// into fp16 values (q - zp) * s and write them straight into TENSOR MEMORY, and the MMAs read
// their A operand from there; the B operand is the caller's fp16 activation matrix, fetched by
// TMA as it lies in memory.  The dequantised weights never exist in shared or global memory
// (the reference materialises them: src/onnx/parse_matmulnbits.cpp:85-158 IR on the ref target).
//
// CTA tile = 128 output columns x 128 activation rows, all of K; persistent over tiles.
// CTA = 480 threads:
//   warp 0       TMA producer: per 128-k group 8 KB of packed weights and 2 x 16 KB of activations
//   warps 2..5, 11..14  dequantise (nibbles -> fp16 pairs with byte permutes, one subtract and
//                one multiply per pair) -> tcgen05.st
//   warps 1, 10  MMA issuers: each owns one fp32 accumulator (128 columns of tensor memory) and
//                half of every group's k-steps, so the order of additions into an accumulator is
//                fixed; the epilogue adds the two
//   warps 6..9   epilogue: tcgen05.ld, add, convert, store (consecutive lanes = consecutive n)
// Only plain TMA loads; every wait is bounded.
#include "common.cuh"
#include "ptx.cuh"
#include <cuda_fp16.h>

namespace mgx {

constexpr int PF_ROWS    = 128; // output columns (weight rows) per tile = UMMA M
constexpr int PF_TOKENS  = 128; // activation rows per tile = UMMA N
constexpr int PF_GROUP_K = 128;
constexpr int PF_STAGES  = 5;
constexpr int PF_W_BYTES = PF_ROWS * PF_GROUP_K / 2;      // 8192
constexpr int PF_A_ATOM  = PF_TOKENS * 128;               // 16384: 128 rows x 64 fp16
constexpr int PF_STAGE   = PF_W_BYTES + 2 * PF_A_ATOM;    // 40960
constexpr int PF_TSTAGES = 4;                             // A operand buffers in tensor memory
constexpr int PF_A_COL0  = 256;
constexpr int PF_A_COLS  = PF_GROUP_K / 2;                // 64 columns per group
constexpr int PF_SMEM    = PF_STAGES * PF_STAGE + 512 + 1024;
constexpr int PF_THREADS = 480;

struct pf_params
{
    const __half* scales;
    const uint8_t* zp; // may be null
    __half* D;
    int64_t M, N, K, ldd;
    int group, groups_per_row, zp_const;
    int tiles_m, num_tiles;
};

__global__ void __launch_bounds__(PF_THREADS, 1)
    w4a16_prefill_kernel(const __grid_constant__ CUtensorMap tmap_w,
                         const __grid_constant__ CUtensorMap tmap_a,
                         const pf_params p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem           = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint8_t* bar_base       = smem + PF_STAGES * PF_STAGE;
    uint64_t* full_bar      = reinterpret_cast<uint64_t*>(bar_base);
    uint64_t* empty_bar     = full_bar + PF_STAGES;  // weights read (256) + MMAs retired (2)
    uint64_t* unp_bar       = empty_bar + PF_STAGES; // A operand in tensor memory
    uint64_t* tfree_bar     = unp_bar + PF_TSTAGES;  // MMAs that read it retired (2)
    uint64_t* accf_bar      = tfree_bar + PF_TSTAGES;
    uint64_t* acce_bar      = accf_bar + 1;
    uint32_t* tmem_slot     = reinterpret_cast<uint32_t*>(acce_bar + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    grid_launch_dependents();
    if(threadIdx.x == 0)
    {
        for(int s = 0; s < PF_STAGES; ++s)
        {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 256 + 2);
        }
        for(int s = 0; s < PF_TSTAGES; ++s)
        {
            mbar_init(&unp_bar[s], 256);
            mbar_init(&tfree_bar[s], 2);
        }
        mbar_init(accf_bar, 2);
        mbar_init(acce_bar, 4);
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

    const int G      = static_cast<int>(p.K / PF_GROUP_K);
    const int rshift = 31 - __clz(p.group / PF_GROUP_K); // groups are powers of two
    const int issuer = warp == 1 ? 0 : (warp == 10 ? 1 : -1);

    if(warp == 0)
    {
        // ---------------------------------------------------- TMA producer
        if(lane == 0)
        {
            grid_dependency_wait(); // the activations are the previous kernel's output
            uint32_t it = 0;
            bool ok     = true;
            for(int t = blockIdx.x; ok and t < p.num_tiles; t += gridDim.x)
            {
                const int n0 = (t / p.tiles_m) * PF_ROWS;
                const int m0 = (t % p.tiles_m) * PF_TOKENS;
                for(int g = 0; g < G; ++g, ++it)
                {
                    const uint32_t s  = it % PF_STAGES;
                    const uint32_t ph = (it / PF_STAGES) & 1u;
                    if(not mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, 2))
                    {
                        ok = false;
                        break;
                    }
                    uint8_t* st = smem + s * PF_STAGE;
                    mbar_expect_tx(&full_bar[s], PF_STAGE);
                    tma_load_2d(st, &tmap_w, &full_bar[s], g * (PF_GROUP_K / 2), n0);
                    tma_load_2d(st + PF_W_BYTES, &tmap_a, &full_bar[s], g * PF_GROUP_K, m0);
                    tma_load_2d(st + PF_W_BYTES + PF_A_ATOM, &tmap_a, &full_bar[s],
                                g * PF_GROUP_K + 64, m0);
                }
            }
        }
    }
    else if(issuer >= 0)
    {
        // ---------------------------------------------------- MMA issuers
        if(lane == 0)
        {
            // D f32 += A f16 (weights, tensor memory) * B f16 (activation rows, K-major shared
            // memory); M = 128, N = 128, K = 16 per instruction
            constexpr uint32_t idesc = make_idesc(1u, 0u, 0u, PF_ROWS, PF_TOKENS);
            const uint32_t d_tmem    = tmem_base + issuer * PF_TOKENS;
            uint32_t it = 0, lt = 0;
            bool ok     = true;
            grid_dependency_wait(); // the bounded waits below must not count the previous kernel's time
            for(int t = blockIdx.x; ok and t < p.num_tiles; t += gridDim.x, ++lt)
            {
                if(not mbar_wait_bounded(acce_bar, (lt & 1u) ^ 1u, abort_flag, 4))
                    break;
                tc_fence_after_sync();
                for(int g = 0; g < G; ++g, ++it)
                {
                    const uint32_t s  = it % PF_STAGES;
                    const uint32_t ts = it % PF_TSTAGES;
                    const uint32_t tp = (it / PF_TSTAGES) & 1u;
                    // implies that the stage's TMA requests have landed
                    if(not mbar_wait_bounded(&unp_bar[ts], tp, abort_flag, 5))
                    {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t b_smem =
                        smem_u32(smem + s * PF_STAGE + PF_W_BYTES + issuer * PF_A_ATOM);
                    const uint64_t bdesc  = make_smem_desc_sw128(b_smem);
                    const uint32_t a_tmem = tmem_base + PF_A_COL0 + ts * PF_A_COLS + issuer * 32;
#pragma unroll
                    for(int k = 0; k < 4; ++k)
                        mma_f16_tmem_a(d_tmem, a_tmem + k * 8, bdesc + static_cast<uint64_t>((k * 32) >> 4),
                                       idesc, (g != 0 or k != 0) ? 1u : 0u);
                    tc_commit(&tfree_bar[ts]);
                    tc_commit(&empty_bar[s]);
                }
                if(ok)
                    tc_commit(accf_bar);
            }
        }
    }
    else if(warp < 6 or warp >= 11)
    {
        // ---------------------------------------------------- dequantise: nibbles -> fp16
        // Two threads per weight row (warps 2..5 take the first 64 k of a group, warps 11..14 the
        // second): 32 packed bytes (64-byte swizzle: a quarter warp's 16-byte reads fall in eight
        // different bank groups) -> 32 words of two fp16 each, in k order, to this row's lane of
        // tensor memory.
        const int row            = (warp & 3) * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const int sw             = (row >> 1) & 3;
        uint32_t it              = 0;
        bool ok                  = true;
        for(int t = blockIdx.x; ok and t < p.num_tiles; t += gridDim.x)
        {
            const int n  = min((t / p.tiles_m) * PF_ROWS + row, static_cast<int>(p.N) - 1);
            const unsigned short* srow =
                reinterpret_cast<const unsigned short*>(p.scales) + static_cast<int64_t>(n) * p.groups_per_row;
            const uint8_t* zrow = p.zp == nullptr ? nullptr : p.zp + static_cast<int64_t>(n) * p.groups_per_row;
            // scale and zero point of the next group are fetched one group ahead
            unsigned short s_next = __ldg(srow);
            int z_next            = zrow == nullptr ? p.zp_const : static_cast<int>(__ldg(zrow));
            for(int g = 0; g < G; ++g, ++it)
            {
                const uint32_t s  = it % PF_STAGES;
                const uint32_t ph = (it / PF_STAGES) & 1u;
                const uint32_t ts = it % PF_TSTAGES;
                const uint32_t tp = (it / PF_TSTAGES) & 1u;
                const unsigned short s_cur = s_next;
                const int z_cur            = z_next;
                if(g + 1 < G)
                {
                    const int gi = (g + 1) >> rshift;
                    s_next       = __ldg(srow + gi);
                    z_next       = zrow == nullptr ? p.zp_const : static_cast<int>(__ldg(zrow + gi));
                }
                // the tensor-memory stores below are warp-wide: leave only as a whole warp
                if(not __all_sync(0xffffffffu, mbar_wait_bounded(&full_bar[s], ph, abort_flag, 1)) or
                   not __all_sync(0xffffffffu, mbar_wait_bounded(&tfree_bar[ts], tp ^ 1u, abort_flag, 8)))
                {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                // (1024 + q) - (1024 + zp) is exact in fp16; one rounding in the multiply
                const uint32_t zz = 0x64006400u + static_cast<uint32_t>(z_cur) * 0x00010001u;
                const uint32_t ss = static_cast<uint32_t>(s_cur) * 0x00010001u;
                const __half2 zz2 = *reinterpret_cast<const __half2*>(&zz);
                const __half2 ss2 = *reinterpret_cast<const __half2*>(&ss);
                const uint8_t* pk = smem + s * PF_STAGE + row * 64;
                const int half = warp >= 11 ? 1 : 0;
                {
                    uint32_t u[32];
#pragma unroll
                    for(int c = 0; c < 2; ++c)
                    {
                        const uint4 w4 =
                            *reinterpret_cast<const uint4*>(pk + (((half * 2 + c) ^ sw) << 4));
                        const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                        for(int i = 0; i < 4; ++i)
                        {
                            const uint32_t lo = ww[i] & 0x0F0F0F0Fu;        // k 0 2 4 6
                            const uint32_t hi = (ww[i] >> 4) & 0x0F0F0F0Fu; // k 1 3 5 7
                            const uint32_t t01 = __byte_perm(lo, hi, 0x5140); // k 0 1 2 3
                            const uint32_t t23 = __byte_perm(lo, hi, 0x7362); // k 4 5 6 7
                            uint32_t h[4];
                            h[0] = __byte_perm(t01, 0x64646464u, 0x4140);
                            h[1] = __byte_perm(t01, 0x64646464u, 0x4342);
                            h[2] = __byte_perm(t23, 0x64646464u, 0x4140);
                            h[3] = __byte_perm(t23, 0x64646464u, 0x4342);
#pragma unroll
                            for(int j = 0; j < 4; ++j)
                            {
                                const __half2 x = __hmul2(
                                    __hsub2(*reinterpret_cast<const __half2*>(&h[j]), zz2), ss2);
                                u[(c * 4 + i) * 4 + j] = *reinterpret_cast<const uint32_t*>(&x);
                            }
                        }
                    }
                    tmem_st_32x32b_x32(tmem_base + lane_addr + PF_A_COL0 + ts * PF_A_COLS + half * 32, u);
                }
                mbar_arrive(&empty_bar[s]); // the packed block is in registers
                tmem_st_wait();
                tc_fence_before_sync();
                mbar_arrive(&unp_bar[ts]);
            }
        }
    }
    else
    {
        // ---------------------------------------------------- epilogue
        grid_dependency_wait(); // D may still be read by the previous kernel
        const int quarter = warp & 3;
        uint32_t lt       = 0;
        for(int t = blockIdx.x; t < p.num_tiles; t += gridDim.x, ++lt)
        {
            const int64_t n  = static_cast<int64_t>(t / p.tiles_m) * PF_ROWS + quarter * 32 + lane;
            const int64_t m0 = static_cast<int64_t>(t % p.tiles_m) * PF_TOKENS;
            if(not __all_sync(0xffffffffu, mbar_wait_bounded(accf_bar, lt & 1u, abort_flag, 3)))
                break;
            tc_fence_after_sync();
            const uint32_t tbase = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
            for(int c = 0; c < PF_TOKENS / 32; ++c)
            {
                uint32_t a0[32], a1[32];
                tmem_ld_32x32b_x32(tbase + c * 32, a0);
                tmem_ld_32x32b_x32(tbase + PF_TOKENS + c * 32, a1);
                tmem_ld_wait();
                if(n < p.N)
                {
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                    {
                        const int64_t m = m0 + c * 32 + j;
                        if(m < p.M)
                            p.D[m * p.ldd + n] =
                                __float2half_rn(__uint_as_float(a0[j]) + __uint_as_float(a1[j]));
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if(lane == 0)
                mbar_arrive(acce_bar);
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

int encode_rows(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t inner,
                uint64_t rows, uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows,
                CUtensorMapSwizzle swz)
{
    cuTensorMapEncodeTiled_t encode = get_tensor_map_encoder();
    if(encode == nullptr)
        return MGX_E_DRIVER;
    cuuint64_t dims[2]    = {inner, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2]     = {box_inner, box_rows};
    cuuint32_t estr[2]    = {1u, 1u};
    CUresult r = encode(map, type, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MGX_OK : MGX_E_INVALID_ARG;
}

} // namespace

bool w4a16_prefill_applicable(const mgx_w4_desc& d, const void* A, const void* Bp)
{
    const int64_t ratio = d.group / PF_GROUP_K;
    return d.M > 16 and d.K % PF_GROUP_K == 0 and d.group % PF_GROUP_K == 0 and
           (ratio & (ratio - 1)) == 0 and d.act == MGX_ACT_NONE and d.lda % 8 == 0 and
           ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(Bp)) & 15u) == 0 and
           ceil_div(d.N, PF_ROWS) * ceil_div(d.M, PF_TOKENS) < (int64_t{1} << 30) and
           d.N * (d.K / d.group) < (int64_t{1} << 40);
}

int w4a16_prefill_launch(const mgx_w4_desc& d, const void* A, const void* Bp, const void* scales,
                         const void* zp, void* D, cudaStream_t stream)
{
    CUtensorMap tw, ta;
    int rc = encode_rows(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, Bp, static_cast<uint64_t>(d.K / 2),
                         static_cast<uint64_t>(d.N), static_cast<uint64_t>(d.K / 2), PF_GROUP_K / 2,
                         PF_ROWS, CU_TENSOR_MAP_SWIZZLE_64B);
    if(rc != MGX_OK)
        return rc;
    rc = encode_rows(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT16, A, static_cast<uint64_t>(d.K),
                     static_cast<uint64_t>(d.M), static_cast<uint64_t>(d.lda) * 2, 64, PF_TOKENS,
                     CU_TENSOR_MAP_SWIZZLE_128B);
    if(rc != MGX_OK)
        return rc;
    pf_params p{};
    p.scales         = static_cast<const __half*>(scales);
    p.zp             = static_cast<const uint8_t*>(zp);
    p.D              = static_cast<__half*>(D);
    p.M              = d.M;
    p.N              = d.N;
    p.K              = d.K;
    p.ldd            = d.ldd;
    p.group          = d.group;
    p.groups_per_row = static_cast<int>(d.K / d.group);
    p.zp_const       = d.zp_const;
    p.tiles_m        = static_cast<int>(ceil_div(d.M, PF_TOKENS));
    p.num_tiles      = static_cast<int>(ceil_div(d.N, PF_ROWS)) * p.tiles_m;
    rc = ensure_smem_optin(reinterpret_cast<const void*>(w4a16_prefill_kernel), PF_SMEM);
    if(rc != MGX_OK)
        return rc;
    const int sms  = device_sm_count();
    const int grid = p.num_tiles < sms ? p.num_tiles : sms;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = dim3(static_cast<unsigned>(grid));
    cfg.blockDim         = dim3(PF_THREADS);
    cfg.dynamicSmemBytes = PF_SMEM;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs                                          = attr;
    cfg.numAttrs                                       = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, w4a16_prefill_kernel, tw, ta, p));
}

int w4a16_prefill_status(unsigned int* out) { return read_and_clear_status(out); }

} // namespace mgx
