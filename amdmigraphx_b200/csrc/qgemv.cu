// quant_dot for at most 16 rows of A (decode-sized batches) with the weights [N, K]
// K-contiguous: bound by the HBM stream of the weights, so the roles of the operands are
// swapped with respect to the tiled GEMM.  The WEIGHTS are the tcgen05 A operand (128 output
// columns per MMA, straight from the TMA-filled shared memory), the few activation rows are
// the B operand (N = 16), and the accumulator holds D transposed: TMEM lane = output column,
// TMEM column = row of A.  Work is the flat list of (128-column tile, 128-byte k-block) items,
// split evenly over one CTA per SM; tiles shared between CTAs are completed by the last warp
// to arrive, which adds the partial sums in slot order (int32: exact; fp32: fixed order).
// The epilogue is the tiled GEMM's arithmetic (dequantizelinear, bias, activation, fp32 / fp16 /
// raw int32 output; op::quant_dot + dequantizelinear.hpp:60-82 + the fused pointwise module).
//
// CTA = 192 threads: warp 0 TMA producer, warp 1 MMA issuer + tensor-memory owner, warps 2..5
// epilogue.  Only plain TMA loads; every wait is bounded.
#include "common.cuh"
#include "ptx.cuh"
#include "qgemm_math.cuh"
#include <cuda_fp16.h>
#include <type_traits>

namespace mgx {

constexpr int GV_ROWS    = 128; // output columns (weight rows) per tile = UMMA M
constexpr int GV_MB      = 16;  // padded rows of A = UMMA N
constexpr int GV_BK      = 128; // bytes of K per item
constexpr int GV_STAGES  = 10;
constexpr int GV_W_BYTES = GV_ROWS * GV_BK; // 16384
constexpr int GV_A_BYTES = GV_MB * GV_BK;   // 2048
constexpr int GV_STAGE   = GV_W_BYTES + GV_A_BYTES;
constexpr int GV_SMEM    = GV_STAGES * GV_STAGE + 256 + 1024;
constexpr int GV_THREADS = 192;

struct gv_params
{
    void* D;
    const float* scale;
    const float* bias;
    uint32_t* partial; // [slots][M][N] raw accumulators
    int* counters;     // [tiles][4], zeroed by the kernel launched before
    int64_t M, N, K, ldd;
    int scale_mode, act;
    int items_total, items_per_cta, kblocks;
};

__global__ void qgemv_zero_kernel(int* counters, int n)
{
    grid_launch_dependents();
    grid_dependency_wait(); // the previous kernel of the stream may still use the workspace
    for(int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        counters[i] = 0;
}

// walks a CTA's items tile by tile
struct gv_walk
{
    int tile, kb, left, KB;
    __device__ gv_walk(int f_lo, int f_hi, int kblocks)
        : tile(f_lo / kblocks), kb(f_lo - (f_lo / kblocks) * kblocks), left(f_hi - f_lo), KB(kblocks)
    {
    }
    // next segment: the items of one tile
    __device__ bool next(int& tile_out, int& kb0, int& count)
    {
        if(left <= 0)
            return false;
        tile_out = tile;
        kb0      = kb;
        count    = min(left, KB - kb);
        left -= count;
        kb = 0;
        ++tile;
        return true;
    }
};

template <bool IS_INT, class OutT>
__global__ void __launch_bounds__(GV_THREADS, 1)
    qgemv_kernel(const __grid_constant__ CUtensorMap tmap_w,
                 const __grid_constant__ CUtensorMap tmap_a,
                 const gv_params p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem           = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint8_t* bar_base       = smem + GV_STAGES * GV_STAGE;
    uint64_t* full_bar      = reinterpret_cast<uint64_t*>(bar_base);
    uint64_t* empty_bar     = full_bar + GV_STAGES;
    uint64_t* accf_bar      = empty_bar + GV_STAGES; // [2]
    uint64_t* acce_bar      = accf_bar + 2;          // [2]
    uint32_t* tmem_slot     = reinterpret_cast<uint32_t*>(acce_bar + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    grid_launch_dependents();
    if(threadIdx.x == 0)
    {
        for(int s = 0; s < GV_STAGES; ++s)
        {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for(int b = 0; b < 2; ++b)
        {
            mbar_init(&accf_bar[b], 1);
            mbar_init(&acce_bar[b], 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmap_w);
        prefetch_tensormap(&tmap_a);
    }
    if(warp == 1)
    {
        tmem_alloc(tmem_slot, 32);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int f_lo = min(p.items_total, static_cast<int>(blockIdx.x) * p.items_per_cta);
    const int f_hi = min(p.items_total, f_lo + p.items_per_cta);

    if(warp == 0)
    {
        // ---------------------------------------------------- TMA producer
        if(lane == 0)
        {
            grid_dependency_wait(); // A is the previous kernel's output
            int tile = f_lo / p.kblocks, kb = f_lo - tile * p.kblocks;
            for(int i = 0; i < f_hi - f_lo; ++i)
            {
                const uint32_t s  = i % GV_STAGES;
                const uint32_t ph = (i / GV_STAGES) & 1u;
                if(not mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, 2))
                    break;
                uint8_t* st = smem + s * GV_STAGE;
                // bytes past the end of K or N are zero-filled and still counted
                mbar_expect_tx(&full_bar[s], GV_STAGE);
                tma_load_2d(st, &tmap_w, &full_bar[s], kb * GV_BK, tile * GV_ROWS);
                tma_load_2d(st + GV_W_BYTES, &tmap_a, &full_bar[s], kb * GV_BK, 0);
                if(++kb == p.kblocks)
                {
                    kb = 0;
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
            // D (s32 | f32) += A (weights) * B (rows of A); M = 128, N = 16, K = 32 bytes
            constexpr uint32_t idesc = IS_INT ? make_idesc(2u, 1u, 1u, GV_ROWS, GV_MB)
                                              : make_idesc(1u, 0u, 0u, GV_ROWS, GV_MB);
            gv_walk walk(f_lo, f_hi, p.kblocks);
            int tile, kb0, count;
            bool ok = true;
            int i   = 0;
            grid_dependency_wait(); // the bounded waits below must not count the previous kernel's time
            for(uint32_t sc = 0; ok and walk.next(tile, kb0, count); ++sc)
            {
                const uint32_t buf = sc & 1u;
                if(not mbar_wait_bounded(&acce_bar[buf], ((sc >> 1) & 1u) ^ 1u, abort_flag, 4))
                    break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * GV_MB;
                for(int j = 0; j < count; ++j, ++i)
                {
                    const uint32_t s  = i % GV_STAGES;
                    const uint32_t ph = (i / GV_STAGES) & 1u;
                    if(not mbar_wait_bounded(&full_bar[s], ph, abort_flag, 1))
                    {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t st    = smem_u32(smem + s * GV_STAGE);
                    const uint64_t adesc = make_smem_desc_sw128(st);
                    const uint64_t bdesc = make_smem_desc_sw128(st + GV_W_BYTES);
#pragma unroll
                    for(int k = 0; k < 4; ++k)
                    {
                        const uint64_t koff = static_cast<uint64_t>((k * 32) >> 4);
                        if constexpr(IS_INT)
                            mma_i8(d_tmem, adesc + koff, bdesc + koff, idesc, (j != 0 or k != 0) ? 1u : 0u);
                        else
                            mma_f8(d_tmem, adesc + koff, bdesc + koff, idesc, (j != 0 or k != 0) ? 1u : 0u);
                    }
                    tc_commit(&empty_bar[s]);
                }
                if(ok)
                    tc_commit(&accf_bar[buf]);
            }
        }
    }
    else
    {
        // ---------------------------------------------------- epilogue
        grid_dependency_wait(); // counters zeroed, D free to overwrite
        const int quarter = warp & 3;
        const float tensor_scale = p.scale_mode == MGX_SCALE_PER_TENSOR ? __ldg(p.scale) : 1.0f;
        // raw accumulator -> output value, as in the tiled GEMM's epilogue
        auto finish = [&](uint32_t raw, float s, float b) {
            float x;
            if constexpr(IS_INT)
            {
                const int32_t a = static_cast<int32_t>(raw);
                x = p.scale_mode == MGX_SCALE_NONE ? (fits_small(a) ? int_to_float_small(a) : __int2float_rn(a))
                                                   : dequant_i32(a, s);
            }
            else
            {
                x = __uint_as_float(raw);
                if(p.scale_mode != MGX_SCALE_NONE)
                    x = __fmul_rn(x, s);
            }
            if(p.bias != nullptr)
                x = __fadd_rn(x, b);
            switch(p.act)
            {
            case MGX_ACT_RELU: return apply_act<MGX_ACT_RELU>(x);
            case MGX_ACT_GELU_ERF: return apply_act<MGX_ACT_GELU_ERF>(x);
            case MGX_ACT_GELU_TANH: return apply_act<MGX_ACT_GELU_TANH>(x);
            case MGX_ACT_SILU: return apply_act<MGX_ACT_SILU>(x);
            default: return x;
            }
        };
        auto store = [&](int64_t m, int64_t n, uint32_t raw, float s, float b) {
            if constexpr(std::is_same<OutT, int32_t>::value)
                static_cast<int32_t*>(p.D)[m * p.ldd + n] = static_cast<int32_t>(raw);
            else if constexpr(std::is_same<OutT, float>::value)
                static_cast<float*>(p.D)[m * p.ldd + n] = finish(raw, s, b);
            else
                static_cast<__half*>(p.D)[m * p.ldd + n] = __float2half_rz(finish(raw, s, b));
        };
        gv_walk walk(f_lo, f_hi, p.kblocks);
        int tile, kb0, count;
        for(uint32_t sc = 0; walk.next(tile, kb0, count); ++sc)
        {
            const uint32_t buf = sc & 1u;
            const int64_t n    = static_cast<int64_t>(tile) * GV_ROWS + quarter * 32 + lane;
            const bool n_ok    = n < p.N;
            float s = tensor_scale, b = 0.0f;
            if(n_ok)
            {
                if(p.scale_mode == MGX_SCALE_PER_COL)
                    s = __ldg(p.scale + n);
                if(p.bias != nullptr)
                    b = __ldg(p.bias + n);
            }
            if(not __all_sync(0xffffffffu, mbar_wait_bounded(&accf_bar[buf], (sc >> 1) & 1u, abort_flag, 3)))
                break;
            tc_fence_after_sync();
            uint32_t acc[GV_MB];
            tmem_ld_32x32b_x16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * GV_MB, acc);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if(lane == 0)
                mbar_arrive(&acce_bar[buf]);
            const bool whole = kb0 == 0 and count == p.kblocks;
            if(whole)
            {
                if(n_ok)
                {
#pragma unroll
                    for(int m = 0; m < GV_MB; ++m)
                        if(m < p.M)
                            store(m, n, acc[m], s, b);
                }
                continue;
            }
            const int first = (tile * p.kblocks) / p.items_per_cta;
            const int last  = ((tile + 1) * p.kblocks - 1) / p.items_per_cta;
            const int slot  = static_cast<int>(blockIdx.x) - first;
            if(n_ok)
            {
#pragma unroll
                for(int m = 0; m < GV_MB; ++m)
                    if(m < p.M)
                        p.partial[(static_cast<int64_t>(slot) * p.M + m) * p.N + n] = acc[m];
            }
            // the counting atomic releases this warp's stores (ordered before it by the warp
            // barrier) and acquires those of the warps that counted themselves in before
            __syncwarp();
            int old = 0;
            if(lane == 0)
                asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;"
                             : "=r"(old)
                             : "l"(p.counters + tile * 4 + quarter)
                             : "memory");
            old = __shfl_sync(0xffffffffu, old, 0);
            if(old == last - first and n_ok)
            {
                uint32_t tot[GV_MB];
#pragma unroll
                for(int m = 0; m < GV_MB; ++m)
                    tot[m] = IS_INT ? 0u : __float_as_uint(0.0f);
#pragma unroll 2
                for(int sl = 0; sl <= last - first; ++sl)
                {
                    uint32_t t[GV_MB];
#pragma unroll
                    for(int m = 0; m < GV_MB; ++m)
                        t[m] = m < p.M ? __ldcg(p.partial + (static_cast<int64_t>(sl) * p.M + m) * p.N + n) : 0u;
#pragma unroll
                    for(int m = 0; m < GV_MB; ++m)
                    {
                        if constexpr(IS_INT)
                            tot[m] += t[m];
                        else
                            tot[m] = __float_as_uint(__uint_as_float(tot[m]) + __uint_as_float(t[m]));
                    }
                }
#pragma unroll
                for(int m = 0; m < GV_MB; ++m)
                    if(m < p.M)
                        store(m, n, tot[m], s, b);
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
        tmem_dealloc(tmem_base, 32);
    }
}

// ------------------------------------------------------------------ host
namespace {

struct gv_plan
{
    int tiles, kblocks, items_total, items_per_cta, grid, slots;
    size_t off_partial, total;
};

gv_plan make_gv_plan(const mgx_qgemm_desc& d)
{
    gv_plan pl{};
    pl.tiles         = static_cast<int>(ceil_div(d.N, GV_ROWS));
    pl.kblocks       = static_cast<int>(ceil_div(d.K, GV_BK));
    pl.items_total   = pl.tiles * pl.kblocks;
    pl.items_per_cta = static_cast<int>(ceil_div(pl.items_total, device_sm_count()));
    pl.grid          = static_cast<int>(ceil_div(pl.items_total, pl.items_per_cta));
    pl.slots         = (pl.kblocks - 1) / pl.items_per_cta + 2;
    pl.off_partial   = (static_cast<size_t>(pl.tiles) * 4 * sizeof(int) + 255) / 256 * 256;
    pl.total         = pl.off_partial + static_cast<size_t>(pl.slots) * d.M * d.N * 4;
    return pl;
}

int encode_k_major(CUtensorMap* map, const void* base, uint64_t k, uint64_t rows, uint64_t pitch,
                   uint32_t box_rows)
{
    cuTensorMapEncodeTiled_t encode = get_tensor_map_encoder();
    if(encode == nullptr)
        return MGX_E_DRIVER;
    cuuint64_t dims[2]    = {k, rows};
    cuuint64_t strides[1] = {pitch};
    cuuint32_t box[2]     = {GV_BK, box_rows};
    cuuint32_t estr[2]    = {1u, 1u};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MGX_OK : MGX_E_INVALID_ARG;
}

template <bool IS_INT, class OutT>
int launch_gv(int grid, const CUtensorMap& tw, const CUtensorMap& ta, const gv_params& p, cudaStream_t stream)
{
    auto kernel = qgemv_kernel<IS_INT, OutT>;
    int rc      = ensure_smem_optin(reinterpret_cast<const void*>(kernel), GV_SMEM);
    if(rc != MGX_OK)
        return rc;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = dim3(static_cast<unsigned>(grid));
    cfg.blockDim         = dim3(GV_THREADS);
    cfg.dynamicSmemBytes = GV_SMEM;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs                                          = attr;
    cfg.numAttrs                                       = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, tw, ta, p));
}

} // namespace

// the skinny-M kernel covers: one batch, at most 16 rows of A, weights [N, K] K-contiguous, no
// residual, no fused quantizelinear output, no per-row scale
bool qgemv_applicable(const mgx_qgemm_desc& d, bool has_residual, bool has_qout)
{
    return d.M <= GV_MB and d.batch == 1 and d.b_layout == MGX_B_NK and not has_residual and
           not has_qout and d.scale_mode != MGX_SCALE_PER_ROW and
           ceil_div(d.N, GV_ROWS) * ceil_div(d.K, GV_BK) < (int64_t{1} << 30);
}

size_t qgemv_workspace(const mgx_qgemm_desc& d) { return make_gv_plan(d).total + 256; }

int qgemv_launch(const mgx_qgemm_desc& d, const void* A, const void* B, void* D, const float* scale,
                 const float* bias, int64_t ldb, void* workspace, size_t workspace_bytes,
                 cudaStream_t stream)
{
    const gv_plan pl = make_gv_plan(d);
    auto addr          = reinterpret_cast<uintptr_t>(workspace);
    const size_t shift = (256 - (addr & 255u)) & 255u;
    if(workspace == nullptr or workspace_bytes < shift + pl.total)
        return MGX_E_WORKSPACE;
    auto* ws = static_cast<uint8_t*>(workspace) + shift;
    CUtensorMap tw, ta;
    int rc = encode_k_major(&tw, B, static_cast<uint64_t>(d.K), static_cast<uint64_t>(d.N),
                            static_cast<uint64_t>(ldb), GV_ROWS);
    if(rc != MGX_OK)
        return rc;
    rc = encode_k_major(&ta, A, static_cast<uint64_t>(d.K), static_cast<uint64_t>(d.M),
                        static_cast<uint64_t>(d.lda), GV_MB);
    if(rc != MGX_OK)
        return rc;
    gv_params p{};
    p.D             = D;
    p.scale         = scale;
    p.bias          = bias;
    p.counters      = reinterpret_cast<int*>(ws);
    p.partial       = reinterpret_cast<uint32_t*>(ws + pl.off_partial);
    p.M             = d.M;
    p.N             = d.N;
    p.K             = d.K;
    p.ldd           = d.ldd;
    p.scale_mode    = d.scale_mode;
    p.act           = d.act;
    p.items_total   = pl.items_total;
    p.items_per_cta = pl.items_per_cta;
    p.kblocks       = pl.kblocks;
    {
        // zero the tile counters; chained so that the main kernel starts (and streams weights)
        // while this one runs
        cudaLaunchConfig_t cfg{};
        const int n          = pl.tiles * 4;
        cfg.gridDim          = dim3(static_cast<unsigned>(ceil_div(n, 256) < 64 ? ceil_div(n, 256) : 64));
        cfg.blockDim         = dim3(256);
        cfg.dynamicSmemBytes = 0;
        cfg.stream           = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs    = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, qgemv_zero_kernel, p.counters, n);
        if(e != cudaSuccess)
            return static_cast<int>(e);
    }
    const bool is_int = d.ab_type == MGX_I8;
    if(d.out_type == MGX_I32)
        return launch_gv<true, int32_t>(pl.grid, tw, ta, p, stream);
    if(d.out_type == MGX_F16)
        return is_int ? launch_gv<true, __half>(pl.grid, tw, ta, p, stream)
                      : launch_gv<false, __half>(pl.grid, tw, ta, p, stream);
    return is_int ? launch_gv<true, float>(pl.grid, tw, ta, p, stream)
                  : launch_gv<false, float>(pl.grid, tw, ta, p, stream);
}

int qgemv_status(unsigned int* out) { return read_and_clear_status(out); }

} // namespace mgx
