// Reductions over the innermost axis and softmax: one thread block per row, 16-byte loads where
// the row allows, warp shuffles + one shared-memory step.  HBM-bound: x is read once by the
// reductions, and once by softmax when a row fits the block's registers (cols <= 8192), twice
// otherwise.
#include "common.cuh"
#include "qgemm_math.cuh"
#include <cuda_fp16.h>
#include <cfloat>

namespace mgx {

template <class T>
__device__ __forceinline__ float rd_load(const T* p, int64_t i)
{
    if constexpr(std::is_same<T, float>::value)
        return p[i];
    else
        return __half2float(p[i]);
}

template <class T>
__device__ __forceinline__ void rd_store(T* p, int64_t i, float v)
{
    if constexpr(std::is_same<T, float>::value)
        p[i] = v;
    else
        p[i] = __float2half_rz(v); // migraphx::half truncates
}

template <class T>
__device__ __forceinline__ float rd_round(float v)
{
    if constexpr(std::is_same<T, float>::value)
        return v;
    else
        return truncate_to_half_precision(v);
}

template <int OP>
__device__ __forceinline__ float rd_combine(float a, float b)
{
    if constexpr(OP == MGX_REDUCE_MAX)
        return fmaxf(a, b);
    else if constexpr(OP == MGX_REDUCE_MIN)
        return fminf(a, b);
    else
        return a + b;
}

template <int OP>
__device__ __forceinline__ float rd_identity()
{
    if constexpr(OP == MGX_REDUCE_MAX)
        return -FLT_MAX;
    else if constexpr(OP == MGX_REDUCE_MIN)
        return FLT_MAX;
    else
        return 0.0f;
}

// block-wide reduction; every thread gets the result
template <int OP>
__device__ __forceinline__ float block_reduce(float v, float* scratch)
{
#pragma unroll
    for(int o = 16; o > 0; o >>= 1)
        v = rd_combine<OP>(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads(); // scratch may still be read from a previous call
    if(lane == 0)
        scratch[warp] = v;
    __syncthreads();
    v = lane < nw ? scratch[lane] : rd_identity<OP>();
#pragma unroll
    for(int o = 16; o > 0; o >>= 1)
        v = rd_combine<OP>(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

template <class T, int OP>
__global__ void __launch_bounds__(256) reduce_rows_kernel(const T* __restrict__ x, int64_t ldx, int64_t rows,
                                                          int64_t cols, T* __restrict__ y)
{
    __shared__ float scratch[32];
    constexpr int BOP = OP == MGX_REDUCE_MEAN ? MGX_REDUCE_SUM : OP;
    for(int64_t r = blockIdx.x; r < rows; r += gridDim.x)
    {
        const T* row = x + r * ldx;
        float acc    = rd_identity<BOP>();
        for(int64_t c = threadIdx.x; c < cols; c += blockDim.x)
            acc = rd_combine<BOP>(acc, rd_load(row, c));
        acc = block_reduce<BOP>(acc, scratch);
        if(threadIdx.x == 0)
        {
            if constexpr(OP == MGX_REDUCE_MEAN)
                acc = acc / static_cast<float>(cols);
            rd_store(y, r, acc);
        }
    }
}

// PER: elements a thread keeps in registers (row length up to 256 * PER), 0: re-read the row
template <class T, int PER>
__global__ void __launch_bounds__(256) softmax_rows_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ y,
                                                           int64_t ldy, int64_t rows, int64_t cols)
{
    __shared__ float scratch[32];
    for(int64_t r = blockIdx.x; r < rows; r += gridDim.x)
    {
        const T* row = x + r * ldx;
        T* out       = y + r * ldy;
        float v[PER > 0 ? PER : 1];
        float mx = -FLT_MAX;
        if constexpr(PER > 0)
        {
#pragma unroll
            for(int i = 0; i < PER; ++i)
            {
                const int64_t c = threadIdx.x + static_cast<int64_t>(i) * 256;
                v[i]            = c < cols ? rd_load(row, c) : -FLT_MAX;
                mx              = fmaxf(mx, v[i]);
            }
        }
        else
        {
            for(int64_t c = threadIdx.x; c < cols; c += 256)
                mx = fmaxf(mx, rd_load(row, c));
        }
        mx = block_reduce<MGX_REDUCE_MAX>(mx, scratch);
        // exponentials take the output type before they are summed (as the reference stores them)
        float sum = 0.0f;
        if constexpr(PER > 0)
        {
#pragma unroll
            for(int i = 0; i < PER; ++i)
            {
                const int64_t c = threadIdx.x + static_cast<int64_t>(i) * 256;
                v[i]            = c < cols ? rd_round<T>(expf(v[i] - mx)) : 0.0f;
                sum += v[i];
            }
        }
        else
        {
            for(int64_t c = threadIdx.x; c < cols; c += 256)
                sum += rd_round<T>(expf(rd_load(row, c) - mx));
        }
        sum = block_reduce<MGX_REDUCE_SUM>(sum, scratch);
        if constexpr(PER > 0)
        {
#pragma unroll
            for(int i = 0; i < PER; ++i)
            {
                const int64_t c = threadIdx.x + static_cast<int64_t>(i) * 256;
                if(c < cols)
                    rd_store(out, c, v[i] / sum);
            }
        }
        else
        {
            for(int64_t c = threadIdx.x; c < cols; c += 256)
                rd_store(out, c, rd_round<T>(expf(rd_load(row, c) - mx)) / sum);
        }
    }
}

// exp(t) for t <= 0 as one multiply and one ex2.approx (relative error about 2e-7 + 6e-8 |t|;
// results below 2^-126 flush to zero)
__device__ __forceinline__ float fast_exp(float t)
{
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t * 1.4426950408889634f));
    return e;
}

// a / b from a reciprocal of b and one Newton step on the quotient: the correctly rounded
// quotient except in rare last-place cases
__device__ __forceinline__ float fast_div(float a, float b, float rcp)
{
    const float q = a * rcp;
    return fmaf(fmaf(-b, q, a), rcp, q);
}

// ---- vector variants: rows whose base and length allow 16-byte accesses -------------------
template <class T>
struct vec_of;
template <>
struct vec_of<float>
{
    static constexpr int n = 4;
    __device__ static void load(const float* p, float (&v)[4])
    {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
    }
    __device__ static void store(float* p, const float (&v)[4])
    {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <>
struct vec_of<__half>
{
    static constexpr int n = 8;
    __device__ static void load(const __half* p, float (&v)[8])
    {
        const uint4 t     = *reinterpret_cast<const uint4*>(p);
        const __half2* h2 = reinterpret_cast<const __half2*>(&t);
#pragma unroll
        for(int i = 0; i < 4; ++i)
        {
            const float2 f = __half22float2(h2[i]);
            v[2 * i]       = f.x;
            v[2 * i + 1]   = f.y;
        }
    }
    __device__ static void store(__half* p, const float (&v)[8])
    {
        uint4 t;
        __half2* h2 = reinterpret_cast<__half2*>(&t);
#pragma unroll
        for(int i = 0; i < 4; ++i)
            h2[i] = __halves2half2(__float2half_rz(v[2 * i]), __float2half_rz(v[2 * i + 1]));
        *reinterpret_cast<uint4*>(p) = t;
    }
};

// reduction over WPR warps of a block of 8 (WPR = 1: shuffles only; WPR = 8: one shared-memory step)
template <int OP, int WPR>
__device__ __forceinline__ float group_reduce(float v, float* scratch)
{
#pragma unroll
    for(int o = 16; o > 0; o >>= 1)
        v = rd_combine<OP>(v, __shfl_xor_sync(0xffffffffu, v, o));
    if constexpr(WPR > 1)
    {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        __syncthreads();
        if(lane == 0)
            scratch[warp] = v;
        __syncthreads();
        v = scratch[lane & (WPR - 1)];
#pragma unroll
        for(int o = WPR / 2; o > 0; o >>= 1)
            v = rd_combine<OP>(v, __shfl_xor_sync(0xffffffffu, v, o));
    }
    return v;
}

// WPR warps per row (1: eight rows per block, 8: one row per block)
template <class T, int OP, int WPR>
__global__ void __launch_bounds__(256) reduce_rows_vec_kernel(const T* __restrict__ x, int64_t ldx, int64_t rows,
                                                              int64_t cols, T* __restrict__ y)
{
    __shared__ float scratch[8];
    constexpr int BOP = OP == MGX_REDUCE_MEAN ? MGX_REDUCE_SUM : OP;
    constexpr int N   = vec_of<T>::n;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rpb  = 8 / WPR;                              // rows per block
    const int sub  = WPR == 1 ? lane : threadIdx.x;        // position within the row's threads
    const int64_t nv = cols / N;
    // every block runs the same number of trips (the shared-memory step has barriers)
    for(int64_t r0 = static_cast<int64_t>(blockIdx.x) * rpb; r0 < rows; r0 += static_cast<int64_t>(gridDim.x) * rpb)
    {
        const int64_t r = r0 + (WPR == 1 ? warp : 0);
        float acc[4]    = {rd_identity<BOP>(), rd_identity<BOP>(), rd_identity<BOP>(), rd_identity<BOP>()};
        if(r < rows)
        {
            const T* row = x + r * ldx;
            for(int64_t c = sub; c < nv; c += 32 * WPR)
            {
                float v[N];
                vec_of<T>::load(row + c * N, v);
#pragma unroll
                for(int i = 0; i < N; ++i)
                    acc[i & 3] = rd_combine<BOP>(acc[i & 3], v[i]);
            }
        }
        float a = rd_combine<BOP>(rd_combine<BOP>(acc[0], acc[1]), rd_combine<BOP>(acc[2], acc[3]));
        a       = group_reduce<BOP, WPR>(a, scratch);
        if(r < rows and sub == 0)
        {
            if constexpr(OP == MGX_REDUCE_MEAN)
                a = a / static_cast<float>(cols);
            rd_store(y, r, a);
        }
    }
}

// The row stays in registers: VPL vectors per thread, WPR warps per row.
template <class T, int VPL, int WPR>
__global__ void __launch_bounds__(256) softmax_rows_vec_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ y,
                                                               int64_t ldy, int64_t rows, int64_t cols)
{
    __shared__ float scratch[8];
    constexpr int N = vec_of<T>::n;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rpb  = 8 / WPR;
    const int sub  = WPR == 1 ? lane : threadIdx.x;
    const int64_t nv = cols / N;
    for(int64_t r0 = static_cast<int64_t>(blockIdx.x) * rpb; r0 < rows; r0 += static_cast<int64_t>(gridDim.x) * rpb)
    {
        const int64_t r  = r0 + (WPR == 1 ? warp : 0);
        const bool live  = r < rows;
        const T* row     = x + (live ? r : 0) * ldx;
        float v[VPL][N];
        float mx = -FLT_MAX;
#pragma unroll
        for(int k = 0; k < VPL; ++k)
        {
            const int64_t c = sub + static_cast<int64_t>(k) * 32 * WPR;
            if(live and c < nv)
                vec_of<T>::load(row + c * N, v[k]);
            else
            {
#pragma unroll
                for(int i = 0; i < N; ++i)
                    v[k][i] = -FLT_MAX;
            }
#pragma unroll
            for(int i = 0; i < N; ++i)
                mx = fmaxf(mx, v[k][i]);
        }
        mx        = group_reduce<MGX_REDUCE_MAX, WPR>(mx, scratch);
        float sum = 0.0f;
#pragma unroll
        for(int k = 0; k < VPL; ++k)
        {
            const bool in = sub + static_cast<int64_t>(k) * 32 * WPR < nv;
#pragma unroll
            for(int i = 0; i < N; ++i)
            {
                // exponentials take the output type before they are summed
                v[k][i] = in ? rd_round<T>(fast_exp(v[k][i] - mx)) : 0.0f;
                sum += v[k][i];
            }
        }
        sum = group_reduce<MGX_REDUCE_SUM, WPR>(sum, scratch);
        const float rcp = __frcp_rn(sum);
        if(live)
        {
            T* out = y + r * ldy;
#pragma unroll
            for(int k = 0; k < VPL; ++k)
            {
                const int64_t c = sub + static_cast<int64_t>(k) * 32 * WPR;
                if(c < nv)
                {
#pragma unroll
                    for(int i = 0; i < N; ++i)
                        v[k][i] = fast_div(v[k][i], sum, rcp);
                    vec_of<T>::store(out + c * N, v[k]);
                }
            }
        }
    }
}

// blocks of 256 threads that are resident at once on the whole device, at most `blocks`
template <class K>
static int resident_grid(K kernel, int64_t blocks)
{
    int n = 0;
    if(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, 256, 0) != cudaSuccess or n < 1)
        n = 4;
    const int64_t cap = static_cast<int64_t>(device_sm_count()) * n;
    return static_cast<int>(blocks < cap ? blocks : cap);
}

template <class T>
static bool rows_vectorisable(const void* p, int64_t ld, int64_t cols)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0 and (ld * sizeof(T)) % 16 == 0 and cols % vec_of<T>::n == 0;
}

template <class T>
int launch_reduce(const void* x, int64_t ldx, int64_t rows, int64_t cols, int op, void* y, cudaStream_t s)
{
    const int grid = static_cast<int>(rows < 148 * 8 ? rows : 148 * 8);
    const T* xp    = static_cast<const T*>(x);
    T* yp          = static_cast<T*>(y);
    if(rows_vectorisable<T>(x, ldx, cols) and op >= MGX_REDUCE_SUM and op <= MGX_REDUCE_MIN)
    {
        // short rows: a warp each; long rows: a block each
        const bool wide      = cols * static_cast<int64_t>(sizeof(T)) >= 8192;
        const int64_t blocks = wide ? rows : ceil_div(rows, int64_t{8});
        const int g          = static_cast<int>(blocks < 148 * 8 ? blocks : 148 * 8);
#define MGX_RED(OP)                                                                           \
    if(wide)                                                                                  \
        reduce_rows_vec_kernel<T, OP, 8><<<g, 256, 0, s>>>(xp, ldx, rows, cols, yp);          \
    else                                                                                      \
        reduce_rows_vec_kernel<T, OP, 1><<<g, 256, 0, s>>>(xp, ldx, rows, cols, yp)
        switch(op)
        {
        case MGX_REDUCE_SUM: MGX_RED(MGX_REDUCE_SUM); break;
        case MGX_REDUCE_MEAN: MGX_RED(MGX_REDUCE_MEAN); break;
        case MGX_REDUCE_MAX: MGX_RED(MGX_REDUCE_MAX); break;
        default: MGX_RED(MGX_REDUCE_MIN); break;
        }
#undef MGX_RED
        return static_cast<int>(cudaGetLastError());
    }
    switch(op)
    {
    case MGX_REDUCE_SUM: reduce_rows_kernel<T, MGX_REDUCE_SUM><<<grid, 256, 0, s>>>(xp, ldx, rows, cols, yp); break;
    case MGX_REDUCE_MEAN: reduce_rows_kernel<T, MGX_REDUCE_MEAN><<<grid, 256, 0, s>>>(xp, ldx, rows, cols, yp); break;
    case MGX_REDUCE_MAX: reduce_rows_kernel<T, MGX_REDUCE_MAX><<<grid, 256, 0, s>>>(xp, ldx, rows, cols, yp); break;
    case MGX_REDUCE_MIN: reduce_rows_kernel<T, MGX_REDUCE_MIN><<<grid, 256, 0, s>>>(xp, ldx, rows, cols, yp); break;
    default: return MGX_E_INVALID_ARG;
    }
    return static_cast<int>(cudaGetLastError());
}

template <class T>
int launch_softmax(const void* x, int64_t ldx, void* y, int64_t ldy, int64_t rows, int64_t cols, cudaStream_t s)
{
    const int grid = static_cast<int>(rows < 148 * 8 ? rows : 148 * 8);
    const T* xp    = static_cast<const T*>(x);
    T* yp          = static_cast<T*>(y);
    if(rows_vectorisable<T>(x, ldx, cols) and rows_vectorisable<T>(y, ldy, cols))
    {
        constexpr int N  = vec_of<T>::n;
        const int64_t nv = cols / N;
        bool done        = true;
        // grid = one wave of resident blocks (the kernels loop over rows)
#define MGX_SOFTMAX(VPL, WPR)                                                                             \
    {                                                                                                     \
        auto k = softmax_rows_vec_kernel<T, VPL, WPR>;                                                    \
        k<<<resident_grid(k, ceil_div(rows, int64_t{8 / WPR})), 256, 0, s>>>(xp, ldx, yp, ldy, rows, cols); \
    }
        if(nv <= 32)
            MGX_SOFTMAX(1, 1)
        else if(nv <= 64)
            MGX_SOFTMAX(2, 1)
        else if(nv <= 128)
            MGX_SOFTMAX(4, 1)
        else if(nv <= 256)
            MGX_SOFTMAX(1, 8)
        else if(nv <= 512)
            MGX_SOFTMAX(2, 8)
        else if(nv <= 1024)
            MGX_SOFTMAX(4, 8)
        else
            done = false;
#undef MGX_SOFTMAX
        if(done)
            return static_cast<int>(cudaGetLastError());
    }
    if(cols <= 256 * 4)
        softmax_rows_kernel<T, 4><<<grid, 256, 0, s>>>(xp, ldx, yp, ldy, rows, cols);
    else if(cols <= 256 * 16)
        softmax_rows_kernel<T, 16><<<grid, 256, 0, s>>>(xp, ldx, yp, ldy, rows, cols);
    else if(cols <= 256 * 32)
        softmax_rows_kernel<T, 32><<<grid, 256, 0, s>>>(xp, ldx, yp, ldy, rows, cols);
    else
        softmax_rows_kernel<T, 0><<<grid, 256, 0, s>>>(xp, ldx, yp, ldy, rows, cols);
    return static_cast<int>(cudaGetLastError());
}

} // namespace mgx

using namespace mgx;

extern "C" int mgx_cuda_reduce(const void* x, int type, int64_t ldx, int64_t rows, int64_t cols, int op,
                               void* y, void* stream)
{
    if(rows < 0 or cols <= 0 or ldx < cols)
        return MGX_E_INVALID_ARG;
    if(rows == 0)
        return MGX_OK;
    if(x == nullptr or y == nullptr)
        return MGX_E_INVALID_ARG;
    if(type == MGX_F32)
        return launch_reduce<float>(x, ldx, rows, cols, op, y, static_cast<cudaStream_t>(stream));
    if(type == MGX_F16)
        return launch_reduce<__half>(x, ldx, rows, cols, op, y, static_cast<cudaStream_t>(stream));
    return MGX_E_UNSUPPORTED;
}

extern "C" int mgx_cuda_softmax(const void* x, int type, int64_t ldx, void* y, int64_t ldy, int64_t rows,
                                int64_t cols, void* stream)
{
    if(rows < 0 or cols <= 0 or ldx < cols or ldy < cols)
        return MGX_E_INVALID_ARG;
    if(rows == 0)
        return MGX_OK;
    if(x == nullptr or y == nullptr)
        return MGX_E_INVALID_ARG;
    if(type == MGX_F32)
        return launch_softmax<float>(x, ldx, y, ldy, rows, cols, static_cast<cudaStream_t>(stream));
    if(type == MGX_F16)
        return launch_softmax<__half>(x, ldx, y, ldy, rows, cols, static_cast<cudaStream_t>(stream));
    return MGX_E_UNSUPPORTED;
}
