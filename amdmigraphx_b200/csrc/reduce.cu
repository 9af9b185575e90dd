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

template <class T>
int launch_reduce(const void* x, int64_t ldx, int64_t rows, int64_t cols, int op, void* y, cudaStream_t s)
{
    const int grid = static_cast<int>(rows < 148 * 8 ? rows : 148 * 8);
    const T* xp    = static_cast<const T*>(x);
    T* yp          = static_cast<T*>(y);
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
