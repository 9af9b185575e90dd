// gather along one axis and strided row copies (concat): byte movers, HBM-bound.  Elements are
// moved in the widest unit (16, 8, 4, 2 or 1 bytes) that the row length and the pointers allow.
#include "common.cuh"

namespace mgx {

template <int U>
struct unit_type;
template <>
struct unit_type<16>
{
    using type = uint4;
};
template <>
struct unit_type<8>
{
    using type = uint2;
};
template <>
struct unit_type<4>
{
    using type = uint32_t;
};
template <>
struct unit_type<2>
{
    using type = uint16_t;
};
template <>
struct unit_type<1>
{
    using type = uint8_t;
};

// out[o, j, :] = data[o, idx[j], :] over rows of `per` units; an index outside
// [-axis_len, axis_len) yields zeros (the reference throws on the host)
template <int U, class IdxT>
__global__ void __launch_bounds__(256)
    gather_kernel(const uint8_t* __restrict__ data, const IdxT* __restrict__ idx, uint8_t* __restrict__ out,
                  int64_t total, int64_t axis_len, int64_t per, int64_t nidx)
{
    using T = typename unit_type<U>::type;
    const T* src = reinterpret_cast<const T*>(data);
    T* dst       = reinterpret_cast<T*>(out);
    for(int64_t t = blockIdx.x * int64_t{256} + threadIdx.x; t < total; t += gridDim.x * int64_t{256})
    {
        const int64_t u  = t % per;
        const int64_t oj = t / per;
        const int64_t j  = oj % nidx;
        const int64_t o  = oj / nidx;
        int64_t k        = static_cast<int64_t>(__ldg(idx + j));
        k                = k < 0 ? k + axis_len : k;
        T v{};
        if(k >= 0 and k < axis_len)
            v = src[(o * axis_len + k) * per + u];
        dst[t] = v;
    }
}

template <int U>
__global__ void __launch_bounds__(256)
    copy_rows_kernel(const uint8_t* __restrict__ src, int64_t src_pitch, uint8_t* __restrict__ dst,
                     int64_t dst_pitch, int64_t total, int64_t per)
{
    using T = typename unit_type<U>::type;
    for(int64_t t = blockIdx.x * int64_t{256} + threadIdx.x; t < total; t += gridDim.x * int64_t{256})
    {
        const int64_t u = t % per;
        const int64_t r = t / per;
        *reinterpret_cast<T*>(dst + r * dst_pitch + u * U) =
            *reinterpret_cast<const T*>(src + r * src_pitch + u * U);
    }
}

static int widest_unit(uintptr_t bits)
{
    for(int u : {16, 8, 4, 2})
        if(bits % static_cast<uintptr_t>(u) == 0)
            return u;
    return 1;
}

static unsigned grid_for(int64_t total)
{
    const int64_t blocks = ceil_div(total, int64_t{256});
    const int64_t cap    = int64_t{148} * 16;
    return static_cast<unsigned>(blocks < cap ? blocks : cap);
}

} // namespace mgx

using namespace mgx;

extern "C" int mgx_cuda_gather(const void* data, int64_t outer, int64_t axis_len, int64_t inner_bytes,
                               const void* indices, int index_type, int64_t nidx, void* out, void* stream_)
{
    if(outer < 0 or axis_len <= 0 or inner_bytes <= 0 or nidx < 0)
        return MGX_E_INVALID_ARG;
    if(index_type != MGX_I32 and index_type != MGX_I64)
        return MGX_E_UNSUPPORTED;
    if(outer == 0 or nidx == 0)
        return MGX_OK;
    if(data == nullptr or indices == nullptr or out == nullptr)
        return MGX_E_INVALID_ARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int u = widest_unit(reinterpret_cast<uintptr_t>(data) | reinterpret_cast<uintptr_t>(out) |
                              static_cast<uintptr_t>(inner_bytes));
    const int64_t per   = inner_bytes / u;
    const int64_t total = outer * nidx * per;
    const auto* d       = static_cast<const uint8_t*>(data);
    auto* o             = static_cast<uint8_t*>(out);
    const unsigned grid = grid_for(total);
#define MGX_GATHER(U)                                                                                        \
    if(index_type == MGX_I32)                                                                                \
        gather_kernel<U, int32_t><<<grid, 256, 0, stream>>>(d, static_cast<const int32_t*>(indices), o, total, \
                                                            axis_len, per, nidx);                            \
    else                                                                                                     \
        gather_kernel<U, int64_t><<<grid, 256, 0, stream>>>(d, static_cast<const int64_t*>(indices), o, total, \
                                                            axis_len, per, nidx)
    switch(u)
    {
    case 16: MGX_GATHER(16); break;
    case 8: MGX_GATHER(8); break;
    case 4: MGX_GATHER(4); break;
    case 2: MGX_GATHER(2); break;
    default: MGX_GATHER(1); break;
    }
#undef MGX_GATHER
    return static_cast<int>(cudaGetLastError());
}

extern "C" int mgx_cuda_copy_rows(const void* src, int64_t src_pitch, void* dst, int64_t dst_pitch,
                                  int64_t rows, int64_t row_bytes, void* stream_)
{
    if(rows < 0 or row_bytes < 0 or src_pitch < row_bytes or dst_pitch < row_bytes)
        return MGX_E_INVALID_ARG;
    if(rows == 0 or row_bytes == 0)
        return MGX_OK;
    if(src == nullptr or dst == nullptr)
        return MGX_E_INVALID_ARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int u = widest_unit(reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) |
                              static_cast<uintptr_t>(row_bytes) | static_cast<uintptr_t>(src_pitch) |
                              static_cast<uintptr_t>(dst_pitch));
    const int64_t per   = row_bytes / u;
    const int64_t total = rows * per;
    const auto* s       = static_cast<const uint8_t*>(src);
    auto* d             = static_cast<uint8_t*>(dst);
    const unsigned grid = grid_for(total);
    switch(u)
    {
    case 16: copy_rows_kernel<16><<<grid, 256, 0, stream>>>(s, src_pitch, d, dst_pitch, total, per); break;
    case 8: copy_rows_kernel<8><<<grid, 256, 0, stream>>>(s, src_pitch, d, dst_pitch, total, per); break;
    case 4: copy_rows_kernel<4><<<grid, 256, 0, stream>>>(s, src_pitch, d, dst_pitch, total, per); break;
    case 2: copy_rows_kernel<2><<<grid, 256, 0, stream>>>(s, src_pitch, d, dst_pitch, total, per); break;
    default: copy_rows_kernel<1><<<grid, 256, 0, stream>>>(s, src_pitch, d, dst_pitch, total, per); break;
    }
    return static_cast<int>(cudaGetLastError());
}
