// The decoder's KV-cache and rotary-embedding operators ("next" rows of the quantized-GEMM path:
// what sits between the int4 projections of a Llama-shaped layer).
//
// concat_past_present: appends the new keys / values of a step to the cache in place
// (src/include/migraphx/op/concat_past_present.hpp:84-155: per batch entry and KV head the chunk of
// L rows goes to row seqlens_k[b] of the cache when L = 1 - decode - and to row 0 otherwise -
// prompt).  A byte mover: 16-byte units where pointers and rows allow.
//
// gqa_rotary_embedding: rotary position embedding of the Q and K heads of a packed
// [batch, heads + 2 kv_heads, seq, head] tensor, V copied through
// (src/include/migraphx/op/gqa_rotary_embedding.hpp:72-221), with the reference's roundings for fp16:
// x * cos is a half product (truncated), sign * x' * sin stays in fp32, the sum is stored as half.
#include "common.cuh"
#include "qgemm_math.cuh"
#include <cuda_fp16.h>

namespace mgx {

struct cpp_params
{
    const uint8_t* present;
    uint8_t* past;
    const void* seqlens;
    int seqlens_i64;
    int64_t sb, sh, sl; // byte strides of present along batch, head, row
    int64_t kv_heads, seq, row_bytes, cache_seq;
};

template <int V> // bytes per access
__global__ void concat_past_present_kernel(const cpp_params p)
{
    const int64_t bh   = blockIdx.y;
    const int64_t b    = bh / p.kv_heads, h = bh % p.kv_heads;
    int64_t pos        = 0;
    if(p.seq == 1)
        pos = p.seqlens_i64 ? static_cast<const int64_t*>(p.seqlens)[b]
                            : static_cast<int64_t>(static_cast<const int32_t*>(p.seqlens)[b]);
    const int64_t per_row = p.row_bytes / V;
    const int64_t total   = p.seq * per_row;
    for(int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
        i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        const int64_t l = i / per_row, c = i - l * per_row;
        if(pos + l < 0 or pos + l >= p.cache_seq)
            continue; // beyond the cache: nothing is written (the reference would write out of bounds)
        const uint8_t* src = p.present + b * p.sb + h * p.sh + l * p.sl + c * V;
        uint8_t* dst       = p.past + ((bh * p.cache_seq + pos + l) * p.row_bytes) + c * V;
        if constexpr(V == 16)
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
        else if constexpr(V == 4)
            *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(src);
        else
            *dst = *src;
    }
}

struct rope_params
{
    const void* qkv;
    void* out;
    const void* cosc;
    const void* sinc;
    const void* seqlens;
    int seqlens_i64;
    int64_t batch, heads, kv_heads, seq, head, max_seq;
    int rot; // rotary dimension = 2 * columns of the caches
    int interleaved;
};

template <class T>
__device__ __forceinline__ float rope_load(const T* p, int64_t i)
{
    if constexpr(std::is_same<T, float>::value)
        return p[i];
    else
        return __half2float(p[i]);
}

// one thread per element of the packed tensor
template <class T>
__global__ void gqa_rotary_kernel(const rope_params p)
{
    const int64_t total_heads = p.heads + 2 * p.kv_heads;
    const int64_t n           = p.batch * total_heads * p.seq * p.head;
    const T* in               = static_cast<const T*>(p.qkv);
    T* out                    = static_cast<T*>(p.out);
    const T* cosc             = static_cast<const T*>(p.cosc);
    const T* sinc             = static_cast<const T*>(p.sinc);
    const int half            = p.rot / 2;
    for(int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < n;
        idx += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        const int i       = static_cast<int>(idx % p.head);
        const int64_t s   = (idx / p.head) % p.seq;
        const int64_t hd  = (idx / (p.head * p.seq)) % total_heads;
        const int64_t b   = idx / (p.head * p.seq * total_heads);
        if(hd >= p.heads + p.kv_heads or i >= p.rot)
        {
            out[idx] = in[idx]; // V heads and the columns beyond the rotary dimension pass through
            continue;
        }
        int64_t pos = s;
        if(p.seq == 1)
            pos = p.seqlens_i64 ? static_cast<const int64_t*>(p.seqlens)[b]
                                : static_cast<int64_t>(static_cast<const int32_t*>(p.seqlens)[b]);
        pos = pos < 0 ? 0 : (pos >= p.max_seq ? p.max_seq - 1 : pos);
        int ci, j;
        float sign;
        if(p.interleaved)
        {
            ci   = (i / 2) % half;
            sign = (i % 2 == 0) ? -1.0f : 1.0f;
            j    = (i % 2 == 0) ? i + 1 : i - 1;
        }
        else
        {
            ci   = i % half;
            sign = i < half ? -1.0f : 1.0f;
            j    = (i + half) % p.rot;
        }
        const float x  = rope_load(in, idx);
        const float xj = rope_load(in, idx - i + j);
        const float c  = rope_load(cosc, pos * half + ci);
        const float sn = rope_load(sinc, pos * half + ci);
        if constexpr(std::is_same<T, float>::value)
            out[idx] = __fadd_rn(__fmul_rn(x, c), __fmul_rn(__fmul_rn(sign, xj), sn));
        else
        {
            // half * half -> half (truncated); float(sign) * half * half stays fp32; the sum is stored as half
            const float t1 = truncate_to_half_precision(__fmul_rn(x, c));
            const float t2 = __fmul_rn(__fmul_rn(sign, xj), sn);
            out[idx]       = __float2half_rz(__fadd_rn(t1, t2));
        }
    }
}

// The rotation of the rotary_embedding builder (src/op/builder/rotary_embedding.cpp:177-230,
// non-interleaved): out = x * cos + concat(x[half:], x[:half]) * (signs * sin), every product and the
// sum stored in T (half: truncated) as the builder's separate mul / mul / mul / add operators do;
// cos / sin rows gathered at positions[b, s].  x: [batch, heads, seq, head] with element strides
// sb / sh / ss (rows contiguous); out packed.
struct rope_builder_params
{
    const void* x;
    void* out;
    const void* cosc;
    const void* sinc;
    const void* pos;
    int pos_i64;
    int64_t sb, sh, ss;
    int64_t batch, heads, seq, head, max_pos;
};

template <class T>
__global__ void rotary_builder_kernel(const rope_builder_params p)
{
    const int64_t n = p.batch * p.heads * p.seq * p.head;
    const T* in     = static_cast<const T*>(p.x);
    T* out          = static_cast<T*>(p.out);
    const T* cosc   = static_cast<const T*>(p.cosc);
    const T* sinc   = static_cast<const T*>(p.sinc);
    const int half  = static_cast<int>(p.head / 2);
    for(int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < n;
        idx += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        const int i      = static_cast<int>(idx % p.head);
        const int64_t s  = (idx / p.head) % p.seq;
        const int64_t h  = (idx / (p.head * p.seq)) % p.heads;
        const int64_t b  = idx / (p.head * p.seq * p.heads);
        int64_t pos      = p.pos_i64 ? static_cast<const int64_t*>(p.pos)[b * p.seq + s]
                                     : static_cast<int64_t>(static_cast<const int32_t*>(p.pos)[b * p.seq + s]);
        if(pos < 0)
            pos += p.max_pos; // gathernd counts negative indices from the end
        pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
        const T* row   = in + b * p.sb + h * p.sh + s * p.ss;
        const int ci   = i < half ? i : i - half;
        const float x  = rope_load(row, i);
        const float xr = rope_load(row, i < half ? i + half : i - half);
        const float c  = rope_load(cosc, pos * half + ci);
        const float sn = rope_load(sinc, pos * half + ci);
        const float ss = i < half ? -sn : sn; // signs * sin: exact
        if constexpr(std::is_same<T, float>::value)
            out[idx] = __fadd_rn(__fmul_rn(x, c), __fmul_rn(xr, ss));
        else
        {
            const float t1 = truncate_to_half_precision(__fmul_rn(x, c));
            const float t2 = truncate_to_half_precision(__fmul_rn(xr, ss));
            out[idx]       = __float2half_rz(__fadd_rn(t1, t2));
        }
    }
}

} // namespace mgx

extern "C" int mgx_cuda_rotary_embedding(const void* x, int type, const int64_t x_strides[3], int64_t batch,
                                         int64_t heads, int64_t seq, int64_t head, const void* positions,
                                         int positions_type, const void* cos_cache, const void* sin_cache,
                                         int64_t max_pos, void* out, void* stream_)
{
    using namespace mgx;
    if(x == nullptr or out == nullptr or cos_cache == nullptr or sin_cache == nullptr or positions == nullptr or
       x_strides == nullptr)
        return MGX_E_INVALID_ARG;
    if(batch <= 0 or heads <= 0 or seq <= 0 or head <= 0 or head % 2 != 0 or max_pos <= 0)
        return MGX_E_INVALID_ARG;
    if(type != MGX_F16 and type != MGX_F32)
        return MGX_E_UNSUPPORTED;
    if(positions_type != MGX_I32 and positions_type != MGX_I64)
        return MGX_E_UNSUPPORTED;
    rope_builder_params p{};
    p.x = x, p.out = out, p.cosc = cos_cache, p.sinc = sin_cache, p.pos = positions;
    p.pos_i64 = positions_type == MGX_I64 ? 1 : 0;
    p.sb = x_strides[0], p.sh = x_strides[1], p.ss = x_strides[2];
    p.batch = batch, p.heads = heads, p.seq = seq, p.head = head, p.max_pos = max_pos;
    const int64_t n       = batch * heads * seq * head;
    const unsigned blocks = static_cast<unsigned>((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    cudaStream_t stream   = static_cast<cudaStream_t>(stream_);
    if(type == MGX_F16)
        rotary_builder_kernel<__half><<<blocks, 256, 0, stream>>>(p);
    else
        rotary_builder_kernel<float><<<blocks, 256, 0, stream>>>(p);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int mgx_cuda_concat_past_present(const void* present, const int64_t present_strides[3], int64_t batch,
                                            int64_t kv_heads, int64_t seq, int64_t head_bytes, const void* seqlens,
                                            int seqlens_type, void* past, int64_t cache_seq, void* stream_)
{
    using namespace mgx;
    if(present == nullptr or past == nullptr or present_strides == nullptr)
        return MGX_E_INVALID_ARG;
    if(batch <= 0 or kv_heads <= 0 or seq <= 0 or head_bytes <= 0 or cache_seq <= 0)
        return MGX_E_INVALID_ARG;
    if(seq == 1 and seqlens == nullptr)
        return MGX_E_INVALID_ARG;
    if(seqlens_type != MGX_I32 and seqlens_type != MGX_I64)
        return MGX_E_UNSUPPORTED;
    if(batch * kv_heads > 65535)
        return MGX_E_TOO_LARGE;
    cpp_params p{};
    p.present     = static_cast<const uint8_t*>(present);
    p.past        = static_cast<uint8_t*>(past);
    p.seqlens     = seqlens;
    p.seqlens_i64 = seqlens_type == MGX_I64 ? 1 : 0;
    p.sb = present_strides[0], p.sh = present_strides[1], p.sl = present_strides[2];
    p.kv_heads  = kv_heads;
    p.seq       = seq;
    p.row_bytes = head_bytes;
    p.cache_seq = cache_seq;
    auto aligned = [&](int a) {
        return (reinterpret_cast<uintptr_t>(present) % a) == 0 and (reinterpret_cast<uintptr_t>(past) % a) == 0 and
               head_bytes % a == 0 and p.sb % a == 0 and p.sh % a == 0 and p.sl % a == 0;
    };
    const int v           = aligned(16) ? 16 : (aligned(4) ? 4 : 1);
    const int64_t work    = seq * (head_bytes / v);
    const unsigned blocks = static_cast<unsigned>(work < 256 ? 1 : (work + 255) / 256 > 1024 ? 1024 : (work + 255) / 256);
    const dim3 grid(blocks, static_cast<unsigned>(batch * kv_heads));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if(v == 16)
        concat_past_present_kernel<16><<<grid, 256, 0, stream>>>(p);
    else if(v == 4)
        concat_past_present_kernel<4><<<grid, 256, 0, stream>>>(p);
    else
        concat_past_present_kernel<1><<<grid, 256, 0, stream>>>(p);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int mgx_cuda_gqa_rotary_embedding(const void* qkv, int type, int64_t batch, int64_t heads, int64_t kv_heads,
                                             int64_t seq, int64_t head, const void* cos_cache, const void* sin_cache,
                                             int64_t max_seq, int64_t rotary_dim, const void* seqlens, int seqlens_type,
                                             int interleaved, void* out, void* stream_)
{
    using namespace mgx;
    if(qkv == nullptr or out == nullptr or cos_cache == nullptr or sin_cache == nullptr)
        return MGX_E_INVALID_ARG;
    if(batch <= 0 or heads <= 0 or kv_heads <= 0 or seq <= 0 or head <= 0 or max_seq <= 0 or rotary_dim <= 0 or
       rotary_dim % 2 != 0 or rotary_dim > head)
        return MGX_E_INVALID_ARG;
    if(type != MGX_F16 and type != MGX_F32)
        return MGX_E_UNSUPPORTED;
    if(seq == 1 and seqlens == nullptr)
        return MGX_E_INVALID_ARG;
    if(seqlens != nullptr and seqlens_type != MGX_I32 and seqlens_type != MGX_I64)
        return MGX_E_UNSUPPORTED;
    rope_params p{};
    p.qkv = qkv, p.out = out, p.cosc = cos_cache, p.sinc = sin_cache, p.seqlens = seqlens;
    p.seqlens_i64 = seqlens_type == MGX_I64 ? 1 : 0;
    p.batch = batch, p.heads = heads, p.kv_heads = kv_heads, p.seq = seq, p.head = head, p.max_seq = max_seq;
    p.rot         = static_cast<int>(rotary_dim);
    p.interleaved = interleaved != 0 ? 1 : 0;
    const int64_t n       = batch * (heads + 2 * kv_heads) * seq * head;
    const unsigned blocks = static_cast<unsigned>((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    cudaStream_t stream   = static_cast<cudaStream_t>(stream_);
    if(type == MGX_F16)
        gqa_rotary_kernel<__half><<<blocks, 256, 0, stream>>>(p);
    else
        gqa_rotary_kernel<float><<<blocks, 256, 0, stream>>>(p);
    return static_cast<int>(cudaGetLastError());
}
