// Tensor-parallel exchange step: an in-place sum all-reduce over NCCL (NVLink / NVSwitch),
// enqueued on the caller's stream.  The reference has no collective anywhere; this is the one
// exchange the row-split linears (o_proj, down_proj) of a tensor-parallel decoder need.
// NCCL is resolved at run time (dlopen of libnccl.so.2, or the path in MGX_NCCL_LIB) so that
// single-GPU users carry no dependency on it.
#include "common.cuh"
#include <dlfcn.h>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace {

struct nccl_api
{
    // signatures of nccl.h (ncclResult_t = int, ncclComm_t = opaque pointer, ncclUniqueId = 128 bytes)
    int (*GetUniqueId)(void* id)                                                   = nullptr;
    int (*CommInitRank)(void** comm, int nranks, const void* id_by_value, int rank) = nullptr;
    int (*CommDestroy)(void* comm)                                                 = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t)    = nullptr;
    const char* (*GetErrorString)(int)                                             = nullptr;
    bool ok = false;
};

struct unique_id
{
    char bytes[128];
};

nccl_api& api()
{
    static nccl_api a;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* env = std::getenv("MGX_NCCL_LIB");
        void* h         = nullptr;
        if(env != nullptr and env[0] != 0)
            h = dlopen(env, RTLD_NOW | RTLD_GLOBAL);
        if(h == nullptr)
            h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if(h == nullptr)
            return;
        a.GetUniqueId    = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        a.CommDestroy    = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        a.AllReduce      = reinterpret_cast<decltype(a.AllReduce)>(dlsym(h, "ncclAllReduce"));
        a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
        a.CommInitRank   = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        a.ok = a.GetUniqueId and a.CommDestroy and a.AllReduce and a.CommInitRank;
    });
    return a;
}

void* g_default_comm = nullptr;

// ncclDataType_t values of nccl.h
int nccl_type(int t)
{
    switch(t)
    {
    case MGX_F32: return 7;  // ncclFloat32
    case MGX_F16: return 6;  // ncclFloat16
    case MGX_I32: return 2;  // ncclInt32
    case MGX_I8: return 0;   // ncclInt8
    case MGX_U8: return 1;   // ncclUint8
    default: return -1;
    }
}

} // namespace

extern "C" int mgx_cuda_comm_unique_id(void* id128)
{
    if(id128 == nullptr)
        return MGX_E_INVALID_ARG;
    if(not api().ok)
        return MGX_E_DRIVER;
    unique_id id{};
    const int r = api().GetUniqueId(&id);
    if(r != 0)
        return 2000 + r;
    std::memcpy(id128, id.bytes, sizeof(id.bytes));
    return MGX_OK;
}

extern "C" int mgx_cuda_comm_create(const void* id128, int nranks, int rank, void** comm)
{
    if(id128 == nullptr or comm == nullptr or nranks < 1 or rank < 0 or rank >= nranks)
        return MGX_E_INVALID_ARG;
    if(not api().ok)
        return MGX_E_DRIVER;
    unique_id id{};
    std::memcpy(id.bytes, id128, sizeof(id.bytes));
    // ncclCommInitRank takes the 128-byte id BY VALUE
    auto init = reinterpret_cast<int (*)(void**, int, unique_id, int)>(api().CommInitRank);
    const int r = init(comm, nranks, id, rank);
    return r == 0 ? MGX_OK : 2000 + r;
}

extern "C" int mgx_cuda_comm_destroy(void* comm)
{
    if(comm == nullptr)
        return MGX_OK;
    if(not api().ok)
        return MGX_E_DRIVER;
    if(comm == g_default_comm)
        g_default_comm = nullptr;
    const int r = api().CommDestroy(comm);
    return r == 0 ? MGX_OK : 2000 + r;
}

extern "C" void mgx_cuda_comm_set_default(void* comm) { g_default_comm = comm; }
extern "C" void* mgx_cuda_comm_default(void) { return g_default_comm; }

extern "C" int mgx_cuda_all_reduce(void* buf, size_t count, int dtype, void* comm, void* stream)
{
    if(count == 0)
        return MGX_OK;
    if(buf == nullptr)
        return MGX_E_INVALID_ARG;
    if(comm == nullptr)
        comm = g_default_comm;
    if(comm == nullptr)
        return MGX_E_INVALID_ARG;
    const int t = nccl_type(dtype);
    if(t < 0)
        return MGX_E_UNSUPPORTED;
    if(not api().ok)
        return MGX_E_DRIVER;
    const int r = api().AllReduce(buf, buf, count, t, 0 /* ncclSum */, comm, static_cast<cudaStream_t>(stream));
    return r == 0 ? MGX_OK : 2000 + r;
}
