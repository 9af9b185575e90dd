// Library-wide host helpers: driver entry point lookup, per-device caches,
// status reporting.
#include "common.cuh"
#include "ptx.cuh"
#include <atomic>
#include <mutex>

namespace mgx {

// One thread waits, with a time limit, on a barrier phase that nothing ever completes: the
// expiry path every kernel of this library shares (status word written, abort flag raised, the
// kernel returns normally) exercised by itself.  Nothing faults and the context stays usable.
__global__ void bounded_wait_probe_kernel(unsigned long long limit_ns, unsigned int code,
                                          unsigned int* gave_up)
{
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if(threadIdx.x == 0)
    {
        mbar_init(&bar, 1);
        abort_flag = 0;
        fence_barrier_init();
        const bool done = mbar_wait_bounded(&bar, 0u, &abort_flag, code, limit_ns);
        if(gave_up != nullptr)
            *gave_up = done ? 0u : abort_flag;
    }
}

static int runtime_status(unsigned int* out) { return read_and_clear_status(out); }

cuTensorMapEncodeTiled_t get_tensor_map_encoder()
{
    static std::atomic<void*> cached{nullptr};
    void* fn = cached.load(std::memory_order_acquire);
    if(fn != nullptr)
        return reinterpret_cast<cuTensorMapEncodeTiled_t>(fn);
    cudaDriverEntryPointQueryResult q;
    void* p = nullptr;
    if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess or
       q != cudaDriverEntryPointSuccess)
        return nullptr;
    cached.store(p, std::memory_order_release);
    return reinterpret_cast<cuTensorMapEncodeTiled_t>(p);
}

constexpr int max_devices = 64;

int device_sm_count()
{
    static std::atomic<int> cache[max_devices];
    int dev = 0;
    if(cudaGetDevice(&dev) != cudaSuccess or dev < 0 or dev >= max_devices)
        return 148;
    int v = cache[dev].load(std::memory_order_relaxed);
    if(v > 0)
        return v;
    if(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess or v <= 0)
        return 148;
    cache[dev].store(v, std::memory_order_relaxed);
    return v;
}

int ensure_smem_optin(const void* kernel, int bytes)
{
    // (kernel, device) pairs already configured; small, append-only.
    struct entry
    {
        const void* k;
        int dev;
    };
    static std::mutex m;
    static entry done[512];
    static int ndone = 0;
    int dev          = 0;
    cudaError_t e    = cudaGetDevice(&dev);
    if(e != cudaSuccess)
        return static_cast<int>(e);
    std::lock_guard<std::mutex> lock(m);
    for(int i = 0; i < ndone; ++i)
        if(done[i].k == kernel and done[i].dev == dev)
            return MGX_OK;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if(e != cudaSuccess)
        return static_cast<int>(e);
    if(ndone < 512)
        done[ndone++] = entry{kernel, dev};
    return MGX_OK;
}

} // namespace mgx

extern "C" int mgx_cuda_device_status(int* status)
{
    if(status == nullptr)
        return MGX_E_INVALID_ARG;
    cudaError_t e = cudaDeviceSynchronize();
    if(e != cudaSuccess)
        return static_cast<int>(e);
    unsigned int a = 0, b = 0, c = 0, d = 0, g = 0, r = 0;
    int rc = mgx::runtime_status(&r);
    if(rc != 0)
        return rc;
    rc = mgx::qgemm_status(&a);
    if(rc != 0)
        return rc;
    rc = mgx::w4a16_status(&b);
    if(rc != 0)
        return rc;
    rc = mgx::w4a16_tc_status(&c);
    if(rc != 0)
        return rc;
    rc = mgx::w4a16_prefill_status(&d);
    if(rc != 0)
        return rc;
    rc = mgx::qgemv_status(&g);
    if(rc != 0)
        return rc;
    *status = static_cast<int>(a != 0 ? a : (b != 0 ? b : (c != 0 ? c : (d != 0 ? d : (g != 0 ? g : r)))));
    return MGX_OK;
}

extern "C" int mgx_cuda_selftest_bounded_wait(uint64_t limit_ns, void* gave_up, void* stream)
{
    if(limit_ns == 0 or limit_ns > 100000000ull)
        return MGX_E_INVALID_ARG; // at most 0.1 s: this is a probe, not a way to park a GPU
    mgx::bounded_wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        limit_ns, 99u, static_cast<unsigned int*>(gave_up));
    return static_cast<int>(cudaGetLastError());
}

extern "C" const char* mgx_cuda_status_string(int code)
{
    switch(code)
    {
    case MGX_OK: return "ok";
    case MGX_E_INVALID_ARG: return "invalid argument";
    case MGX_E_UNSUPPORTED: return "unsupported case (no kernel; there is no CPU fallback)";
    case MGX_E_ALIGNMENT: return "pointer or leading dimension not aligned as required";
    case MGX_E_WORKSPACE: return "workspace missing or too small";
    case MGX_E_TOO_LARGE: return "size beyond the supported maximum";
    case MGX_E_DRIVER: return "CUDA driver entry point unavailable";
    case MGX_E_DEVICE_TIMEOUT: return "a bounded wait inside a kernel expired";
    default: break;
    }
    if(code > 0)
        return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown status";
}

extern "C" const char* mgx_cuda_version(void) { return "mgx_cuda sm_100a kernels 1"; }
