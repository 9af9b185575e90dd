// The MIGraphX `cuda` target for B200: context, target, passes and models.
//
// Plug-in boundary (MIGraphX): src/include/migraphx/target.hpp:130-146 (name / get_passes /
// get_context / copy_to / copy_from / allocate), context.hpp:93-111, operation.hpp:504-557,
// register_target.hpp:53-73.  Everything below that boundary is host code that enqueues the
// kernels of include/mgx_cuda.h on the context's CUDA stream.  There is no CPU fallback: an
// instruction the target has no kernel for makes compile() throw.
#ifndef MGX_CUDA_TARGET_HPP
#define MGX_CUDA_TARGET_HPP

#include <migraphx/config.hpp>
#include <migraphx/argument.hpp>
#include <migraphx/compile_options.hpp>
#include <migraphx/context.hpp>
#include <migraphx/instruction_ref.hpp>
#include <migraphx/operation.hpp>
#include <migraphx/pass.hpp>
#include <migraphx/shape.hpp>
#include <migraphx/value.hpp>
#include <migraphx/any_ptr.hpp>
#include <cuda_runtime.h>
#include <functional>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

namespace migraphx {
inline namespace MIGRAPHX_INLINE_NS {
struct module;
struct module_pass_manager;
namespace cuda {

#define MGX_CUDA_EXPORT __attribute__((visibility("default")))

// Throws a migraphx::exception when a CUDA runtime call or a kernel-library call failed.
void check_cuda(cudaError_t e, const char* what);
void check_mgx(int status, const char* what);

// Device buffer of s.bytes() (+1, so that empty shapes still own an address) owned by the
// returned argument (cudaFree on release).
MGX_CUDA_EXPORT argument allocate_device(const shape& s);
MGX_CUDA_EXPORT argument to_device(const argument& host);
MGX_CUDA_EXPORT argument from_device(const argument& dev);

struct context_state
{
    int device = 0;
    std::vector<cudaStream_t> streams; // owned
    std::vector<cudaEvent_t> events;   // owned, created on demand
    std::size_t current   = 0;
    cudaStream_t external = nullptr; // a caller's queue bound with set_queue()
    bool has_external     = false;
    cudaEvent_t begin_event  = nullptr;
    cudaEvent_t finish_event = nullptr;
    std::unordered_map<std::string, argument> preallocations;
    // page-locked host buffers handed out for results copied back to the host (offload_copy):
    // a buffer is reused once the caller has dropped the argument that referred to it
    std::vector<std::pair<std::size_t, std::shared_ptr<void>>> host_pool;
    bool ready = false;
    // CUDA-graph replay of the instruction stream (cuda::graph_run)
    enum class graph_mode
    {
        off,       // not used for this program
        warm,      // still executing instruction by instruction
        capturing, // this eval is being captured
        ready      // a graph is instantiated for `graph_params`
    };
    graph_mode gmode        = graph_mode::off;
    int warm_evals          = 0;
    std::vector<argument> graph_results; // what the recorded submodule returned
    cudaGraph_t graph       = nullptr;
    cudaGraphExec_t gexec   = nullptr;
    std::vector<const void*> graph_params; // parameter buffers the graph was captured with
    context_state(int dev, std::size_t nstreams);
    void init(); // creates the streams and events (first use)
    ~context_state();
    context_state(const context_state&)            = delete;
    context_state& operator=(const context_state&) = delete;
};

// One per compiled program (program::compile, src/program.cpp:327); copies share state.
struct MGX_CUDA_EXPORT context
{
    explicit context(int device = 0, std::size_t nstreams = 1);

    int device() const { return state->device; }
    std::size_t nstreams() const { return state->streams.size(); }
    cudaStream_t stream() const;
    void set_stream(std::size_t n);
    cudaEvent_t event(std::size_t id);
    // page-locked host buffer of s.bytes() that nobody else holds (see context_state::host_pool)
    argument pinned_host(const shape& s);
    void store_preallocation(const std::string& id, const argument& a);
    argument get_preallocation(const std::string& id) const;
    // true while a captured graph stands in for the instruction stream: operators that would
    // launch work return their output buffer instead
    void enable_graph();
    // runs body() - the evaluation of a submodule - or, once it has been recorded for these
    // parameter buffers, launches the recorded graph instead and returns the recorded results
    std::vector<argument> run_graph(const std::vector<const void*>& params,
                                    const std::function<std::vector<argument>()>& body);

    // migraphx::context interface
    void finish() const;
    value to_value() const;
    void from_value(const value& v);
    any_ptr get_queue();
    void set_queue(any_ptr queue);
    void restore_queue();
    void wait_for(any_ptr queue);
    void finish_on(any_ptr queue);

    std::shared_ptr<context_state> state;
};

struct MGX_CUDA_EXPORT target
{
    std::string name() const;
    std::vector<pass> get_passes(migraphx::context& ctx, const compile_options& options) const;
    migraphx::context get_context() const;
    argument copy_to(const argument& arg) const;
    argument copy_from(const argument& arg) const;
    argument allocate(const shape& s) const;
};

// allocation_model (src/include/migraphx/allocation_model.hpp:62-75)
struct allocation_model
{
    std::string name() const { return "cuda::allocate"; }
    std::string copy() const { return "cuda::copy"; }
    operation allocate(const shape& s) const;
    operation preallocate(const shape& s, const std::string& id) const;
    bool needs_out_params() const { return true; }
};

// schedule_model (src/include/migraphx/schedule_model.hpp:65-78)
struct schedule_model
{
    std::size_t streams = 1;
    std::size_t concurrency() const { return streams; }
    void sched(module& m, instruction_ref ins, std::size_t n) const;
    void wait(module& m, instruction_ref ins, std::size_t wait_id) const;
    void record(module& m, instruction_ref ins, std::size_t wait_id) const;
    std::size_t weight(const operation& op) const;
};

// ---- passes -------------------------------------------------------------------------
// Puts the instructions of `pointwise` sub-modules (the output of fuse_pointwise) back
// into the enclosing module so that the lowering sees plain operator chains.
struct inline_pointwise
{
    std::string name() const { return "cuda::inline_pointwise"; }
    void apply(module& m) const;
};

// Replaces the quantized-GEMM sub-graphs by cuda::* operators and throws on anything the
// target cannot run.
struct lowering
{
    context* ctx      = nullptr;
    bool offload_copy = false;
    std::string name() const { return "cuda::lowering"; }
    void apply(module_pass_manager& mpm) const;
};

// @literal -> cuda::literal (device-resident constant, uploaded at finalize).
struct write_literals
{
    std::string name() const { return "cuda::write_literals"; }
    void apply(module& m) const;
};

// Merges a cuda::pointwise whose result has a single user into that user when the user is a
// cuda::pointwise too (what fuse_pointwise does for the reference's targets): chains of
// element-wise operators become one launch.
struct fuse_cuda_pointwise
{
    std::string name() const { return "cuda::fuse_pointwise"; }
    void apply(module& m) const;
};

// Moves the instructions of the main module into a submodule behind ONE cuda::graph_run
// instruction: the first two eval() calls evaluate the submodule instruction by instruction, the
// third records it with stream capture, and from then on an eval() is one cudaGraphLaunch - the
// submodule's instructions (hundreds of literals, views and launches) are not visited at all -
// as long as the caller passes the same parameter buffers (src/program.cpp:472-565 is the loop
// this short-cuts).  With offload_copy the host-to-device and device-to-host copies stay in the
// main module around the call (their device buffers are arena addresses, which never change).  Not applied with several streams or collectives; MIGRAPHX_CUDA_GRAPH=0 turns it off.
struct insert_graph_ops
{
    context* ctx      = nullptr;
    bool offload_copy = false;
    std::string name() const { return "cuda::insert_graph_ops"; }
    void apply(module_pass_manager& mpm) const;
};

// Synchronises the stream before results copied to the host are returned.
struct sync_device
{
    std::string name() const { return "cuda::sync_device"; }
    void apply(module& m) const;
};

} // namespace cuda
} // namespace MIGRAPHX_INLINE_NS
} // namespace migraphx
#endif
