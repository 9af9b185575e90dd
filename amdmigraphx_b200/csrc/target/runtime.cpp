// cuda::context, device memory helpers and the memory / stream operators of the `cuda`
// target.  Structural counterparts in the reference's HIP target (not ported, re-written
// for the CUDA runtime): src/targets/gpu/include/migraphx/gpu/context.hpp:56-448,
// src/targets/gpu/include/migraphx/gpu/hip.hpp:73-296, src/targets/gpu/hip.cpp:99-308.
#include "cuda_target.hpp"
#include "cuda_ops.hpp"
#include <migraphx/check_shapes.hpp>
#include <migraphx/errors.hpp>
#include <migraphx/register_op.hpp>
#include <migraphx/env.hpp>
#include "../../../include/mgx_cuda.h"
#include <cstring>
#include <migraphx/module.hpp>

namespace migraphx {
inline namespace MIGRAPHX_INLINE_NS {
namespace cuda {

void check_cuda(cudaError_t e, const char* what)
{
    if(e != cudaSuccess)
        MIGRAPHX_THROW(std::string("cuda target: ") + what + ": " + cudaGetErrorString(e));
}

void check_mgx(int status, const char* what)
{
    if(status != MGX_OK)
        MIGRAPHX_THROW(std::string("cuda target: ") + what + ": " + mgx_cuda_status_string(status));
}

argument allocate_device(const shape& s)
{
    void* p = nullptr;
    check_cuda(cudaMalloc(&p, s.bytes() + 1), "cudaMalloc");
    std::shared_ptr<void> owner(p, [](void* q) { (void)cudaFree(q); });
    return argument{s, owner};
}

argument to_device(const argument& host)
{
    argument dev = allocate_device(host.get_shape());
    if(host.get_shape().bytes() > 0)
        check_cuda(cudaMemcpy(dev.data(), host.data(), host.get_shape().bytes(),
                              cudaMemcpyHostToDevice),
                   "cudaMemcpy host to device");
    return dev;
}

argument from_device(const argument& dev)
{
    argument host{dev.get_shape()};
    if(dev.get_shape().bytes() > 0)
        check_cuda(cudaMemcpy(host.data(), dev.data(), dev.get_shape().bytes(),
                              cudaMemcpyDeviceToHost),
                   "cudaMemcpy device to host");
    return host;
}

// ------------------------------------------------------------------ context
// Streams and events are created on first use, so that a program can be taken through the
// pass pipeline (everything before finalize) on a machine without a GPU.
context_state::context_state(int dev, std::size_t nstreams) : device(dev)
{
    streams.assign(nstreams < 1 ? 1 : nstreams, nullptr);
}

void context_state::init()
{
    if(ready)
        return;
    check_cuda(cudaSetDevice(device), "cudaSetDevice");
    for(auto& s : streams)
        check_cuda(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreate");
    check_cuda(cudaEventCreateWithFlags(&begin_event, cudaEventDisableTiming), "cudaEventCreate");
    check_cuda(cudaEventCreateWithFlags(&finish_event, cudaEventDisableTiming), "cudaEventCreate");
    ready = true;
}

context_state::~context_state()
{
    for(auto s : streams)
        if(s != nullptr)
            (void)cudaStreamDestroy(s);
    for(auto e : events)
        (void)cudaEventDestroy(e);
    if(begin_event != nullptr)
        (void)cudaEventDestroy(begin_event);
    if(finish_event != nullptr)
        (void)cudaEventDestroy(finish_event);
    if(gexec != nullptr)
        (void)cudaGraphExecDestroy(gexec);
    if(graph != nullptr)
        (void)cudaGraphDestroy(graph);
}

context::context(int device, std::size_t nstreams)
    : state(std::make_shared<context_state>(device, nstreams))
{
}

cudaStream_t context::stream() const
{
    state->init();
    if(state->has_external and state->current == 0)
        return state->external;
    return state->streams.at(state->current);
}

void context::set_stream(std::size_t n)
{
    if(n >= state->streams.size())
        MIGRAPHX_THROW("cuda target: stream index out of range");
    state->current = n;
}

cudaEvent_t context::event(std::size_t id)
{
    state->init();
    while(state->events.size() <= id)
    {
        cudaEvent_t e = nullptr;
        check_cuda(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
        state->events.push_back(e);
    }
    return state->events[id];
}

argument context::pinned_host(const shape& s)
{
    const std::size_t bytes = s.bytes() + 1;
    for(auto& e : state->host_pool)
        if(e.first >= bytes and e.first <= 2 * bytes and e.second.use_count() == 1)
            return argument{s, e.second};
    void* p = nullptr;
    check_cuda(cudaHostAlloc(&p, bytes, cudaHostAllocDefault), "cudaHostAlloc");
    std::shared_ptr<void> owner(p, [](void* q) { (void)cudaFreeHost(q); });
    state->host_pool.emplace_back(bytes, owner);
    return argument{s, owner};
}

void context::store_preallocation(const std::string& id, const argument& a)
{
    state->preallocations[id] = a;
}

argument context::get_preallocation(const std::string& id) const
{
    auto it = state->preallocations.find(id);
    if(it == state->preallocations.end())
        MIGRAPHX_THROW("cuda target: no preallocation named " + id);
    return it->second;
}

void context::finish() const
{
    if(not state->ready)
        return; // nothing was ever submitted
    check_cuda(cudaSetDevice(state->device), "cudaSetDevice");
    for(auto s : state->streams)
        check_cuda(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    if(state->has_external)
        check_cuda(cudaStreamSynchronize(state->external), "cudaStreamSynchronize");
    int dev_status = 0;
    check_mgx(mgx_cuda_device_status(&dev_status), "mgx_cuda_device_status");
    if(dev_status != 0)
        MIGRAPHX_THROW("cuda target: a kernel reported an expired bounded wait (code " +
                       std::to_string(dev_status) + ")");
}

value context::to_value() const
{
    value v;
    v["device"]   = state->device;
    v["nstreams"] = state->streams.size();
    return v;
}

void context::from_value(const value& v)
{
    const int dev          = v.contains("device") ? v.at("device").to<int>() : 0;
    const std::size_t nstr = v.contains("nstreams") ? v.at("nstreams").to<std::size_t>() : 1;
    int count = 0;
    if(cudaGetDeviceCount(&count) != cudaSuccess)
        count = 0;
    state = std::make_shared<context_state>(dev < count ? dev : 0, nstr);
}

any_ptr context::get_queue()
{
    cudaStream_t s = stream();
    return s == nullptr ? any_ptr{} : any_ptr{s};
}

void context::set_queue(any_ptr queue)
{
    state->external     = queue.unsafe_get() == nullptr ? nullptr : queue.get<cudaStream_t>();
    state->has_external = true;
}

void context::restore_queue() { state->has_external = false; }

void context::wait_for(any_ptr queue)
{
    state->init();
    check_cuda(cudaEventRecord(state->begin_event, queue.get<cudaStream_t>()), "cudaEventRecord");
    check_cuda(cudaStreamWaitEvent(stream(), state->begin_event, 0), "cudaStreamWaitEvent");
}

void context::finish_on(any_ptr queue)
{
    state->init();
    check_cuda(cudaEventRecord(state->finish_event, stream()), "cudaEventRecord");
    check_cuda(cudaStreamWaitEvent(queue.get<cudaStream_t>(), state->finish_event, 0),
               "cudaStreamWaitEvent");
}

// ------------------------------------------------------------------ CUDA-graph replay
void context::enable_graph()
{
    if(state->gmode == context_state::graph_mode::off)
        state->gmode = context_state::graph_mode::warm;
}

std::vector<argument> context::run_graph(const std::vector<const void*>& params,
                                         const std::function<std::vector<argument>()>& body)
{
    using mode = context_state::graph_mode;
    auto& st   = *state;
    if(st.gmode == mode::ready)
    {
        if(params == st.graph_params)
        {
            check_cuda(cudaGraphLaunch(st.gexec, stream()), "cudaGraphLaunch");
            return st.graph_results;
        }
        // other buffers: evaluate instruction by instruction and record again
        (void)cudaGraphExecDestroy(st.gexec);
        (void)cudaGraphDestroy(st.graph);
        st.gexec = nullptr;
        st.graph = nullptr;
        st.graph_results.clear();
        st.gmode      = mode::warm;
        st.warm_evals = 1;
        return body();
    }
    // the first two evaluations run eagerly: one-time set-up (kernel attributes, entry point
    // look-ups) must not happen inside a capture
    if(st.gmode == mode::warm and ++st.warm_evals > 2)
    {
        check_cuda(cudaStreamBeginCapture(stream(), cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
        st.gmode = mode::off; // whatever fails below, no second attempt
        std::vector<argument> results;
        try
        {
            results = body();
        }
        catch(...)
        {
            cudaGraph_t broken = nullptr;
            (void)cudaStreamEndCapture(stream(), &broken);
            if(broken != nullptr)
                (void)cudaGraphDestroy(broken);
            throw;
        }
        check_cuda(cudaStreamEndCapture(stream(), &st.graph), "cudaStreamEndCapture");
        check_cuda(cudaGraphInstantiate(&st.gexec, st.graph, 0), "cudaGraphInstantiate");
        // nothing of this evaluation has run yet: the recorded work is launched as the new graph
        check_cuda(cudaGraphLaunch(st.gexec, stream()), "cudaGraphLaunch");
        st.graph_params  = params;
        st.graph_results = results;
        st.gmode         = mode::ready;
        return results;
    }
    return body();
}

shape op_graph_run::compute_shape(const std::vector<shape>& inputs, std::vector<module_ref> mods) const
{
    if(mods.size() != 1 or inputs.size() != params.size())
        MIGRAPHX_THROW("cuda::graph_run: expects one submodule and one input per parameter name");
    return shape(mods.front()->get_output_shapes());
}

argument op_graph_run::compute(context& ctx,
                               const shape&,
                               const std::vector<argument>& args,
                               const std::vector<module_ref>& mods,
                               const std::function<std::vector<argument>(
                                   module_ref&, const std::unordered_map<std::string, argument>&)>& run) const
{
    std::vector<const void*> ptrs;
    ptrs.reserve(args.size());
    for(const auto& a : args)
        ptrs.push_back(a.empty() ? nullptr : a.data());
    module_ref mod = mods.front();
    auto results   = ctx.run_graph(ptrs, [&] {
        std::unordered_map<std::string, argument> pm;
        for(std::size_t i = 0; i < args.size(); ++i)
            pm[params[i]] = args[i];
        return run(mod, pm);
    });
    return argument{results};
}

// ------------------------------------------------------------------ memory operators
shape op_allocate::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(0);
    return s;
}
argument op_allocate::compute(context&, const shape& out, const std::vector<argument>&) const
{
    return allocate_device(out);
}

shape op_preallocate::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(0);
    return s;
}
argument op_preallocate::compute(context& ctx, const shape&, const std::vector<argument>&) const
{
    return ctx.get_preallocation(id);
}
void op_preallocate::finalize(context& ctx, const shape&, const std::vector<shape>&) const
{
    (void)ctx.stream(); // selects the context's device
    ctx.store_preallocation(id, allocate_device(s));
}

shape op_literal::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(0);
    return l.get_shape();
}
argument op_literal::compute(context& ctx, const shape&, const std::vector<argument>&) const
{
    return ctx.get_preallocation(id);
}
void op_literal::finalize(context& ctx, const shape&, const std::vector<shape>&) const
{
    (void)ctx.stream(); // selects the context's device
    ctx.store_preallocation(id, to_device(l.get_argument()));
}

shape op_copy_to::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(2).same_type();
    return inputs.at(1);
}
argument op_copy_to::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto& s = args[0].get_shape();
    if(not s.standard() and not s.packed())
        MIGRAPHX_THROW("cuda::copy_to: host argument must be packed");
    if(s.bytes() > 0)
        check_cuda(cudaMemcpyAsync(args[1].data(), args[0].data(), s.bytes(),
                                   cudaMemcpyHostToDevice, ctx.stream()),
                   "cudaMemcpyAsync host to device");
    return args[1];
}

shape op_copy_from::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(1);
    return inputs.at(0);
}
argument op_copy_from::compute(context& ctx, const shape& out, const std::vector<argument>& args) const
{
    // page-locked, so that the copy runs at the link's speed and truly asynchronously
    argument host = ctx.pinned_host(out);
    if(out.bytes() > 0)
    {
        check_cuda(cudaMemcpyAsync(host.data(), args[0].data(), out.bytes(), cudaMemcpyDeviceToHost,
                                   ctx.stream()),
                   "cudaMemcpyAsync device to host");
        // the caller reads the host buffer right after eval(): it must be complete
        check_cuda(cudaStreamSynchronize(ctx.stream()), "cudaStreamSynchronize");
    }
    return host;
}

shape op_copy::compute_shape(const std::vector<shape>& inputs) const
{
    check_shapes{inputs, *this}.has(2).same_type().standard();
    return inputs.at(1);
}
argument op_copy::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    const auto bytes = args[0].get_shape().bytes();
    if(bytes > 0)
        check_cuda(cudaMemcpyAsync(args[1].data(), args[0].data(), bytes, cudaMemcpyDeviceToDevice,
                                   ctx.stream()),
                   "cudaMemcpyAsync device to device");
    return args[1];
}

shape op_sync_stream::compute_shape(const std::vector<shape>& inputs) const
{
    if(inputs.empty())
        return {};
    return inputs.front();
}
argument op_sync_stream::compute(context& ctx, const shape&, const std::vector<argument>& args) const
{
    check_cuda(cudaStreamSynchronize(ctx.stream()), "cudaStreamSynchronize");
    if(args.empty())
        return {};
    return args.front();
}

// ------------------------------------------------------------------ stream scheduling operators
shape op_set_stream::compute_shape(const std::vector<shape>&) const { return {}; }
argument op_set_stream::compute(context& ctx, const shape&, const std::vector<argument>&) const
{
    ctx.set_stream(stream);
    return {};
}
void op_set_stream::finalize(context& ctx, const shape&, const std::vector<shape>&) const
{
    ctx.set_stream(stream);
}

shape op_record_event::compute_shape(const std::vector<shape>&) const { return {}; }
argument op_record_event::compute(context& ctx, const shape&, const std::vector<argument>&) const
{
    check_cuda(cudaEventRecord(ctx.event(event), ctx.stream()), "cudaEventRecord");
    return {};
}
void op_record_event::finalize(context& ctx, const shape&, const std::vector<shape>&) const
{
    (void)ctx.event(event);
}

shape op_wait_event::compute_shape(const std::vector<shape>&) const { return {}; }
argument op_wait_event::compute(context& ctx, const shape&, const std::vector<argument>&) const
{
    check_cuda(cudaStreamWaitEvent(ctx.stream(), ctx.event(event), 0), "cudaStreamWaitEvent");
    return {};
}

MIGRAPHX_REGISTER_OP(op_allocate)
MIGRAPHX_REGISTER_OP(op_preallocate)
MIGRAPHX_REGISTER_OP(op_literal)
MIGRAPHX_REGISTER_OP(op_copy_to)
MIGRAPHX_REGISTER_OP(op_copy_from)
MIGRAPHX_REGISTER_OP(op_copy)
MIGRAPHX_REGISTER_OP(op_sync_stream)
MIGRAPHX_REGISTER_OP(op_graph_run)
MIGRAPHX_REGISTER_OP(op_set_stream)
MIGRAPHX_REGISTER_OP(op_record_event)
MIGRAPHX_REGISTER_OP(op_wait_event)

} // namespace cuda
} // namespace MIGRAPHX_INLINE_NS
} // namespace migraphx
