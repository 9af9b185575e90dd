// cuda::target: the pass pipeline, the allocation / schedule models and the registration
// with MIGraphX (MIGRAPHX_REGISTER_TARGET, src/include/migraphx/register_target.hpp:53-73).
// The pipeline is the short counterpart of the HIP target's
// (src/targets/gpu/target.cpp:118-239): target-independent passes are MIGraphX's own,
// unchanged; the cuda:: passes are the ones of this library.
#include "cuda_ops.hpp"
#include <migraphx/register_target.hpp>
#include <migraphx/adjust_allocation.hpp>
#include <migraphx/check_context.hpp>
#include <migraphx/dead_code_elimination.hpp>
#include <migraphx/eliminate_allocation.hpp>
#include <migraphx/eliminate_common_subexpression.hpp>
#include <migraphx/eliminate_identity.hpp>
#include <migraphx/env.hpp>
#include <migraphx/instruction.hpp>
#include <migraphx/make_op.hpp>
#include <migraphx/memory_coloring.hpp>
#include <migraphx/module.hpp>
#include <migraphx/normalize_ops.hpp>
#include <migraphx/preallocate_param.hpp>
#include <migraphx/replace_allocate.hpp>
#include <migraphx/schedule.hpp>
#include <migraphx/simplify_qdq.hpp>
#include <migraphx/stringutils.hpp>

namespace migraphx {
inline namespace MIGRAPHX_INLINE_NS {
namespace cuda {

MIGRAPHX_DECLARE_ENV_VAR(MIGRAPHX_CUDA_DEVICE)
MIGRAPHX_DECLARE_ENV_VAR(MIGRAPHX_CUDA_NSTREAMS)

// ------------------------------------------------------------------ models
operation allocation_model::allocate(const shape& s) const
{
    return make_op(name(), {{"shape", to_value(s)}});
}

operation allocation_model::preallocate(const shape& s, const std::string& id) const
{
    return make_op("cuda::preallocate", {{"shape", to_value(s)}, {"id", id}});
}

void schedule_model::sched(module& m, instruction_ref ins, std::size_t n) const
{
    auto last = std::prev(ins);
    if(last != m.end() and last->name() == "cuda::set_stream")
    {
        auto v = last->get_operator().to_value();
        if(v.at("stream").to<std::size_t>() == n)
            return;
    }
    m.insert_instruction(ins, make_op("cuda::set_stream", {{"stream", n}}));
}

void schedule_model::wait(module& m, instruction_ref ins, std::size_t wait_id) const
{
    m.insert_instruction(ins, make_op("cuda::wait_event", {{"event", wait_id}}));
}

void schedule_model::record(module& m, instruction_ref ins, std::size_t wait_id) const
{
    m.insert_instruction(std::next(ins), make_op("cuda::record_event", {{"event", wait_id}}));
}

std::size_t schedule_model::weight(const operation& op) const
{
    const auto n = op.name();
    if(n == "cuda::qgemm" or n == "cuda::w4a16")
        return 8;
    if(starts_with(n, "cuda::") and not contains(n, "allocate") and not contains(n, "literal"))
        return 2;
    return 0;
}

// ------------------------------------------------------------------ target
std::string target::name() const { return "cuda"; }

migraphx::context target::get_context() const
{
    int dev = 0;
    if(not string_value_of(MIGRAPHX_CUDA_DEVICE{}).empty())
        dev = static_cast<int>(value_of(MIGRAPHX_CUDA_DEVICE{}, 0));
    else
        (void)cudaGetDevice(&dev);
    const std::size_t nstreams = value_of(MIGRAPHX_CUDA_NSTREAMS{}, 1);
    return context{dev, nstreams};
}

std::vector<pass> target::get_passes(migraphx::context& gctx, const compile_options& options) const
{
    auto& ctx = any_cast<context>(gctx);
    return {
        normalize_ops{},
        dead_code_elimination{},
        eliminate_identity{},
        dead_code_elimination{},
        // Q/DQ pairs around dot become quant_dot + dequantizelinear (MIGraphX's own pass)
        simplify_qdq{},
        dead_code_elimination{},
        eliminate_common_subexpression{},
        dead_code_elimination{},
        // programs that already went through fuse_pointwise: open the sub-modules again
        inline_pointwise{},
        dead_code_elimination{},
        lowering{&ctx, options.offload_copy},
        dead_code_elimination{},
        fuse_cuda_pointwise{},
        dead_code_elimination{},
        replace_allocate{allocation_model{}, options.offload_copy},
        dead_code_elimination{},
        adjust_allocation{allocation_model{}},
        dead_code_elimination{},
        write_literals{},
        schedule{schedule_model{ctx.nstreams()}, ctx.nstreams() > 1},
        memory_coloring{"cuda::allocate"},
        sync_device{},
        preallocate_param{"scratch", allocation_model{}},
        dead_code_elimination{},
        eliminate_allocation{"cuda::allocate"},
        check_context<context>{},
        dead_code_elimination{},
        insert_graph_ops{&ctx, options.offload_copy},
    };
}

argument target::copy_to(const argument& arg) const { return to_device(arg); }
argument target::copy_from(const argument& arg) const { return from_device(arg); }
argument target::allocate(const shape& s) const { return allocate_device(s); }

MIGRAPHX_REGISTER_TARGET(target);

} // namespace cuda
} // namespace MIGRAPHX_INLINE_NS
} // namespace migraphx
