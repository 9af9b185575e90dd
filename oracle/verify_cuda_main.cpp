// Entry point of the reference's own cross-target verify harness (test/verify/run_verify.cpp,
// verify_program.cpp, auto_print.cpp, compiled where they lie by oracle/build_verify.py) with the
// `cuda` target linked in: run_verify::verify picks up every registered target
// (test/verify/run_verify.cpp:186-199), compiles each verify program for it, round-trips the
// compiled program through save / load (:60-67, :105) and compares with the ref target.
// What this file adds is the per-target validation the reference registers for its own GPU
// target in test/verify/main.cpp:36-64: no stream races, and a dry run leaves the context shared.
//
// TEST INFRASTRUCTURE: links the plug-in (the thing under test) and MIGraphX's ref target (the
// checker).
#include "run_verify.hpp"
#include "test.hpp"
#include <migraphx/analyze_streams.hpp>
#include <migraphx/instruction.hpp>
#include <migraphx/iterator_for.hpp>
#include <migraphx/ranges.hpp>
#include <iostream>
#include <unordered_map>

namespace {

// the stream model of the cuda target's scheduling instructions
struct cuda_stream_model
{
    std::size_t max_stream = 0;
    std::unordered_map<migraphx::instruction_ref, std::size_t> ins2stream{};
    std::size_t get_nstream() const { return max_stream + 1; }
    std::size_t get_stream(migraphx::instruction_ref ins) const { return ins2stream.at(ins); }
    std::size_t get_event_id(migraphx::instruction_ref ins) const
    {
        return ins->get_operator().to_value()["event"].to<std::size_t>();
    }
    bool has_stream(migraphx::instruction_ref ins) const { return ins2stream.count(ins) > 0; }
    bool is_record(migraphx::instruction_ref ins) const { return ins->name() == "cuda::record_event"; }
    bool is_wait(migraphx::instruction_ref ins) const { return ins->name() == "cuda::wait_event"; }
};

void validate_cuda(const migraphx::program& p, const migraphx::parameter_map& m)
{
    const auto* mm = p.get_main_module();
    cuda_stream_model sm;
    std::size_t stream = 0;
    for(auto ins : migraphx::iterator_for(*mm))
    {
        if(ins->name() == "cuda::set_stream")
        {
            stream        = ins->get_operator().to_value()["stream"].to<std::size_t>();
            sm.max_stream = std::max(stream, sm.max_stream);
        }
        if(ins->get_operator().is_context_free())
            continue;
        if(migraphx::contains({"cuda::preallocate", "cuda::literal", "@param"}, ins->name()))
            continue;
        sm.ins2stream[ins] = stream;
    }
    for(auto&& race : migraphx::analyze_streams(*mm, sm))
    {
        std::cout << "FAILED: race condition detected for: ";
        mm->debug_print(race.ins);
        std::cout << "should happen after: ";
        mm->debug_print(race.before);
        EXPECT(false);
    }
    // a dry run must not replace the program's context
    auto ctx = p.get_context();
    EXPECT(is_shared(ctx, p.get_context()));
    p.dry_run(m);
    EXPECT(is_shared(ctx, p.get_context()));
}

} // namespace

int main(int argc, const char* argv[])
{
    run_verify rv;
    rv.add_validation_for("cuda", &validate_cuda);
    rv.run(argc, argv);
}
