// The plug-in route a MIGraphX application takes: this program links libmigraphx.so ONLY.
// make_target("cuda") makes MIGraphX dlopen libmigraphx_cuda.so.<so-major> (src/register_target.cpp:
// 56-80), whose static initialiser registers the target (MIGRAPHX_REGISTER_TARGET,
// src/include/migraphx/register_target.hpp:53-73) and its operators; the same call with "ref" loads
// MIGraphX's CPU interpreter as the checker.  Three programs of the quantized path are compiled,
// evaluated on both and compared; one JSON line per program, exit code 0 when all agree.
#include "programs.hpp"
#include <migraphx/register_target.hpp>
#include <migraphx/verify.hpp>
#include <iostream>

namespace {

bool agree(const migraphx::argument& a, const migraphx::argument& b, double rtol, double atol, double& worst)
{
    bool ok = a.get_shape().lens() == b.get_shape().lens() and a.get_shape().type() == b.get_shape().type();
    if(not ok)
        return false;
    a.visit([&](auto va) {
        b.visit([&](auto vb) {
            for(std::size_t i = 0; i < va.size(); ++i)
            {
                const double x = static_cast<double>(va[i]), y = static_cast<double>(vb[i]);
                const double d = std::abs(x - y);
                worst          = std::max(worst, d);
                if(not(d <= atol + rtol * std::abs(y)))
                    ok = false;
            }
        });
    });
    return ok;
}

} // namespace

int main()
{
    using namespace mgx_programs;
    int failures = 0;
    try
    {
        const auto before = migraphx::get_targets();
        auto cuda_t       = migraphx::make_target("cuda");
        auto ref_t        = migraphx::make_target("ref");
        std::cout << "{\"targets_before\": " << before.size() << ", \"cuda\": \"" << cuda_t.name() << "\", \"ref\": \""
                  << ref_t.name() << "\"}" << std::endl;
        std::vector<std::pair<std::string, test_case>> cases;
        cases.emplace_back("int8_relu", qdq_linear(64, 256, 96, shape::int8_type, "relu", true, 1));
        cases.emplace_back("fp8_gelu", qdq_linear(48, 128, 64, shape::fp8e4m3fn_type, "gelu", true, 2));
        cases.emplace_back("int4", int4_linear(4, 256, 512, 128, true, 3));
        for(auto& [name, t] : cases)
        {
            migraphx::program pc = t.prog, pr = t.prog;
            migraphx::compile_options opts;
            opts.offload_copy = true;
            pc.compile(cuda_t, opts);
            pr.compile(ref_t);
            auto rc = pc.eval(t.params);
            auto rr = pr.eval(t.params);
            double worst = 0;
            bool ok      = rc.size() == rr.size();
            for(std::size_t i = 0; ok and i < rc.size(); ++i)
                ok = agree(rc[i], rr[i], t.rtol, t.atol, worst);
            std::cout << "{\"case\": \"" << name << "\", \"max_abs\": " << worst << ", \"pass\": " << (ok ? "true" : "false")
                      << "}" << std::endl;
            failures += ok ? 0 : 1;
        }
    }
    catch(const std::exception& e)
    {
        std::cout << "{\"error\": \"" << e.what() << "\", \"pass\": false}" << std::endl;
        return 2;
    }
    return failures == 0 ? 0 : 1;
}
