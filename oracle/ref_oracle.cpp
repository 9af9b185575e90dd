// C-ABI window onto the UNMODIFIED MIGraphX `ref` target (oracle/_ref/lib/libmigraphx.so
// + libmigraphx_ref.so, built by oracle/build_ref.py from the reference sources).
//
// TEST INFRASTRUCTURE ONLY: used to pin the numpy restatement (oracle/mgx_oracle.py), to
// generate the golden fixtures under tests/golden/ and as the timed CPU baseline.  The
// product never links or loads this library.
//
// ref_run_op() builds a one-instruction MIGraphX program out of public API calls
// (module::add_parameter / add_instruction(make_op(name, attrs)) / add_return), compiles
// it for the "ref" target (src/targets/ref/target.cpp) and evaluates it
// (program::eval, src/program.cpp:623-704).  Evaluating a chain op by op through this
// function is what the ref interpreter does for a whole program: it runs the
// instructions one after another, each on the previous one's output buffer.
#include <migraphx/program.hpp>
#include <migraphx/module.hpp>
#include <migraphx/make_op.hpp>
#include <migraphx/json.hpp>
#include <migraphx/register_target.hpp>
#include <migraphx/argument.hpp>
#include <migraphx/shape.hpp>
#include <migraphx/instruction.hpp>
#include <migraphx/stringutils.hpp>
#include <chrono>
#include <cstring>
#include <string>
#include <thread>
#include <vector>
// the program builders the product's benchmark and parity driver use (header-only, MIGraphX
// public API only): the CPU baseline evaluates the very same programs
#include "../amdmigraphx_b200/csrc/target/programs.hpp"

namespace {

thread_local std::string last_error;

bool parse_type(const std::string& name, migraphx::shape::type_t& out)
{
#define REF_ORACLE_TYPE_CASE(x, t)   \
    if(name == #x)                   \
    {                                \
        out = migraphx::shape::x;    \
        return true;                 \
    }
    MIGRAPHX_SHAPE_VISIT_TYPES(REF_ORACLE_TYPE_CASE)
#undef REF_ORACLE_TYPE_CASE
    return false;
}

} // namespace

extern "C" {

struct ref_tensor
{
    const char* type; // migraphx::shape::type_t enumerator name, e.g. "float_type"
    int ndim;
    const int64_t* lens;
    const int64_t* strides; // may be null (packed row-major)
    void* data;
};

__attribute__((visibility("default"))) const char* ref_last_error() { return last_error.c_str(); }

__attribute__((visibility("default"))) int ref_hardware_threads()
{
    return static_cast<int>(std::thread::hardware_concurrency());
}

// Runs `op_name` with JSON attributes `attrs_json` ("" or "{}" for none) on the ref
// target.  The result is copied to out->data (packed); out->type/lens must describe the
// expected result and are checked.  repeat >= 1 evaluations are made; *seconds (may be
// null) receives the wall-clock time of the fastest one (compile time excluded).
// Returns 0 on success, non-zero on failure (see ref_last_error()).
__attribute__((visibility("default"))) int ref_run_op(const char* op_name,
                                                       const char* attrs_json,
                                                       int n_inputs,
                                                       const ref_tensor* inputs,
                                                       const ref_tensor* out,
                                                       int repeat,
                                                       double* seconds)
{
    try
    {
        migraphx::program p;
        auto* mm = p.get_main_module();
        std::vector<migraphx::instruction_ref> args;
        migraphx::parameter_map params;
        for(int i = 0; i < n_inputs; ++i)
        {
            migraphx::shape::type_t t;
            if(not parse_type(inputs[i].type, t))
            {
                last_error = std::string("unknown type ") + inputs[i].type;
                return 2;
            }
            std::vector<std::size_t> lens(inputs[i].lens, inputs[i].lens + inputs[i].ndim);
            migraphx::shape s{t, lens};
            if(inputs[i].strides != nullptr)
            {
                std::vector<std::size_t> strides(inputs[i].strides,
                                                 inputs[i].strides + inputs[i].ndim);
                s = migraphx::shape{t, lens, strides};
            }
            const std::string name = "x" + std::to_string(i);
            args.push_back(mm->add_parameter(name, s));
            params[name] = migraphx::argument(s, inputs[i].data);
        }
        const bool has_attrs = attrs_json != nullptr and std::strlen(attrs_json) > 2;
        auto op = has_attrs ? migraphx::make_op(op_name, migraphx::from_json_string(attrs_json))
                            : migraphx::make_op(op_name);
        auto r  = mm->add_instruction(op, args);
        mm->add_return({r});
        p.compile(migraphx::make_target("ref"));
        double best = -1.0;
        migraphx::argument result;
        for(int it = 0; it < (repeat < 1 ? 1 : repeat); ++it)
        {
            auto t0     = std::chrono::steady_clock::now();
            auto res    = p.eval(params);
            auto t1     = std::chrono::steady_clock::now();
            double secs = std::chrono::duration<double>(t1 - t0).count();
            if(best < 0 or secs < best)
                best = secs;
            result = res.at(0);
        }
        if(seconds != nullptr)
            *seconds = best;
        migraphx::shape::type_t ot;
        if(not parse_type(out->type, ot))
        {
            last_error = std::string("unknown type ") + out->type;
            return 2;
        }
        const auto& rs = result.get_shape();
        std::vector<std::size_t> olens(out->lens, out->lens + out->ndim);
        if(rs.type() != ot or rs.lens() != olens)
        {
            last_error = "result shape mismatch: ref produced " + migraphx::to_string(rs);
            return 3;
        }
        if(not rs.standard())
        {
            // make packed: run through contiguous on ref
            migraphx::program q;
            auto* qm = q.get_main_module();
            auto x   = qm->add_parameter("x", rs);
            qm->add_return({qm->add_instruction(migraphx::make_op("contiguous"), x)});
            q.compile(migraphx::make_target("ref"));
            result = q.eval({{"x", result}}).at(0);
        }
        std::memcpy(out->data, result.data(), result.get_shape().bytes());
        return 0;
    }
    catch(const std::exception& e)
    {
        last_error = e.what();
        return 1;
    }
    catch(...)
    {
        last_error = "unknown exception";
        return 1;
    }
}


// The BERT-shaped int8 encoder program of the benchmark (amdmigraphx_b200/csrc/target/programs.hpp,
// `layers` layers, `batch` sequences of `seq` tokens, typical fixed activation scales) compiled
// for the ref target and evaluated `warmup` (untimed) + `repeat` times.  *seconds: the sum over the
// `repeat` timed eval() calls;
// *quant_ops: 2*M*N*K summed over its QDQ linears.  simplify_qdq is applied first, so that the
// linears run as quant_dot (ref's own integer GEMM) like on every GPU target.
__attribute__((visibility("default"))) int ref_time_bert(int64_t batch, int64_t seq, int64_t layers,
                                                          int64_t hidden, int64_t heads, int64_t ffn,
                                                          int64_t vocab, int warmup, int repeat,
                                                          double* seconds, double* quant_ops)
{
    try
    {
        mgx_programs::bert_config c;
        c.batch  = static_cast<std::size_t>(batch);
        c.seq    = static_cast<std::size_t>(seq);
        c.layers = static_cast<std::size_t>(layers);
        c.hidden = static_cast<std::size_t>(hidden);
        c.heads  = static_cast<std::size_t>(heads);
        c.ffn    = static_cast<std::size_t>(ffn);
        c.vocab  = static_cast<std::size_t>(vocab);
        auto bp  = mgx_programs::bert_encoder_int8_calibrated(c, false);
        migraphx::run_passes(bp.prog, {migraphx::simplify_qdq{}, migraphx::dead_code_elimination{}});
        bp.prog.compile(migraphx::make_target("ref"));
        migraphx::parameter_map pm;
        pm["ids"]   = mgx_programs::bert_ids(c, 7);
        for(int it = 0; it < warmup; ++it)
            (void)bp.prog.eval(pm);
        auto t0 = std::chrono::steady_clock::now();
        for(int it = 0; it < (repeat < 1 ? 1 : repeat); ++it)
            (void)bp.prog.eval(pm);
        if(seconds != nullptr)
            *seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if(quant_ops != nullptr)
            *quant_ops = bp.quant_ops;
        return 0;
    }
    catch(const std::exception& e)
    {
        last_error = e.what();
        return 1;
    }
}

} // extern "C"
