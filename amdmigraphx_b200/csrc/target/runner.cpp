// libmgx_cuda_runner.so: a small C ABI over "build a MIGraphX program of this repository's
// workloads, compile it for the `cuda` target, evaluate it" - the calls a user of MIGraphX makes
// (make_target("cuda") -> program::compile -> program::eval, src/program.cpp:327-353, 623-704),
// packaged so that a benchmark written in another language can time them.  Nothing here runs
// kernels by itself: every launch comes out of program::eval through the plug-in.
//
// Device timing: CUDA events recorded on the compiled program's own stream (the context's
// queue) around a run of eval() calls; host timing: steady_clock around the same run.
#include "programs.hpp"
#include "cuda_target.hpp"
#include <migraphx/context.hpp>
#include <migraphx/iterator_for.hpp>
#include <cuda_runtime.h>
#include <sstream>

using namespace mgx_programs;

namespace {

thread_local std::string g_error;

struct runner
{
    migraphx::program prog;
    migraphx::target tgt = migraphx::make_target("cuda");
    migraphx::parameter_map params;
    std::vector<migraphx::argument> last_out;
    std::shared_ptr<void> pinned_ids; // offload mode: the caller-side input buffer
    std::size_t ids_bytes = 0;
    bool offload          = false;
    double quant_ops      = 0;
    std::size_t tokens    = 0;
    std::map<std::string, int> op_counts;
    int launches = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    ~runner()
    {
        if(e0 != nullptr)
            (void)cudaEventDestroy(e0);
        if(e1 != nullptr)
            (void)cudaEventDestroy(e1);
    }
};

bool launching(const std::string& n)
{
    static const char* names[] = {"cuda::quantizelinear", "cuda::dequantizelinear", "cuda::qgemm", "cuda::w4a16",
                                  "cuda::unpack_int4",    "cuda::pack_int4",        "cuda::copy",  "cuda::pointwise",
                                  "cuda::reduce",         "cuda::softmax",          "cuda::gather", "cuda::concat",
                                  "cuda::pad_rows",       "cuda::layernorm",        "cuda::attention",
                                  "cuda::concat_past_present", "cuda::gqa_rotary_embedding",
                                  "cuda::gqa_decode_attention", "cuda::rotary_embedding"};
    for(auto* s : names)
        if(n == s)
            return true;
    return false;
}

template <class F>
int guarded(F f)
{
    try
    {
        return f();
    }
    catch(const std::exception& e)
    {
        g_error = e.what();
        return -1;
    }
}

} // namespace

extern "C" {

#define MGX_RUNNER_API __attribute__((visibility("default")))

struct mgx_bert_desc
{
    int64_t batch, seq, layers, hidden, heads, ffn, vocab;
    uint32_t seed;
    int32_t offload_copy; // 1: eval() takes host arguments and returns host results
    int32_t fixed_scales; // 1: typical fixed activation scales instead of a calibration run
    int32_t reserved;
};

MGX_RUNNER_API const char* mgx_runner_last_error() { return g_error.c_str(); }

// Builds the BERT-shaped int8 encoder program (calibrating its activation scales with one run of
// the un-quantised fp16 program on the device), compiles it for `cuda`, and prepares parameters.
MGX_RUNNER_API int mgx_runner_create_bert(const mgx_bert_desc* d, void** out)
{
    return guarded([&] {
        auto r = std::make_unique<runner>();
        bert_config c;
        c.batch  = static_cast<std::size_t>(d->batch);
        c.seq    = static_cast<std::size_t>(d->seq);
        c.layers = static_cast<std::size_t>(d->layers);
        c.hidden = static_cast<std::size_t>(d->hidden);
        c.heads  = static_cast<std::size_t>(d->heads);
        c.ffn    = static_cast<std::size_t>(d->ffn);
        c.vocab  = static_cast<std::size_t>(d->vocab);
        c.seed   = d->seed;
        // programs of one configuration and seed share their activation scales: calibrate once
        static std::map<std::string, std::vector<float>> scale_cache;
        std::ostringstream key;
        key << c.batch << "/" << c.seq << "/" << c.layers << "/" << c.hidden << "/" << c.heads << "/" << c.ffn << "/"
            << c.vocab << "/" << c.seed;
        auto cached = scale_cache.find(key.str());
        if(cached != scale_cache.end())
            c.act_scales = cached->second;
        bert_program bp;
        if(d->fixed_scales != 0)
            bp = bert_encoder_int8_calibrated(c, false);
        else if(c.calibrate())
        {
            bp = bert_encoder_int8_calibrated(c, true, &c.act_scales);
            scale_cache[key.str()] = c.act_scales;
        }
        else
            bp = bert_encoder_int8(c);
        r->prog      = std::move(bp.prog);
        r->quant_ops = bp.quant_ops;
        r->tokens    = bp.tokens;
        r->offload   = d->offload_copy != 0;
        migraphx::compile_options opts;
        opts.offload_copy = r->offload;
        r->prog.compile(r->tgt, opts);
        // every module: the compiled body sits in a submodule behind cuda::graph_run
        for(auto* mod : r->prog.get_modules())
            for(auto ins : migraphx::iterator_for(*mod))
            {
                ++r->op_counts[ins->name()];
                if(launching(ins->name()))
                    ++r->launches;
            }
        auto& ctx = migraphx::any_cast<migraphx::cuda::context>(r->prog.get_context());
        r->stream = ctx.stream();
        if(cudaEventCreate(&r->e0) != cudaSuccess or cudaEventCreate(&r->e1) != cudaSuccess)
            MIGRAPHX_THROW("cudaEventCreate failed");
        for(const auto& ps : r->prog.get_parameter_shapes())
        {
            if(ps.first == "ids")
            {
                r->ids_bytes = ps.second.bytes();
                if(r->offload)
                {
                    void* p = nullptr;
                    if(cudaHostAlloc(&p, r->ids_bytes, cudaHostAllocDefault) != cudaSuccess)
                        MIGRAPHX_THROW("cudaHostAlloc failed");
                    r->pinned_ids = std::shared_ptr<void>(p, [](void* q) { (void)cudaFreeHost(q); });
                    r->params[ps.first] = migraphx::argument{ps.second, r->pinned_ids};
                }
                else
                    r->params[ps.first] = r->tgt.allocate(ps.second);
            }
            else
                r->params[ps.first] = r->tgt.allocate(ps.second);
        }
        *out = r.release();
        return 0;
    });
}

// One Llama-shaped decoder layer at a decode step (programs.hpp: llama_decoder_layer) compiled for
// the cuda target with device-resident parameters (activations, KV caches, past lengths, filled with
// the case's seeded values).  mgx_runner_eval / _launches / _op_counts work on the handle.
struct mgx_llama_desc
{
    int64_t batch, hidden, heads, kv_heads, head, ffn, cache, group;
    uint32_t seed;
    int32_t reserved;
};

MGX_RUNNER_API int mgx_runner_create_llama_layer(const mgx_llama_desc* d, void** out)
{
    return guarded([&] {
        if(d == nullptr or out == nullptr)
            MIGRAPHX_THROW("mgx_runner_create_llama_layer: null argument");
        auto r = std::make_unique<runner>();
        auto t = llama_decoder_layer(static_cast<std::size_t>(d->batch), static_cast<std::size_t>(d->hidden),
                                     static_cast<std::size_t>(d->heads), static_cast<std::size_t>(d->kv_heads),
                                     static_cast<std::size_t>(d->head), static_cast<std::size_t>(d->ffn),
                                     static_cast<std::size_t>(d->cache), static_cast<std::size_t>(d->group), d->seed);
        r->prog   = std::move(t.prog);
        r->tokens = static_cast<std::size_t>(d->batch);
        r->prog.compile(r->tgt, migraphx::compile_options{});
        for(auto* mod : r->prog.get_modules())
            for(auto ins : migraphx::iterator_for(*mod))
            {
                ++r->op_counts[ins->name()];
                if(launching(ins->name()))
                    ++r->launches;
            }
        auto& ctx = migraphx::any_cast<migraphx::cuda::context>(r->prog.get_context());
        r->stream = ctx.stream();
        if(cudaEventCreate(&r->e0) != cudaSuccess or cudaEventCreate(&r->e1) != cudaSuccess)
            MIGRAPHX_THROW("cudaEventCreate failed");
        for(const auto& ps : r->prog.get_parameter_shapes())
        {
            auto it = t.params.find(ps.first);
            r->params[ps.first] = it != t.params.end() ? r->tgt.copy_to(it->second) : r->tgt.allocate(ps.second);
        }
        *out = r.release();
        return 0;
    });
}

MGX_RUNNER_API void mgx_runner_destroy(void* h) { delete static_cast<runner*>(h); }

// Token ids of the next eval()s.  Device-resident mode: copied to the device now (outside any
// timed region); offload mode: copied into the page-locked host buffer eval() reads.
MGX_RUNNER_API int mgx_runner_set_ids(void* h, const int32_t* ids, size_t count)
{
    return guarded([&] {
        auto* r = static_cast<runner*>(h);
        if(count * sizeof(int32_t) != r->ids_bytes)
            MIGRAPHX_THROW("mgx_runner_set_ids: wrong number of ids");
        auto& a = r->params.at("ids");
        if(r->offload)
            std::memcpy(a.data(), ids, r->ids_bytes);
        else if(cudaMemcpy(a.data(), ids, r->ids_bytes, cudaMemcpyHostToDevice) != cudaSuccess)
            MIGRAPHX_THROW("cudaMemcpy failed");
        return 0;
    });
}

// `steps` eval() calls, rotating over the n programs in hs (so that consecutive steps do not find
// their weights in L2).  device_ms: CUDA events around the run on the programs' streams (each
// eval() ends synchronised, so the run is serial on the device); wall_ms: host clock.
MGX_RUNNER_API int mgx_runner_eval(void* const* hs, int n, int steps, float* device_ms, double* wall_ms)
{
    return guarded([&] {
        if(n <= 0 or steps <= 0)
            MIGRAPHX_THROW("mgx_runner_eval: nothing to run");
        auto* first = static_cast<runner*>(hs[0]);
        auto* last  = static_cast<runner*>(hs[(steps - 1) % n]);
        if(cudaEventRecord(first->e0, first->stream) != cudaSuccess)
            MIGRAPHX_THROW("cudaEventRecord failed");
        const auto t0 = std::chrono::steady_clock::now();
        for(int i = 0; i < steps; ++i)
        {
            auto* r     = static_cast<runner*>(hs[i % n]);
            r->last_out = r->prog.eval(r->params);
        }
        const auto t1 = std::chrono::steady_clock::now();
        if(cudaEventRecord(last->e1, last->stream) != cudaSuccess or cudaEventSynchronize(last->e1) != cudaSuccess)
            MIGRAPHX_THROW("cudaEventRecord failed");
        float ms = 0;
        if(cudaEventElapsedTime(&ms, first->e0, last->e1) != cudaSuccess)
            MIGRAPHX_THROW("cudaEventElapsedTime failed");
        if(device_ms != nullptr)
            *device_ms = ms;
        if(wall_ms != nullptr)
            *wall_ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
        last->prog.finish(); // also reads the kernels' status word
        return 0;
    });
}

// The first result of the last eval(), as bytes on the host.
MGX_RUNNER_API int mgx_runner_read_output(void* h, void* host, size_t bytes)
{
    return guarded([&] {
        auto* r = static_cast<runner*>(h);
        if(r->last_out.empty())
            MIGRAPHX_THROW("mgx_runner_read_output: no eval() yet");
        const auto& o = r->last_out.front();
        if(o.get_shape().bytes() != bytes)
            MIGRAPHX_THROW("mgx_runner_read_output: size mismatch");
        if(r->offload)
            std::memcpy(host, o.data(), bytes);
        else if(cudaMemcpy(host, o.data(), bytes, cudaMemcpyDeviceToHost) != cudaSuccess)
            MIGRAPHX_THROW("cudaMemcpy failed");
        return 0;
    });
}

MGX_RUNNER_API double mgx_runner_quant_ops(void* h) { return static_cast<runner*>(h)->quant_ops; }
MGX_RUNNER_API int64_t mgx_runner_tokens(void* h) { return static_cast<int64_t>(static_cast<runner*>(h)->tokens); }
MGX_RUNNER_API int mgx_runner_launches(void* h) { return static_cast<runner*>(h)->launches; }
MGX_RUNNER_API size_t mgx_runner_output_bytes(void* h)
{
    return static_cast<runner*>(h)->prog.get_output_shapes().front().bytes();
}

// {"cuda::qgemm": 72, ...}: instructions of the compiled program by operator name.
MGX_RUNNER_API int mgx_runner_op_counts(void* h, char* buf, size_t len)
{
    auto* r = static_cast<runner*>(h);
    std::ostringstream os;
    os << "{";
    bool sep = false;
    for(const auto& kv : r->op_counts)
    {
        os << (sep ? ", " : "") << "\"" << kv.first << "\": " << kv.second;
        sep = true;
    }
    os << "}";
    const auto s = os.str();
    if(s.size() + 1 > len)
        return -1;
    std::memcpy(buf, s.c_str(), s.size() + 1);
    return 0;
}

} // extern "C"
