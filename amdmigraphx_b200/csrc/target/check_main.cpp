// cuda_target_check: builds MIGraphX programs of the quantized-GEMM path with the public
// module API, runs them on MIGraphX's CPU `ref` target and on the `cuda` target and compares
// the results - the same scheme as the reference's cross-target verify harness
// (test/verify/run_verify.cpp:176-259), for the programs this target supports.
//
//   cuda_target_check passes <case>          print the program after the cuda pass pipeline
//                                            (no GPU needed: finalize is not run)
//   cuda_target_check run <case> [offload]   compile + eval on ref and cuda, print one JSON line
//   cuda_target_check list
#include "programs.hpp"
#include <migraphx/register_target.hpp>
#include "../../../include/mgx_cuda.h"
#include <cuda_runtime.h>
#include <fstream>
#include <thread>

using namespace mgx_programs;

namespace {

bool g_have_device = true; // false in `passes` mode: nothing may touch a GPU

// the rows the CPU interpreter can evaluate in a few seconds (about 4 GOP at ~1 GOP/s)
std::size_t ref_rows_for(std::size_t m, std::size_t n, std::size_t k)
{
    const double per_row = 2.0 * static_cast<double>(n) * static_cast<double>(k);
    std::size_t r        = static_cast<std::size_t>(4.0e9 / per_row);
    r                    = std::max<std::size_t>(4, r / 4 * 4);
    return std::min(m, r);
}

test_case c3_point(std::size_t m, std::size_t n, std::size_t k)
{
    const unsigned seed = static_cast<unsigned>((m * 1315423911u) ^ (n * 2654435761u) ^ (k * 97u));
    return qdq_linear_sampled(m, k, n, shape::fp8e4m3fn_type, "gelu", false, seed, ref_rows_for(m, n, k));
}

test_case int8_point(std::size_t m, std::size_t n, std::size_t k)
{
    const unsigned seed = static_cast<unsigned>((m * 31u) ^ (n * 131u) ^ (k * 7u));
    auto t = qdq_linear_sampled(m, k, n, shape::int8_type, "gelu", true, seed, ref_rows_for(m, n, k));
    // ref runs the simplify_qdq-rewritten program: exact int32 quant_dot, then the same fp32
    // dequantizelinear / add / GELU operators (libm's erf against the kernel's: 1e-5)
    t.ref_simplify_qdq = true;
    return t;
}

test_case w4_point(std::size_t m, std::size_t n, std::size_t k, bool heavy_tail = false)
{
    const unsigned seed = static_cast<unsigned>((m * 17u) ^ (n * 257u) ^ (k * 3u));
    return int4_linear_sampled(m, n, k, 128, false, seed, ref_rows_for(m, n, k), heavy_tail);
}

// config 2 at its real dimensions: embedding + `layers` encoder layers on `batch` sequences of 384
test_case c2_encoder(std::size_t batch, std::size_t layers)
{
    bert_config c;
    c.batch  = batch;
    c.layers = layers;
    c.seed   = 31;
    auto bp  = bert_encoder_int8_calibrated(c, g_have_device);
    test_case t;
    t.prog          = bp.prog;
    t.params["ids"] = bert_ids(c, 99);
    // fp16 model: ref rounds (truncates) every operator's result to half, the fused epilogues
    // and the tensor cores' fp32 accumulation round once
    t.ref_simplify_qdq = true;
    t.rtol = 2e-2;
    t.atol = 1e-2;
    // quantizer flips behind the fused attention and the fp32 LayerNorm sums (see test_case): a layer
    // has four activation quantisers, and a flipped int8 value moves a few results of every layer
    // after it by a quantisation step, so the allowance grows with the depth
    t.outlier_fraction = 2e-3 * static_cast<double>(layers);
    t.outlier_atol     = 0.1;
    return t;
}

std::map<std::string, std::function<test_case()>> cases()
{
    std::map<std::string, std::function<test_case()>> big;
    // config 3: the whole fp8 sweep
    for(std::size_t m : {1, 16, 128, 1024, 4096, 8192})
        for(auto nk : std::vector<std::pair<std::size_t, std::size_t>>{{4096, 4096}, {8192, 8192}, {14336, 4096}})
            big["c3_m" + std::to_string(m) + "_n" + std::to_string(nk.first) + "_k" + std::to_string(nk.second)] =
                [=] { return c3_point(m, nk.first, nk.second); };
    // the int8 GEMM the 70 %-of-peak figure is quoted on, and the encoder's shapes at batch 8 and 1
    big["int8_8192"] = [] { return int8_point(8192, 8192, 8192); };
    big["int8_8192_raw"] = [] { return raw_quant_dot_sampled(8192, 8192, 8192, 77, ref_rows_for(8192, 8192, 8192)); };
    for(std::size_t m : {3072, 384})
    {
        big["c2_qkv_m" + std::to_string(m)]  = [=] { return int8_point(m, 768, 768); };
        big["c2_ffn1_m" + std::to_string(m)] = [=] { return int8_point(m, 3072, 768); };
        big["c2_ffn2_m" + std::to_string(m)] = [=] { return int8_point(m, 768, 3072); };
    }
    // config 4: the seven linears of a Llama-2-7B-shaped layer (four distinct shapes) at decode
    // batch 1 / 16 and prefill 512; config 5: the Llama-2-70B-shaped ones, whole and split two ways
    const std::vector<std::pair<std::size_t, std::size_t>> c4 = {{4096, 4096}, {11008, 4096}, {4096, 11008}};
    for(std::size_t m : {1, 16, 512})
        for(auto nk : c4)
            big["c4_m" + std::to_string(m) + "_n" + std::to_string(nk.first) + "_k" + std::to_string(nk.second)] =
                [=] { return w4_point(m, nk.first, nk.second); };
    const std::vector<std::pair<std::size_t, std::size_t>> c5 = {
        {8192, 8192}, {1024, 8192}, {28672, 8192}, {8192, 28672},    // q/o, k/v, gate/up, down
        {4096, 8192}, {512, 8192}, {14336, 8192}, {8192, 14336},     // the same, TP 2 (o: K split)
        {8192, 4096}};
    for(auto nk : c5)
        big["c5_m16_n" + std::to_string(nk.first) + "_k" + std::to_string(nk.second)] =
            [=] { return w4_point(16, nk.first, nk.second); };
    big["int4_heavy_tail_m1"]  = [] { return w4_point(1, 4096, 4096, true); };
    big["int4_heavy_tail_m16"] = [] { return w4_point(16, 11008, 4096, true); };
    big["int4_heavy_tail_m512"] = [] { return w4_point(512, 4096, 4096, true); };
    // group sizes whose K / group is not a power of two (K = 28672 and 11008 of the Llama shapes)
    big["int4_group_k28672"] = [] { return int4_linear(2, 64, 28672, 128, false, 41); };
    big["int4_group_k96"]    = [] { return int4_linear(3, 64, 96, 32, true, 42); };
    big["quant_dot_transposed_a"] = [] { return quant_dot_transposed_a(43); };
    // programs produced by MIGraphX's own quantisation entry points
    big["pass_quantize_int8"]  = [] { return quantized_mlp(96, 256, 320, 128, false, "ref", 51); };
    big["pass_quantize_fp8"]   = [] { return quantized_mlp(96, 256, 320, 128, true, "ref", 52); };
    big["pass_int4_weights_decode"]  = [] { return int4_weights_pass_linear(4, 512, 384, 54); };
    big["pass_int4_weights_prefill"] = [] { return int4_weights_pass_linear(160, 512, 384, 55); };
    // decoder attention with an fp16 KV cache, grouped-query heads and rotary embedding
    big["gqa_decode_small"]  = [] { return gqa_attention(2, 4, 2, 32, 1, 48, false, 61); };
    big["gqa_prompt_small"]  = [] { return gqa_attention(1, 4, 2, 32, 16, 48, false, 62); };
    big["gqa_decode_rotary_op"] = [] { return gqa_attention(2, 4, 2, 32, 1, 48, true, 63); };
    big["gqa_decode_d64_f4"]    = [] { return gqa_attention(3, 8, 2, 64, 1, 200, false, 67); };
    big["gqa_decode_d128_f2"]   = [] { return gqa_attention(2, 4, 2, 128, 1, 333, false, 68); };
    big["gqa_decode_d64_f8"]    = [] { return gqa_attention(2, 8, 1, 64, 1, 1100, false, 69); };
    big["c4_attention_decode"]  = [] { return gqa_attention(1, 32, 32, 128, 1, 2048, false, 64); };
    big["c4_attention_decode_b16"] = [] { return gqa_attention(16, 32, 32, 128, 1, 2048, false, 65); };
    big["c5_attention_decode_tp8"] = [] { return gqa_attention(16, 8, 1, 128, 1, 4096, false, 66); };
    // whole decoder layers at a decode step: RMSNorm, int4 linears, GQA with KV cache, SwiGLU
    big["llama_layer_small"]     = [] { return llama_decoder_layer(2, 256, 4, 2, 64, 512, 96, 128, 71); };
    big["llama_layer_small_d128"] = [] { return llama_decoder_layer(3, 512, 4, 4, 128, 1024, 160, 128, 72); };
    big["c4_layer_decode"]       = [] { return llama_decoder_layer(1, 4096, 32, 32, 128, 11008, 2048, 128, 73); };
    big["c5_layer_decode_tp8"]   = [] { return llama_decoder_layer(16, 8192, 8, 1, 128, 3584, 4096, 128, 74); };
    // one rank's shard of a tensor-parallel int4 MLP with cuda::all_reduce inside the program (run as
    // one process per GPU with MGX_TP_RANK / MGX_TP_WORLD / MGX_TP_ID_FILE set; a single process is
    // rank 0 of 1, whose all-reduce needs no communicator partner but still a communicator)
    big["tp_int4_mlp"] = [] {
        const char* r = std::getenv("MGX_TP_RANK");
        const char* w = std::getenv("MGX_TP_WORLD");
        return tp_int4_mlp(r != nullptr ? std::stoul(r) : 0, w != nullptr ? std::stoul(w) : 1, 16, 1024, 2048, 128, 91);
    };
    big["c2_layer"]   = [] { return c2_encoder(1, 1); };
    big["c2_layers2"] = [] { return c2_encoder(1, 2); };
    big["c2_full"]    = [] { return c2_encoder(1, 12); }; // the whole 12-layer program, one sequence
    std::map<std::string, std::function<test_case()>> small = {
        {"c1", [] { auto t = qdq_linear(256, 1024, 1024, shape::int8_type, "relu", true, 0); t.exact = true; return t; }},
        {"c1_small", [] { auto t = qdq_linear(64, 256, 96, shape::int8_type, "relu", true, 1); t.exact = true; return t; }},
        {"c1_semantic", [] { return qdq_linear(64, 256, 96, shape::int8_type, "relu", true, 1); }},
        {"int8_gelu", [] { return qdq_linear(128, 256, 320, shape::int8_type, "gelu", true, 2); }},
        {"int8_per_tensor", [] { auto t = qdq_linear(100, 128, 72, shape::int8_type, "none", false, 3); t.exact = true; return t; }},
        {"fp8_gelu", [] { return qdq_linear(128, 512, 256, shape::fp8e4m3fn_type, "gelu", false, 4); }},
        {"int4_decode", [] { return int4_linear(1, 256, 512, 128, false, 5); }},
        {"int4_batch16_zp", [] { return int4_linear(16, 128, 1024, 32, true, 6); }},
        {"int4_batch8_zp", [] { return int4_linear(8, 384, 1024, 128, true, 7); }},
        {"int4_prefill", [] { return int4_linear(96, 256, 512, 128, true, 8); }},
        {"pw_gelu_f16", [] { return pw_gelu_f16(9); }},
        {"pw_arith_f32", [] { return pw_arith_f32(10); }},
        {"pw_transcendental_f32", [] { return pw_transcendental_f32(11); }},
        {"layernorm_f32", [] { return layernorm(shape::float_type, 2, 48, 768, 12); }},
        {"layernorm_f16", [] { return layernorm(shape::half_type, 3, 20, 1000, 13); }},
        {"layernorm_f32_odd", [] { return layernorm(shape::float_type, 2, 30, 770, 26); }},
        {"layernorm_f16_odd", [] { return layernorm(shape::half_type, 2, 30, 1004, 27); }},
        {"reduce_axes", [] { return reduce_axes(24); }},
        {"softmax_f32", [] { return softmax_rows(shape::float_type, 2, 4, 56, 200, 14); }},
        {"softmax_f16", [] { return softmax_rows(shape::half_type, 1, 3, 40, 1500, 15); }},
        {"softmax_f32_long", [] { return softmax_rows(shape::float_type, 1, 1, 6, 9000, 16); }},
        {"attention_f16", [] { return attention_f16(2, 4, 64, 32, 17); }},
        {"attention_f16_d64", [] { return attention_f16(2, 3, 200, 64, 25); }},
        {"dot_f16_const", [] { return dot_f16(1, 200, 136, 264, true, 18); }},
        {"dot_f16_batched", [] { return dot_f16(3, 72, 50, 96, false, 19); }},
        {"dot_f16_odd_k", [] { return dot_f16(2, 50, 64, 197, false, 22); }},
        {"dot_f16_odd_k_const", [] { return dot_f16(1, 33, 40, 13, true, 23); }},
        {"bert_layer_int8", [] { return bert_layer_int8(2, 64, 4, 64, 1024, 20); }},
        {"embed_rope_f16", [] { return embed_rope_f16(2, 24, 40, 128, 500, 21); }},
        {"q_dq_ops", [] { return q_dq_ops(7); }},
        {"mlp_fused_q", [] { return qdq_mlp(96, 256, 320, 128, false, 9); }},
        {"mlp_two_outputs", [] { return qdq_mlp(96, 256, 320, 128, true, 10); }},
        {"raw_quant_dot", [] { return raw_quant_dot(8); }},
    };
    small.insert(big.begin(), big.end());
    return small;
}

struct cmp_result
{
    double max_abs = 0, max_rel = 0, rms_err = 0, rms_ref = 0;
    std::size_t mismatched = 0, n = 0;
};

cmp_result compare(const migraphx::argument& ref, migraphx::argument got, bool exact, double rtol,
                   double atol, const std::vector<std::size_t>* sample_rows = nullptr, bool atol_row_rms = false)
{
    cmp_result r;
    if(sample_rows != nullptr)
    {
        // ref holds rows sample_rows[i] of the full problem
        const auto& gs = got.get_shape();
        if(gs.ndim() != 2 or ref.get_shape().ndim() != 2 or ref.get_shape().lens()[0] != sample_rows->size())
        {
            r.mismatched = 1u << 30;
            return r;
        }
        got = take_rows(got, *sample_rows);
    }
    if(ref.get_shape().lens() != got.get_shape().lens() or ref.get_shape().type() != got.get_shape().type())
    {
        r.mismatched = 1u << 30;
        return r;
    }
    r.n = ref.get_shape().elements();
    if(exact)
    {
        const auto es = ref.get_shape().type_size();
        for(std::size_t i = 0; i < r.n; ++i)
            if(std::memcmp(ref.data() + i * es, got.data() + i * es, es) != 0)
                ++r.mismatched;
        return r;
    }
    std::vector<double> a(r.n), b(r.n);
    ref.visit([&](auto v) { std::size_t i = 0; for(auto x : v) a[i++] = static_cast<double>(x); });
    got.visit([&](auto v) { std::size_t i = 0; for(auto x : v) b[i++] = static_cast<double>(x); });
    const std::size_t cols = ref.get_shape().ndim() == 0 ? 1 : ref.get_shape().lens().back();
    double row_atol        = atol;
    for(std::size_t i = 0; i < r.n; ++i)
    {
        if(atol_row_rms and i % cols == 0)
        {
            double ss = 0;
            for(std::size_t j = i; j < i + cols; ++j)
                ss += a[j] * a[j];
            row_atol = atol * std::max(1.0, std::sqrt(ss / static_cast<double>(cols)));
        }
        const double d = std::fabs(a[i] - b[i]);
        r.max_abs      = std::max(r.max_abs, d);
        if(std::fabs(a[i]) > 0)
            r.max_rel = std::max(r.max_rel, d / std::fabs(a[i]));
        r.rms_err += d * d;
        r.rms_ref += a[i] * a[i];
        if(not(d <= row_atol + rtol * std::fabs(a[i])))
            ++r.mismatched;
    }
    r.rms_err = std::sqrt(r.rms_err / static_cast<double>(std::max<std::size_t>(1, r.n)));
    r.rms_ref = std::sqrt(r.rms_ref / static_cast<double>(std::max<std::size_t>(1, r.n)));
    return r;
}

// the case's acceptance rule (see test_case::outlier_fraction)
bool within(const cmp_result& c, const test_case& t)
{
    if(c.mismatched == 0)
        return true;
    return not t.exact and static_cast<double>(c.mismatched) <= t.outlier_fraction * static_cast<double>(c.n) and
           c.max_abs <= t.outlier_atol;
}

} // namespace

// One process per GPU: rank 0 makes the NCCL id and leaves it in MGX_TP_ID_FILE, the others wait for
// the file (at most a minute); every rank creates its communicator and makes it the default one,
// which is what cuda::all_reduce uses.  The device of the rank is chosen by MIGRAPHX_CUDA_DEVICE.
void join_tensor_parallel_group()
{
    const int rank  = std::stoi(std::getenv("MGX_TP_RANK"));
    const int world = std::stoi(std::getenv("MGX_TP_WORLD"));
    const std::string path = std::getenv("MGX_TP_ID_FILE");
    const char* dev = std::getenv("MIGRAPHX_CUDA_DEVICE");
    if(cudaSetDevice(dev != nullptr ? std::stoi(dev) : rank) != cudaSuccess)
        throw std::runtime_error("cudaSetDevice failed");
    std::vector<char> id(128, 0);
    if(rank == 0)
    {
        if(mgx_cuda_comm_unique_id(id.data()) != 0)
            throw std::runtime_error("mgx_cuda_comm_unique_id failed");
        std::ofstream f(path + ".tmp", std::ios::binary);
        f.write(id.data(), 128);
        f.close();
        std::rename((path + ".tmp").c_str(), path.c_str());
    }
    else
    {
        bool got = false;
        for(int i = 0; i < 600 and not got; ++i)
        {
            std::ifstream f(path, std::ios::binary);
            if(f.good() and f.read(id.data(), 128) and f.gcount() == 128)
                got = true;
            else
                std::this_thread::sleep_for(std::chrono::milliseconds(100));
        }
        if(not got)
            throw std::runtime_error("no NCCL id from rank 0 within a minute");
    }
    void* comm = nullptr;
    const int rc = mgx_cuda_comm_create(id.data(), world, rank, &comm);
    if(rc != 0)
        throw std::runtime_error("mgx_cuda_comm_create failed: " + std::to_string(rc));
    mgx_cuda_comm_set_default(comm);
}

int main(int argc, char** argv)
{
    const auto all = cases();
    if(argc < 2 or std::string(argv[1]) == "list")
    {
        for(const auto& c : all)
            std::cout << c.first << "\n";
        return 0;
    }
    const std::string mode = argv[1];
    const std::string name = argc > 2 ? argv[2] : "c1_small";
    const bool offload     = argc > 3 and std::string(argv[3]) == "offload";
    const bool prefused    = argc > 3 and std::string(argv[3]) == "prefused";
    if(all.count(name) == 0)
    {
        std::cerr << "unknown case " << name << "\n";
        return 2;
    }
    try
    {
        g_have_device = mode != "passes";
        if(mode != "passes" and std::getenv("MGX_TP_ID_FILE") != nullptr)
            join_tensor_parallel_group();
        const auto tb0 = std::chrono::steady_clock::now();
        test_case t = all.at(name)();
        const double build_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - tb0).count();
        auto cuda_t = migraphx::make_target("cuda");
        if(mode == "passes")
        {
            migraphx::program p = t.prog;
            auto ctx            = cuda_t.get_context();
            migraphx::compile_options opts;
            opts.offload_copy = offload;
            if(prefused)
                migraphx::run_passes(p, {migraphx::simplify_qdq{}, migraphx::dead_code_elimination{},
                                         migraphx::fuse_pointwise{}, migraphx::dead_code_elimination{}});
            const auto tp0 = std::chrono::steady_clock::now();
            migraphx::run_passes(p, cuda_t.get_passes(ctx, opts));
            std::cerr << "build " << build_s << " s, passes "
                      << std::chrono::duration<double>(std::chrono::steady_clock::now() - tp0).count() << " s\n";
            std::cout << p << std::endl;
            return 0;
        }
        // reference result
        migraphx::program pr = t.sampled ? t.ref_prog : t.prog;
        if(t.exact or t.ref_simplify_qdq)
            migraphx::run_passes(pr, {migraphx::simplify_qdq{}, migraphx::dead_code_elimination{}});
        pr.compile(migraphx::make_target("ref"));
        auto t0       = std::chrono::steady_clock::now();
        auto ref_out  = pr.eval(t.sampled ? t.ref_params : t.params);
        const std::vector<std::size_t>* rows = t.sampled ? &t.sample_rows : nullptr;
        double ref_s  = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        // cuda result
        migraphx::program pc = t.prog;
        if(prefused)
            migraphx::run_passes(pc, {migraphx::simplify_qdq{}, migraphx::dead_code_elimination{},
                                      migraphx::fuse_pointwise{}, migraphx::dead_code_elimination{}});
        migraphx::compile_options opts;
        opts.offload_copy = offload;
        pc.compile(cuda_t, opts);
        migraphx::parameter_map pm;
        for(const auto& ps : pc.get_parameter_shapes())
        {
            if(t.params.count(ps.first) > 0)
                pm[ps.first] = offload ? t.params.at(ps.first) : cuda_t.copy_to(t.params.at(ps.first));
            else
                pm[ps.first] = cuda_t.allocate(ps.second);
        }
        auto cuda_out = pc.eval(pm);
        // the target runs the first evals instruction by instruction and then records them as
        // a CUDA graph: time the steady state
        for(int i = 0; i < 4; ++i)
            cuda_out = pc.eval(pm);
        pc.finish();
        auto t1 = std::chrono::steady_clock::now();
        const int reps = 100;
        for(int i = 0; i < reps; ++i)
            cuda_out = pc.eval(pm);
        pc.finish();
        double cuda_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t1).count() / reps;
        bool ok = ref_out.size() == cuda_out.size();
        std::cout << "{\"case\": \"" << name << "\", \"ref_rows\": "
                  << (t.sampled ? t.sample_rows.size() : std::size_t{0}) << ", \"offload\": " << (offload ? "true" : "false")
                  << ", \"prefused\": " << (prefused ? "true" : "false") << ", \"outputs\": [";
        for(std::size_t i = 0; i < ref_out.size() and i < cuda_out.size(); ++i)
        {
            auto host = offload ? cuda_out[i] : cuda_t.copy_from(cuda_out[i]);
            auto c    = compare(ref_out[i], host, t.exact, t.rtol, t.atol, rows, t.atol_row_rms);
            ok        = ok and within(c, t);
            std::cout << (i ? ", " : "") << "{\"n\": " << c.n << ", \"mismatched\": " << c.mismatched
                      << ", \"max_abs\": " << c.max_abs << ", \"max_rel\": " << c.max_rel
                      << ", \"rms_err\": " << c.rms_err << ", \"rms_ref\": " << c.rms_ref << "}";
        }
        // the same program with other parameter buffers (the recorded graph does not apply:
        // the target has to notice, run instruction by instruction and record again)
        bool rebind_ok = true;
        if(not offload)
        {
            migraphx::parameter_map pm2;
            for(const auto& ps : pc.get_parameter_shapes())
            {
                if(t.params.count(ps.first) > 0)
                    pm2[ps.first] = cuda_t.copy_to(t.params.at(ps.first));
                else
                    pm2[ps.first] = cuda_t.allocate(ps.second);
            }
            std::vector<migraphx::argument> out2;
            for(int i = 0; i < 5; ++i)
                out2 = pc.eval(pm2);
            pc.finish();
            rebind_ok = out2.size() == ref_out.size();
            for(std::size_t i = 0; i < ref_out.size() and i < out2.size(); ++i)
                rebind_ok = rebind_ok and
                            within(compare(ref_out[i], cuda_t.copy_from(out2[i]), t.exact, t.rtol, t.atol, rows, t.atol_row_rms), t);
            ok = ok and rebind_ok;
        }
        std::cout << "], \"exact\": " << (t.exact ? "true" : "false") << ", \"ref_seconds\": " << ref_s
                  << ", \"cuda_seconds\": " << cuda_s << ", \"rebind\": " << (rebind_ok ? "true" : "false")
                  << ", \"pass\": " << (ok ? "true" : "false") << "}"
                  << std::endl;
        return ok ? 0 : 1;
    }
    catch(const std::exception& e)
    {
        std::cout << "{\"case\": \"" << name << "\", \"error\": \"" << e.what() << "\", \"pass\": false}"
                  << std::endl;
        return 3;
    }
}
