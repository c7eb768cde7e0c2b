// Times the UNMODIFIED reference engine (Cyxuan0311/Forge) on its CUDA backend, through its own public API
// and stock code path: EngineRegistry::create("llama") -> InferenceEngine::forward(ids, start_pos), the call
// that its Generator, its CLI benchmark (src/cli/forge_cli.cpp:242-321) and its Python `ctx.forward` make,
// and Sampler::sample for the greedy token (src/inference/generator.cpp:84-99).  Nothing of this project's
// engine is linked here.  Built by baseline/build_reference.py; run by `bench.py --impl reference`.
//
//   ref_bench LAYERS HIDDEN HEADS KV_HEADS HEAD_DIM INTERMEDIATE VOCAB THETA EPS MAX_SEQ PROMPT_LEN PREFILL_TOKENS STEPS WARMUP
//
// Weights are FP32 (the reference computes in FP32; it has no bf16 path), drawn N(0, 0.02) on the host with a
// counter-based generator and put into Model::weights() under the reference's canonical names, on the CUDA
// device, as its loaders would leave them.  One sequence at a time: the reference's batched CUDA path copies
// device memory with host memcpy (src/inference/engines/transformer_engine.cpp:236-240) and is not run.
// Prints one line of JSON numbers on stdout.
#include <cuda_runtime.h>

#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <string>
#include <vector>

#include "forge/arch_registry.h"
#include "forge/context.h"
#include "forge/engine.h"
#include "forge/engines/transformer_engine.h"
#include "forge/logger.h"
#include "forge/model.h"
#include "forge/sampler.h"

using namespace forge;
using clk = std::chrono::high_resolution_clock;

static inline uint64_t mix(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// N(0, std) by the sum of four uniforms (variance 4/12, scaled): cheap, and the timing does not depend on it
static TensorPtr random_tensor(std::vector<int64_t> shape, uint64_t tag, float std_, float mean = 0.f) {
    auto t = std::make_shared<Tensor>(DataType::FP32, shape, DeviceType::CPU);
    float* p = static_cast<float*>(t->data());
    const int64_t n = t->numel();
    const float k = std_ * std::sqrt(3.0f);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const uint64_t r = mix(tag * 0x100000001B3ull + (uint64_t)i);
        const float u = ((r & 0xFFFF) + ((r >> 16) & 0xFFFF) + ((r >> 32) & 0xFFFF) + ((r >> 48) & 0xFFFF)) * (1.0f / 65535.0f) - 2.0f;
        p[i] = mean + u * k;
    }
    t->to_device(DeviceType::CUDA);
    return t;
}

static TensorPtr ids_on_device(const std::vector<int32_t>& v) {
    auto t = std::make_shared<Tensor>(DataType::INT32, std::vector<int64_t>{(int64_t)v.size()}, DeviceType::CPU);
    std::memcpy(t->data(), v.data(), v.size() * sizeof(int32_t));
    t->to_device(DeviceType::CUDA);
    return t;
}

int main(int argc, char** argv) {
    (void)forge::_arch_registrations_linked;
    if (argc < 15) {
        std::fprintf(stderr, "usage: ref_bench L H NH NKV HD I V theta eps max_seq prompt_len prefill_tokens steps warmup\n");
        return 2;
    }
    int a = 1;
    const int L = std::atoi(argv[a++]), H = std::atoi(argv[a++]), NH = std::atoi(argv[a++]), NKV = std::atoi(argv[a++]);
    const int HD = std::atoi(argv[a++]), I = std::atoi(argv[a++]), V = std::atoi(argv[a++]);
    const float theta = std::atof(argv[a++]), eps = std::atof(argv[a++]);
    const int max_seq = std::atoi(argv[a++]), prompt_len = std::atoi(argv[a++]), prefill_tokens = std::atoi(argv[a++]);
    const int steps = std::atoi(argv[a++]), warmup = std::atoi(argv[a++]);
    Logger::instance().set_level(static_cast<LogLevel>(0));

    ModelConfig cfg;
    cfg.arch_type = "llama";
    cfg.vocab_size = V; cfg.hidden_dim = H; cfg.intermediate_dim = I; cfg.num_layers = L;
    cfg.num_heads = NH; cfg.num_kv_heads = NKV; cfg.head_dim = HD;
    cfg.rope_theta = theta; cfg.rms_norm_eps = eps; cfg.tie_embeddings = false;
    cfg.max_seq_len = max_seq;

    Model m;
    m.set_config(cfg);
    m.set_device(DeviceType::CUDA);
    auto& ws = m.weights();
    uint64_t tag = 1;
    ws.set("token_embedding", random_tensor({V, H}, tag++, 0.02f));
    ws.set("output_norm", random_tensor({H}, tag++, 0.f, 1.f));
    ws.set("output_weight", random_tensor({V, H}, tag++, 0.02f));
    for (int l = 0; l < L; ++l) {
        const std::string p = "layers." + std::to_string(l) + ".";
        ws.set(p + "attn_norm", random_tensor({H}, tag++, 0.f, 1.f));
        ws.set(p + "wq", random_tensor({NH * HD, H}, tag++, 0.02f));
        ws.set(p + "wk", random_tensor({NKV * HD, H}, tag++, 0.02f));
        ws.set(p + "wv", random_tensor({NKV * HD, H}, tag++, 0.02f));
        ws.set(p + "wo", random_tensor({H, NH * HD}, tag++, 0.02f));
        ws.set(p + "ffn_norm", random_tensor({H}, tag++, 0.f, 1.f));
        ws.set(p + "gate_proj", random_tensor({I, H}, tag++, 0.02f));
        ws.set(p + "up_proj", random_tensor({I, H}, tag++, 0.02f));
        ws.set(p + "down_proj", random_tensor({H, I}, tag++, 0.02f));
    }

    ContextParams params;
    params.device = DeviceType::CUDA;
    params.gpu_layers = -1;
    params.max_seq_len = max_seq;
    InferenceContext ctx(m, params);
    auto engine = EngineRegistry::instance().create("llama", m, ctx);
    if (!engine) { std::fprintf(stderr, "no engine registered for llama\n"); return 4; }
    if (auto* te = dynamic_cast<TransformerEngine*>(engine.get())) te->set_gpu_layers(-1);
    InferenceEngine* e = engine.get();

    std::vector<int32_t> prompt(prefill_tokens > prompt_len ? prefill_tokens : prompt_len);
    for (size_t i = 0; i < prompt.size(); ++i) prompt[i] = (int32_t)(mix(777 + i) % (uint64_t)V);
    auto sync = [] {
        cudaError_t err = cudaDeviceSynchronize();
        if (err != cudaSuccess) { std::fprintf(stderr, "CUDA error: %s\n", cudaGetErrorString(err)); std::exit(5); }
    };

    // ---- prefill: PREFILL_TOKENS in one forward, from an empty cache (as report/base.py:112-133 measures it)
    double prefill_ms = 0;
    {
        std::vector<int32_t> pf(prompt.begin(), prompt.begin() + prefill_tokens);
        for (int i = 0; i < 2; ++i) { e->reset(); auto lg = e->forward(ids_on_device(pf), 0); sync(); }
        const int reps = 3;
        auto t0 = clk::now();
        for (int i = 0; i < reps; ++i) { e->reset(); auto lg = e->forward(ids_on_device(pf), 0); }
        sync();
        prefill_ms = std::chrono::duration<double, std::milli>(clk::now() - t0).count() / reps;
    }

    // ---- decode: a PROMPT_LEN-token prompt, then single tokens.  Device-timed: forward only, the input token
    // already on the device.  End to end: every step copies its token to the device, runs forward, takes the
    // greedy token with the reference's Sampler (device argmax + 4-byte read back) and feeds it to the next step.
    e->reset();
    std::vector<int32_t> pp(prompt.begin(), prompt.begin() + prompt_len);
    { auto lg = e->forward(ids_on_device(pp), 0); sync(); }
    int64_t pos = prompt_len;
    auto one = ids_on_device({1});
    for (int i = 0; i < warmup; ++i) { auto lg = e->forward(one, pos++); }
    sync();
    cudaEvent_t ev0, ev1;
    cudaEventCreate(&ev0); cudaEventCreate(&ev1);
    cudaEventRecord(ev0, 0);
    for (int i = 0; i < steps; ++i) { auto lg = e->forward(one, pos++); }
    cudaEventRecord(ev1, 0);
    sync();
    float dev_ms = 0;
    cudaEventElapsedTime(&dev_ms, ev0, ev1);

    SamplerConfig sc;
    sc.do_sample = false;
    Sampler sampler(sc);
    int32_t tok = 1;
    for (int i = 0; i < warmup; ++i) { auto lg = e->forward(ids_on_device({tok}), pos++); tok = sampler.sample(lg, pos); }
    sync();
    auto t0 = clk::now();
    for (int i = 0; i < steps; ++i) { auto lg = e->forward(ids_on_device({tok}), pos++); tok = sampler.sample(lg, pos); }
    sync();
    const double e2e_ms = std::chrono::duration<double, std::milli>(clk::now() - t0).count();

    std::printf("{\"prefill_ms\": %.4f, \"prefill_tokens\": %d, \"decode_ms_per_step\": %.5f, \"e2e_ms_per_step\": %.5f, "
                "\"steps\": %d, \"warmup\": %d, \"context_start\": %d, \"last_token\": %d}\n",
                prefill_ms, prefill_tokens, dev_ms / steps, e2e_ms / steps, steps, warmup, prompt_len, (int)tok);
    return 0;
}
