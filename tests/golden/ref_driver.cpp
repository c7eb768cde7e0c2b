// Drives the UNMODIFIED reference CPU engine (Cyxuan0311/Forge, scalar build) on a tiny
// random LLaMA model and dumps its logits.  Used once by make_golden.py; not part of the
// product and not needed to run the tests (its outputs are committed beside it).
//
// usage: ref_driver WEIGHTS.bin OUT.bin  < spec on stdin
// stdin: vocab hidden inter layers heads kv_heads head_dim theta eps tie bias n_steps
//        then per step: start_pos n_tokens id...
// WEIGHTS.bin: fp32 tensors in the fixed order written by make_golden.py.
#include <cstdio>
#include <cstring>
#include <iostream>
#include <vector>

#include "forge/arch_registry.h"
#include "forge/context.h"
#include "forge/engine.h"
#include "forge/engines/transformer_engine.h"
#include "forge/model.h"

using namespace forge;

static TensorPtr read_tensor(FILE* f, std::vector<int64_t> shape) {
    auto t = std::make_shared<Tensor>(DataType::FP32, shape, DeviceType::CPU);
    size_t n = static_cast<size_t>(t->numel());
    if (fread(t->data(), sizeof(float), n, f) != n) {
        std::cerr << "short read\n";
        std::exit(2);
    }
    return t;
}

int main(int argc, char** argv) {
    (void)forge::_arch_registrations_linked;
    if (argc < 3) return 1;
    int V, H, I, L, NH, NKV, HD, tie, bias, n_steps;
    float theta, eps;
    std::cin >> V >> H >> I >> L >> NH >> NKV >> HD >> theta >> eps >> tie >> bias >> n_steps;

    ModelConfig cfg;
    cfg.arch_type = "llama";
    cfg.vocab_size = V; cfg.hidden_dim = H; cfg.intermediate_dim = I; cfg.num_layers = L;
    cfg.num_heads = NH; cfg.num_kv_heads = NKV; cfg.head_dim = HD;
    cfg.rope_theta = theta; cfg.rms_norm_eps = eps; cfg.tie_embeddings = tie != 0;
    cfg.max_seq_len = 512;

    Model m;
    m.set_config(cfg);
    m.set_device(DeviceType::CPU);
    FILE* f = fopen(argv[1], "rb");
    if (!f) return 3;
    auto& ws = m.weights();
    ws.set("token_embedding", read_tensor(f, {V, H}));
    ws.set("output_norm", read_tensor(f, {H}));
    if (!tie) ws.set("output_weight", read_tensor(f, {V, H}));
    for (int l = 0; l < L; ++l) {
        std::string p = "layers." + std::to_string(l) + ".";
        ws.set(p + "attn_norm", read_tensor(f, {H}));
        ws.set(p + "wq", read_tensor(f, {NH * HD, H}));
        ws.set(p + "wk", read_tensor(f, {NKV * HD, H}));
        ws.set(p + "wv", read_tensor(f, {NKV * HD, H}));
        if (bias) {
            ws.set(p + "bq", read_tensor(f, {NH * HD}));
            ws.set(p + "bk", read_tensor(f, {NKV * HD}));
            ws.set(p + "bv", read_tensor(f, {NKV * HD}));
        }
        ws.set(p + "wo", read_tensor(f, {H, NH * HD}));
        ws.set(p + "ffn_norm", read_tensor(f, {H}));
        ws.set(p + "gate_proj", read_tensor(f, {I, H}));
        ws.set(p + "up_proj", read_tensor(f, {I, H}));
        ws.set(p + "down_proj", read_tensor(f, {H, I}));
    }
    fclose(f);

    ContextParams params;
    params.device = DeviceType::CPU;
    params.gpu_layers = 0;
    params.max_seq_len = 512;
    InferenceContext ctx(m, params);
    auto e = EngineRegistry::instance().create("llama", m, ctx);
    if (!e) { std::cerr << "no engine\n"; return 4; }
    e->set_gpu_layers(0);

    FILE* out = fopen(argv[2], "wb");
    bool head_fixed = false;
    for (int s = 0; s < n_steps; ++s) {
        long start; int n;
        std::cin >> start >> n;
        auto ids = std::make_shared<Tensor>(DataType::INT32, std::vector<int64_t>{n}, DeviceType::CPU);
        for (int i = 0; i < n; ++i) { int v; std::cin >> v; static_cast<int32_t*>(ids->data())[i] = v; }
        if (!head_fixed) {
            // The CPU engine re-quantizes an FP32 lm_head to Q8_0 when it initialises its weights
            // (src/model/model_weights.cpp:40-67); put the FP32 tensor back so the oracle is FP32.
            // Weight init happens lazily, so run once, then patch, then reset and run for real.
            e->forward(ids, start);
            auto* te = dynamic_cast<TransformerEngine*>(e.get());
            if (te) te->weights().output_weight = ws.get(tie ? "token_embedding" : "output_weight");
            e->reset();
            head_fixed = true;
        }
        auto logits = e->forward(ids, start);
        fwrite(logits->data(), sizeof(float), static_cast<size_t>(logits->numel()), out);
    }
    fclose(out);
    return 0;
}
