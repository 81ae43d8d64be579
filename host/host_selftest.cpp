// Self-test of the C++ host mirror: builds a tiny synthetic Llama through the reference-shaped interface, runs
// Model::generate, prints the greedy ids as JSON.  tests/test_host_cpp_gpu.py compares them with the oracle.
// `host_selftest --sampler seed temperature vocab logits.bin` needs no GPU: it runs the mirror's LogitsProcessor over the f32 rows
// of logits.bin and prints the sampled ids (tests/test_sampling_cpu.py compares them with the oracle).
// Build: g++ -std=c++17 -O2 host/host_selftest.cpp -o host/_build/host_selftest -Lfastllm_b200 -lfastllm_b200 -Wl,-rpath,...
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "fastllm_host.hpp"

int main(int argc, char** argv) {
    if (argc == 6 && std::strcmp(argv[1], "--sampler") == 0) {
        try {
            const uint64_t seed = std::strtoull(argv[2], nullptr, 10);
            const double temperature = std::atof(argv[3]);
            const size_t vocab = (size_t)std::strtoull(argv[4], nullptr, 10);
            FILE* lf = std::fopen(argv[5], "rb");
            if (!lf || vocab == 0) throw std::runtime_error("cannot open logits");
            fastllm::LogitsProcessor lp(seed, temperature < 0 ? std::nullopt : std::optional<double>(temperature));
            std::vector<float> row(vocab);
            std::printf("[");
            for (int i = 0; std::fread(row.data(), 4, vocab, lf) == vocab; ++i) std::printf("%s%u", i ? "," : "", lp.sample(row.data(), vocab));
            std::printf("]\n");
            std::fclose(lf);
            return 0;
        } catch (const std::exception& e) {
            std::fprintf(stderr, "host_selftest --sampler failed: %s\n", e.what());
            return 1;
        }
    }
    if (argc > 5 && std::strcmp(argv[1], "--layered") == 0) {
        // host_selftest --layered max_tokens max_batch prefill_chunk id id / id id id / ...: a two-layer synthetic layered decoder
        // (gated linear attention + dense feed-forward, windowed latent attention + experts) through the C++ MixedBatcher, exact mode
        try {
            const int max_tokens = std::atoi(argv[2]), max_batch = std::atoi(argv[3]), chunk = std::atoi(argv[4]);
            std::vector<std::vector<uint32_t>> prompts(1);
            for (int i = 5; i < argc; ++i) {
                if (std::strcmp(argv[i], "/") == 0) prompts.emplace_back();
                else prompts.back().push_back((uint32_t)std::strtoul(argv[i], nullptr, 10));
            }
            fastllm::check(fl_init(0));
            fl_stack_config sc{};
            sc.arch = FL_ARCH_NIFUNEX; sc.vocab = 48; sc.width = 32; sc.norm_eps = 1e-5f; sc.compute_dtype = FL_DTYPE_F32;
            std::vector<fl_layer_desc> ly(2);
            ly[0].mixer = FL_MIXER_GLA; ly[0].heads = 2; ly[0].dim = 8; ly[0].vdim = 8; ly[0].decay_rank = 4; ly[0].tau = 8.0f; ly[0].kv_from = -1;
            ly[0].ffn = FL_FFN_DENSE; ly[0].ff = 24; ly[0].limit = 1.5f;
            ly[1].mixer = FL_MIXER_LATENT_ATTN; ly[1].heads = 2; ly[1].dim = 8; ly[1].vdim = 8; ly[1].rot_dim = 4; ly[1].kv_rank = 16; ly[1].kv_from = -1;
            ly[1].window = 9; ly[1].rot_dims = 4; ly[1].rot_base = 10000.0; ly[1].scale = 0.28867513f;
            ly[1].ffn = FL_FFN_MOE; ly[1].ff = 16; ly[1].limit = 1.0f; ly[1].experts = 4; ly[1].top = 2; ly[1].shared_ff = 24; ly[1].shared_limit = 0.75f;
            fastllm::LayeredModel model(sc, ly, /*seed=*/5, /*std=*/0.3f);
            fastllm::MixedBatcher mb(model, max_batch, chunk, std::nullopt, 256);
            const auto outs = mb.generate(prompts, max_tokens);
            std::printf("[");
            for (size_t r = 0; r < outs.size(); ++r) {
                std::printf("%s[", r ? "," : "");
                for (size_t i = 0; i < outs[r].size(); ++i) std::printf("%s%u", i ? "," : "", outs[r][i]);
                std::printf("]");
            }
            std::printf("]\n");
            const auto ps = mb.cache.pool_stats();
            std::fprintf(stderr, "mixed steps: %d, pool %d/%d free\n", mb.steps, ps.second, ps.first);
            return ps.first == ps.second ? 0 : 1;
        } catch (const std::exception& e) {
            std::fprintf(stderr, "host_selftest --layered failed: %s\n", e.what());
            return 1;
        }
    }
    // argv: weights.bin (concatenated f32 tensors in manifest order), manifest.txt (name ndim dims...), prompt ids...
    if (argc < 4) { std::fprintf(stderr, "usage: host_selftest manifest.txt weights.bin max_tokens id...\n"); return 2; }
    try {
        FILE* mf = std::fopen(argv[1], "r");
        FILE* wf = std::fopen(argv[2], "rb");
        if (!mf || !wf) throw std::runtime_error("cannot open inputs");
        fastllm::ConfigFile cfg;
        int nkv = 0, maxpos = 0;
        double theta = 0;
        if (std::fscanf(mf, "%d %d %d %d %d %d %lf %lf %d", &cfg.hidden_size, &cfg.intermediate_size, &cfg.vocab_size, &cfg.num_hidden_layers,
                        &cfg.num_attention_heads, &nkv, &cfg.rms_norm_eps, &theta, &maxpos) != 9) throw std::runtime_error("bad manifest header");
        cfg.num_key_value_heads = nkv; cfg.rope_theta = theta; cfg.max_position_embeddings = maxpos;
        std::vector<std::vector<float>> storage;
        fastllm::TensorMap tensors;
        char name[256];
        int nd;
        while (std::fscanf(mf, "%255s %d", name, &nd) == 2) {
            std::vector<int64_t> shape(nd);
            size_t n = 1;
            for (int i = 0; i < nd; ++i) { long long d; if (std::fscanf(mf, "%lld", &d) != 1) throw std::runtime_error("bad shape"); shape[i] = d; n *= (size_t)d; }
            storage.emplace_back(n);
            if (std::fread(storage.back().data(), 4, n, wf) != n) throw std::runtime_error("short weights file");
            tensors[name] = fastllm::HostTensor{FL_DTYPE_F32, shape, storage.back().data()};
        }
        const int max_tokens = std::atoi(argv[3]);
        if (argc > 5 && std::strcmp(argv[4], "--batch") == 0) {
            // host_selftest manifest weights max_tokens --batch max_batch id id / id id id / ...: the C++ ContinuousBatcher over sequence slots
            const int max_batch = std::atoi(argv[5]);
            std::vector<std::vector<uint32_t>> prompts(1);
            for (int i = 6; i < argc; ++i) {
                if (std::strcmp(argv[i], "/") == 0) prompts.emplace_back();
                else prompts.back().push_back((uint32_t)std::strtoul(argv[i], nullptr, 10));
            }
            auto pr = fastllm::LlamaWithConfig::initialize_model(cfg, tensors, 0);
            fastllm::ContinuousBatcher<fastllm::LlamaWithConfig> cb(pr.first, max_batch, std::nullopt);
            const auto outs = cb.generate(prompts, max_tokens);
            std::printf("[");
            for (size_t r = 0; r < outs.size(); ++r) {
                std::printf("%s[", r ? "," : "");
                for (size_t i = 0; i < outs[r].size(); ++i) std::printf("%s%u", i ? "," : "", outs[r][i]);
                std::printf("]");
            }
            std::printf("]\n");
            std::fprintf(stderr, "ragged steps: %d\n", cb.steps);
            return 0;
        }
        std::vector<uint32_t> prompt;
        for (int i = 4; i < argc; ++i) prompt.push_back((uint32_t)std::strtoul(argv[i], nullptr, 10));
        auto pair = fastllm::LlamaWithConfig::initialize_model(cfg, tensors, 0);
        fastllm::Model<fastllm::LlamaWithConfig> model{std::move(pair.first), std::move(pair.second), std::nullopt};
        const auto ids = model.generate(prompt, max_tokens);
        std::printf("[");
        for (size_t i = 0; i < ids.size(); ++i) std::printf("%s%u", i ? "," : "", ids[i]);
        std::printf("]\n");
        // failure point parity: multi-token forward on a non-empty Llama cache must be an error, not a crash
        try {
            model.model.forward(prompt.data(), 1, (int)prompt.size(), prompt.size(), model.cache);
            std::printf("ERROR: expected failure\n");
            return 1;
        } catch (const fastllm::Error& e) { std::fprintf(stderr, "expected error: %s\n", e.what()); }
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "host_selftest failed: %s\n", e.what());
        return 1;
    }
}
