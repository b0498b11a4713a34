// Drives the UNMODIFIED reference project (spymaster2h/spyinfer) on its CUDA backend for the
// benchmark's decode workload and prints timings.  Nothing of the reference is copied here: this
// file includes its headers and is linked against its own sources (build_reference.py), and nothing
// of this repository's engine is used.
//
// What it calls is the reference's stock model code: Qwen3::forward and Qwen3::compute_logits
// (src/models/qwen3.hpp:93-308) through CUDABackend, with the batch description that its
// ModelRunner::execute_model builds for a decoding step (src/engine/model_runner.cpp:49-100):
// Context::set_context / set_context_device, token ids and positions as int32 tensors, then the
// logits copied to the host, widened from half and argmax'ed per sequence (:102-134).  Two things
// of the reference's engine are gone around, and the JSON line says so:
//  * LLMEngine takes chat messages through a tokenizer (src/engine/llm_engine.cpp:32-45) and has no
//    entry for token ids; a random-weights model has no tokenizer files.
//  * execute_model's CUDA branch reads its host copy of the logits after the vector that holds it
//    has gone out of scope (model_runner.cpp:102-118); here the vector lives as long as it is read.
// A step never brings 100 or more tokens (the model's scratch holds 100 rows: qwen3.hpp:13, 97),
// and the cache is sized for the batch through the reference's own num_kvcache_blocks /
// kvcache_block_size (src/config.hpp:26-27).  The caches start zeroed instead of prefilled: the
// decode step's work does not depend on what the keys hold, and the reference's CUDA prefill
// cannot take 100 tokens.
//
// usage: reference_decode MODEL_DIR BLOCK_SIZE WARMUP BATCHxCONTEXTxSTEPS [BATCHxCONTEXTxSTEPS ...]
// prints one line a workload: {"ms_per_step": device ms, "wall_ms_per_step": host ms, "tokens_per_s": ..., ...}
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <numeric>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "backends/cuda/cuda_backend.hpp"
#include "models/qwen3.hpp"
#include "utils/constant_table.hpp"
#include "utils/context.hpp"
#include "utils/precision.hpp"

#define CK(call)                                                                          \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess) {                                                          \
            std::fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e_));              \
            return 3;                                                                     \
        }                                                                                 \
    } while (0)

static int run(std::shared_ptr<spyinfer::CUDABackend> backend, Qwen3& model, const ModelConfig& cfg, int batch, int context, int steps, int warmup,
               int block_size, double load_s)
{
    const int blocks_per_seq = (context + block_size - 1) / block_size;
    const int num_blocks = batch * blocks_per_seq;
    const int64_t kv_width = (int64_t)cfg.num_key_value_heads * cfg.head_dim;
    auto k_cache = backend->create_tensor({cfg.num_hidden_layers, num_blocks, block_size, kv_width}, spyinfer::DataType::fp16_t);
    auto v_cache = backend->create_tensor({cfg.num_hidden_layers, num_blocks, block_size, kv_width}, spyinfer::DataType::fp16_t);
    CK(cudaMemset(k_cache->data_ptr<uint16_t>(), 0, k_cache->numel() * sizeof(uint16_t)));
    CK(cudaMemset(v_cache->data_ptr<uint16_t>(), 0, v_cache->numel() * sizeof(uint16_t)));
    Context::getInstance().set_kv_cache(k_cache, v_cache);

    // sequence s holds blocks s * blocks_per_seq ..., as a sequence admitted alone would get them
    std::vector<int> block_tables((size_t)batch * blocks_per_seq);
    std::iota(block_tables.begin(), block_tables.end(), 0);
    std::vector<int> tokens(batch), positions(batch), slots(batch), ctx_lens(batch), seq_idx(batch), cu(batch + 1);
    unsigned rng = 12345u;
    for (int s = 0; s < batch; ++s) {
        rng = rng * 1664525u + 1013904223u;
        tokens[s] = (int)(rng % (unsigned)cfg.vocab_size);
        seq_idx[s] = s;
    }
    std::iota(cu.begin(), cu.end(), 0);
    std::vector<float> host_logits((size_t)batch * cfg.vocab_size);   // lives for the whole run

    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0));
    CK(cudaEventCreate(&e1));
    std::chrono::steady_clock::time_point w0;
    int len = context - (steps + warmup) - 1;   // tokens each sequence holds before the first step
    long long sampled = 0;
    for (int i = 0; i < steps + warmup; ++i) {
        if (i == warmup) {
            CK(cudaDeviceSynchronize());
            w0 = std::chrono::steady_clock::now();
            CK(cudaEventRecord(e0));
        }
        for (int s = 0; s < batch; ++s) {
            positions[s] = len;
            slots[s] = block_tables[(size_t)s * blocks_per_seq + len / block_size] * block_size + len % block_size;
            ctx_lens[s] = len + 1;
        }
        Context::getInstance().set_context(false, batch, slots.data(), ctx_lens.data(), block_tables.data(), seq_idx.data(), cu.data(), 1, blocks_per_seq);
        Context::getInstance().set_context_device(slots, ctx_lens, block_tables, seq_idx, cu);
        auto ids_t = backend->create_tensor({1, 1, 1, batch}, spyinfer::DataType::int32_t);
        backend->copy_data_from_cpu(ids_t->data_ptr<int>(), tokens.data(), batch * sizeof(int));
        auto pos_t = backend->create_tensor({1, 1, 1, batch}, spyinfer::DataType::int32_t);
        backend->copy_data_from_cpu(pos_t->data_ptr<int>(), positions.data(), batch * sizeof(int));
        auto logits = model.compute_logits(model.forward(ids_t, pos_t));
        backend->copy_data_to_cpu(host_logits.data(), logits->data_ptr<uint16_t>(), logits->numel() * sizeof(uint16_t));
        for (long long j = (long long)logits->numel() - 1; j >= 0; --j)
            host_logits[j] = half_to_float(reinterpret_cast<uint16_t*>(host_logits.data())[j]);
        for (int s = 0; s < batch; ++s) {
            const float* row = host_logits.data() + (size_t)s * cfg.vocab_size;
            tokens[s] = (int)std::distance(row, std::max_element(row, row + cfg.vocab_size));
            sampled += tokens[s];
        }
        Context::getInstance().reset_context();
        ++len;
    }
    CK(cudaEventRecord(e1));
    CK(cudaDeviceSynchronize());
    const double wall_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - w0).count();
    float dev_ms = 0.f;
    CK(cudaEventElapsedTime(&dev_ms, e0, e1));
    CK(cudaGetLastError());
    std::printf("\n{\"ms_per_step\": %.4f, \"wall_ms_per_step\": %.4f, \"tokens_per_s\": %.2f, \"wall_tokens_per_s\": %.2f, \"batch\": %d, "
                "\"context\": %d, \"steps\": %d, \"warmup\": %d, \"block_size\": %d, \"load_s\": %.1f, \"h2d_bytes_per_step\": %lld, "
                "\"d2h_bytes_per_step\": %lld, \"checksum\": %lld}\n",
                dev_ms / steps, wall_ms / steps, batch * steps / (dev_ms / 1e3), batch * steps / (wall_ms / 1e3), batch, context, steps, warmup,
                block_size, load_s, (long long)(4LL * (6 * batch + 1 + (long long)batch * blocks_per_seq)),
                (long long)(2LL * batch * cfg.vocab_size), sampled);
    std::fflush(stdout);
    return 0;
}

int main(int argc, char** argv)
{
    if (argc < 5) {
        std::fprintf(stderr, "usage: reference_decode MODEL_DIR BLOCK_SIZE WARMUP BATCHxCONTEXTxSTEPS [BATCHxCONTEXTxSTEPS ...]\n");
        return 2;
    }
    const std::string model_dir = argv[1];
    const int block_size = std::atoi(argv[2]), warmup = std::atoi(argv[3]);
    struct Work {
        int batch, context, steps;
    };
    std::vector<Work> works;
    ModelConfig cfg(model_dir + "/config.json");
    for (int a = 4; a < argc; ++a) {
        Work w{0, 0, 0};
        if (std::sscanf(argv[a], "%dx%dx%d", &w.batch, &w.context, &w.steps) != 3 || w.batch <= 0 || w.batch >= max_temp_size || w.steps <= 0 ||
            w.context <= w.steps + warmup + 1 || w.context > cfg.max_position_embeddings || block_size <= 0 || warmup < 0) {
            std::fprintf(stderr, "reference_decode: %s: the batch must lie in 1..99 (the reference's scratch), the context above steps + warmup + 1 and "
                                 "within max_position_embeddings\n", argv[a]);
            return 2;
        }
        works.push_back(w);
    }
    auto backend = std::make_shared<spyinfer::CUDABackend>();
    backend->set_compute_dtype(spyinfer::DataType::fp16_t);
    Qwen3 model(cfg, backend);
    const auto t_load = std::chrono::steady_clock::now();
    model.load_model(model_dir);
    CK(cudaDeviceSynchronize());
    const double load_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_load).count();
    ConstantTable::GetInstance().BuildRopeTable(cfg.max_position_embeddings, cfg.head_dim, cfg.rope_theta);
    for (const Work& w : works)
        if (int rc = run(backend, model, cfg, w.batch, w.context, w.steps, warmup, block_size, load_s)) return rc;
    return 0;
}
