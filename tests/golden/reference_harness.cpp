// Drives the reference project's own CPU model code (spymaster2h/spyinfer, src/models/qwen3.hpp
// through its CPUBackend) on hand-built batches and writes the logits it computes.
// It is compiled against the reference's sources by make_golden.py; nothing of the
// reference is copied here, and nothing of the package under test is used.
//
// usage: reference_harness MODEL_DIR PLAN_FILE OUT_FILE
// PLAN_FILE: first line "block_size num_blocks", then one line a step, seven
// '|'-separated integer lists:
//   tokens | positions | slot_mapping | seq_idx_of_token | context_lens | max_blocks | block_tables
// OUT_FILE: the logits of every token of every step, in order, as little-endian float32.
#include <cstdio>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "backends/cpu/cpu_backend.hpp"
#include "models/qwen3.hpp"
#include "utils/constant_table.hpp"
#include "utils/context.hpp"

static std::vector<int> parse_ints(const std::string& s)
{
    std::vector<int> out;
    std::istringstream in(s);
    int v;
    while (in >> v) out.push_back(v);
    return out;
}

int main(int argc, char** argv)
{
    if (argc != 4)
    {
        std::cerr << "usage: reference_harness MODEL_DIR PLAN_FILE OUT_FILE" << std::endl;
        return 2;
    }
    const std::string model_dir = argv[1];
    std::ifstream plan(argv[2]);
    std::FILE* out = std::fopen(argv[3], "wb");
    if (!plan || !out) return 2;

    ModelConfig cfg(model_dir + "/config.json");
    auto backend = std::make_shared<spyinfer::CPUBackend>(2);
    backend->set_compute_dtype(spyinfer::DataType::fp32_t);
    Qwen3 model(cfg, backend);
    model.load_model(model_dir);

    std::string line;
    std::getline(plan, line);
    auto head = parse_ints(line);
    const int block_size = head.at(0), num_blocks = head.at(1);
    auto k_cache = backend->create_tensor({cfg.num_hidden_layers, num_blocks, block_size, cfg.num_key_value_heads * cfg.head_dim},
                                          spyinfer::DataType::fp32_t);
    auto v_cache = backend->create_tensor({cfg.num_hidden_layers, num_blocks, block_size, cfg.num_key_value_heads * cfg.head_dim},
                                          spyinfer::DataType::fp32_t);
    Context::getInstance().set_kv_cache(k_cache, v_cache);
    ConstantTable::GetInstance().BuildRopeTable(cfg.max_position_embeddings, cfg.head_dim, cfg.rope_theta);

    while (std::getline(plan, line))
    {
        if (line.empty()) continue;
        std::vector<std::vector<int>> f;
        std::istringstream in(line);
        std::string part;
        while (std::getline(in, part, '|')) f.push_back(parse_ints(part));
        if (f.size() != 7) return 3;
        auto &tokens = f[0], &positions = f[1], &slots = f[2], &seq_idx = f[3], &ctx_lens = f[4], &tables = f[6];
        const int max_blocks = f[5].at(0);
        const int T = (int)tokens.size();
        std::vector<int> cu(ctx_lens.size() + 1, 0);
        Context::getInstance().set_context(false, (int)ctx_lens.size(), slots.data(), ctx_lens.data(), tables.data(), seq_idx.data(),
                                           cu.data(), 0, max_blocks);
        auto ids_t = backend->create_tensor({1, 1, 1, T}, spyinfer::DataType::int32_t);
        auto pos_t = backend->create_tensor({1, 1, 1, T}, spyinfer::DataType::int32_t);
        std::copy(tokens.begin(), tokens.end(), ids_t->data_ptr<int>());
        std::copy(positions.begin(), positions.end(), pos_t->data_ptr<int>());
        auto logits = model.compute_logits(model.forward(ids_t, pos_t));
        std::fwrite(logits->data_ptr<float>(), sizeof(float), (size_t)T * cfg.vocab_size, out);
    }
    std::fclose(out);
    return 0;
}
