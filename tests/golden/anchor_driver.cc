// Runs nireo/chibillm's own host code on a tiny model folder and writes what
// it computes, as golden files for this repository's tests.
//
// Linked with the reference's unmodified .cc files and metal_cpu_shim.cc
// (which supplies the device layer on the CPU).  Everything called here is
// the reference's: load_qwen3_config, safetensors_file::open_model,
// load_qwen_weights, embed_tokens, run_qwen_layers, rms_norm, linear,
// encode_greedy, prepare_paged_batch, metal_model_state, scheduler and
// inference_engine.  The model adapter below does what
// qwen_model_runner::execute does (src/qwen/qwen_model_runner.cc:198-239)
// without the tokenizer that qwen_model_runner::make insists on, the way the
// reference's own layer test drives the stack
// (tests/qwen_weights_test.cc:963-1043).
//
//   anchor_driver MODEL_DIR JOB.json OUT_DIR
//
// JOB.json: {"block_size": n, "requests": [{"id": 1, "tokens": [...]}, ...],
//            "generate": [{"name": "...", "max_new_tokens": n, "max_sequences": n,
//                          "max_batch_tokens": n, "prefill_chunk_tokens": n,
//                          "kv_block_count": n}, ...]}
// Writes, per request: whole_<id>.f32 (logits of every position, the prompt
// run as one batch through a permuted block table) and steps_<id>.f32 (the
// same positions fed one token at a time); per generate entry, in
// generated.json, the greedy tokens of every request through the reference's
// scheduler and engine, and gen_<name>_<id>.f32, the logits of the rows that
// were sampled.
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <iostream>
#include <map>
#include <numeric>
#include <stdexcept>
#include <string>
#include <vector>

#include <nlohmann/json.hpp>

#include "inference_engine.h"
#include "metal/metal_kv_cache.h"
#include "metal/metal_model_state.h"
#include "model_batch.h"
#include "model_format/safetensors.h"
#include "model_runner.h"
#include "qwen/qwen_configs.h"
#include "qwen/qwen_layer.h"
#include "qwen/qwen_weights.h"
#include "tensor/attention.h"
#include "tensor/functions.h"

using namespace chibillm;
using json = nlohmann::json;

namespace {

[[noreturn]] void
die(const std::string& what)
{
    throw std::runtime_error(what);
}

template <typename Result>
auto
must(Result&& result, const char* what) -> decltype(std::move(*result))
{
    if (!result)
        die(std::string(what) + ": " + describe_error(result.error()));
    return std::move(*result);
}

template <typename Result>
void
must_ok(Result&& result, const char* what)
{
    if (!result)
        die(std::string(what) + ": " + describe_error(result.error()));
}

void
write_floats(const std::filesystem::path& path, const std::vector<float>& values)
{
    std::ofstream file(path, std::ios::binary);
    file.write(reinterpret_cast<const char*>(values.data()),
               static_cast<std::streamsize>(values.size() * sizeof(float)));
    if (!file)
        die("cannot write " + path.string());
}

struct loaded_model {
    metal_context context;
    qwen3_config config;
    qwen_weights weights;
};

// logits of every row of final hidden states: the final norm, then the
// vocabulary product (what encode_greedy computes before its argmax,
// src/tensor/functions.cc:287-363)
std::vector<float>
all_logits(const loaded_model& model, const metal_tensor& hidden)
{
    auto normed =
        must(rms_norm(model.context, hidden, model.weights.final_norm, model.config.rms_epsilon),
             "final norm");
    auto logits = must(linear(model.context, normed, model.weights.vocabulary()), "vocabulary");
    const auto bytes = logits.buffer().bytes();
    std::vector<float> values(bytes.size() / sizeof(float));
    std::memcpy(values.data(), bytes.data(), bytes.size());
    return values;
}

// One request alone, with hand-made paging (pages in reverse order, so a
// logical page never sits at its own index), either as one batch of all rows
// or one row at a time.
std::vector<float>
run_alone(const loaded_model& model, const std::vector<token_id>& tokens, std::size_t block_size,
          bool one_by_one)
{
    const auto& config = model.config;
    const std::size_t blocks = (tokens.size() - 1) / block_size + 1;
    auto cache = must(metal_kv_cache::make(model.context,
                                           {
                                               .layer_count = config.layer_count,
                                               .block_count = blocks + 1,
                                               .block_size = block_size,
                                               .kv_head_count = config.kv_head_count,
                                               .head_dimension = config.head_dimension,
                                           }),
                      "kv cache");
    std::vector<std::uint32_t> table(blocks);
    for (std::size_t b = 0; b < blocks; ++b)
        table[b] = static_cast<std::uint32_t>(blocks - b);      // blocks .. 1, page 0 unused
    std::vector<float> result;
    const std::size_t vocabulary = config.vocabulary_size;
    const auto run = [&](std::size_t first, std::size_t count) {
        std::vector<token_id> ids(tokens.begin() + first, tokens.begin() + first + count);
        std::vector<std::uint32_t> positions(count), slots(count), offsets(count, 0),
            lengths(count, static_cast<std::uint32_t>(blocks));
        for (std::size_t i = 0; i < count; ++i) {
            const std::size_t p = first + i;
            positions[i] = static_cast<std::uint32_t>(p);
            slots[i] = static_cast<std::uint32_t>(table[p / block_size] * block_size + p % block_size);
        }
        auto hidden = must(embed_tokens(model.context, model.weights.token_embedding, ids), "embed");
        auto final_hidden = must(run_qwen_layers(model.context, config, model.weights,
                                                 std::move(hidden),
                                                 attention_metadata {
                                                     .positions = positions,
                                                     .slots = slots,
                                                     .block_table = table,
                                                     .block_table_offsets = offsets,
                                                     .block_table_lengths = lengths,
                                                 },
                                                 cache),
                                 "layers");
        auto logits = all_logits(model, final_hidden);
        if (logits.size() != count * vocabulary)
            die("unexpected logits size");
        result.insert(result.end(), logits.begin(), logits.end());
    };
    if (one_by_one)
        for (std::size_t p = 0; p < tokens.size(); ++p)
            run(p, 1);
    else
        run(0, tokens.size());
    return result;
}

// The model adapter the reference's engine drives.
class anchor_runner final : public model_runner {
public:
    anchor_runner(const loaded_model& model, std::size_t block_size, std::size_t block_count)
        : model_(model)
        , cache_config_ { .layer_count = model.config.layer_count,
                          .block_count = block_count,
                          .block_size = block_size,
                          .kv_head_count = model.config.kv_head_count,
                          .head_dimension = model.config.head_dimension }
        , info_ { .id = "anchor",
                  .max_context_tokens =
                      std::min(model.config.max_position_embeddings, block_count * block_size),
                  .eos_token = model.config.eos_token_id }
    {}

    result<std::unique_ptr<model_state>, model_runner_error>
    make_state(scheduler_config config) const override
    {
        auto geometry = cache_config_;
        geometry.block_count = config.kv_block_count;
        auto state = metal_model_state::make(model_.context, geometry);
        if (!state)
            return fail(model_runner_errc::backend_failure, state.error(), "create model state");
        return std::move(*state);
    }

    const model_info&
    info() const noexcept override
    {
        return info_;
    }

    result<encoded_prompt, model_runner_error>
    encode_chat(std::span<const chat_message>) override
    {
        return fail(model_runner_errc::invalid_chat);
    }

    result<std::string, model_runner_error>
    decode(std::span<const token_id>) const override
    {
        return std::string();
    }

    result<std::vector<token_id>, model_runner_error>
    execute(const model_batch& batch, model_state& state) override
    {
        auto* paged_state = dynamic_cast<metal_model_state*>(&state);
        if (!paged_state)
            return fail(model_runner_errc::inconsistent_batch);
        auto& cache = paged_state->cache();
        auto metadata = prepare_paged_batch(batch, model_.config.max_position_embeddings,
                                            cache.block_count(), cache.block_size());
        if (!metadata)
            return fail(model_runner_errc::inconsistent_batch, metadata.error(), "prepare batch");
        auto hidden = embed_tokens(model_.context, model_.weights.token_embedding, batch.tokens);
        if (!hidden)
            return fail(model_runner_errc::backend_failure, hidden.error(), "embedding");
        auto final_hidden = run_qwen_layers(model_.context, model_.config, model_.weights,
                                            std::move(*hidden),
                                            {
                                                .positions = batch.positions,
                                                .slots = metadata->slots,
                                                .block_table = metadata->block_table,
                                                .block_table_offsets = metadata->table_offsets,
                                                .block_table_lengths = metadata->table_lengths,
                                            },
                                            cache);
        if (!final_hidden)
            return fail(model_runner_errc::backend_failure, final_hidden.error(), "layers");
        steps_.push_back({ batch.phase == batch_phase::prefill ? "prefill" : "decode",
                           batch.tokens.size(), batch.items.size() });
        if (metadata->logits_indices.empty())
            return std::vector<token_id> {};
        auto encoded = encode_greedy(model_.context, model_.weights.final_norm,
                                     model_.weights.vocabulary(), model_.config.rms_epsilon,
                                     *final_hidden, metadata->logits_indices);
        if (!encoded)
            return fail(model_runner_errc::backend_failure, encoded.error(), "greedy output");
        auto tokens = read_greedy(*encoded);

        // the logits behind those tokens, for the record
        const auto logits = all_logits(model_, *final_hidden);
        const std::size_t vocabulary = model_.config.vocabulary_size;
        std::size_t sampled = 0;
        for (const auto& item : batch.items) {
            if (!item.logits_index)
                continue;
            auto& rows = sampled_logits_[item.id];
            const auto* row = logits.data() + *item.logits_index * vocabulary;
            rows.insert(rows.end(), row, row + vocabulary);
            ++sampled;
        }
        if (sampled != tokens.size())
            return fail(model_runner_errc::inconsistent_batch);
        return tokens;
    }

    struct step_record {
        std::string phase;
        std::size_t tokens;
        std::size_t sequences;
    };

    std::map<seq_id, std::vector<float>> sampled_logits_;
    std::vector<step_record> steps_;

private:
    const loaded_model& model_;
    kv_cache_config cache_config_;
    model_info info_;
};

} // namespace

int
main(int argc, char** argv)
{
    try {
        if (argc != 4)
            die("usage: anchor_driver MODEL_DIR JOB.json OUT_DIR");
        const std::filesystem::path model_dir = argv[1];
        const std::filesystem::path out_dir = argv[3];
        std::filesystem::create_directories(out_dir);
        json job;
        {
            std::ifstream file(argv[2]);
            if (!file)
                die("cannot read the job file");
            file >> job;
        }
        const std::size_t block_size = job.at("block_size").get<std::size_t>();

        auto config = must(load_qwen3_config(model_dir / "config.json"), "config");
        auto file = must(safetensors_file::open_model(model_dir), "safetensors");
        auto context = must(metal_context::make(""), "context");
        auto weights = must(load_qwen_weights(context, file, config), "weights");
        loaded_model model { std::move(context), std::move(config), std::move(weights) };

        std::vector<std::pair<seq_id, std::vector<token_id>>> requests;
        for (const auto& r : job.at("requests"))
            requests.emplace_back(r.at("id").get<seq_id>(), r.at("tokens").get<std::vector<token_id>>());

        for (const auto& [id, tokens] : requests) {
            write_floats(out_dir / ("whole_" + std::to_string(id) + ".f32"),
                         run_alone(model, tokens, block_size, false));
            write_floats(out_dir / ("steps_" + std::to_string(id) + ".f32"),
                         run_alone(model, tokens, block_size, true));
        }

        json generated = json::object();
        for (const auto& g : job.value("generate", json::array())) {
            const auto name = g.at("name").get<std::string>();
            scheduler_config sc {
                .max_sequences = g.at("max_sequences").get<std::size_t>(),
                .max_batch_tokens = g.at("max_batch_tokens").get<std::size_t>(),
                .kv_block_count = g.at("kv_block_count").get<std::size_t>(),
                .kv_block_size = block_size,
                .prefill_chunk_tokens = g.at("prefill_chunk_tokens").get<std::size_t>(),
                .prefix_cache_bytes = 0,
                .prefix_cache_min_tokens = 64,
            };
            anchor_runner runner(model, block_size, sc.kv_block_count);
            auto engine = must(inference_engine::make(sc, runner), "engine");
            std::map<seq_id, std::vector<token_id>> produced;
            std::map<seq_id, std::string> reasons;
            std::size_t next = 0;
            const auto admit = [&] {
                // first come first served; a request that does not fit now waits
                // for a finish (src/serving_runtime.cc:243-247)
                while (next < requests.size()) {
                    auto sequence = must(seq::make(requests[next].first, requests[next].second,
                                                   generation_params {
                                                       .max_new_tokens =
                                                           g.at("max_new_tokens").get<std::size_t>(),
                                                       .ignore_eos = g.value("ignore_eos", true),
                                                   }),
                                         "sequence");
                    const auto admitted = must(engine.try_add(sequence), "admission");
                    if (admitted == admission_result::too_large)
                        die("a request is too large for the pool");
                    if (admitted == admission_result::deferred)
                        break;
                    ++next;
                }
            };
            admit();
            while (!engine.is_finished() || next < requests.size()) {
                auto updates = must(engine.step(), "step");
                bool finished_one = false;
                for (const auto& update : updates) {
                    produced[update.id].push_back(update.token);
                    if (update.reason != finish_reason::none) {
                        reasons[update.id] = update.reason == finish_reason::eos ? "eos"
                            : update.reason == finish_reason::len_limit          ? "len_limit"
                                                                                   : "cancelled";
                        must_ok(engine.remove(update.id), "remove");
                        finished_one = true;
                    }
                }
                if (finished_one || engine.is_finished())
                    admit();
            }
            json entry = json::object();
            json tokens_out = json::object();
            json reasons_out = json::object();
            for (const auto& [id, tokens] : produced) {
                tokens_out[std::to_string(id)] = tokens;
                reasons_out[std::to_string(id)] = reasons[id];
                write_floats(out_dir / ("gen_" + name + "_" + std::to_string(id) + ".f32"),
                             runner.sampled_logits_[id]);
            }
            json steps_out = json::array();
            for (const auto& s : runner.steps_)
                steps_out.push_back({ s.phase, s.tokens, s.sequences });
            entry["tokens"] = tokens_out;
            entry["reasons"] = reasons_out;
            entry["steps"] = steps_out;
            generated[name] = entry;
        }
        std::ofstream(out_dir / "generated.json") << generated.dump(1) << "\n";
        return 0;
    } catch (const std::exception& error) {
        std::cerr << "anchor_driver: " << error.what() << "\n";
        return 1;
    }
}
