// A CPU stand-in for the device layer of nireo/chibillm, for tests only.
//
// The reference's host code (configuration, safetensors reader, weight
// packing, layer loop, op validation, attention metadata, paging, scheduler,
// engine) is plain C++ behind three pimpl classes whose bodies live in
// Objective-C++ files that only an Apple machine can build:
//   metal_buffer, metal_context       (src/metal/metal_context.h:63-156)
//   metal_kernels::dispatch_*         (src/metal/metal_kernels.h:7-180)
// This file defines those symbols over malloc'ed memory, so that the
// reference's own, unmodified .cc files can be compiled and linked on any
// machine and its real model code produces logits for the tiny test models.
//
// What is the reference's code and what is restated here: everything above
// the dispatch_* calls runs as the reference wrote it.  Each dispatch_* below
// restates the arithmetic of the Metal kernel that the .mm file would launch
// (cited at each function), one thread's work at a time in plain loops.  Where
// a Metal kernel adds with simd_sum, whose order the hardware chooses, the
// loop here adds in index order.  No reference source is copied into this
// repository; the build takes it from the directory that make_goldens.py is
// given.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>

#include "metal/metal_context.h"
#include "metal/metal_kernels.h"

namespace chibillm {

// ------------------------------------------------------------------ buffers
struct metal_buffer::implementation {
    std::byte* data = nullptr;
    std::size_t size = 0;
    ~implementation() { std::free(data); }
};

metal_buffer::metal_buffer(std::unique_ptr<implementation> implementation) noexcept
    : implementation_(std::move(implementation))
{}
metal_buffer::metal_buffer(metal_buffer&&) noexcept = default;
metal_buffer& metal_buffer::operator=(metal_buffer&&) noexcept = default;
metal_buffer::~metal_buffer() = default;

std::size_t
metal_buffer::size_bytes() const noexcept
{
    return implementation_ ? implementation_->size : 0;
}

std::span<std::byte>
metal_buffer::bytes() noexcept
{
    return implementation_ ? std::span<std::byte>(implementation_->data, implementation_->size)
                           : std::span<std::byte>();
}

std::span<const std::byte>
metal_buffer::bytes() const noexcept
{
    return implementation_ ? std::span<const std::byte>(implementation_->data, implementation_->size)
                           : std::span<const std::byte>();
}

// ------------------------------------------------------------------ context
struct metal_context::implementation {
    bool pass_open = false;
};

metal_context::metal_context(std::unique_ptr<implementation> implementation) noexcept
    : implementation_(std::move(implementation))
{}
metal_context::metal_context(metal_context&&) noexcept = default;
metal_context& metal_context::operator=(metal_context&&) noexcept = default;
metal_context::~metal_context() = default;

result<metal_context, metal_error>
metal_context::make(std::string_view)
{
    return metal_context { std::make_unique<implementation>() };
}

std::string_view
metal_context::device_name() const noexcept
{
    return "cpu stand-in";
}

// Work runs at once, so a pass only remembers that it is open
// (src/metal/metal_context.mm:404-475 collects and waits).
result<void, metal_error>
metal_context::begin_compute_pass()
{
    if (implementation_->pass_open)
        return std::unexpected(metal_error { metal_errc::invalid_input, "a pass is already open" });
    implementation_->pass_open = true;
    return {};
}

result<void, metal_error>
metal_context::end_compute_pass()
{
    if (!implementation_->pass_open)
        return std::unexpected(metal_error { metal_errc::invalid_input, "no pass is open" });
    implementation_->pass_open = false;
    return {};
}

void
metal_context::abort_compute_pass() noexcept
{
    implementation_->pass_open = false;
}

// Zero-filled, as a new Metal buffer is; size 0 is refused
// (src/metal/metal_context.mm:476-503).
result<metal_buffer, metal_error>
metal_context::make_shared_buffer(std::size_t size_bytes) const
{
    if (size_bytes == 0)
        return std::unexpected(
            metal_error { metal_errc::invalid_input, "Metal buffer size must be nonzero" });
    auto impl = std::make_unique<metal_buffer::implementation>();
    impl->data = static_cast<std::byte*>(std::calloc(size_bytes, 1));
    if (!impl->data)
        return std::unexpected(
            metal_error { metal_errc::buffer_creation_failed, "calloc failed" });
    impl->size = size_bytes;
    return metal_buffer { std::move(impl) };
}

// ------------------------------------------------------------------ helpers
namespace {

template <typename T>
const T*
in(const metal_buffer& buffer)
{
    return reinterpret_cast<const T*>(buffer.bytes().data());
}

template <typename T>
T*
out(metal_buffer& buffer)
{
    return reinterpret_cast<T*>(buffer.bytes().data());
}

// bf16 storage to float: the bits shifted up (src/metal/kernels/common.metalh:26-30).
float
bf16_to_float(std::uint16_t bits)
{
    const std::uint32_t wide = std::uint32_t(bits) << 16;
    float value;
    std::memcpy(&value, &wide, sizeof(value));
    return value;
}

// One output feature of a projection: sum over k of input[k] * float(w[row,k])
// (src/metal/kernels/linear.metal:152-156; the one-row kernels add the same
// products lane by lane and finish with simd_sum, common.metalh:40-65).
float
dot_row(const float* input, const std::uint16_t* weight, std::size_t columns, std::size_t row)
{
    float accumulator = 0.0F;
    const std::uint16_t* w = weight + row * columns;
    for (std::size_t k = 0; k < columns; ++k)
        accumulator += input[k] * bf16_to_float(w[k]);
    return accumulator;
}

std::unexpected<metal_error>
refuse(const char* what)
{
    return std::unexpected(metal_error { metal_errc::invalid_input, what });
}

// rms_norm_bf16 (src/metal/kernels/tensor_ops.metal:53-106): one group per row.
void
rms_norm_rows(const float* input,
              const std::uint16_t* weight,
              float* output,
              std::size_t rows,
              std::size_t width,
              float epsilon,
              float weight_offset)
{
    for (std::size_t row = 0; row < rows; ++row) {
        const float* x = input + row * width;
        float sum = 0.0F;
        for (std::size_t f = 0; f < width; ++f)
            sum += x[f] * x[f];
        const float mean_square = sum / float(width);
        const float inverse_rms = 1.0F / std::sqrt(mean_square + epsilon);
        for (std::size_t f = 0; f < width; ++f) {
            const float weight_value = bf16_to_float(weight[f]) + weight_offset;
            output[row * width + f] = x[f] * inverse_rms * weight_value;
        }
    }
}

struct paged_view {
    const std::uint32_t* positions;
    const std::uint32_t* block_table;
    const std::uint32_t* offsets;
    const std::uint32_t* lengths;
    const float* keys;
    const float* values;
    std::size_t query_heads, kv_heads, head_dim, block_size, slot_count, layer, table_entries;

    // [layer][slot][kv head][feature] (src/metal/kernels/attention.metal:108-113)
    std::size_t
    cache_base(std::uint32_t table_offset, std::uint32_t token, std::size_t kv_head) const
    {
        const std::uint32_t physical = block_table[table_offset + token / block_size];
        const std::size_t slot = std::size_t(physical) * block_size + token % block_size;
        return ((layer * slot_count + slot) * kv_heads + kv_head) * head_dim;
    }

    bool
    row_ok(std::uint32_t table_offset, std::uint32_t table_length, std::uint32_t last_position) const
    {
        return !(table_offset > table_entries || table_length > table_entries - table_offset
                 || last_position / block_size >= table_length);
    }
};

// The token-by-token online softmax of paged_attention_f32 and of one chunk of
// paged_attention_partial_f32 (src/metal/kernels/attention.metal:98-158,520-558).
struct running_softmax {
    float maximum = -std::numeric_limits<float>::infinity();
    float denominator = 0.0F;
    std::vector<float> accumulator;
};

void
attend_range(const paged_view& v,
             const float* query,
             std::uint32_t table_offset,
             std::size_t kv_head,
             std::uint32_t begin,
             std::uint32_t end,
             running_softmax& state)
{
    const float attention_scale = 1.0F / std::sqrt(float(v.head_dim));
    state.accumulator.assign(v.head_dim, 0.0F);
    for (std::uint32_t token = begin; token < end; ++token) {
        const std::size_t base = v.cache_base(table_offset, token, kv_head);
        float score = 0.0F;
        for (std::size_t f = 0; f < v.head_dim; ++f)
            score += query[f] * v.keys[base + f];
        score *= attention_scale;
        const float new_max = std::max(state.maximum, score);
        const float rescale = std::exp(state.maximum - new_max);
        const float weight = std::exp(score - new_max);
        state.maximum = new_max;
        state.denominator = state.denominator * rescale + weight;
        for (std::size_t f = 0; f < v.head_dim; ++f)
            state.accumulator[f] = state.accumulator[f] * rescale + v.values[base + f] * weight;
    }
}

} // namespace

// ------------------------------------------------------------------ products
// Host side: src/metal/metal_kernels_linear.mm:12-73 (dense branch); kernels
// linear_split_bf16(_decode) and linear_add_bf16_decode, and add_f32 after a
// product of several rows with a residual.
result<void, metal_error>
metal_kernels::dispatch_projection(const metal_buffer& input,
                                   matrix_view weight,
                                   const std::array<metal_buffer*, 3>& outputs,
                                   std::size_t rows,
                                   const std::array<std::size_t, 3>& widths,
                                   const metal_buffer* residual) const
{
    if (!weight.supported() || !weight.dense())
        return refuse("the stand-in takes dense bf16 matrices only");
    const auto columns = weight.shape().dimensions()[1];
    const auto total = weight.shape().dimensions()[0];
    const auto* w = in<std::uint16_t>(weight.dense()->buffer());
    const auto* x = in<float>(input);
    if (residual) {
        // only the first output is written (linear_add: one output, full width)
        float* y = out<float>(*outputs[0]);
        const auto* r = in<float>(*residual);
        for (std::size_t row = 0; row < rows; ++row)
            for (std::size_t c = 0; c < total; ++c)
                y[row * total + c] = r[row * total + c] + dot_row(x + row * columns, w, columns, c);
        return {};
    }
    if (widths[0] + widths[1] + widths[2] != total)
        return refuse("split widths do not add up to the weight's rows");
    for (std::size_t row = 0; row < rows; ++row) {
        std::size_t c = 0;
        for (std::size_t part = 0; part < 3; ++part) {
            float* y = widths[part] ? out<float>(*outputs[part]) : nullptr;
            for (std::size_t local = 0; local < widths[part]; ++local, ++c)
                y[row * widths[part] + local] = dot_row(x + row * columns, w, columns, c);
        }
    }
    return {};
}

// embedding_bf16 (src/metal/kernels/tensor_ops.metal:3-37)
result<void, metal_error>
metal_kernels::dispatch_embedding(const metal_buffer& token_ids,
                                  matrix_view weight,
                                  metal_buffer& output,
                                  std::size_t token_count) const
{
    if (!weight.supported() || !weight.dense())
        return refuse("the stand-in takes dense bf16 matrices only");
    const auto hidden = weight.shape().dimensions()[1];
    const auto* w = in<std::uint16_t>(weight.dense()->buffer());
    const auto* ids = in<std::int32_t>(token_ids);
    float* y = out<float>(output);
    for (std::size_t t = 0; t < token_count; ++t)
        for (std::size_t h = 0; h < hidden; ++h)
            y[t * hidden + h] = bf16_to_float(w[std::size_t(ids[t]) * hidden + h]);
    return {};
}

// src/metal/metal_kernels.mm:16-53: weight offset 1 if zero centred, else 0.
result<void, metal_error>
metal_kernels::dispatch_rms_norm_bf16(const metal_buffer& input,
                                      const metal_buffer& weight,
                                      metal_buffer& output,
                                      std::size_t rows,
                                      std::size_t hidden_size,
                                      float epsilon,
                                      bool zero_centered) const
{
    // input and output may be the same buffer (in-place q/k norm); each row is
    // read completely before its first write only through the sum, and every
    // element is rewritten from its own old value, so in place is safe.
    rms_norm_rows(in<float>(input), in<std::uint16_t>(weight), out<float>(output), rows,
                  hidden_size, epsilon, zero_centered ? 1.0F : 0.0F);
    return {};
}

// silu_mul_f32 (src/metal/kernels/tensor_ops.metal:108-124)
result<void, metal_error>
metal_kernels::dispatch_silu_mul_f32(const metal_buffer& gate,
                                     const metal_buffer& up,
                                     metal_buffer& output,
                                     std::size_t element_count,
                                     bool sigmoid_only) const
{
    const auto* g = in<float>(gate);
    const auto* u = in<float>(up);
    float* y = out<float>(output);
    for (std::size_t i = 0; i < element_count; ++i) {
        const float x = g[i];
        const float silu = (sigmoid_only ? 1.0F : x) / (1.0F + std::exp(-x));
        y[i] = silu * u[i];
    }
    return {};
}

// add_f32 (src/metal/kernels/tensor_ops.metal:126-138)
result<void, metal_error>
metal_kernels::dispatch_add_f32(const metal_buffer& lhs,
                                const metal_buffer& rhs,
                                metal_buffer& output,
                                std::size_t element_count) const
{
    const auto* a = in<float>(lhs);
    const auto* b = in<float>(rhs);
    float* y = out<float>(output);
    for (std::size_t i = 0; i < element_count; ++i)
        y[i] = a[i] + b[i];
    return {};
}

// split_heads_f32 (src/metal/kernels/tensor_ops.metal:140-155); not on the Qwen3 path.
result<void, metal_error>
metal_kernels::dispatch_split_heads_f32(const metal_buffer& input,
                                        metal_buffer& first,
                                        metal_buffer& second,
                                        std::size_t rows,
                                        std::size_t head_count,
                                        std::size_t head_dimension) const
{
    const auto width = head_count * head_dimension;
    const auto* x = in<float>(input);
    float* a = out<float>(first);
    float* b = out<float>(second);
    for (std::size_t row = 0; row < rows; ++row)
        for (std::size_t column = 0; column < width; ++column) {
            const auto source = row * width * 2 + (column / head_dimension) * head_dimension * 2
                + column % head_dimension;
            a[row * width + column] = x[source];
            b[row * width + column] = x[source + head_dimension];
        }
    return {};
}

// rope_f32 (src/metal/kernels/tensor_ops.metal:157-198) with the frequency
// table of the host side: powf(theta, -2 * pair / rotary) in float
// (src/metal/metal_kernels.mm:186-191).
result<void, metal_error>
metal_kernels::dispatch_rope_f32(const metal_buffer& input,
                                 const metal_buffer& positions,
                                 metal_buffer& output,
                                 std::size_t rows,
                                 std::size_t head_count,
                                 std::size_t head_dimension,
                                 float theta,
                                 std::size_t rotary_dimension) const
{
    std::vector<float> frequencies(rotary_dimension / 2);
    for (std::size_t pair = 0; pair < frequencies.size(); ++pair) {
        const auto exponent = -2.0F * static_cast<float>(pair) / static_cast<float>(rotary_dimension);
        frequencies[pair] = std::pow(theta, exponent);
    }
    const auto* x = in<float>(input);
    const auto* pos = in<std::uint32_t>(positions);
    float* y = out<float>(output);
    const std::size_t half_dimension = head_dimension / 2;
    const std::size_t half_rotary = rotary_dimension / 2;
    for (std::size_t row = 0; row < rows; ++row)
        for (std::size_t head = 0; head < head_count; ++head) {
            const std::size_t head_offset = (row * head_count + head) * head_dimension;
            for (std::size_t pair = 0; pair < half_dimension; ++pair) {
                if (pair >= half_rotary) {
                    const auto tail = head_offset + rotary_dimension + 2 * (pair - half_rotary);
                    y[tail] = x[tail];
                    y[tail + 1] = x[tail + 1];
                    continue;
                }
                const auto first_index = head_offset + pair;
                const auto second_index = first_index + half_rotary;
                const float angle = float(pos[row]) * frequencies[pair];
                const float cosine = std::cos(angle);
                const float sine = std::sin(angle);
                const float first = x[first_index];
                const float second = x[second_index];
                y[first_index] = first * cosine - second * sine;
                y[second_index] = second * cosine + first * sine;
            }
        }
    return {};
}

// store_kv_f32 (src/metal/kernels/attention.metal:3-33)
result<void, metal_error>
metal_kernels::dispatch_store_kv_f32(const metal_buffer& keys,
                                     const metal_buffer& values,
                                     const metal_buffer& slot_mapping,
                                     metal_buffer& key_cache,
                                     metal_buffer& value_cache,
                                     std::size_t rows,
                                     std::size_t feature_count,
                                     std::size_t layer,
                                     std::size_t slot_count) const
{
    const auto* k = in<float>(keys);
    const auto* v = in<float>(values);
    const auto* slots = in<std::uint32_t>(slot_mapping);
    float* kc = out<float>(key_cache);
    float* vc = out<float>(value_cache);
    for (std::size_t row = 0; row < rows; ++row) {
        const std::size_t slot = slots[row];
        if (slot >= slot_count)
            continue;
        for (std::size_t f = 0; f < feature_count; ++f) {
            const auto index = (layer * slot_count + slot) * feature_count + f;
            kc[index] = k[row * feature_count + f];
            vc[index] = v[row * feature_count + f];
        }
    }
    return {};
}

// Host side: src/metal/metal_kernels_attention.mm:141-296.  A lone row at
// position 63 or later is cut into chunks of 64 keys whose partial results
// are merged (paged_attention_partial_f32 + paged_attention_reduce_f32,
// src/metal/kernels/attention.metal:446-615); everything else runs
// paged_attention_f32 (attention.metal:35-159).  Head sizes above 128 on
// several rows would take paged_attention_simd_f32, which Qwen3 does not reach.
result<void, metal_error>
metal_kernels::dispatch_paged_attention_f32(const metal_buffer& queries,
                                            const metal_buffer& positions,
                                            const metal_buffer& block_table,
                                            const metal_buffer& block_table_offsets,
                                            const metal_buffer& block_table_lengths,
                                            const metal_buffer& key_cache,
                                            const metal_buffer& value_cache,
                                            metal_buffer& output,
                                            std::size_t rows,
                                            std::size_t query_head_count,
                                            std::size_t kv_head_count,
                                            std::size_t head_dimension,
                                            std::size_t block_size,
                                            std::size_t slot_count,
                                            std::size_t layer,
                                            std::size_t block_table_entry_count) const
{
    const paged_view v { in<std::uint32_t>(positions),
                         in<std::uint32_t>(block_table),
                         in<std::uint32_t>(block_table_offsets),
                         in<std::uint32_t>(block_table_lengths),
                         in<float>(key_cache),
                         in<float>(value_cache),
                         query_head_count,
                         kv_head_count,
                         head_dimension,
                         block_size,
                         slot_count,
                         layer,
                         block_table_entry_count };
    const auto* q = in<float>(queries);
    float* y = out<float>(output);
    const std::size_t group = query_head_count / kv_head_count;

    constexpr std::uint32_t chunk_size = 64;
    const std::uint32_t decode_position = rows == 1 ? v.positions[0] : 0;
    const std::size_t chunk_count = rows == 1 ? decode_position / chunk_size + 1 : 1;
    const bool chunked = chunk_count > 1 && decode_position >= chunk_size - 1;

    for (std::size_t row = 0; row < rows; ++row) {
        const std::uint32_t position = v.positions[row];
        const std::uint32_t table_offset = v.offsets[row];
        if (!v.row_ok(table_offset, v.lengths[row], position))
            continue;       // the kernels return without writing
        for (std::size_t head = 0; head < query_head_count; ++head) {
            const std::size_t query_base = (row * query_head_count + head) * head_dimension;
            const std::size_t kv_head = head / group;
            if (!chunked) {
                running_softmax state;
                attend_range(v, q + query_base, table_offset, kv_head, 0, position + 1, state);
                for (std::size_t f = 0; f < head_dimension; ++f)
                    y[query_base + f] = state.accumulator[f] / state.denominator;
                continue;
            }
            std::vector<running_softmax> parts(chunk_count);
            for (std::size_t chunk = 0; chunk < chunk_count; ++chunk) {
                const std::uint32_t begin = std::uint32_t(chunk) * chunk_size;
                const std::uint32_t end = std::min(position + 1, begin + chunk_size);
                if (begin >= end) {
                    parts[chunk].accumulator.assign(head_dimension, 0.0F);
                    continue;
                }
                attend_range(v, q + query_base, table_offset, kv_head, begin, end, parts[chunk]);
            }
            float global_max = -std::numeric_limits<float>::infinity();
            for (const auto& part : parts)
                global_max = std::max(global_max, part.maximum);
            std::vector<float> scales(chunk_count);
            float denominator = 0.0F;
            for (std::size_t chunk = 0; chunk < chunk_count; ++chunk) {
                scales[chunk] = std::exp(parts[chunk].maximum - global_max);
                denominator += parts[chunk].denominator * scales[chunk];
            }
            for (std::size_t f = 0; f < head_dimension; ++f) {
                float accumulator = 0.0F;
                for (std::size_t chunk = 0; chunk < chunk_count; ++chunk)
                    accumulator += parts[chunk].accumulator[f] * scales[chunk];
                y[query_base + f] = accumulator / denominator;
            }
        }
    }
    return {};
}

// paged_flash_attention_prefill_f32 (src/metal/kernels/attention.metal:246-444):
// a tile of up to 8 query rows against key tiles of 16; masked scores are
// -inf; one maximum and one rescale per key tile.  Head sizes above
// 4 * simd width (128) fall back as the host side does
// (src/metal/metal_kernels_attention.mm:72-82).
result<void, metal_error>
metal_kernels::dispatch_paged_flash_attention_prefill_f32(const metal_buffer& queries,
                                                          const metal_buffer& positions,
                                                          const metal_buffer& block_table,
                                                          const metal_buffer& block_table_offsets,
                                                          const metal_buffer& block_table_lengths,
                                                          const metal_buffer& key_cache,
                                                          const metal_buffer& value_cache,
                                                          const metal_buffer& query_tile_starts,
                                                          const metal_buffer& query_tile_lengths,
                                                          metal_buffer& output,
                                                          std::size_t rows,
                                                          std::size_t query_head_count,
                                                          std::size_t kv_head_count,
                                                          std::size_t head_dimension,
                                                          std::size_t block_size,
                                                          std::size_t slot_count,
                                                          std::size_t layer,
                                                          std::size_t block_table_entry_count,
                                                          std::size_t query_tile_count) const
{
    if (head_dimension > 128)
        return dispatch_paged_attention_f32(queries, positions, block_table, block_table_offsets,
                                            block_table_lengths, key_cache, value_cache, output,
                                            rows, query_head_count, kv_head_count, head_dimension,
                                            block_size, slot_count, layer, block_table_entry_count);
    if (query_tile_count == 0
        || query_tile_starts.size_bytes() < query_tile_count * sizeof(std::uint32_t)
        || query_tile_lengths.size_bytes() < query_tile_count * sizeof(std::uint32_t))
        return refuse("paged FlashAttention dimensions are invalid");
    const paged_view v { in<std::uint32_t>(positions),
                         in<std::uint32_t>(block_table),
                         in<std::uint32_t>(block_table_offsets),
                         in<std::uint32_t>(block_table_lengths),
                         in<float>(key_cache),
                         in<float>(value_cache),
                         query_head_count,
                         kv_head_count,
                         head_dimension,
                         block_size,
                         slot_count,
                         layer,
                         block_table_entry_count };
    const auto* q = in<float>(queries);
    const auto* starts = in<std::uint32_t>(query_tile_starts);
    const auto* lengths = in<std::uint32_t>(query_tile_lengths);
    float* y = out<float>(output);
    constexpr std::uint32_t query_tile_size = 8;
    constexpr std::uint32_t key_tile_size = 16;
    const std::size_t group = query_head_count / kv_head_count;
    const float attention_scale = 1.0F / std::sqrt(float(head_dimension));
    const float minus_infinity = -std::numeric_limits<float>::infinity();

    for (std::size_t tile = 0; tile < query_tile_count; ++tile) {
        const std::uint32_t row_start = starts[tile];
        const std::uint32_t tile_rows = lengths[tile];
        if (tile_rows == 0 || tile_rows > query_tile_size || row_start >= rows
            || tile_rows > rows - row_start)
            continue;
        const std::uint32_t table_offset = v.offsets[row_start];
        const std::uint32_t final_position = v.positions[row_start + tile_rows - 1];
        if (!v.row_ok(table_offset, v.lengths[row_start], final_position))
            continue;
        for (std::size_t head = 0; head < query_head_count; ++head) {
            const std::size_t kv_head = head / group;
            std::vector<float> accumulators(std::size_t(tile_rows) * head_dimension, 0.0F);
            float maxima[query_tile_size], sums[query_tile_size], rescales[query_tile_size];
            float scores[query_tile_size * key_tile_size];
            for (std::uint32_t query = 0; query < query_tile_size; ++query) {
                maxima[query] = minus_infinity;
                sums[query] = 0.0F;
            }
            for (std::uint32_t key_begin = 0; key_begin <= final_position; key_begin += key_tile_size) {
                const std::uint32_t tile_keys = std::min(key_tile_size, final_position + 1 - key_begin);
                for (std::uint32_t key = 0; key < tile_keys; ++key) {
                    const std::uint32_t token = key_begin + key;
                    const std::size_t base = v.cache_base(table_offset, token, kv_head);
                    for (std::uint32_t query = 0; query < tile_rows; ++query) {
                        const float* qv =
                            q + ((row_start + query) * query_head_count + head) * head_dimension;
                        float score = 0.0F;
                        for (std::size_t f = 0; f < head_dimension; ++f)
                            score += qv[f] * v.keys[base + f];
                        score *= attention_scale;
                        scores[query * key_tile_size + key] =
                            token <= v.positions[row_start + query] ? score : minus_infinity;
                    }
                }
                for (std::uint32_t query = 0; query < tile_rows; ++query) {
                    float tile_maximum = minus_infinity;
                    for (std::uint32_t key = 0; key < tile_keys; ++key)
                        tile_maximum = std::max(tile_maximum, scores[query * key_tile_size + key]);
                    const float new_maximum = std::max(maxima[query], tile_maximum);
                    const float old_rescale = std::exp(maxima[query] - new_maximum);
                    float tile_sum = 0.0F;
                    for (std::uint32_t key = 0; key < tile_keys; ++key) {
                        const float weight = std::exp(scores[query * key_tile_size + key] - new_maximum);
                        scores[query * key_tile_size + key] = weight;
                        tile_sum += weight;
                    }
                    maxima[query] = new_maximum;
                    sums[query] = sums[query] * old_rescale + tile_sum;
                    rescales[query] = old_rescale;
                }
                for (std::size_t f = 0; f < head_dimension; ++f) {
                    for (std::uint32_t query = 0; query < tile_rows; ++query)
                        accumulators[query * head_dimension + f] *= rescales[query];
                    for (std::uint32_t key = 0; key < tile_keys; ++key) {
                        const float value =
                            v.values[v.cache_base(table_offset, key_begin + key, kv_head) + f];
                        for (std::uint32_t query = 0; query < tile_rows; ++query)
                            accumulators[query * head_dimension + f] +=
                                scores[query * key_tile_size + key] * value;
                    }
                }
            }
            for (std::uint32_t query = 0; query < tile_rows; ++query) {
                float* o = y + ((row_start + query) * query_head_count + head) * head_dimension;
                for (std::size_t f = 0; f < head_dimension; ++f)
                    o[f] = accumulators[query * head_dimension + f] / sums[query];
            }
        }
    }
    return {};
}

// Row gather, final norm in place, vocabulary product with the best (score,
// index) of every 64 outputs, then the best of those; equal scores go to the
// lower index (src/metal/kernels/sampling.metal:11-22,24-104,131-170; host
// side src/metal/metal_kernels_linear.mm:298-403).
result<void, metal_error>
metal_kernels::dispatch_greedy_vocabulary(const metal_buffer& hidden_states,
                                          const metal_buffer& row_indices,
                                          const metal_buffer& norm_weight,
                                          matrix_view vocabulary_weight,
                                          metal_buffer& normalized,
                                          metal_buffer& partial_maxima,
                                          metal_buffer& token_ids,
                                          std::size_t rows,
                                          std::size_t partial_count,
                                          float epsilon,
                                          bool zero_centered) const
{
    if (!vocabulary_weight.supported() || !vocabulary_weight.dense())
        return refuse("the stand-in takes dense bf16 matrices only");
    const auto hidden = vocabulary_weight.shape().dimensions()[1];
    const auto vocabulary = vocabulary_weight.shape().dimensions()[0];
    constexpr std::size_t group_outputs = greedy_argmax_outputs_per_threadgroup;
    if (partial_count != (vocabulary + group_outputs - 1) / group_outputs)
        return refuse("GPU sampling partial buffer has the wrong size");
    const auto* w = in<std::uint16_t>(vocabulary_weight.dense()->buffer());
    const auto* x = in<float>(hidden_states);
    const auto* indices = in<std::uint32_t>(row_indices);
    float* n = out<float>(normalized);
    for (std::size_t row = 0; row < rows; ++row)
        std::memcpy(n + row * hidden, x + std::size_t(indices[row]) * hidden, hidden * sizeof(float));
    rms_norm_rows(n, in<std::uint16_t>(norm_weight), n, rows, hidden, epsilon,
                  zero_centered ? 1.0F : 0.0F);
    struct pair {
        float score;
        std::uint32_t index;
    };
    auto* partials = reinterpret_cast<pair*>(partial_maxima.bytes().data());
    auto* ids = out<std::uint32_t>(token_ids);
    const auto better = [](float score, std::uint32_t index, const pair& best) {
        return score > best.score || (score == best.score && index < best.index);
    };
    for (std::size_t row = 0; row < rows; ++row) {
        for (std::size_t part = 0; part < partial_count; ++part) {
            pair best { -std::numeric_limits<float>::infinity(), 0xffffffffU };
            for (std::size_t local = 0; local < group_outputs; ++local) {
                const std::size_t feature = part * group_outputs + local;
                if (feature >= vocabulary)
                    break;
                const float score = dot_row(n + row * hidden, w, hidden, feature);
                if (better(score, std::uint32_t(feature), best))
                    best = { score, std::uint32_t(feature) };
            }
            partials[row * partial_count + part] = best;
        }
        pair best { -std::numeric_limits<float>::infinity(), 0xffffffffU };
        for (std::size_t part = 0; part < partial_count; ++part) {
            const pair& candidate = partials[row * partial_count + part];
            if (better(candidate.score, candidate.index, best))
                best = candidate;
        }
        ids[row] = best.index;
    }
    return {};
}

// ------------------------------------------------------------------ not on this path
// The other architecture's kernels (src/metal/kernels/deltanet.metal) are not
// restated; reaching one is an error, not a wrong number.
result<void, metal_error>
metal_kernels::dispatch_causal_conv1d_silu(const metal_buffer&, const metal_buffer&, metal_buffer&,
                                           metal_buffer&, std::size_t, std::size_t, std::size_t,
                                           std::size_t) const
{
    return refuse("not restated in the CPU stand-in");
}

result<void, metal_error>
metal_kernels::dispatch_gated_delta_rule(const metal_buffer&, const metal_buffer&,
                                         const metal_buffer&, const metal_buffer&,
                                         const metal_buffer&, metal_buffer&, metal_buffer&,
                                         std::size_t, std::size_t, std::size_t, std::size_t,
                                         std::size_t, float, std::size_t, bool) const
{
    return refuse("not restated in the CPU stand-in");
}

result<void, metal_error>
metal_kernels::dispatch_rms_norm_gated(const metal_buffer&, const metal_buffer&,
                                       const metal_buffer&, metal_buffer&, std::size_t,
                                       std::size_t, float) const
{
    return refuse("not restated in the CPU stand-in");
}

} // namespace chibillm
