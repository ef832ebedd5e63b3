// Plain C++ restatements of the device operations, one loop nest each, 32-bit throughout.
//
// They stand beside the CUDA kernels as what each kernel has to compute: same arguments (paged
// caches, block tables, the step's index arrays), no tiling, no fusion, no reordering of sums
// beyond index order.  Nothing on the path of generation calls them: the tests compare every
// kernel with them (and them with the PyTorch restatements) at small, odd sizes.  The formulas are
// those of the reference's kernels, cited at each function.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <vector>

#if defined(_WIN32)
#define REF_API extern "C" __declspec(dllexport)
#else
#define REF_API extern "C" __attribute__((visibility("default")))
#endif

// out[t, :] = table[tokens[t], :]  (src/metal/kernels/tensor_ops.metal:12-24).  Returns the number of
// token ids outside [0, vocab) (their rows are left untouched).
REF_API int chibi_ref_embed(const int* tokens, const float* table, float* out, long long T, int hidden, int vocab)
{
    int bad = 0;
    for (long long t = 0; t < T; ++t) {
        if (tokens[t] < 0 || tokens[t] >= vocab) {
            ++bad;
            continue;
        }
        for (int j = 0; j < hidden; ++j)
            out[t * hidden + j] = table[(long long)tokens[t] * hidden + j];
    }
    return bad;
}

// Every run of n values is one group: y = (x * rsqrt(mean(x^2) + eps)) * (w + offset)
// (src/metal/kernels/tensor_ops.metal:76-105; the product with the statistic comes first).
REF_API void chibi_ref_rmsnorm(const float* x, const float* w, float* out, long long groups, int n, float eps,
                               float offset)
{
    for (long long g = 0; g < groups; ++g) {
        float ss = 0.f;
        for (int j = 0; j < n; ++j)
            ss += x[g * n + j] * x[g * n + j];
        const float inv = 1.f / std::sqrt(ss / (float)n + eps);
        for (int j = 0; j < n; ++j)
            out[g * n + j] = (x[g * n + j] * inv) * (w[j] + offset);
    }
}

// out[m, n] = sum_k x[m, k] * w[n, k] (+ residual[m, n]); w is stored [out, in]
// (src/metal/kernels/linear.metal:136-156).  out may be the residual itself.
REF_API void chibi_ref_linear(const float* x, const float* w, const float* residual, float* out, long long M, int N,
                              int K)
{
    for (long long m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            float acc = 0.f;
            for (int k = 0; k < K; ++k)
                acc += x[m * K + k] * w[(long long)n * K + k];
            out[m * N + n] = residual ? residual[m * N + n] + acc : acc;
        }
}

// out[t, i] = silu(gate[t, i]) * up[t, i] with gate_up = [gate | up]
// (src/tensor/functions.cc:241-252; src/metal/kernels/tensor_ops.metal:120-123).
REF_API void chibi_ref_swiglu(const float* gate_up, float* out, long long T, int inter)
{
    for (long long t = 0; t < T; ++t)
        for (int i = 0; i < inter; ++i) {
            const float g = gate_up[t * 2 * inter + i], u = gate_up[t * 2 * inter + inter + i];
            out[t * inter + i] = (g / (1.f + std::exp(-g))) * u;
        }
}

// out[r, :] = x[rows[r], :]
REF_API void chibi_ref_gather_rows(const float* x, const int* rows, float* out, int R, int width)
{
    for (int r = 0; r < R; ++r)
        for (int j = 0; j < width; ++j)
            out[(long long)r * width + j] = x[(long long)rows[r] * width + j];
}

// Per head of q and k: RMSNorm over the head's d features with one weight for all heads (when
// given), then the split-half rotation of the first `rot` features with angle
// float(position) * inv_freq[j] (src/qwen/qwen_layer.cc:56-101 and :20-30;
// src/metal/kernels/tensor_ops.metal:168-197); q goes to q_out, k and v to the token's slot of the
// paged caches [pages][nkv][page_size][d].  Without caches (k_cache null) qkv holds q only.
// Returns the number of tokens whose block table has no valid page (nothing is written for them).
REF_API int chibi_ref_qk_norm_rope_append(const float* qkv, long long T, float* q_out, float* k_cache, float* v_cache,
                                          const float* q_norm_w, const float* k_norm_w, const float* inv_freq, int rot,
                                          float eps, float offset, const int* positions, const int* seq_of_token,
                                          const int* block_table, int table_stride, int nq, int nkv, int d,
                                          int page_size, int num_pages)
{
    const bool append = k_cache != nullptr;
    const int width = append ? (nq + 2 * nkv) * d : nq * d;
    int bad = 0;
    std::vector<float> x(d);
    for (long long t = 0; t < T; ++t) {
        const int pos = positions[t];
        long long slot = -1;
        if (append) {
            const int page = block_table[(long long)seq_of_token[t] * table_stride + pos / page_size];
            if (page < 0 || page >= num_pages)
                ++bad;
            else
                slot = ((long long)page * nkv * page_size + pos % page_size) * d;
        }
        const int heads = append ? nq + 2 * nkv : nq;
        for (int h = 0; h < heads; ++h) {
            const float* src = qkv + t * width + (long long)h * d;
            const bool is_q = h < nq, is_v = h >= nq + nkv;
            if (!is_q && slot < 0)
                continue;
            for (int j = 0; j < d; ++j)
                x[j] = src[j];
            const float* w = is_q ? q_norm_w : k_norm_w;
            if (!is_v && w) {
                float ss = 0.f;
                for (int j = 0; j < d; ++j)
                    ss += x[j] * x[j];
                const float inv = 1.f / std::sqrt(ss / (float)d + eps);
                for (int j = 0; j < d; ++j)
                    x[j] = (x[j] * inv) * (w[j] + offset);
            }
            if (!is_v) {
                const int half = rot / 2;
                for (int j = 0; j < half; ++j) {
                    const float a = (float)pos * inv_freq[j];
                    const float c = std::cos(a), s = std::sin(a);
                    const float x0 = x[j], x1 = x[j + half];
                    x[j] = x0 * c - x1 * s;
                    x[j + half] = x1 * c + x0 * s;
                }
            }
            float* dst;
            if (is_q)
                dst = q_out + (t * nq + h) * d;
            else if (!is_v)
                dst = k_cache + slot + (long long)(h - nq) * page_size * d;
            else
                dst = v_cache + slot + (long long)(h - nq - nkv) * page_size * d;
            for (int j = 0; j < d; ++j)
                dst[j] = x[j];
        }
    }
    return bad;
}

// Causal grouped-query attention of every token over its sequence's pages: token t of sequence s
// at position p sees keys max(0, p - window + 1) .. p (all of 0 .. p without a window); query head h
// reads kv head h / (nq / nkv); softmax in 32-bit over scale * (q . k)
// (src/metal/kernels/attention.metal:81-158).  Returns the number of page ids outside the pool.
REF_API int chibi_ref_attention(const float* q, const float* k_cache, const float* v_cache, float* out,
                                const int* block_table, int table_stride, const int* positions,
                                const int* seq_of_token, long long T, int nq, int nkv, int d, int page_size,
                                int num_pages, float scale, int window)
{
    const int group = nq / nkv;
    int bad = 0;
    std::vector<float> score, acc(d);
    for (long long t = 0; t < T; ++t) {
        const int pos = positions[t];
        const int first = window > 0 && pos - window + 1 > 0 ? pos - window + 1 : 0;
        const int* table = block_table + (long long)seq_of_token[t] * table_stride;
        for (int h = 0; h < nq; ++h) {
            const int kvh = h / group;
            const float* qv = q + (t * nq + h) * d;
            score.assign(pos - first + 1, 0.f);
            float mx = -std::numeric_limits<float>::infinity();
            bool ok = true;
            for (int key = first; key <= pos; ++key) {
                const int page = table[key / page_size];
                if (page < 0 || page >= num_pages) {
                    ok = false;
                    break;
                }
                const float* kv = k_cache + (((long long)page * nkv + kvh) * page_size + key % page_size) * d;
                float dot = 0.f;
                for (int j = 0; j < d; ++j)
                    dot += qv[j] * kv[j];
                score[key - first] = dot * scale;
                mx = std::max(mx, score[key - first]);
            }
            if (!ok) {
                ++bad;
                continue;
            }
            float sum = 0.f;
            std::fill(acc.begin(), acc.end(), 0.f);
            for (int key = first; key <= pos; ++key) {
                const float p = std::exp(score[key - first] - mx);
                sum += p;
                const int page = table[key / page_size];
                const float* vv = v_cache + (((long long)page * nkv + kvh) * page_size + key % page_size) * d;
                for (int j = 0; j < d; ++j)
                    acc[j] += p * vv[j];
            }
            for (int j = 0; j < d; ++j)
                out[(t * nq + h) * d + j] = acc[j] / sum;
        }
    }
    return bad;
}

// Greedy rows (no temperature given, or temperature <= 0): the arg max, ties to the lowest id
// (src/metal/kernels/sampling.metal:55-60,145-149).  Other rows: the inverse CDF of
// softmax(logits / temperature) at uniform[r], probabilities and their running sum in 64-bit;
// the last id if rounding leaves the sum below the uniform.
REF_API void chibi_ref_sample(const float* logits, long long stride, int rows, int vocab, const float* temperature,
                              const float* uniform, int* out)
{
    for (int r = 0; r < rows; ++r) {
        const float* row = logits + (long long)r * stride;
        int best = 0;
        for (int i = 1; i < vocab; ++i)
            if (row[i] > row[best])
                best = i;
        if (!temperature || temperature[r] <= 0.f) {
            out[r] = best;
            continue;
        }
        const double t = temperature[r];
        double total = 0.0;
        for (int i = 0; i < vocab; ++i)
            total += std::exp(((double)row[i] - (double)row[best]) / t);
        const double target = (double)uniform[r] * total;
        double run = 0.0;
        int pick = vocab - 1;
        for (int i = 0; i < vocab; ++i) {
            run += std::exp(((double)row[i] - (double)row[best]) / t);
            if (run > target) {
                pick = i;
                break;
            }
        }
        out[r] = pick;
    }
}
