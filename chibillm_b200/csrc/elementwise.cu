// Row-wise kernels: embedding gather, RMSNorm, the fused per-head norm +
// rotation + cache append, SwiGLU, row gather, casts.  All statistics, angles
// and activations are computed in 32-bit; element types of inputs, weights and
// outputs are template parameters so the same code serves the bfloat16 and the
// 32-bit engine.
#define CHIBI_UNIT elementwise
#define CHIBI_UNIT_ID 1
#include "common.cuh"

namespace chibi {

// ---------------------------------------------------------------- embedding
// out[t, :] = float(table[token[t], :]).  Ids outside the table leave zeros and
// raise the error word (the host checks ids before the launch; this guard only
// keeps a bad id from reading outside the table).
template <typename TW, typename TO>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                             TO* __restrict__ out, int hidden, int vocab, int* __restrict__ error)
{
    pdl_enter();
    const int t = blockIdx.x;
    const int id = tokens[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0 && error)
        atomicExch(error, 1);
    const TW* row = table + (size_t)(ok ? id : 0) * hidden;
    TO* dst = out + (size_t)t * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x)
        dst[j] = from_f32<TO>(ok ? to_f32(row[j]) : 0.f);
}

// ---------------------------------------------------------------- RMSNorm
// One block per group of n features: inv = rsqrt(sum(x^2)/n + eps);
// y = (x * inv) * (w + offset).
template <typename TX, typename TW, typename TO>
__global__ void rmsnorm_kernel(const TX* x, const TW* __restrict__ w, TO* out,   // out may be x
                               int n, long long x_stride,
                               long long out_stride, float eps, float offset)
{
    pdl_enter();
    __shared__ float scratch[33];
    const TX* row = x + (size_t)blockIdx.x * x_stride;
    TO* dst = out + (size_t)blockIdx.x * out_stride;
    float s = 0.f;
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        const float v = to_f32(row[j]);
        s = fmaf(v, v, s);
    }
    s = block_sum(s, scratch);
    const float inv = rsqrtf(s / (float)n + eps);
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        const float v = to_f32(row[j]);
        dst[j] = from_f32<TO>((v * inv) * (to_f32(w[j]) + offset));
    }
}

// The same for 32-bit rows and bfloat16 weights and output, n a multiple of 4
// and at most 16 * blockDim.x: the row stays in registers between the two passes.
__global__ void __launch_bounds__(512)
rmsnorm_f32_bf16_kernel(const float* x, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* out, int n,
                        long long x_stride, long long out_stride, float eps, float offset)
{
    pdl_enter();
    __shared__ float scratch[33];
    const float4* row = reinterpret_cast<const float4*>(x + (size_t)blockIdx.x * x_stride);
    __nv_bfloat16* dst = out + (size_t)blockIdx.x * out_stride;
    const int n4 = n >> 2;
    float4 v[4];
    uint2 wq[4];                  // the weights travel together with the row, not after the sum
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int j = threadIdx.x + i * blockDim.x;
        v[i] = j < n4 ? row[j] : make_float4(0.f, 0.f, 0.f, 0.f);
        wq[i] = j < n4 ? *reinterpret_cast<const uint2*>(w + 4 * j) : make_uint2(0u, 0u);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        s = fmaf(v[i].x, v[i].x, s);
        s = fmaf(v[i].y, v[i].y, s);
        s = fmaf(v[i].z, v[i].z, s);
        s = fmaf(v[i].w, v[i].w, s);
    }
    s = block_sum(s, scratch);
    const float inv = rsqrtf(s / (float)n + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int j = threadIdx.x + i * blockDim.x;
        if (j < n4) {
            const uint2 wv = wq[i];
            const __nv_bfloat162 w01 = *reinterpret_cast<const __nv_bfloat162*>(&wv.x);
            const __nv_bfloat162 w23 = *reinterpret_cast<const __nv_bfloat162*>(&wv.y);
            const __nv_bfloat162 o01 = __floats2bfloat162_rn((v[i].x * inv) * (__low2float(w01) + offset),
                                                             (v[i].y * inv) * (__high2float(w01) + offset));
            const __nv_bfloat162 o23 = __floats2bfloat162_rn((v[i].z * inv) * (__low2float(w23) + offset),
                                                             (v[i].w * inv) * (__high2float(w23) + offset));
            uint2 ov;
            ov.x = *reinterpret_cast<const uint32_t*>(&o01);
            ov.y = *reinterpret_cast<const uint32_t*>(&o23);
            *reinterpret_cast<uint2*>(dst + 4 * j) = ov;
        }
    }
}

// ------------------------------------------- per-head norm + rotation + append
// grid (tokens, ceil(jobs / warps)), one warp per head job.  Jobs 0..nq-1 are
// query heads, nq..nq+nkv-1 key heads, the rest value heads.  Query and key
// heads are normalised over their d features (when a norm weight is given),
// rotated (split-half pairs (j, j + rot/2), angle = float(pos) * inv_freq[j];
// the block computes the token's cosines and sines once) and written to q_out
// or to the key cache; value heads are copied to the value cache.  Cache
// layout: [page][kv_head][slot][d]; page = block_table[row][pos / page_size],
// slot = pos % page_size.
template <typename TX, typename TW, typename TC>
__global__ void qk_norm_rope_append_kernel(
    const TX* __restrict__ qkv, long long qkv_stride, TX* __restrict__ q_out,
    TC* __restrict__ k_cache, TC* __restrict__ v_cache, const TW* __restrict__ q_norm_w,
    const TW* __restrict__ k_norm_w, const float* __restrict__ inv_freq,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ seq_rows, const int* __restrict__ block_table, int table_stride, int nq,
    int nkv, int d, int rot, int page_size, int num_pages, float eps, float norm_offset, int append,
    int* __restrict__ error)
{
    pdl_enter();
    extern __shared__ float smem[];
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    const int half = rot >> 1;
    float* cs = smem;                       // [half] cosines, [half] sines
    float* buf = smem + 2 * half + (size_t)warp * d;
    const int pos = positions[t];
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float a = (float)pos * inv_freq[j];
        float sn, c;
        sincosf(a, &sn, &c);
        cs[j] = c;
        cs[half + j] = sn;
    }
    __syncthreads();
    const int jobs = append ? nq + 2 * nkv : nq;
    const int job = blockIdx.y * warps + warp;
    if (job >= jobs)
        return;
    const TX* src = qkv + (size_t)t * qkv_stride + (size_t)job * d;   // q | k | v are consecutive columns
    const bool is_q = job < nq;
    const bool is_k = !is_q && job < nq + nkv;
    const int head = is_q ? job : (is_k ? job - nq : job - nq - nkv);

    long long cache_base = -1;
    if (!is_q) {
        const int seq = seq_of_token[t];
        const int table_row = seq_rows ? seq_rows[seq] : seq;
        const int page = block_table[(size_t)table_row * table_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0 && error)
                atomicExch(error, 2);
            return;
        }
        cache_base = (((long long)page * nkv + head) * page_size + (pos % page_size)) * d;
    }
    if (!is_q && !is_k) {
        TC* dst = v_cache + cache_base;
        for (int j = lane; j < d; j += 32)
            dst[j] = from_f32<TC>(to_f32(src[j]));
        return;
    }
    const TW* w = is_q ? q_norm_w : k_norm_w;
    float s = 0.f;
    for (int j = lane; j < d; j += 32) {
        const float v = to_f32(src[j]);
        buf[j] = v;
        s = fmaf(v, v, s);
    }
    s = warp_sum(s);
    __syncwarp();
    if (w) {
        const float inv = rsqrtf(s / (float)d + eps);
        for (int j = lane; j < d; j += 32)
            buf[j] = (buf[j] * inv) * (to_f32(w[j]) + norm_offset);
        __syncwarp();
    }
    // every lane reads its pairs before any lane writes (d <= 256: at most 4 pairs per lane)
    float lo[4], hi[4];
    int cnt = 0;
    for (int j = lane; j < half; j += 32, ++cnt) {
        const float c = cs[j], sn = cs[half + j];
        const float x0 = buf[j], x1 = buf[j + half];
        lo[cnt] = x0 * c - x1 * sn;
        hi[cnt] = x1 * c + x0 * sn;
    }
    __syncwarp();
    cnt = 0;
    for (int j = lane; j < half; j += 32, ++cnt) {
        buf[j] = lo[cnt];
        buf[j + half] = hi[cnt];
    }
    __syncwarp();
    if (is_q) {
        TX* dst = q_out + ((size_t)t * nq + head) * d;
        for (int j = lane; j < d; j += 32)
            dst[j] = from_f32<TX>(buf[j]);
    } else {
        TC* dst = k_cache + cache_base;
        for (int j = lane; j < d; j += 32)
            dst[j] = from_f32<TC>(buf[j]);
    }
}

// The same with four features per lane (d a multiple of 4) and, optionally, the
// input given as the partial sums of a split matrix product: `splits` arrays of
// 32-bit [tokens, row stride], `split_stride` values apart, added in split order.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4])
    {
        const float4 q = *reinterpret_cast<const float4*>(p);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4])
    {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4])
    {
        const uint2 q = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4])
    {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 q;
        q.x = *reinterpret_cast<const uint32_t*>(&a);
        q.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = q;
    }
};

// A row copied with a change of type, four features per thread and step (n a
// multiple of 4, rows 16-byte aligned); a thread's loads all go out before its
// stores.  Used by the embedding (row = table[token]) and the row gather.
template <typename TX, typename TO>
__device__ __forceinline__ void copy_row_vec4(const TX* __restrict__ src, TO* __restrict__ dst, int n, bool ok)
{
    const int n4 = n >> 2;
    for (int j0 = threadIdx.x; j0 < n4; j0 += 4 * blockDim.x) {
        float v[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = j0 + u * blockDim.x;
            if (ok && j < n4)
                Vec4<TX>::load(src + 4 * j, v[u]);
            else
                v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = j0 + u * blockDim.x;
            if (j < n4)
                Vec4<TO>::store(dst + 4 * j, v[u]);
        }
    }
}

template <typename TW, typename TO>
__global__ void embed_vec4_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                  TO* __restrict__ out, int hidden, int vocab, int* __restrict__ error)
{
    pdl_enter();
    const int id = tokens[blockIdx.x];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0 && error)
        atomicExch(error, 1);
    copy_row_vec4(table + (size_t)(ok ? id : 0) * hidden, out + (size_t)blockIdx.x * hidden, hidden, ok);
}

template <typename TX, typename TO>
__global__ void gather_rows_vec4_kernel(const TX* __restrict__ x, const int* __restrict__ rows,
                                        TO* __restrict__ out, int n, long long x_rows)
{
    pdl_enter();
    const int r = rows[blockIdx.x];
    const bool ok = r >= 0 && r < x_rows;
    copy_row_vec4(x + (size_t)(ok ? r : 0) * n, out + (size_t)blockIdx.x * n, n, ok);
}

// JPW head jobs per warp.  Every launch uses 1 (as many warps as possible side by
// side); more per warp measured slower, and many tokens with 128-feature heads
// take the per-token kernel below.
template <int JPW, typename TX, typename TQ, typename TW, typename TC>
__global__ void qk_norm_rope_append_vec4_kernel(
    const TX* __restrict__ qkv, long long qkv_stride, int splits, long long split_stride,
    TQ* __restrict__ q_out, TC* __restrict__ k_cache, TC* __restrict__ v_cache,
    const TW* __restrict__ q_norm_w, const TW* __restrict__ k_norm_w,
    const float* __restrict__ inv_freq, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ seq_rows,
    const int* __restrict__ block_table, int table_stride, int nq, int nkv, int d, int rot,
    int page_size, int num_pages, float eps, float norm_offset, int append, int* __restrict__ error)
{
    pdl_trigger();
    extern __shared__ float smem[];
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    const int half = rot >> 1;
    float* cs = smem;
    float* buf = smem + 2 * half + (size_t)warp * JPW * d;
    // The step's index arrays and the block table were written before the step's first
    // kernel: the token's cache slot and its cosines and sines are worked out while the
    // kernel before this one still runs.
    const int pos = positions[t];
    const int jobs = append ? nq + 2 * nkv : nq;
    const int job0 = (blockIdx.y * warps + warp) * JPW;
    long long cache_base = -1;                // the token's slot in the caches, head 0
    if (append && job0 + JPW > nq) {
        const int seq = seq_of_token[t];
        const int table_row = seq_rows ? seq_rows[seq] : seq;
        const int page = block_table[(size_t)table_row * table_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0 && error)
                atomicExch(error, 2);
        } else {
            cache_base = ((long long)page * nkv * page_size + (pos % page_size)) * d;
        }
    }
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float a = (float)pos * inv_freq[j];
        float sn, c;
        sincosf(a, &sn, &c);
        cs[j] = c;
        cs[half + j] = sn;
    }
    pdl_wait();
    float s[JPW];
#pragma unroll
    for (int jj = 0; jj < JPW; ++jj) {
        s[jj] = 0.f;
        const int job = job0 + jj;
        if (job >= jobs)
            continue;
        const bool is_v = job >= nq + nkv;
        if (job >= nq && cache_base < 0)
            continue;
        const TX* src = qkv + (size_t)t * qkv_stride + (size_t)job * d;
        for (int j = lane * 4; j < d; j += 128) {
            float v[4];
            Vec4<TX>::load(src + j, v);
            for (int sp0 = 1; sp0 < splits; sp0 += 8) {      // eight loads in flight, added in split order
                float q[8][4];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (sp0 + u < splits)
                        Vec4<TX>::load(src + (sp0 + u) * split_stride + j, q[u]);
                    else
                        q[u][0] = q[u][1] = q[u][2] = q[u][3] = 0.f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    v[0] += q[u][0]; v[1] += q[u][1]; v[2] += q[u][2]; v[3] += q[u][3];
                }
            }
            if (is_v) {
                Vec4<TC>::store(v_cache + cache_base + (long long)(job - nq - nkv) * page_size * d + j, v);
            } else {
                float* b = buf + jj * d;
                b[j] = v[0]; b[j + 1] = v[1]; b[j + 2] = v[2]; b[j + 3] = v[3];
                s[jj] = fmaf(v[0], v[0], s[jj]);
                s[jj] = fmaf(v[1], v[1], s[jj]);
                s[jj] = fmaf(v[2], v[2], s[jj]);
                s[jj] = fmaf(v[3], v[3], s[jj]);
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int jj = 0; jj < JPW; ++jj) {
        const int job = job0 + jj;
        if (job >= jobs || job >= nq + nkv)
            continue;
        const bool is_q = job < nq;
        if (!is_q && cache_base < 0)
            continue;
        float* b = buf + jj * d;
        const TW* w = is_q ? q_norm_w : k_norm_w;
        const float sum = warp_sum(s[jj]);
        if (w) {
            const float inv = rsqrtf(sum / (float)d + eps);
            for (int j = lane; j < d; j += 32)
                b[j] = (b[j] * inv) * (to_f32(w[j]) + norm_offset);
            __syncwarp();
        }
        float lo[4], hi[4];
        int cnt = 0;
        for (int j = lane; j < half; j += 32, ++cnt) {
            const float c = cs[j], sn = cs[half + j];
            const float x0 = b[j], x1 = b[j + half];
            lo[cnt] = x0 * c - x1 * sn;
            hi[cnt] = x1 * c + x0 * sn;
        }
        __syncwarp();
        cnt = 0;
        for (int j = lane; j < half; j += 32, ++cnt) {
            b[j] = lo[cnt];
            b[j + half] = hi[cnt];
        }
        __syncwarp();
        for (int j = lane * 4; j < d; j += 128) {
            const float v[4] = { b[j], b[j + 1], b[j + 2], b[j + 3] };
            if (is_q)
                Vec4<TQ>::store(q_out + ((size_t)t * nq + job) * d + j, v);
            else
                Vec4<TC>::store(k_cache + cache_base + (long long)(job - nq) * page_size * d + j, v);
        }
    }
}

// Many tokens, heads of 128 features rotated whole: one block of eight warps per
// token; the heads stay in registers.  A lane holds features 4*lane .. 4*lane+3 of a head, so
// the partner of a feature in the rotation (64 features away) sits 16 lanes away
// and comes by one shuffle.  Warp w takes heads w, w+8, ...  The token's cache
// slot, the norm weights and its cosines and sines (once per block, in shared
// memory) are ready before the kernel waits for the q | k | v product.
constexpr int ROWS_KERNEL_WARPS = 8;
constexpr int ROWS_KERNEL_MAX_JOBS = 8;       // heads per warp: nq + 2 * nkv <= 64

template <typename TX, typename TW, typename TC>
__global__ void __launch_bounds__(ROWS_KERNEL_WARPS * 32) qk_norm_rope_append_d128_kernel(
    const TX* __restrict__ qkv, long long qkv_stride, TX* __restrict__ q_out, TC* __restrict__ k_cache,
    TC* __restrict__ v_cache, const TW* __restrict__ q_norm_w, const TW* __restrict__ k_norm_w,
    const float* __restrict__ inv_freq, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ seq_rows,
    const int* __restrict__ block_table, int table_stride, int nq, int nkv, int page_size,
    int num_pages, float eps, float norm_offset, int append, int* __restrict__ error)
{
    pdl_trigger();
    constexpr int D = 128;
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[t];
    const int jobs = append ? nq + 2 * nkv : nq;
    long long cache_base = -1;
    if (append) {
        const int seq = seq_of_token[t];
        const int table_row = seq_rows ? seq_rows[seq] : seq;
        const int page = block_table[(size_t)table_row * table_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0 && error)
                atomicExch(error, 2);
        } else {
            cache_base = ((long long)page * nkv * page_size + (pos % page_size)) * D;
        }
    }
    float wq[4], wk[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        wq[u] = q_norm_w ? to_f32(q_norm_w[lane * 4 + u]) + norm_offset : 1.f;
        wk[u] = k_norm_w ? to_f32(k_norm_w[lane * 4 + u]) + norm_offset : 1.f;
    }
    // the token's 64 cosines and sines, each computed once per block
    __shared__ __align__(16) float cs[D];
    if (threadIdx.x < D / 2) {
        float sn, cn;
        sincosf((float)pos * inv_freq[threadIdx.x], &sn, &cn);
        cs[threadIdx.x] = cn;
        cs[D / 2 + threadIdx.x] = sn;
    }
    // all of the above reads what was there before the step's first kernel
    pdl_wait();
    const TX* src = qkv + (size_t)t * qkv_stride + lane * 4;
    float v[ROWS_KERNEL_MAX_JOBS][4];
#pragma unroll
    for (int jj = 0; jj < ROWS_KERNEL_MAX_JOBS; ++jj) {
        const int job = warp + jj * ROWS_KERNEL_WARPS;
        if (job < jobs && (job < nq || cache_base >= 0))
            Vec4<TX>::load(src + (size_t)job * D, v[jj]);
        else
            v[jj][0] = v[jj][1] = v[jj][2] = v[jj][3] = 0.f;
    }
    __syncthreads();
    float c[4], s[4];
    {
        const float4 cv = *reinterpret_cast<const float4*>(cs + (lane & 15) * 4);
        const float4 sv = *reinterpret_cast<const float4*>(cs + D / 2 + (lane & 15) * 4);
        const float sign = lane < 16 ? -1.f : 1.f;     // low half: x0 * c - x1 * s; high half: x1 * c + x0 * s
        c[0] = cv.x; c[1] = cv.y; c[2] = cv.z; c[3] = cv.w;
        s[0] = sign * sv.x; s[1] = sign * sv.y; s[2] = sign * sv.z; s[3] = sign * sv.w;
    }
#pragma unroll
    for (int jj = 0; jj < ROWS_KERNEL_MAX_JOBS; ++jj) {
        const int job = warp + jj * ROWS_KERNEL_WARPS;
        if (job >= jobs || (job >= nq && cache_base < 0))
            continue;
        if (job >= nq + nkv) {
            Vec4<TC>::store(v_cache + cache_base + (long long)(job - nq - nkv) * page_size * D + lane * 4, v[jj]);
            continue;
        }
        const bool is_q = job < nq;
        const bool normed = is_q ? q_norm_w != nullptr : k_norm_w != nullptr;
        float x[4] = { v[jj][0], v[jj][1], v[jj][2], v[jj][3] };
        if (normed) {
            float sum = 0.f;
#pragma unroll
            for (int u = 0; u < 4; ++u)
                sum = fmaf(x[u], x[u], sum);
            sum = warp_sum(sum);
            const float inv = rsqrtf(sum / (float)D + eps);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                x[u] = (x[u] * inv) * (is_q ? wq[u] : wk[u]);
        }
        float out[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float partner = __shfl_xor_sync(0xffffffffu, x[u], 16);
            out[u] = x[u] * c[u] + partner * s[u];
        }
        if (is_q)
            Vec4<TX>::store(q_out + ((size_t)t * nq + job) * D + lane * 4, out);
        else
            Vec4<TC>::store(k_cache + cache_base + (long long)(job - nq) * page_size * D + lane * 4, out);
    }
}

// ---------------------------------------------------------------- SwiGLU
// gate_up[t, 0:I] = gate, gate_up[t, I:2I] = up; out = gate / (1 + exp(-gate)) * up.
template <typename TX, typename TO>
__global__ void swiglu_kernel(const TX* __restrict__ gate_up, TO* __restrict__ out, long long rows,
                              int inter)
{
    pdl_enter();
    const long long total = rows * inter;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / inter;
        const int c = (int)(i - r * inter);
        const float g = to_f32(gate_up[r * 2 * inter + c]);
        const float u = to_f32(gate_up[r * 2 * inter + inter + c]);
        out[i] = from_f32<TO>((g / (1.f + expf(-g))) * u);
    }
}

// bfloat16 in and out, inter a multiple of 8: eight values per thread.
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up,
                                     __nv_bfloat16* __restrict__ out, int inter)
{
    pdl_enter();
    const int chunks = inter >> 3;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= chunks)
        return;
    const size_t row = blockIdx.y;
    const uint4 g = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + 8 * c);
    const uint4 u = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + inter + 8 * c);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 gf = __bfloat1622float2(gp[i]), uf = __bfloat1622float2(up[i]);
        op[i] = __floats2bfloat162_rn((gf.x / (1.f + expf(-gf.x))) * uf.x, (gf.y / (1.f + expf(-gf.y))) * uf.y);
    }
    *reinterpret_cast<uint4*>(out + row * inter + 8 * c) = o;
}

// ---------------------------------------------------------------- row gather
template <typename TX, typename TO>
__global__ void gather_rows_kernel(const TX* __restrict__ x, const int* __restrict__ rows,
                                   TO* __restrict__ out, int n, long long x_rows)
{
    pdl_enter();
    const int r = rows[blockIdx.x];
    const bool ok = r >= 0 && r < x_rows;
    for (int j = threadIdx.x; j < n; j += blockDim.x)
        out[(size_t)blockIdx.x * n + j] = from_f32<TO>(ok ? to_f32(x[(size_t)r * n + j]) : 0.f);
}

// ---------------------------------------------------------------- cast / add
template <typename TX, typename TO>
__global__ void cast_kernel(const TX* __restrict__ x, TO* __restrict__ out, long long total)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(to_f32(x[i]));
}

// acc (32-bit) += x
template <typename TX>
__global__ void add_into_kernel(float* __restrict__ acc, const TX* __restrict__ x, long long total)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x)
        acc[i] += to_f32(x[i]);
}

// updates = [count, (row, index, page) * count]: table[row][index] = page.
__global__ void apply_table_updates_kernel(int* __restrict__ table, int table_stride, int table_rows,
                                           const int* __restrict__ updates, int capacity,
                                           int* __restrict__ error)
{
    pdl_enter();
    int n = updates[0];
    if (n > capacity) {
        n = capacity;
        if (threadIdx.x == 0 && blockIdx.x == 0 && error)
            atomicExch(error, 4);
    }
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int row = updates[1 + 3 * i], index = updates[2 + 3 * i], page = updates[3 + 3 * i];
        if (row < 0 || row >= table_rows || index < 0 || index >= table_stride) {
            if (error)
                atomicExch(error, 4);
            continue;
        }
        table[(size_t)row * table_stride + index] = page;
    }
}

static int grid_for(long long total, int block)
{
    long long g = (total + block - 1) / block;
    if (g > 148LL * 32)
        g = 148LL * 32;
    if (g < 1)
        g = 1;
    return (int)g;
}

} // namespace chibi

using namespace chibi;

CHIBI_API int chibi_embed(const int* tokens, const void* table, int table_type, void* out,
                          int out_type, long long rows, int hidden, int vocab, int* error,
                          cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    const int block = hidden >= 1024 ? 256 : 128;
    const bool vec = hidden % 4 == 0 && (reinterpret_cast<uintptr_t>(table) & 15) == 0
        && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    CHIBI_DISPATCH_TYPE(table_type, TW, CHIBI_DISPATCH_TYPE(out_type, TO, {
        if (vec)
            launch_ordered(embed_vec4_kernel<TW, TO>, dim3((unsigned)rows), dim3(block), 0, stream,
                           tokens, (const TW*)table, (TO*)out, hidden, vocab, error);
        else
            launch_ordered(embed_kernel<TW, TO>, dim3((unsigned)rows), dim3(block), 0, stream,
                           tokens, (const TW*)table, (TO*)out, hidden, vocab, error);
    }));
    return launch_status();
}

CHIBI_API int chibi_rmsnorm(const void* x, int x_type, const void* w, int w_type, void* out,
                            int out_type, long long groups, int n, long long x_stride,
                            long long out_stride, float eps, float offset, cudaStream_t stream)
{
    if (groups <= 0)
        return CHIBI_OK;
    int block = 32;
    while (block < n && block < 512)
        block <<= 1;
    if (x_type == CHIBI_F32 && w_type == CHIBI_BF16 && out_type == CHIBI_BF16 && n % 4 == 0
        && n <= 16 * 512 && x_stride % 4 == 0 && out_stride % 4 == 0
        && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 7) == 0
        && (reinterpret_cast<uintptr_t>(w) & 7) == 0 && x != out) {
        int fast = 32;
        while (fast * 16 < n)
            fast <<= 1;
        if (fast < 128 && n >= 512)
            fast = 128;
        launch(rmsnorm_f32_bf16_kernel, dim3((unsigned)groups), dim3(fast), 0, stream, 
            (const float*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, n, x_stride, out_stride, eps,
            offset);
        return launch_status();
    }
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(w_type, TW, CHIBI_DISPATCH_TYPE(out_type, TO, {
        launch(rmsnorm_kernel<TX, TW, TO>, dim3((unsigned)groups), dim3(block), 0, stream, 
            (const TX*)x, (const TW*)w, (TO*)out, n, x_stride, out_stride, eps, offset);
    })));
    return launch_status();
}

CHIBI_API int chibi_qk_norm_rope_append(
    const void* qkv, int x_type, long long qkv_stride, void* q_out, void* k_cache, void* v_cache,
    int cache_type, const void* q_norm_w, const void* k_norm_w, int w_type, const float* inv_freq,
    const int* positions, const int* seq_of_token, const int* seq_rows, const int* block_table,
    int table_stride,
    long long tokens, int nq, int nkv, int d, int rot, int page_size, int num_pages, float eps,
    float norm_offset, int append, int* error, cudaStream_t stream)
{
    if (tokens <= 0)
        return CHIBI_OK;
    if (d <= 0 || d > 256 || rot < 0 || rot > d || (rot & 1))
        return CHIBI_ERR_UNSUPPORTED;
    const int jobs = append ? nq + 2 * nkv : nq;
    const int warps = jobs < 8 ? jobs : 8;
    const size_t smem = (size_t)(warps * d + rot) * sizeof(float);
    const dim3 grid((unsigned)tokens, (unsigned)((jobs + warps - 1) / warps));
    if (tokens > 2147483647LL || grid.y > 65535)
        return CHIBI_ERR_UNSUPPORTED;
    const bool aligned = d % 4 == 0 && qkv_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(qkv) & 15) == 0
        && (reinterpret_cast<uintptr_t>(q_out) & 15) == 0 && (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0
        && (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0;
    if (aligned && d == 128 && rot == d && tokens >= 32 && jobs <= ROWS_KERNEL_WARPS * ROWS_KERNEL_MAX_JOBS) {
        CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(w_type, TW, CHIBI_DISPATCH_TYPE(cache_type, TC, {
            launch(qk_norm_rope_append_d128_kernel<TX, TW, TC>, dim3((unsigned)tokens),
                   dim3(ROWS_KERNEL_WARPS * 32), 0, stream, (const TX*)qkv, qkv_stride, (TX*)q_out, (TC*)k_cache,
                   (TC*)v_cache, (const TW*)q_norm_w, (const TW*)k_norm_w, inv_freq, positions, seq_of_token,
                   seq_rows, block_table, table_stride, nq, nkv, page_size, num_pages, eps, norm_offset, append,
                   error);
        })));
        return launch_status();
    }
    if (aligned) {
        // one head per warp: four per warp measured slower at 2,048 tokens (68 us against 51 us)
        const dim3 grid4((unsigned)tokens, (unsigned)((jobs + warps - 1) / warps));
        const size_t smem4 = (size_t)(warps * d + rot) * sizeof(float);
        CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(w_type, TW, CHIBI_DISPATCH_TYPE(cache_type, TC, {
            launch(qk_norm_rope_append_vec4_kernel<1, TX, TX, TW, TC>, dim3(grid4), dim3(warps * 32), smem4,
                   stream, (const TX*)qkv, qkv_stride, 1, 0, (TX*)q_out, (TC*)k_cache, (TC*)v_cache,
                   (const TW*)q_norm_w, (const TW*)k_norm_w, inv_freq, positions, seq_of_token, seq_rows,
                   block_table, table_stride, nq, nkv, d, rot, page_size, num_pages, eps, norm_offset,
                   append, error);
        })));
        return launch_status();
    }
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(w_type, TW, CHIBI_DISPATCH_TYPE(cache_type, TC, {
        launch(qk_norm_rope_append_kernel<TX, TW, TC>, dim3(grid), dim3(warps * 32), smem, stream, 
            (const TX*)qkv, qkv_stride, (TX*)q_out, (TC*)k_cache, (TC*)v_cache,
            (const TW*)q_norm_w, (const TW*)k_norm_w, inv_freq, positions, seq_of_token, seq_rows,
            block_table, table_stride, nq, nkv, d, rot, page_size, num_pages, eps, norm_offset,
            append, error);
    })));
    return launch_status();
}

// The same on the partial sums of a split matrix product ([splits][tokens][width]
// 32-bit); q_out and the caches are bfloat16.
CHIBI_API int chibi_qk_norm_rope_append_partial(
    const float* partial, int splits, long long tokens, long long width, void* q_out, void* k_cache,
    void* v_cache, const void* q_norm_w, const void* k_norm_w, int w_type, const float* inv_freq,
    const int* positions, const int* seq_of_token, const int* seq_rows, const int* block_table,
    int table_stride, int nq, int nkv, int d, int rot, int page_size, int num_pages, float eps,
    float norm_offset, int append, int* error, cudaStream_t stream)
{
    if (tokens <= 0)
        return CHIBI_OK;
    if (d <= 0 || d > 256 || d % 4 != 0 || rot < 0 || rot > d || (rot & 1) || width % 4 != 0
        || splits < 1 || (reinterpret_cast<uintptr_t>(partial) & 15))
        return CHIBI_ERR_UNSUPPORTED;
    const int jobs = append ? nq + 2 * nkv : nq;
    const int warps = jobs < 8 ? jobs : 8;
    const int per_block = warps;
    const size_t smem = (size_t)(per_block * d + rot) * sizeof(float);
    const dim3 grid((unsigned)tokens, (unsigned)((jobs + per_block - 1) / per_block));
    if (tokens > 65535 || grid.y > 65535)
        return CHIBI_ERR_UNSUPPORTED;
    CHIBI_DISPATCH_TYPE(w_type, TW, {
        launch(qk_norm_rope_append_vec4_kernel<1, float, __nv_bfloat16, TW, __nv_bfloat16>, dim3(grid),
               dim3(warps * 32), smem, stream,
                partial, width, splits, tokens * width, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
                (__nv_bfloat16*)v_cache, (const TW*)q_norm_w, (const TW*)k_norm_w, inv_freq, positions,
                seq_of_token, seq_rows, block_table, table_stride, nq, nkv, d, rot, page_size, num_pages,
                eps, norm_offset, append, error);
    });
    return launch_status();
}

CHIBI_API int chibi_swiglu(const void* gate_up, int x_type, void* out, int out_type,
                           long long rows, int inter, cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (x_type == CHIBI_BF16 && out_type == CHIBI_BF16 && inter % 8 == 0 && rows <= 65535
        && (reinterpret_cast<uintptr_t>(gate_up) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        const dim3 grid((unsigned)((inter / 8 + 255) / 256), (unsigned)rows);
        launch(swiglu_bf16x8_kernel, dim3(grid), dim3(256), 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter);
        return launch_status();
    }
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(out_type, TO, {
        launch(swiglu_kernel<TX, TO>, dim3(grid_for(rows * inter, 256)), dim3(256), 0, stream, 
            (const TX*)gate_up, (TO*)out, rows, inter);
    }));
    return launch_status();
}

CHIBI_API int chibi_gather_rows(const void* x, int x_type, const int* rows, void* out,
                                int out_type, long long count, int n, long long x_rows,
                                cudaStream_t stream)
{
    if (count <= 0)
        return CHIBI_OK;
    const bool vec = n % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0
        && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(out_type, TO, {
        if (vec)
            launch(gather_rows_vec4_kernel<TX, TO>, dim3((unsigned)count), dim3(256), 0, stream,
                   (const TX*)x, rows, (TO*)out, n, x_rows);
        else
            launch(gather_rows_kernel<TX, TO>, dim3((unsigned)count), dim3(256), 0, stream,
                   (const TX*)x, rows, (TO*)out, n, x_rows);
    }));
    return launch_status();
}

CHIBI_API int chibi_cast(const void* x, int x_type, void* out, int out_type, long long total,
                         cudaStream_t stream)
{
    if (total <= 0)
        return CHIBI_OK;
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(out_type, TO, {
        launch(cast_kernel<TX, TO>, dim3(grid_for(total, 256)), dim3(256), 0, stream, (const TX*)x, (TO*)out, total);
    }));
    return launch_status();
}

// x[m, :] *= rsqrt(sum of ssq[m][0 .. parts) / norm_n + eps): the factor of an RMSNorm that a
// matrix product left out of its norm output, for a reader that cannot apply it itself.
namespace chibi {
__global__ void scale_rows_kernel(__nv_bfloat16* x, long long stride, int n, const float* __restrict__ ssq,
                                  int parts, float eps, int norm_n)
{
    pdl_enter();
    const long long m = blockIdx.x;
    float ss = 0.f;
    for (int j = 0; j < parts; ++j)
        ss += ssq[m * parts + j];
    const float inv = rsqrtf(ss / (float)norm_n + eps);
    __nv_bfloat16* row = x + m * stride;
    for (int j = threadIdx.x * 8; j < n; j += blockDim.x * 8) {
        uint4 q = *reinterpret_cast<const uint4*>(row + j);
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            h[e] = __floats2bfloat162_rn(f.x * inv, f.y * inv);
        }
        *reinterpret_cast<uint4*>(row + j) = q;
    }
}
} // namespace chibi

CHIBI_API int chibi_scale_rows(void* x, long long rows, int n, long long stride, const float* ssq, int parts,
                               float eps, int norm_n, cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (n % 8 != 0 || stride % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || parts < 1 || norm_n < 1)
        return CHIBI_ERR_UNSUPPORTED;
    launch(chibi::scale_rows_kernel, dim3((unsigned)rows), dim3(256), 0, stream, static_cast<__nv_bfloat16*>(x),
           stride, n, ssq, parts, eps, norm_n);
    return launch_status();
}

CHIBI_API int chibi_add_into(float* acc, const void* x, int x_type, long long total,
                             cudaStream_t stream)
{
    if (total <= 0)
        return CHIBI_OK;
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        launch(add_into_kernel<TX>, dim3(grid_for(total, 256)), dim3(256), 0, stream, acc, (const TX*)x, total);
    });
    return launch_status();
}

CHIBI_API int chibi_apply_table_updates(int* table, int table_stride, int table_rows,
                                        const int* updates, int capacity, int* error,
                                        cudaStream_t stream)
{
    if (capacity <= 0)
        return CHIBI_OK;
    const int blocks = capacity > 4096 ? 16 : 1;
    launch(apply_table_updates_kernel, dim3(blocks), dim3(256), 0, stream, table, table_stride, table_rows, updates,
                                                           capacity, error);
    return launch_status();
}

// Per-token tables that every layer of a step shares when the q | k | v product finishes its heads
// itself.  rope: [tokens][2 * half], the cosines then the sines of float(position) * inv_freq[j],
// the same arithmetic as the norm + rotation kernels.  slots: the element offset of the token's slot
// in a paged cache [pages][nkv][page_size][d] for kv head 0, or -1 (and error word 2) if the block
// table holds no valid page for the position.
namespace chibi {
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  long long tokens, int half, float* __restrict__ out)
{
    pdl_enter();
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < tokens * half;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / half;
        const int j = (int)(idx - t * half);
        float sn, cn;
        sincosf((float)positions[t] * inv_freq[j], &sn, &cn);
        out[t * 2 * half + j] = cn;
        out[t * 2 * half + half + j] = sn;
    }
}

__global__ void cache_slots_kernel(const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                   const int* __restrict__ seq_rows, const int* __restrict__ block_table,
                                   int table_stride, long long tokens, int nkv, int page_size, int num_pages, int d,
                                   long long* __restrict__ out, int* __restrict__ error)
{
    pdl_enter();
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < tokens;
         t += (long long)gridDim.x * blockDim.x) {
        const int pos = positions[t];
        const int seq = seq_of_token[t];
        const int table_row = seq_rows ? seq_rows[seq] : seq;
        const int page = block_table[(size_t)table_row * table_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (error)
                atomicExch(error, 2);
            out[t] = -1;
        } else {
            out[t] = ((long long)page * nkv * page_size + (pos % page_size)) * d;
        }
    }
}
} // namespace chibi

CHIBI_API int chibi_rope_table(const int* positions, const float* inv_freq, long long tokens, int half, float* out,
                               cudaStream_t stream)
{
    if (tokens <= 0 || half <= 0)
        return CHIBI_OK;
    launch(chibi::rope_table_kernel, dim3(grid_for(tokens * half, 256)), dim3(256), 0, stream, positions, inv_freq,
           tokens, half, out);
    return launch_status();
}

CHIBI_API int chibi_cache_slots(const int* positions, const int* seq_of_token, const int* seq_rows,
                                const int* block_table, int table_stride, long long tokens, int nkv, int page_size,
                                int num_pages, int d, long long* out, int* error, cudaStream_t stream)
{
    if (tokens <= 0)
        return CHIBI_OK;
    if (nkv <= 0 || page_size <= 0 || d <= 0)
        return CHIBI_ERR_ARGUMENT;
    launch(chibi::cache_slots_kernel, dim3(grid_for(tokens, 256)), dim3(256), 0, stream, positions, seq_of_token,
           seq_rows, block_table, table_stride, tokens, nkv, page_size, num_pages, d, out, error);
    return launch_status();
}
