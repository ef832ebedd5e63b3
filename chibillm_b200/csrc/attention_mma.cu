// Causal grouped-query attention over the paged bfloat16 cache on the tensor
// cores, for one head size per compiled library (-DCHIBI_HEAD_DIM=d, d a
// multiple of 16 up to 256).  Two kernels:
//
// * decode: sequences that bring one token.  One CTA per (key range, kv head,
//   sequence); the query heads that share the kv head are the rows of one
//   16-row MMA tile, so every key and value is read once for the whole group.
//   The four warps of a CTA take the 16-key tiles of the CTA's range in turn,
//   each with its own cp.async ring, and merge their (max, sum, output) at the
//   end.  With more than one key range per sequence the partial results go to
//   scratch memory and a second kernel merges them.
// * prefill: sequences that bring several tokens.  The rows of a 64-row tile are
//   (token, head in group) pairs; K and V tiles of 64 keys are loaded once per
//   CTA (double-buffered cp.async) and used by all four warps.
//
// Scores are (q . k) * scale in 32-bit; softmax state (running max and sum) and
// the output accumulator are 32-bit; probabilities are rounded to bfloat16 for
// the second product.  A row sees keys max(0, pos - window + 1) .. pos.
#define CHIBI_UNIT attention_mma
#define CHIBI_UNIT_ID 6
#include "common.cuh"

#ifndef CHIBI_HEAD_DIM
#define CHIBI_HEAD_DIM 128
#endif

namespace chibi {

constexpr int D = CHIBI_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 up to 256");
constexpr int DPAD = D + 8;           // row stride in shared memory (16 bytes of padding)
constexpr int KSTEPS = D / 16;        // k-steps of q . k
constexpr int NTILES_D = D / 8;       // 8-wide output tiles of p . v
constexpr int CHUNKS = D / 8;         // 16-byte chunks per row
constexpr bool Q_IN_REGS = D <= 128;

struct AttnParams {
    const __nv_bfloat16* q;        // [T, nq * D]
    const __nv_bfloat16* k_cache;  // [pages, nkv, page_size, D]
    const __nv_bfloat16* v_cache;
    __nv_bfloat16* out;            // [T, nq * D]
    const int* block_table;
    int table_stride;
    const int* seq_rows;           // [S] row of the block table per sequence, or null (row = s)
    const int* q_start;            // [S + 1]
    const int* ctx_len;            // [S]
    int nq, nkv, group;
    int page_size, num_pages;
    float scale_log2;              // scale * log2(e)
    int window;
    int splits;                    // decode: key ranges per sequence
    float* scratch_o;              // decode: [S, nq, splits, D]
    float* scratch_ml;             // decode: [S, nq, splits, 2]
    // decode, optional: q (and the newest key and value) are not in `q` and the caches yet but
    // still the partial sums of the q | k | v product: the kernel adds them up, applies the per-head
    // norm and the rotation itself and appends the new key and value (head size 128 only)
    __nv_bfloat16* k_cache_out;    // the caches again, to write to
    __nv_bfloat16* v_cache_out;
    const float* partial;          // [partial_splits][tokens][partial_width] or null
    int partial_splits;
    long long partial_split_stride, partial_width;
    const __nv_bfloat16* q_norm_w; // [D] or null
    const __nv_bfloat16* k_norm_w;
    const float* inv_freq;         // [D / 2]
    float norm_eps, norm_offset;
    int append;                    // write the new key and value (0: the layer reads another layer's cache)
    int skip_single;               // prefill: leave one-token sequences to the decode kernel
    int* error;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid)
{
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p)
{
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p)
{
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                 "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Loads 16 keys and their values, positions key0 .. key0 + 15 of one (sequence,
// kv head), into shared memory [16][DPAD] each; rows at or past key_end are
// zeroed.  One warp: lanes 0..15 look up the page of one row each (one division
// per row, shared by K and V), the row offsets travel by shuffle, and every lane
// issues its 16-byte chunks.
// The cache page of lane's key (lane % 16) of the 16-key tile at key0; -1 past the context.
__device__ __forceinline__ int lookup_tile_page(const int* table, int page_size, int key0, int key_end, int lane)
{
    const int key = key0 + (lane & 15);
    return key < key_end ? table[key / page_size] : -1;
}

// Issues the copies of a 16-key tile whose pages `lookup_tile_page` has fetched.
__device__ __forceinline__ void load_kv_tile16_paged(__nv_bfloat16* k_dst, __nv_bfloat16* v_dst,
                                                     const __nv_bfloat16* k_cache, const __nv_bfloat16* v_cache,
                                                     int page, int kv_head, int nkv, int page_size, int num_pages,
                                                     int key0, int key_end, int lane, int* error)
{
    long long off = -1;
    {
        const int key = key0 + (lane & 15);
        if (key < key_end) {
            if (page < 0 || page >= num_pages) {
                if (error)
                    atomicExch(error, 3);
            } else {
                off = (((long long)page * nkv + kv_head) * page_size + key % page_size) * D;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 16 * CHUNKS / 32; ++i) {
        const int c = lane + 32 * i;
        const int row = c / CHUNKS, col = c - row * CHUNKS;
        const long long o = __shfl_sync(0xffffffffu, off, row);
        const bool valid = o >= 0;
        const long long src = valid ? o + col * 8 : 0;
        cp_async16(k_dst + row * DPAD + col * 8, k_cache + src, valid);
        cp_async16(v_dst + row * DPAD + col * 8, v_cache + src, valid);
    }
}

__device__ __forceinline__ void load_kv_tile16(__nv_bfloat16* k_dst, __nv_bfloat16* v_dst,
                                               const __nv_bfloat16* k_cache, const __nv_bfloat16* v_cache,
                                               const int* table, int kv_head, int nkv, int page_size,
                                               int num_pages, int key0, int key_end, int lane, int* error)
{
    load_kv_tile16_paged(k_dst, v_dst, k_cache, v_cache, lookup_tile_page(table, page_size, key0, key_end, lane),
                         kv_head, nkv, page_size, num_pages, key0, key_end, lane, error);
}

// Loads the A fragments of a 16-row query tile from shared memory.
__device__ __forceinline__ void load_q_frags(uint32_t (&qf)[KSTEPS][4], const __nv_bfloat16* q_tile, int lane)
{
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
        ldmatrix_x4(qf[ks], q_tile + (lane & 15) * DPAD + ks * 16 + (lane >> 4) * 8);
}

// s[nt] += q . k^T for `NT` 8-key tiles (NT even) of the K tile at k_tile.
template <int NT>
__device__ __forceinline__ void qk_product(float (&s)[NT][4], const uint32_t (&qf)[KSTEPS][4],
                                           const __nv_bfloat16* q_tile, const __nv_bfloat16* k_tile, int lane)
{
    const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t a[4];
        if constexpr (Q_IN_REGS) {
            a[0] = qf[ks][0]; a[1] = qf[ks][1]; a[2] = qf[ks][2]; a[3] = qf[ks][3];
        } else {
            ldmatrix_x4(a, q_tile + (lane & 15) * DPAD + ks * 16 + (lane >> 4) * 8);
        }
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            uint32_t b[4];
            ldmatrix_x4(b, k_tile + (np * 16 + (mi >> 1) * 8 + r8) * DPAD + ks * 16 + (mi & 1) * 8);
            mma_bf16(s[2 * np], a, b[0], b[1]);
            mma_bf16(s[2 * np + 1], a, b[2], b[3]);
        }
    }
}

// o += p . v for `NT` 8-key tiles of probabilities (already in s, unnormalised).
template <int NT>
__device__ __forceinline__ void pv_product(float (&o)[NTILES_D][4], const float (&s)[NT][4],
                                           const __nv_bfloat16* v_tile, int lane)
{
    const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
    for (int kp = 0; kp < NT / 2; ++kp) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kp][0], s[2 * kp][1]);
        a[1] = pack_bf16(s[2 * kp][2], s[2 * kp][3]);
        a[2] = pack_bf16(s[2 * kp + 1][0], s[2 * kp + 1][1]);
        a[3] = pack_bf16(s[2 * kp + 1][2], s[2 * kp + 1][3]);
#pragma unroll
        for (int nt = 0; nt < NTILES_D; nt += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, v_tile + (kp * 16 + (mi & 1) * 8 + r8) * DPAD + (nt + (mi >> 1)) * 8);
            mma_bf16(o[nt], a, b[0], b[1]);
            mma_bf16(o[nt + 1], a, b[2], b[3]);
        }
    }
}

// Online softmax over NT 8-key tiles.  Scores come in as raw dot products; on
// return s holds exp2(score * scale_log2 - m_new) (0 where masked), m/l are
// updated and o is rescaled.  `pos_lo/hi`: positions of this thread's two rows;
// a key is visible when first_lo/hi <= key <= pos_lo/hi and key < key_end.
template <int NT>
__device__ __forceinline__ void softmax_tile(float (&s)[NT][4], float (&o)[NTILES_D][4], float (&m)[2],
                                             float (&l)[2], float scale_log2, int key0, int key_end,
                                             int pos_lo, int pos_hi, int first_lo, int first_hi, int lane)
{
    const int tig = lane & 3;
    float mx[2] = { -INFINITY, -INFINITY };
    // a tile that every row of the warp sees whole needs no masks (most tiles of a long prompt)
    const int last_key = key0 + NT * 8 - 1;
    const bool whole = __all_sync(0xffffffffu, last_key < key_end && last_key <= pos_lo && last_key <= pos_hi
                                                   && key0 >= first_lo && key0 >= first_hi);
    if (whole) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[nt][e] *= scale_log2;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
            }
        }
    } else
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int key = key0 + nt * 8 + tig * 2 + (e & 1);
            const bool hi = e >= 2;
            const bool vis = key < key_end && key <= (hi ? pos_hi : pos_lo) && key >= (hi ? first_hi : first_lo);
            s[nt][e] = vis ? s[nt][e] * scale_log2 : -INFINITY;
            mx[hi] = fmaxf(mx[hi], s[nt][e]);
        }
    }
    float corr[2], base[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m[h], mx[h]);
        base[h] = m_new == -INFINITY ? 0.f : m_new;       // a row that has seen no key yet
        corr[h] = exp2f(m[h] - base[h]);                  // 0 when m was -inf
        m[h] = m_new;
    }
    float sum[2] = { 0.f, 0.f };
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float p = exp2f(s[nt][e] - base[e >> 1]);
            s[nt][e] = p;
            sum[e >> 1] += p;
        }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
        sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
        l[h] = l[h] * corr[h] + sum[h];
    }
#pragma unroll
    for (int nt = 0; nt < NTILES_D; ++nt) {
        o[nt][0] *= corr[0];
        o[nt][1] *= corr[0];
        o[nt][2] *= corr[1];
        o[nt][3] *= corr[1];
    }
}

// ------------------------------------------------------------------ decode
constexpr int DEC_WARPS = 4;
constexpr int DEC_TILE = 16;                 // keys per warp tile
constexpr int DEC_STAGES = D <= 128 ? 3 : 2;
constexpr int DEC_STAGE_ELEMS = 2 * DEC_TILE * DPAD;   // K tile then V tile
constexpr int DEC_Q_ELEMS = 16 * DPAD;
constexpr size_t DEC_SMEM_PIPE = (size_t)(DEC_Q_ELEMS + DEC_WARPS * DEC_STAGES * DEC_STAGE_ELEMS) * 2;
constexpr size_t DEC_SMEM_MERGE = (size_t)DEC_WARPS * (16 * (D + 1) + 32) * 4;
constexpr size_t DEC_SMEM = DEC_SMEM_PIPE > DEC_SMEM_MERGE ? DEC_SMEM_PIPE : DEC_SMEM_MERGE;

// q of one (sequence, kv head) from the partial sums of the q | k | v product, for head
// size 128 and 128 threads (thread j owns feature j of every head): sum over the splits in
// split order, RMSNorm per head (if a weight is given), split-half rotation with the
// token's cosines and sines `cs` ([0, 64) cosines, [64, 128) sines), bfloat16 into the
// q tile.  With `with_kv` the same for the new key, and the new value as it is, written
// to the cache slot at `cache_base`.  xs: [8][128] floats, red: [4][8] floats.
__device__ __forceinline__ void build_q_from_partial(const AttnParams& p, int t, int kv_head, int head0, int rows,
                                                     bool with_kv, long long cache_base,
                                                     __nv_bfloat16* q_tile, const float* cs, float (*xs)[128],
                                                     float (*red)[8])
{
    const int j = threadIdx.x, warp = j >> 5, lane = j & 31;
    const int heads = rows + (with_kv ? 2 : 0);              // at most 8
    long long col[8];
#pragma unroll
    for (int h = 0; h < 8; ++h) {
        int head = head0 + h;                                 // a query head
        if (h == rows)
            head = p.nq + kv_head;                            // the key head
        else if (h == rows + 1)
            head = p.nq + p.nkv + kv_head;                    // the value head
        col[h] = (long long)t * p.partial_width + (long long)head * 128 + j;
    }
    float acc[8] = { 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f };
    for (int s0 = 0; s0 < p.partial_splits; s0 += 8) {        // 64 loads in flight
        float q[8][8];
#pragma unroll
        for (int h = 0; h < 8; ++h)
#pragma unroll
            for (int u = 0; u < 8; ++u)
                q[h][u] = (h < heads && s0 + u < p.partial_splits)
                    ? p.partial[(long long)(s0 + u) * p.partial_split_stride + col[h]] : 0.f;
#pragma unroll
        for (int h = 0; h < 8; ++h)
#pragma unroll
            for (int u = 0; u < 8; ++u)
                acc[h] += q[h][u];
    }
    // per-head sums of squares (the value head is not normalised)
#pragma unroll
    for (int h = 0; h < 8; ++h) {
        const float ss = warp_sum(acc[h] * acc[h]);
        if (lane == 0)
            red[warp][h] = ss;
    }
    __syncthreads();
    const float wq = p.q_norm_w ? __bfloat162float(p.q_norm_w[j]) + p.norm_offset : 1.f;
    const float wk = p.k_norm_w ? __bfloat162float(p.k_norm_w[j]) + p.norm_offset : 1.f;
#pragma unroll
    for (int h = 0; h < 8; ++h) {
        const bool is_q = h < rows, is_k = with_kv && h == rows;
        if ((is_q && p.q_norm_w) || (is_k && p.k_norm_w)) {
            const float total = (red[0][h] + red[1][h]) + (red[2][h] + red[3][h]);
            const float inv = rsqrtf(total / 128.f + p.norm_eps);
            acc[h] = (acc[h] * inv) * (is_q ? wq : wk);
        }
        xs[h][j] = acc[h];
    }
    __syncthreads();
    const float c = cs[j & 63], sn = cs[64 + (j & 63)];
#pragma unroll
    for (int h = 0; h < 8; ++h) {
        if (h < rows || (with_kv && h == rows)) {
            const float partner = xs[h][j ^ 64];
            const float out = j < 64 ? acc[h] * c - partner * sn : acc[h] * c + partner * sn;
            if (h < rows)
                q_tile[h * DPAD + j] = __float2bfloat16_rn(out);
            else
                p.k_cache_out[cache_base + j] = __float2bfloat16_rn(out);
        } else if (with_kv && h == rows + 1) {
            p.v_cache_out[cache_base + j] = __float2bfloat16_rn(acc[h]);
        }
    }
    for (int r = rows; r < 16; ++r)                           // rows past the group are zero
        q_tile[r * DPAD + j] = __float2bfloat16_rn(0.f);
    if (with_kv)
        __threadfence();                                      // the copies of the last tile read them back
}

__global__ void __launch_bounds__(DEC_WARPS * 32) attn_decode_kernel(const AttnParams p)
{
    pdl_trigger();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* pipe = q_tile + DEC_Q_ELEMS;

    // The index arrays, the block table and every key before the newest one were written
    // before this step's first kernel: the first tiles are on their way while the kernel
    // that writes q and the newest key still runs.
    const int seq = blockIdx.z, split = blockIdx.x;
    const int row_blocks = (p.group + 15) / 16;
    const int kv_head = blockIdx.y / row_blocks, row_block = blockIdx.y - kv_head * row_blocks;
    const int t = p.q_start[seq];
    if (p.q_start[seq + 1] - t != 1)
        return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = p.ctx_len[seq] - 1;
    const int first = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int key_end = pos + 1;
    const int tiles_total = (key_end - first + DEC_TILE - 1) / DEC_TILE;
    const int tiles_per_split = (tiles_total + p.splits - 1) / p.splits;
    const int tile_begin = split * tiles_per_split;
    int tile_end = tile_begin + tiles_per_split;
    if (tile_end > tiles_total)
        tile_end = tiles_total;
    const int* table = p.block_table + (size_t)(p.seq_rows ? p.seq_rows[seq] : seq) * p.table_stride;
    const int rows = min(16, p.group - row_block * 16);          // query heads in this tile
    const int head0 = kv_head * p.group + row_block * 16;

    __nv_bfloat16* my_pipe = pipe + (size_t)warp * DEC_STAGES * DEC_STAGE_ELEMS;
    const int my_first_tile = tile_begin + warp;
    const int my_tiles = my_first_tile < tile_end ? (tile_end - my_first_tile + DEC_WARPS - 1) / DEC_WARPS : 0;

    // the page of tile i + 1 is looked up when tile i is issued, so the dependent read of the
    // block table is never waited for
    auto key0_of = [&](int i) { return first + (my_first_tile + i * DEC_WARPS) * DEC_TILE; };
    int page_ahead = my_tiles > 0 ? lookup_tile_page(table, p.page_size, key0_of(0), key_end, lane) : -1;
    bool waited = false;
    [[maybe_unused]] const bool fused = D == 128 && p.partial != nullptr;
    __shared__ float rope_cs[128];
    __shared__ float head_x[8][128];
    __shared__ float head_ss[DEC_WARPS][8];
    if constexpr (D == 128) {
        if (fused && threadIdx.x < 64) {                     // the token's cosines and sines, before the wait
            float sn, cn;
            sincosf((float)pos * p.inv_freq[threadIdx.x], &sn, &cn);
            rope_cs[threadIdx.x] = cn;
            rope_cs[64 + threadIdx.x] = sn;
        }
    }
    auto issue = [&](int i) {
        if (i < my_tiles) {
            if (!waited && key0_of(i) + DEC_TILE > pos) {        // the tile with the newest key
                pdl_wait();
                waited = true;
            }
            const int page = page_ahead;
            if (i + 1 < my_tiles)
                page_ahead = lookup_tile_page(table, p.page_size, key0_of(i + 1), key_end, lane);
            __nv_bfloat16* st = my_pipe + (size_t)(i % DEC_STAGES) * DEC_STAGE_ELEMS;
            load_kv_tile16_paged(st, st + DEC_TILE * DPAD, p.k_cache, p.v_cache, page, kv_head, p.nkv,
                                 p.page_size, p.num_pages, key0_of(i), key_end, lane, p.error);
        }
        cp_async_commit();
    };
    // The first stages of the pipeline; a stage that needs the newest key waits until that key
    // is there (written by the kernel before this one, or, fused, by this CTA below).
    int resume = DEC_STAGES - 1;
#pragma unroll
    for (int i = 0; i < DEC_STAGES - 1; ++i) {
        if (fused && resume == DEC_STAGES - 1 && i < my_tiles && key0_of(i) + DEC_TILE > pos)
            resume = i;
        if (i < resume)
            issue(i);
    }
    if (!waited) {
        pdl_wait();
        waited = true;
    }
    bool q_built = false;
    if constexpr (D == 128) {
        if (fused) {
            const int last_tile = tiles_total - 1;               // holds the newest key
            const bool with_kv = p.append && tile_begin <= last_tile && last_tile < tile_end;
            long long cache_base = 0;
            bool write_kv = with_kv;
            if (with_kv) {
                const int page = table[pos / p.page_size];
                if (page < 0 || page >= p.num_pages) {
                    if (threadIdx.x == 0 && p.error)
                        atomicExch(p.error, 2);
                    write_kv = false;
                } else {
                    cache_base = (((long long)page * p.nkv + kv_head) * p.page_size + pos % p.page_size) * D;
                }
            }
            __syncthreads();                                     // the cosines and sines are there
            build_q_from_partial(p, t, kv_head, head0, rows, write_kv, cache_base, q_tile, rope_cs, head_x, head_ss);
            q_built = true;
        }
    }
    if (!q_built) {
        // query rows -> shared memory (rows past the group are zero)
        for (int c = threadIdx.x; c < 16 * CHUNKS; c += blockDim.x) {
            const int row = c / CHUNKS, col = c - row * CHUNKS;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < rows)
                v = *reinterpret_cast<const uint4*>(p.q + ((size_t)t * p.nq + head0 + row) * D + col * 8);
            *reinterpret_cast<uint4*>(q_tile + row * DPAD + col * 8) = v;
        }
    }
    __syncthreads();
    timeline_mark(0);                  // the query rows are in shared memory
    for (int i = resume; i < DEC_STAGES - 1; ++i)
        issue(i);
    uint32_t qf[KSTEPS][4];
    if constexpr (Q_IN_REGS)
        load_q_frags(qf, q_tile, lane);

    float o[NTILES_D][4];
#pragma unroll
    for (int nt = 0; nt < NTILES_D; ++nt)
        o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    float m[2] = { -INFINITY, -INFINITY }, l[2] = { 0.f, 0.f };

    for (int i = 0; i < my_tiles; ++i) {
        issue(i + DEC_STAGES - 1);
        cp_async_wait<DEC_STAGES - 1>();
        __syncwarp();
        const __nv_bfloat16* k_tile = my_pipe + (size_t)(i % DEC_STAGES) * DEC_STAGE_ELEMS;
        const __nv_bfloat16* v_tile = k_tile + DEC_TILE * DPAD;
        const int key0 = first + (my_first_tile + i * DEC_WARPS) * DEC_TILE;
        float s[2][4] = { { 0.f, 0.f, 0.f, 0.f }, { 0.f, 0.f, 0.f, 0.f } };
        qk_product<2>(s, qf, q_tile, k_tile, lane);
        softmax_tile<2>(s, o, m, l, p.scale_log2, key0, key_end, pos, pos, first, first, lane);
        pv_product<2>(o, s, v_tile, lane);
        __syncwarp();
    }
    cp_async_wait<0>();
    timeline_mark(1);                  // this warp has walked its tiles
    __syncthreads();

    // merge the warps: [warp][row][D + 1] outputs, then [warp][16] max and sum
    float* mo = reinterpret_cast<float*>(smem_raw);
    float* mm = mo + DEC_WARPS * 16 * (D + 1);
    float* ml = mm + DEC_WARPS * 16;
    {
        const int g = lane >> 2, tig = lane & 3;
        float* base = mo + (size_t)warp * 16 * (D + 1);
#pragma unroll
        for (int nt = 0; nt < NTILES_D; ++nt) {
            base[g * (D + 1) + nt * 8 + tig * 2] = o[nt][0];
            base[g * (D + 1) + nt * 8 + tig * 2 + 1] = o[nt][1];
            base[(g + 8) * (D + 1) + nt * 8 + tig * 2] = o[nt][2];
            base[(g + 8) * (D + 1) + nt * 8 + tig * 2 + 1] = o[nt][3];
        }
        if (tig == 0) {
            mm[warp * 16 + g] = m[0];
            mm[warp * 16 + g + 8] = m[1];
            ml[warp * 16 + g] = l[0];
            ml[warp * 16 + g + 8] = l[1];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows * D; idx += blockDim.x) {
        const int row = idx / D, c = idx - row * D;
        float mmax = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w)
            mmax = fmaxf(mmax, mm[w * 16 + row]);
        const float base = mmax == -INFINITY ? 0.f : mmax;
        float acc = 0.f, lsum = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float f = exp2f(mm[w * 16 + row] - base);
            acc += mo[((size_t)w * 16 + row) * (D + 1) + c] * f;
            lsum += ml[w * 16 + row] * f;
        }
        const int head = head0 + row;
        if (p.splits == 1) {
            p.out[((size_t)t * p.nq + head) * D + c] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
        } else {
            const size_t slot = ((size_t)seq * p.nq + head) * p.splits + split;
            p.scratch_o[slot * D + c] = acc;
            if (c == 0) {
                p.scratch_ml[slot * 2] = mmax;
                p.scratch_ml[slot * 2 + 1] = lsum;
            }
        }
    }
}

// Merges the key ranges of one (sequence, head): one block of D threads.
__global__ void attn_decode_merge_kernel(const AttnParams p)
{
    pdl_trigger();
    const int seq = blockIdx.y, head = blockIdx.x, c = threadIdx.x;
    const int t = p.q_start[seq];                     // written before the step's first kernel
    if (p.q_start[seq + 1] - t != 1)
        return;
    pdl_wait();
    const size_t slot0 = ((size_t)seq * p.nq + head) * p.splits;
    // eight key ranges at a time, all their loads in flight together
    float m_run = -INFINITY, acc = 0.f, lsum = 0.f;
    for (int s0 = 0; s0 < p.splits; s0 += 8) {
        float mv[8], lv[8], ov[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const bool in = s0 + u < p.splits;
            mv[u] = in ? p.scratch_ml[(slot0 + s0 + u) * 2] : -INFINITY;
            lv[u] = in ? p.scratch_ml[(slot0 + s0 + u) * 2 + 1] : 0.f;
            ov[u] = in ? p.scratch_o[(slot0 + s0 + u) * D + c] : 0.f;
        }
        float m_new = m_run;
#pragma unroll
        for (int u = 0; u < 8; ++u)
            m_new = fmaxf(m_new, mv[u]);
        const float base = m_new == -INFINITY ? 0.f : m_new;
        const float keep = exp2f(m_run - base);       // 0 while nothing has been seen
        acc *= keep;
        lsum *= keep;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float f = exp2f(mv[u] - base);
            acc += ov[u] * f;
            lsum += lv[u] * f;
        }
        m_run = m_new;
    }
    p.out[((size_t)t * p.nq + head) * D + c] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
}

// ------------------------------------------------------------------ prefill
constexpr int PRE_WARPS = 4;
constexpr int PRE_ROWS = PRE_WARPS * 16;      // query rows per CTA
constexpr int PRE_KEYS = D <= 128 ? 64 : 32;  // keys per tile
constexpr int PRE_NT = PRE_KEYS / 8;
// When the query fragments stay in registers the query tile is only needed until
// they are loaded: it then shares the memory of the second K/V stage, which is
// first written after that.  Three CTAs fit an SM that way.
constexpr bool PRE_Q_ALIASED = Q_IN_REGS && PRE_ROWS <= 2 * PRE_KEYS;
constexpr size_t PRE_SMEM = (size_t)((PRE_Q_ALIASED ? 0 : PRE_ROWS * DPAD) + 2 * 2 * PRE_KEYS * DPAD) * 2;

__global__ void __launch_bounds__(PRE_WARPS * 32, PRE_Q_ALIASED ? 3 : 1) attn_prefill_kernel(const AttnParams p)
{
    pdl_enter();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* kv = PRE_Q_ALIASED ? base : base + PRE_ROWS * DPAD;   // [stage][K | V][PRE_KEYS][DPAD]
    __nv_bfloat16* q_tile = PRE_Q_ALIASED ? kv + 2 * PRE_KEYS * DPAD : base;

    const int seq = blockIdx.z, kv_head = blockIdx.y;
    const int t0 = p.q_start[seq];
    const int q_len = p.q_start[seq + 1] - t0;
    if (q_len <= 0 || (q_len == 1 && p.skip_single))
        return;
    const int rows_total = q_len * p.group;
    const int row0 = blockIdx.x * PRE_ROWS;
    if (row0 >= rows_total)
        return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2;
    const int pos0 = p.ctx_len[seq] - q_len;
    const int* table = p.block_table + (size_t)(p.seq_rows ? p.seq_rows[seq] : seq) * p.table_stride;

    // query rows -> shared memory; row r is (token r / group, head r % group)
    for (int c = threadIdx.x; c < PRE_ROWS * CHUNKS; c += blockDim.x) {
        const int row = c / CHUNKS, col = c - row * CHUNKS;
        const int r = row0 + row;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows_total) {
            const int tok = r / p.group, h = r - tok * p.group;
            v = *reinterpret_cast<const uint4*>(p.q + ((size_t)(t0 + tok) * p.nq + kv_head * p.group + h) * D + col * 8);
        }
        *reinterpret_cast<uint4*>(q_tile + row * DPAD + col * 8) = v;
    }

    const int last_row = min(rows_total, row0 + PRE_ROWS) - 1;
    const int min_pos = pos0 + row0 / p.group, max_pos = pos0 + last_row / p.group;
    const int key_begin = (p.window > 0 && min_pos - p.window + 1 > 0) ? min_pos - p.window + 1 : 0;
    const int key_end = max_pos + 1;
    const int n_tiles = (key_end - key_begin + PRE_KEYS - 1) / PRE_KEYS;

    // this thread's two rows
    const int r_lo = row0 + warp * 16 + g, r_hi = r_lo + 8;
    const int pos_lo = r_lo < rows_total ? pos0 + r_lo / p.group : -1;
    const int pos_hi = r_hi < rows_total ? pos0 + r_hi / p.group : -1;
    const int first_lo = (p.window > 0 && pos_lo - p.window + 1 > 0) ? pos_lo - p.window + 1 : 0;
    const int first_hi = (p.window > 0 && pos_hi - p.window + 1 > 0) ? pos_hi - p.window + 1 : 0;
    // rows of this warp: positions between warp_min_pos and warp_max_pos
    const int w_first_row = row0 + warp * 16;
    const int w_last_row = min(rows_total, w_first_row + 16) - 1;
    const bool warp_active = w_first_row < rows_total;
    const int warp_max_pos = warp_active ? pos0 + w_last_row / p.group : -1;
    const int warp_min_first = !warp_active ? 0
        : ((p.window > 0 && pos0 + w_first_row / p.group - p.window + 1 > 0)
               ? pos0 + w_first_row / p.group - p.window + 1 : 0);

    auto issue = [&](int i) {
        if (i < n_tiles) {
            __nv_bfloat16* st = kv + (size_t)(i & 1) * 2 * PRE_KEYS * DPAD;
            const int key0 = key_begin + i * PRE_KEYS;
            for (int sub = warp; sub < PRE_KEYS / 16; sub += PRE_WARPS)
                load_kv_tile16(st + sub * 16 * DPAD, st + (PRE_KEYS + sub * 16) * DPAD, p.k_cache, p.v_cache,
                               table, kv_head, p.nkv, p.page_size, p.num_pages, key0 + sub * 16, key_end,
                               lane, p.error);
        }
        cp_async_commit();
    };
    issue(0);
    __syncthreads();                       // q_tile is complete
    uint32_t qf[KSTEPS][4];
    const __nv_bfloat16* my_q = q_tile + warp * 16 * DPAD;
    if constexpr (Q_IN_REGS)
        load_q_frags(qf, my_q, lane);
    if constexpr (PRE_Q_ALIASED)
        __syncthreads();                   // every warp has its fragments: the second stage may be filled

    float o[NTILES_D][4];
#pragma unroll
    for (int nt = 0; nt < NTILES_D; ++nt)
        o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    float m[2] = { -INFINITY, -INFINITY }, l[2] = { 0.f, 0.f };

    for (int i = 0; i < n_tiles; ++i) {
        issue(i + 1);
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* k_tile = kv + (size_t)(i & 1) * 2 * PRE_KEYS * DPAD;
        const __nv_bfloat16* v_tile = k_tile + PRE_KEYS * DPAD;
        const int key0 = key_begin + i * PRE_KEYS;
        // skip tiles that no row of this warp can see
        if (warp_active && key0 <= warp_max_pos && key0 + PRE_KEYS > warp_min_first) {
            float s[PRE_NT][4];
#pragma unroll
            for (int nt = 0; nt < PRE_NT; ++nt)
                s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
            qk_product<PRE_NT>(s, qf, my_q, k_tile, lane);
            softmax_tile<PRE_NT>(s, o, m, l, p.scale_log2, key0, key_end, pos_lo, pos_hi, first_lo, first_hi, lane);
            pv_product<PRE_NT>(o, s, v_tile, lane);
        }
        __syncthreads();                   // the stage may be overwritten by the next issue
    }
    cp_async_wait<0>();

    const int tig = lane & 3;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = h ? r_hi : r_lo;
        if (r >= rows_total)
            continue;
        const int tok = r / p.group, head = kv_head * p.group + (r - tok * p.group);
        const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
        __nv_bfloat16* dst = p.out + ((size_t)(t0 + tok) * p.nq + head) * D;
#pragma unroll
        for (int nt = 0; nt < NTILES_D; ++nt) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(o[nt][2 * h] * inv, o[nt][2 * h + 1] * inv);
            *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8 + tig * 2) = v;
        }
    }
}

} // namespace chibi

using namespace chibi;

CHIBI_API int chibi_attention_mma_head_dim() { return D; }

// Scratch floats that a decode launch with these sizes needs.
CHIBI_API long long chibi_attention_mma_scratch_floats(int seqs, int nq, int splits)
{
    return splits > 1 ? (long long)seqs * nq * splits * (D + 2) : 0;
}

// mode bit 0: run the decode kernel (one-token sequences); bit 1: run the
// prefill kernel (the others; all sequences when bit 0 is clear).
CHIBI_API int chibi_attention_mma(const void* q, const void* k_cache, const void* v_cache, void* out,
                                  const int* block_table, int table_stride, const int* seq_rows,
                                  const int* q_start, const int* ctx_len, int seqs, int nq, int nkv, int page_size,
                                  int num_pages, float scale, int window, int mode, int max_q_len,
                                  int splits, float* scratch, long long scratch_floats, int* error,
                                  cudaStream_t stream)
{
    if (seqs <= 0)
        return CHIBI_OK;
    if (nkv <= 0 || nq % nkv != 0 || window < 0 || page_size <= 0 || splits < 1)
        return CHIBI_ERR_ARGUMENT;
    AttnParams p {};
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
    p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.seq_rows = seq_rows;
    p.q_start = q_start;
    p.ctx_len = ctx_len;
    p.nq = nq;
    p.nkv = nkv;
    p.group = nq / nkv;
    p.page_size = page_size;
    p.num_pages = num_pages;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.window = window;
    p.splits = splits;
    p.error = error;
    p.skip_single = (mode & 1) ? 1 : 0;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DEC_SMEM);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PRE_SMEM);
        if (e != cudaSuccess)
            return (int)e;
        configured = true;
    }
    if (mode & 1) {
        if (splits > 1) {
            const long long need = chibi_attention_mma_scratch_floats(seqs, nq, splits);
            if (!scratch || scratch_floats < need)
                return CHIBI_ERR_ARGUMENT;
            p.scratch_o = scratch;
            p.scratch_ml = scratch + (size_t)seqs * nq * splits * D;
        }
        const int row_blocks = (p.group + 15) / 16;
        const dim3 grid(splits, nkv * row_blocks, seqs);
        launch(attn_decode_kernel, dim3(grid), dim3(DEC_WARPS * 32), DEC_SMEM, stream, p);
        int st = launch_status();
        if (st != CHIBI_OK)
            return st;
        if (splits > 1) {
            launch(attn_decode_merge_kernel, dim3(dim3(nq, seqs)), dim3(D), 0, stream, p);
            st = launch_status();
            if (st != CHIBI_OK)
                return st;
        }
    }
    if (mode & 2) {
        const long long rows = (long long)max_q_len * p.group;
        const dim3 grid((unsigned)((rows + PRE_ROWS - 1) / PRE_ROWS), nkv, seqs);
        launch(attn_prefill_kernel, dim3(grid), dim3(PRE_WARPS * 32), PRE_SMEM, stream, p);
        return launch_status();
    }
    return CHIBI_OK;
}

// The decode kernel on the partial sums of the q | k | v product (32-bit,
// [partial_splits][tokens][partial_width]): every sequence brings one token; the kernel
// adds the partial sums of its heads, applies the per-head RMSNorm (weights bfloat16 or
// null) and the rotation, and the CTA whose key range holds the newest position writes
// the new key and value to the caches (append != 0) before it reads them back.  Takes
// head size 128 with at most 6 query heads per kv head and a rotation of the whole head;
// returns CHIBI_ERR_UNSUPPORTED otherwise.
CHIBI_API int chibi_attention_decode_fused(const float* partial, int partial_splits, long long partial_width,
                                           long long tokens, void* k_cache, void* v_cache, void* out,
                                           const int* block_table, int table_stride, const int* seq_rows,
                                           const int* q_start, const int* ctx_len, int seqs, int nq, int nkv,
                                           int page_size, int num_pages, float scale, int window, int splits,
                                           float* scratch, long long scratch_floats, const void* q_norm_w,
                                           const void* k_norm_w, const float* inv_freq, float eps, float offset,
                                           int append, int* error, cudaStream_t stream)
{
    if (seqs <= 0)
        return CHIBI_OK;
    if (nkv <= 0 || nq % nkv != 0 || window < 0 || page_size <= 0 || splits < 1 || !partial || partial_splits < 1
        || !inv_freq)
        return CHIBI_ERR_ARGUMENT;
    if (D != 128 || nq / nkv > 6 || partial_width < (long long)(append ? nq + 2 * nkv : nq) * D)
        return CHIBI_ERR_UNSUPPORTED;
    AttnParams p {};
    p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
    p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
    p.k_cache_out = static_cast<__nv_bfloat16*>(k_cache);
    p.v_cache_out = static_cast<__nv_bfloat16*>(v_cache);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.seq_rows = seq_rows;
    p.q_start = q_start;
    p.ctx_len = ctx_len;
    p.nq = nq;
    p.nkv = nkv;
    p.group = nq / nkv;
    p.page_size = page_size;
    p.num_pages = num_pages;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.window = window;
    p.splits = splits;
    p.error = error;
    p.skip_single = 1;
    p.partial = partial;
    p.partial_splits = partial_splits;
    p.partial_split_stride = tokens * partial_width;
    p.partial_width = partial_width;
    p.q_norm_w = static_cast<const __nv_bfloat16*>(q_norm_w);
    p.k_norm_w = static_cast<const __nv_bfloat16*>(k_norm_w);
    p.inv_freq = inv_freq;
    p.norm_eps = eps;
    p.norm_offset = offset;
    p.append = append;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)DEC_SMEM);
        if (e != cudaSuccess)
            return (int)e;
        configured = true;
    }
    if (splits > 1) {
        const long long need = chibi_attention_mma_scratch_floats(seqs, nq, splits);
        if (!scratch || scratch_floats < need)
            return CHIBI_ERR_ARGUMENT;
        p.scratch_o = scratch;
        p.scratch_ml = scratch + (size_t)seqs * nq * splits * D;
    }
    launch(attn_decode_kernel, dim3(splits, nkv, seqs), dim3(DEC_WARPS * 32), DEC_SMEM, stream, p);
    int st = launch_status();
    if (st != CHIBI_OK)
        return st;
    if (splits > 1) {
        launch(attn_decode_merge_kernel, dim3(dim3(nq, seqs)), dim3(D), 0, stream, p);
        st = launch_status();
    }
    return st;
}
