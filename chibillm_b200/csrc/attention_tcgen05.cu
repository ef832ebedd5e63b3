// Causal grouped-query attention for prompt portions on the 5th-generation
// tensor cores, for one head size per compiled library (-DCHIBI_HEAD_DIM=d,
// d = 64 or 128).
//
// One CTA owns 128 query rows of one kv head -- the rows are (token, head of the
// group) pairs, so the group's heads share every key and value tile -- and walks
// over the keys in tiles of 128:
//
//   warp 0      loads K and V tiles with TMA, one box per cache page and 64-wide
//               half of the head (128-byte swizzle);
//   warp 1      issues the MMAs:  S = Q K^T  (both K-major) into one of two TMEM
//               buffers, and  O += P V  with P from shared memory and V as the
//               MN-major operand (V is stored [key][d]), accumulating in a third TMEM buffer;
//   warps 2..5  softmax: thread r owns query row r.  It reads its row of S from
//               TMEM, keeps the running maximum and sum in registers and writes
//               P = exp2(S * scale - max) as bfloat16 into one of two buffers in
//               shared memory, in the swizzled K-major layout.  The output accumulates in TMEM over all
//               tiles; it is rescaled there only when a row's maximum has grown by
//               more than 2^8, and read out once at the end.
//
// The MMA of the next S tile is issued before the P V product of the current
// one, so it runs while the softmax threads work.  All waits are bounded.
#define CHIBI_UNIT attention_tcgen05
#define CHIBI_UNIT_ID 7
#include "common.cuh"
#include "sm100.cuh"
#include "tensor_map.cuh"

#ifndef CHIBI_HEAD_DIM
#define CHIBI_HEAD_DIM 128
#endif

namespace chibi {

using namespace sm100;

constexpr int D = CHIBI_HEAD_DIM;
static_assert(D == 64 || D == 128, "the tcgen05 attention kernel takes head sizes 64 and 128");
constexpr int ROWS = 128;                    // query rows per CTA = UMMA M
constexpr int KEYS = 128;                    // keys per tile
constexpr int HALVES = D / 64;               // 64-wide (128-byte) slices of a head
constexpr int ATC_THREADS = 192;
constexpr int Q_BYTES = ROWS * D * 2;
constexpr int KV_TILE_BYTES = KEYS * D * 2;  // one K or V tile
constexpr int P_BYTES = ROWS * KEYS * 2;
constexpr int SMEM_TILES = Q_BYTES + 4 * KV_TILE_BYTES + 2 * P_BYTES;
constexpr int NUM_BARS = 16;
constexpr size_t ATC_SMEM = SMEM_TILES + NUM_BARS * 8 + 16 + 1024;
constexpr uint32_t TMEM_S0 = 0, TMEM_S1 = 128, TMEM_O = 256;

struct AttnTcParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const int* block_table;
    int table_stride;
    const int* seq_rows;
    const int* q_start;
    const int* ctx_len;
    int nq, nkv, group;
    int page_size;
    long long cache_rows;        // pages * nkv * page_size: rows of the [rows, D] view of a cache
    int num_pages;
    float scale_log2;
    int window;
    int skip_single;
    int* error;
    // The kernel with one query tile per CTA may cut the keys of a row tile into kv_splits ranges,
    // one CTA each (few query rows over a long context would leave most SMs idle otherwise): every
    // CTA then leaves its unnormalised output, maximum and sum per row, and
    // attn_prefill_merge_kernel puts the ranges together.
    int kv_splits;                 // 1: none
    float* part_o;                 // [tokens][nq][kv_splits][D]
    float* part_ml;                // [tokens][nq][kv_splits][2]
};

// Byte offset of element (row, col) of a [rows][64] bf16 tile laid out with the
// 128-byte swizzle (what TMA writes and tcgen05.mma reads): 16-byte chunk c of
// row r sits at chunk position c ^ (r % 8).
__device__ __forceinline__ uint32_t swizzled_chunk(int row, int chunk)
{
    return (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}

__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// MN-major operand (here V: [key][d], d contiguous) in the same swizzled tiles:
// leading byte offset = distance between the 64-wide slices of d, stride byte
// offset = 8 keys * 128 B.
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_byte_addr, uint32_t lbo_bytes)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_byte_addr & 0x3ffff) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

__global__ void __launch_bounds__(ATC_THREADS)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const AttnTcParams p)
{
    pdl_enter();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = smem;
    uint8_t* k_s = q_s + Q_BYTES;                  // two stages
    uint8_t* v_s = k_s + 2 * KV_TILE_BYTES;        // two stages
    uint8_t* p_s = v_s + 2 * KV_TILE_BYTES;        // two buffers
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_TILES);
    uint64_t* k_full = bars;          // [2] TMA
    uint64_t* v_full = bars + 2;      // [2] TMA
    uint64_t* k_empty = bars + 4;     // [2] MMA commit
    uint64_t* v_empty = bars + 6;     // [2] MMA commit
    uint64_t* s_full = bars + 8;      // [2] MMA commit
    uint64_t* s_free = bars + 10;     // [2] 128 threads
    uint64_t* p_full = bars + 12;     // [2] 128 threads
    uint64_t* o_full = bars + 14;     // [2] MMA commit: O holds tile j, P buffer j % 2 is free
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);

    // CTAs start in the order of their linear index: the row tiles with the most keys come first,
    // for all kv heads, so that the long ones do not start last
    const int seq = blockIdx.z / p.kv_splits, split = blockIdx.z - seq * p.kv_splits;
    const int linear = blockIdx.x + gridDim.x * blockIdx.y;
    const int kv_head = linear % gridDim.y, tile_rank = linear / gridDim.y;
    const int t0 = p.q_start[seq];
    const int q_len = p.q_start[seq + 1] - t0;
    const int rows_total = q_len * p.group;
    const int row0 = (gridDim.x - 1 - tile_rank) * ROWS;
    if (q_len <= 0 || (q_len == 1 && p.skip_single) || row0 >= rows_total)
        return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos0 = p.ctx_len[seq] - q_len;
    const int* table = p.block_table + (size_t)(p.seq_rows ? p.seq_rows[seq] : seq) * p.table_stride;

    const int last_row = min(rows_total, row0 + ROWS) - 1;
    const int min_pos = pos0 + row0 / p.group, max_pos = pos0 + last_row / p.group;
    int key_begin = (p.window > 0 && min_pos - p.window + 1 > 0) ? min_pos - p.window + 1 : 0;
    key_begin = key_begin / p.page_size * p.page_size;           // tiles start on a page
    const int key_end = max_pos + 1;
    int n_tiles = (key_end - key_begin + KEYS - 1) / KEYS;
    if (p.kv_splits > 1) {
        // this CTA's range of the row tile's key tiles (it may be empty)
        const int per = (n_tiles + p.kv_splits - 1) / p.kv_splits;
        const int lo = split * per;
        n_tiles = max(0, min(per, n_tiles - lo));
        key_begin += lo * KEYS;
    }

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&s_free[i], 128);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&p_full[i], 128);
            mbar_init(&o_full[i], 1);
        }
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    // query rows -> shared memory in the swizzled K-major layout (all threads help)
    {
        // all of a thread's loads go out before the first store
        constexpr int PIECES = (ROWS * (D / 8) + ATC_THREADS - 1) / ATC_THREADS;
        uint4 v[PIECES];
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
            const int c = threadIdx.x + i * ATC_THREADS;
            const int row = c / (D / 8), chunk = c - row * (D / 8);
            const int r = row0 + row;
            v[i] = make_uint4(0, 0, 0, 0);
            if (c < ROWS * (D / 8) && r < rows_total) {
                const int tok = r / p.group, h = r - tok * p.group;
                v[i] = *reinterpret_cast<const uint4*>(p.q + ((size_t)(t0 + tok) * p.nq + kv_head * p.group + h) * D + chunk * 8);
            }
        }
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
            const int c = threadIdx.x + i * ATC_THREADS;
            const int row = c / (D / 8), chunk = c - row * (D / 8);
            if (c < ROWS * (D / 8))
                *reinterpret_cast<uint4*>(q_s + (chunk >> 3) * (ROWS * 128) + swizzled_chunk(row, chunk & 7)) = v[i];
        }
    }
    fence_proxy_async();               // the tensor core reads what these threads wrote
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // Lane i brings page i of every 128-key tile (at most 16 pages: page_size >= 8).
        // A lane looks its page up one tile ahead, so the dependent read of the block
        // table is over by the time the stage is free.
        if (lane == 0) {
            tma_prefetch_descriptor(&map_k);
            tma_prefetch_descriptor(&map_v);
        }
        const int pages_per_tile = KEYS / p.page_size;
        auto first_row_of = [&](int j) -> long long {
            const int key = key_begin + j * KEYS + lane * p.page_size;
            if (lane >= pages_per_tile || key >= key_end)
                return p.cache_rows;      // past the context: read outside the array, zeros
            const int page = table[key / p.page_size];
            if (page < 0 || page >= p.num_pages) {
                if (p.error)
                    atomicExch(p.error, 3);
                return p.cache_rows;
            }
            return ((long long)page * p.nkv + kv_head) * p.page_size;
        };
        long long row = n_tiles > 0 ? first_row_of(0) : 0;
        for (int j = 0; j < n_tiles; ++j) {
            const long long row_next = j + 1 < n_tiles ? first_row_of(j + 1) : 0;
            const int st = j & 1;
            const uint32_t round = j >> 1;
            for (int which = 0; which < 2; ++which) {       // keys, then values
                uint64_t* full = which ? &v_full[st] : &k_full[st];
                uint64_t* empty = which ? &v_empty[st] : &k_empty[st];
                uint8_t* dst = (which ? v_s : k_s) + st * KV_TILE_BYTES;
                if (lane == 0) {
                    if (round > 0)
                        mbar_wait(empty, (round - 1) & 1, p.error, 21);
                    mbar_arrive_expect_tx(full, KV_TILE_BYTES);
                }
                __syncwarp();
                if (lane < pages_per_tile) {
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(dst + h * (KEYS * 128) + lane * p.page_size * 128, which ? &map_v : &map_k,
                                    full, h * 64, (int)row);
                }
            }
            row = row_next;
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc_qk = make_idesc_bf16_f32(ROWS, KEYS);
            constexpr uint32_t idesc_pv = make_idesc_bf16_f32(ROWS, D) | (1u << 16);    // B is MN-major
            const uint32_t q_addr = smem_addr(q_s);
            auto issue_qk = [&](int j) {
                const int st = j & 1;
                mbar_wait(&k_full[st], (j >> 1) & 1, p.error, 22);
                if (j >= 2)
                    mbar_wait(&s_free[st], ((j >> 1) - 1) & 1, p.error, 23);
                tcgen05_fence_after();
                const uint32_t k_addr = smem_addr(k_s + st * KV_TILE_BYTES);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks >> 2) * (ROWS * 128) + (ks & 3) * 32;
                    tcgen05_mma_bf16(tmem_base + (st ? TMEM_S1 : TMEM_S0), make_kmajor_sw128_desc(q_addr + off),
                                     make_kmajor_sw128_desc(k_addr + off), idesc_qk, ks > 0 ? 1u : 0u);
                }
                tcgen05_commit(&s_full[st]);
                tcgen05_commit(&k_empty[st]);
            };
            if (n_tiles > 0)
                issue_qk(0);
            for (int j = 0; j < n_tiles; ++j) {
                if (j + 1 < n_tiles)
                    issue_qk(j + 1);                      // runs while the softmax threads work on tile j
                const int st = j & 1;
                mbar_wait(&p_full[st], (j >> 1) & 1, p.error, 24);    // P(j) is written
                mbar_wait(&v_full[st], (j >> 1) & 1, p.error, 25);
                tcgen05_fence_after();
                const uint32_t v_addr = smem_addr(v_s + st * KV_TILE_BYTES);
                const uint32_t p_addr = smem_addr(p_s + st * P_BYTES);
#pragma unroll
                for (int ks = 0; ks < KEYS / 16; ++ks) {
                    const uint32_t a_off = (ks >> 2) * (ROWS * 128) + (ks & 3) * 32;
                    tcgen05_mma_bf16(tmem_base + TMEM_O, make_kmajor_sw128_desc(p_addr + a_off),
                                     make_mnmajor_sw128_desc(v_addr + ks * 16 * 128, KEYS * 128), idesc_pv,
                                     (j > 0 || ks > 0) ? 1u : 0u);
                }
                tcgen05_commit(&o_full[st]);
                tcgen05_commit(&v_empty[st]);
            }
        }
    } else {
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;                 // this thread's query row = its TMEM lane
        const int r = row0 + row;
        const bool live = r < rows_total;
        const int tok = live ? r / p.group : 0;
        const int pos = live ? pos0 + tok : -1;
        const int first = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        // The output accumulates in TMEM over all tiles.  `m` is the maximum that the exponents are
        // taken against; it follows the true maximum only when that has grown by more than 2^8
        // (then the output so far is rescaled in TMEM, a rare event after the first tiles), so
        // the probabilities stay below 2^8 and most tiles need no rescaling at all.
        float m = -INFINITY, l = 0.f;
        for (int j = 0; j < n_tiles; ++j) {
            const int st = j & 1;
            const int key0 = key_begin + j * KEYS;
            mbar_wait(&s_full[st], (j >> 1) & 1, p.error, 26);
            tcgen05_fence_after();
            const uint32_t s_addr = lane_addr + (st ? TMEM_S1 : TMEM_S0);
            // the whole row of S comes into registers with one wait
            uint32_t sv[KEYS];
#pragma unroll
            for (int c0 = 0; c0 < KEYS; c0 += 32)
                tmem_load_32x32(s_addr + c0, *reinterpret_cast<uint32_t(*)[32]>(&sv[c0]));
            tmem_load_wait();
            tcgen05_fence_before();
            mbar_arrive(&s_free[st]);                        // the MMA thread may fill this buffer again
            // masks only where a row's visible range ends inside the tile; the warp takes one path
            const bool masked = __any_sync(0xffffffffu, key0 + KEYS - 1 > pos || key0 < first);
            if (masked) {
#pragma unroll
                for (int i = 0; i < KEYS; ++i) {
                    const int key = key0 + i;
                    if (!(key <= pos && key >= first))
                        sv[i] = 0xff800000u;                 // -inf
                }
            }
            float mx4[4] = { -INFINITY, -INFINITY, -INFINITY, -INFINITY };   // four short chains, not one long one
#pragma unroll
            for (int i = 0; i < KEYS; i += 4) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    mx4[u] = fmaxf(mx4[u], __uint_as_float(sv[i + u]));
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            mx *= p.scale_log2;                              // the scale is positive
            const bool grow = mx > m + 8.f;                  // also true for the first visible key (m = -inf)
            if (__any_sync(0xffffffffu, grow && m != -INFINITY && j > 0)) {
                // rescale what has accumulated: the product of tile j-1 must have landed first
                mbar_wait(&o_full[(j - 1) & 1], ((j - 1) >> 1) & 1, p.error, 27);
                tcgen05_fence_after();
                const float f = (grow && m != -INFINITY) ? fast_exp2(m - mx) : 1.f;
#pragma unroll
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t ov[32];
                    tmem_load_32x32(lane_addr + TMEM_O + c0, ov);
                    tmem_load_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        ov[i] = __float_as_uint(__uint_as_float(ov[i]) * f);
                    tmem_store_32x32(lane_addr + TMEM_O + c0, ov);
                }
                tmem_store_wait();
                tcgen05_fence_before();
            }
            if (grow) {
                l *= (m == -INFINITY) ? 0.f : fast_exp2(m - mx);
                m = mx;
            }
            const float base = m == -INFINITY ? 0.f : m;
            // this P buffer is free once the product with tile j-2 has completed
            if (j >= 2)
                mbar_wait(&o_full[st], ((j >> 1) - 1) & 1, p.error, 28);
            float sum4[4] = { 0.f, 0.f, 0.f, 0.f };
#pragma unroll
            for (int c = 0; c < KEYS / 8; ++c) {             // 16-byte chunk of the row: 8 keys
                uint32_t packed[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float p0 = fast_exp2(fmaf(__uint_as_float(sv[8 * c + 2 * i]), p.scale_log2, -base));
                    const float p1 = fast_exp2(fmaf(__uint_as_float(sv[8 * c + 2 * i + 1]), p.scale_log2, -base));
                    sum4[i] += p0 + p1;
                    const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    packed[i] = *reinterpret_cast<const uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(p_s + st * P_BYTES + (c >> 3) * (ROWS * 128) + swizzled_chunk(row, c & 7)) =
                    make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            // values past the context may be anything (a page is loaded whole): make them zero, so
            // that 0 * value stays 0.  Only the last tile can hold such keys.
            if (key0 + KEYS > key_end) {
                mbar_wait(&v_full[st], (j >> 1) & 1, p.error, 29);
                uint8_t* v_tile = v_s + st * KV_TILE_BYTES;
                for (int c = row; c < (key0 + KEYS - key_end) * (D / 8); c += 128) {
                    const int krow = key_end - key0 + c / (D / 8), chunk = c % (D / 8);
                    *reinterpret_cast<uint4*>(v_tile + (chunk >> 3) * (KEYS * 128) + swizzled_chunk(krow, chunk & 7)) =
                        make_uint4(0, 0, 0, 0);
                }
            }
            fence_proxy_async();
            tcgen05_fence_before();
            mbar_arrive(&p_full[st]);
        }
        // the last product has landed: normalise and write the rows out
        if (n_tiles > 0)
            mbar_wait(&o_full[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, p.error, 30);
        tcgen05_fence_after();
        const int head = kv_head * p.group + (r - tok * p.group);
        if (p.kv_splits > 1) {
            // one of several key ranges: the row as it stands, with its maximum and sum
            const size_t slot = ((size_t)(t0 + tok) * p.nq + head) * p.kv_splits + split;
            float* dst = p.part_o + slot * D;
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t ov[32];
                if (n_tiles > 0) {
                    tmem_load_32x32(lane_addr + TMEM_O + c0, ov);
                    tmem_load_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        ov[i] = 0;
                }
                if (live) {
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        reinterpret_cast<uint4*>(dst + c0)[c] = make_uint4(ov[4 * c], ov[4 * c + 1], ov[4 * c + 2], ov[4 * c + 3]);
                }
            }
            if (live) {
                p.part_ml[slot * 2] = m;
                p.part_ml[slot * 2 + 1] = l;
            }
        } else {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst_row = p.out + ((size_t)(t0 + tok) * p.nq + head) * D;
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t ov[32];
            tmem_load_32x32(lane_addr + TMEM_O + c0, ov);
            tmem_load_wait();
            if (live) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    __nv_bfloat162 h[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        h[q] = __floats2bfloat162_rn(__uint_as_float(ov[8 * c + 2 * q]) * inv,
                                                     __uint_as_float(ov[8 * c + 2 * q + 1]) * inv);
                    reinterpret_cast<uint4*>(dst_row + c0)[c] = *reinterpret_cast<uint4*>(h);
                }
            }
        }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// Puts the key ranges of attn_prefill_tc_kernel together: one block of D threads for each
// (head, token of a sequence); ranges in order, eight at a time.
__global__ void attn_prefill_merge_kernel(const AttnTcParams p)
{
    pdl_trigger();
    const int seq = blockIdx.z, head = blockIdx.x, c = threadIdx.x;
    const int t0 = p.q_start[seq];
    const int q_len = p.q_start[seq + 1] - t0;
    if ((int)blockIdx.y >= q_len || (q_len == 1 && p.skip_single))
        return;
    pdl_wait();
    const size_t slot0 = ((size_t)(t0 + blockIdx.y) * p.nq + head) * p.kv_splits;
    float m_run = -INFINITY, acc = 0.f, lsum = 0.f;
    for (int s0 = 0; s0 < p.kv_splits; s0 += 8) {
        float mv[8], lv[8], ov[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const bool in = s0 + u < p.kv_splits;
            mv[u] = in ? p.part_ml[(slot0 + s0 + u) * 2] : -INFINITY;
            lv[u] = in ? p.part_ml[(slot0 + s0 + u) * 2 + 1] : 0.f;
            ov[u] = in ? p.part_o[(slot0 + s0 + u) * D + c] : 0.f;
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
    p.out[((size_t)(t0 + blockIdx.y) * p.nq + head) * D + c] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
}


// O[row, :] *= f for this thread's row of an output accumulator in TMEM (a rare
// event: kept out of line so that its registers do not count against the loop).
__device__ __noinline__ void rescale_output_row(uint32_t o_addr, float f)
{
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t ov[32];
        tmem_load_32x32(o_addr + c0, ov);
        tmem_load_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
            ov[i] = __float_as_uint(__uint_as_float(ov[i]) * f);
        tmem_store_32x32(o_addr + c0, ov);
    }
    tmem_store_wait();
}

// ------------------------------------------------------------------ two query tiles per CTA
// The same attention with 256 query rows per CTA: two tiles of 128 rows share
// every key and value tile, each tile has a softmax warp group of its own, and
// P never leaves TMEM (it overwrites the first 64 columns of its S buffer as
// packed bfloat16 and is the A operand of the P V product).  While one group
// works on its S tile the tensor core multiplies for the other.
//
//   warp 0      TMA loader (as above)
//   warp 1      MMA issuer:  S_q = Q_q K^T,  O_q += P_q V  for q = 0, 1 in turn
//   warps 2..5  softmax of tile 0;  warps 6..9  softmax of tile 1
//
// TMEM: S_0 at column 0, S_1 at 128, O_0 at 256, O_1 at 384.
constexpr int ATC2_THREADS = 320;
constexpr int SMEM2_TILES = 2 * Q_BYTES + 4 * KV_TILE_BYTES;
constexpr int NUM_BARS2 = 14;
constexpr size_t ATC2_SMEM = SMEM2_TILES + NUM_BARS2 * 8 + 16 + 1024;

__global__ void __launch_bounds__(ATC2_THREADS, 1)
attn_prefill_tc2_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const AttnTcParams p)
{
    pdl_enter();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = smem;                           // two tiles
    uint8_t* k_s = q_s + 2 * Q_BYTES;              // two stages
    uint8_t* v_s = k_s + 2 * KV_TILE_BYTES;        // two stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM2_TILES);
    uint64_t* k_full = bars;          // [2] TMA
    uint64_t* v_full = bars + 2;      // [2] TMA
    uint64_t* k_empty = bars + 4;     // [2] MMA commit
    uint64_t* v_empty = bars + 6;     // [2] MMA commit
    uint64_t* s_full = bars + 8;      // [2] per query tile, MMA commit
    uint64_t* p_full = bars + 10;     // [2] per query tile, 128 threads
    uint64_t* o_done = bars + 12;     // [2] per query tile, MMA commit
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS2);

    const int seq = blockIdx.z;
    const int linear = blockIdx.x + gridDim.x * blockIdx.y;        // longest row tiles first, for all kv heads
    const int kv_head = linear % gridDim.y, tile_rank = linear / gridDim.y;
    const int t0 = p.q_start[seq];
    const int q_len = p.q_start[seq + 1] - t0;
    const int rows_total = q_len * p.group;
    const int row0 = (gridDim.x - 1 - tile_rank) * (2 * ROWS);
    if (q_len <= 0 || (q_len == 1 && p.skip_single) || row0 >= rows_total)
        return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos0 = p.ctx_len[seq] - q_len;
    const int* table = p.block_table + (size_t)(p.seq_rows ? p.seq_rows[seq] : seq) * p.table_stride;

    // key tiles: all start at key_begin (a page boundary at or before the first key that the
    // CTA's first row sees); tile q needs nt[q] of them, nt[0] <= nt[1] when tile 1 has rows
    const int min_pos = pos0 + row0 / p.group;
    int key_begin = (p.window > 0 && min_pos - p.window + 1 > 0) ? min_pos - p.window + 1 : 0;
    key_begin = key_begin / p.page_size * p.page_size;
    int nt[2], key_end = 0;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const int lo = row0 + q * ROWS;
        if (lo < rows_total) {
            const int last_row = min(rows_total, lo + ROWS) - 1;
            const int end = pos0 + last_row / p.group + 1;
            nt[q] = (end - key_begin + KEYS - 1) / KEYS;
            key_end = max(key_end, end);
        } else {
            nt[q] = 0;
        }
    }
    const int n_tiles = max(nt[0], nt[1]);

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 128);
            mbar_init(&o_done[i], 1);
        }
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    // query rows -> shared memory in the swizzled K-major layout (all threads help)
    {
        // all of a thread's loads go out before the first store
        constexpr int PIECES = (2 * ROWS * (D / 8) + ATC2_THREADS - 1) / ATC2_THREADS;
        uint4 v[PIECES];
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
            const int c = threadIdx.x + i * ATC2_THREADS;
            const int row = c / (D / 8), chunk = c - row * (D / 8);     // row 0 .. 255
            const int r = row0 + row;
            v[i] = make_uint4(0, 0, 0, 0);
            if (c < 2 * ROWS * (D / 8) && r < rows_total) {
                const int tok = r / p.group, h = r - tok * p.group;
                v[i] = *reinterpret_cast<const uint4*>(p.q + ((size_t)(t0 + tok) * p.nq + kv_head * p.group + h) * D + chunk * 8);
            }
        }
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
            const int c = threadIdx.x + i * ATC2_THREADS;
            const int row = c / (D / 8), chunk = c - row * (D / 8);
            if (c < 2 * ROWS * (D / 8))
                *reinterpret_cast<uint4*>(q_s + (row >> 7) * Q_BYTES + (chunk >> 3) * (ROWS * 128)
                                          + swizzled_chunk(row & 127, chunk & 7)) = v[i];
        }
    }
    fence_proxy_async();               // the tensor core reads what these threads wrote
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    timeline_mark(0);                  // the query rows are in shared memory
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_descriptor(&map_k);
            tma_prefetch_descriptor(&map_v);
        }
        const int pages_per_tile = KEYS / p.page_size;
        auto first_row_of = [&](int j) -> long long {
            const int key = key_begin + j * KEYS + lane * p.page_size;
            if (lane >= pages_per_tile || key >= key_end)
                return p.cache_rows;      // past the context: read outside the array, zeros
            const int page = table[key / p.page_size];
            if (page < 0 || page >= p.num_pages) {
                if (p.error)
                    atomicExch(p.error, 3);
                return p.cache_rows;
            }
            return ((long long)page * p.nkv + kv_head) * p.page_size;
        };
        long long row = n_tiles > 0 ? first_row_of(0) : 0;
        for (int j = 0; j < n_tiles; ++j) {
            const long long row_next = j + 1 < n_tiles ? first_row_of(j + 1) : 0;
            const int st = j & 1;
            const uint32_t round = j >> 1;
            for (int which = 0; which < 2; ++which) {       // keys, then values
                uint64_t* full = which ? &v_full[st] : &k_full[st];
                uint64_t* empty = which ? &v_empty[st] : &k_empty[st];
                uint8_t* dst = (which ? v_s : k_s) + st * KV_TILE_BYTES;
                if (lane == 0) {
                    if (round > 0)
                        mbar_wait(empty, (round - 1) & 1, p.error, 41);
                    mbar_arrive_expect_tx(full, KV_TILE_BYTES);
                }
                __syncwarp();
                if (lane < pages_per_tile) {
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(dst + h * (KEYS * 128) + lane * p.page_size * 128, which ? &map_v : &map_k,
                                    full, h * 64, (int)row);
                }
            }
            row = row_next;
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc_qk = make_idesc_bf16_f32(ROWS, KEYS);
            constexpr uint32_t idesc_pv = make_idesc_bf16_f32(ROWS, D) | (1u << 16);    // B is MN-major
            // tile 1 is the last user of a key/value tile that it needs at all
            auto last_user = [&](int q, int j) { return q == (j < nt[1] ? 1 : 0); };
            auto issue_qk = [&](int q, int j) {
                const int st = j & 1;
                mbar_wait(&k_full[st], (j >> 1) & 1, p.error, 42);
                tcgen05_fence_after();
                const uint32_t q_addr = smem_addr(q_s + q * Q_BYTES);
                const uint32_t k_addr = smem_addr(k_s + st * KV_TILE_BYTES);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks >> 2) * (ROWS * 128) + (ks & 3) * 32;
                    tcgen05_mma_bf16(tmem_base + q * 128, make_kmajor_sw128_desc(q_addr + off),
                                     make_kmajor_sw128_desc(k_addr + off), idesc_qk, ks > 0 ? 1u : 0u);
                }
                tcgen05_commit(&s_full[q]);
                if (last_user(q, j))
                    tcgen05_commit(&k_empty[st]);
            };
            auto issue_pv = [&](int q, int j) {
                const int st = j & 1;
                mbar_wait(&p_full[q], j & 1, p.error, 43);            // P_q(j) is in TMEM
                mbar_wait(&v_full[st], (j >> 1) & 1, p.error, 44);
                tcgen05_fence_after();
                const uint32_t v_addr = smem_addr(v_s + st * KV_TILE_BYTES);
#pragma unroll
                for (int ks = 0; ks < KEYS / 16; ++ks)
                    tcgen05_mma_bf16_a_tmem(tmem_base + 256 + q * 128, tmem_base + q * 128 + ks * 8,
                                            make_mnmajor_sw128_desc(v_addr + ks * 16 * 128, KEYS * 128), idesc_pv,
                                            (j > 0 || ks > 0) ? 1u : 0u);
                tcgen05_commit(&o_done[q]);
                if (last_user(q, j))
                    tcgen05_commit(&v_empty[st]);
            };
            for (int q = 0; q < 2; ++q)
                if (nt[q] > 0)
                    issue_qk(q, 0);
            for (int j = 0; j < n_tiles; ++j) {
                for (int q = 0; q < 2; ++q) {
                    if (j < nt[q]) {
                        issue_pv(q, j);
                        if (j + 1 < nt[q])
                            issue_qk(q, j + 1);       // S_q may be overwritten: the products of one thread run in order
                    }
                }
            }
        }
    } else {
        const int q = warp >= 6 ? 1 : 0;                     // this warp group's query tile
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;                 // this thread's row of the tile = its TMEM lane
        const int r = row0 + q * ROWS + row;
        const bool live = r < rows_total;
        const int tok = live ? r / p.group : 0;
        const int pos = live ? pos0 + tok : -1;
        const int first = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const uint32_t s_addr = lane_addr + q * 128;
        const uint32_t o_addr = lane_addr + 256 + q * 128;
        const int my_tiles = nt[q];
        float m = -INFINITY, l = 0.f;
        for (int j = 0; j < my_tiles; ++j) {
            const int st = j & 1;
            const int key0 = key_begin + j * KEYS;
            mbar_wait(&s_full[q], j & 1, p.error, 45);
            tcgen05_fence_after();

            // Two passes over the S row in TMEM, 32 columns at a time (the next piece is on its way
            // while this one is worked on): the maximum, then P = exp2(S * scale - m) as packed
            // bfloat16 pairs, which overwrite the columns of S already read.
            const bool masked = __any_sync(0xffffffffu, key0 + KEYS - 1 > pos || key0 < first);
            auto mask_piece = [&](uint32_t (&v)[32], int c0) {
                if (masked) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = key0 + c0 + i;
                        if (!(key <= pos && key >= first))
                            v[i] = 0xff800000u;              // -inf
                    }
                }
            };
            uint32_t pa[32], pb[32];
            float mx4[4] = { -INFINITY, -INFINITY, -INFINITY, -INFINITY };
            tmem_load_32x32(s_addr, pa);
#pragma unroll
            for (int c0 = 0; c0 < KEYS; c0 += 64) {
                tmem_load_wait();
                tmem_load_32x32(s_addr + c0 + 32, pb);
                mask_piece(pa, c0);
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(pa[i]));
                tmem_load_wait();
                if (c0 + 64 < KEYS)
                    tmem_load_32x32(s_addr + c0 + 64, pa);
                mask_piece(pb, c0 + 32);
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(pb[i]));
            }
            tmem_load_32x32(s_addr, pa);                     // the second pass starts while the maximum settles
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            mx *= p.scale_log2;                              // the scale is positive
            const bool grow = mx > m + 8.f;                  // also true for the first visible key (m = -inf)
            if (__any_sync(0xffffffffu, grow && m != -INFINITY && j > 0)) {
                // rescale what has accumulated: the product of tile j-1 must have landed first
                mbar_wait(&o_done[q], (j - 1) & 1, p.error, 46);
                tcgen05_fence_after();
                tmem_load_wait();
                rescale_output_row(o_addr, (grow && m != -INFINITY) ? fast_exp2(m - mx) : 1.f);
            }
            if (grow) {
                l *= (m == -INFINITY) ? 0.f : fast_exp2(m - mx);
                m = mx;
            }
            const float base = m == -INFINITY ? 0.f : m;
            float sum4[4] = { 0.f, 0.f, 0.f, 0.f };
            auto exp_piece = [&](uint32_t (&v)[32], int c0) {
                mask_piece(v, c0);
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float p0 = fast_exp2(fmaf(__uint_as_float(v[2 * i]), p.scale_log2, -base));
                    const float p1 = fast_exp2(fmaf(__uint_as_float(v[2 * i + 1]), p.scale_log2, -base));
                    sum4[i & 3] += p0 + p1;
                    const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    packed[i] = *reinterpret_cast<const uint32_t*>(&h);
                }
                tmem_store_32x16(s_addr + (c0 >> 1), packed);   // behind the columns still to be read
            };
#pragma unroll
            for (int c0 = 0; c0 < KEYS; c0 += 64) {
                tmem_load_wait();
                tmem_load_32x32(s_addr + c0 + 32, pb);
                exp_piece(pa, c0);
                tmem_load_wait();
                if (c0 + 64 < KEYS)
                    tmem_load_32x32(s_addr + c0 + 64, pa);
                exp_piece(pb, c0 + 32);
            }
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            // values past the context may be anything (a page is loaded whole): make them zero, so
            // that 0 * value stays 0.  Only the CTA's last tile can hold such keys.
            if (key0 + KEYS > key_end) {
                mbar_wait(&v_full[st], (j >> 1) & 1, p.error, 47);
                uint8_t* v_tile = v_s + st * KV_TILE_BYTES;
                for (int c = row; c < (key0 + KEYS - key_end) * (D / 8); c += 128) {
                    const int krow = key_end - key0 + c / (D / 8), chunk = c % (D / 8);
                    *reinterpret_cast<uint4*>(v_tile + (chunk >> 3) * (KEYS * 128) + swizzled_chunk(krow, chunk & 7)) =
                        make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
            }
            tmem_store_wait();
            tcgen05_fence_before();
            mbar_arrive(&p_full[q]);
            if (j == 0)
                timeline_mark(1);      // the first tile's probabilities are written
        }
        timeline_mark(2);              // the last tile's probabilities are written
        // the last product has landed: normalise and write the rows out
        if (my_tiles > 0) {
            mbar_wait(&o_done[q], (my_tiles - 1) & 1, p.error, 48);
            tcgen05_fence_after();
            const int head = kv_head * p.group + (r - tok * p.group);
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst_row = p.out + ((size_t)(t0 + tok) * p.nq + head) * D;
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t ov[32];
                tmem_load_32x32(o_addr + c0, ov);
                tmem_load_wait();
                if (live) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        __nv_bfloat162 h[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            h[u] = __floats2bfloat162_rn(__uint_as_float(ov[8 * c + 2 * u]) * inv,
                                                         __uint_as_float(ov[8 * c + 2 * u + 1]) * inv);
                        reinterpret_cast<uint4*>(dst_row + c0)[c] = *reinterpret_cast<uint4*>(h);
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

} // namespace chibi

using namespace chibi;

CHIBI_API int chibi_attention_tc_head_dim() { return D; }

// Attention of the sequences that bring more than one token (all sequences when
// skip_single is 0).  Returns CHIBI_ERR_UNSUPPORTED for page sizes it does not
// take (the page size must divide 128 and be at least 8).  variant: 0 chooses
// between the kernel with one query tile per CTA (1) and the one with two (2).
CHIBI_API int chibi_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                         const int* block_table, int table_stride, const int* seq_rows,
                                         const int* q_start, const int* ctx_len, int seqs, int nq, int nkv,
                                         int page_size, int num_pages, float scale, int window,
                                         int skip_single, int max_q_len, int variant, int kv_splits,
                                         float* scratch, long long scratch_floats, long long tokens,
                                         int* error, cudaStream_t stream)
{
    if (seqs <= 0)
        return CHIBI_OK;
    if (nkv <= 0 || nq % nkv != 0 || window < 0 || variant < 0 || variant > 2)
        return CHIBI_ERR_ARGUMENT;
    if (page_size < 8 || page_size > 128 || KEYS % page_size != 0
        || (reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15)
        || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
        return CHIBI_ERR_UNSUPPORTED;
    AttnTcParams p {};
    p.q = static_cast<const __nv_bfloat16*>(q);
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
    p.cache_rows = (long long)num_pages * nkv * page_size;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.window = window;
    p.skip_single = skip_single;
    p.error = error;
    p.kv_splits = 1;
    CUtensorMap mk, mv;
    if (!tensor_map_2d(k_cache, p.cache_rows, D, D, page_size, &mk)
        || !tensor_map_2d(v_cache, p.cache_rows, D, D, page_size, &mv))
        return CHIBI_ERR_UNSUPPORTED;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)ATC_SMEM);
        if (e != cudaSuccess)
            return (int)e;
        configured = true;
    }
    const long long rows = (long long)max_q_len * p.group;
    // Two query tiles per CTA share the key and value tiles and keep the tensor core busier, but
    // halve the number of CTAs: taken when that still gives every SM a CTA (or when asked for).
    const long long ctas2 = ((rows + 2 * ROWS - 1) / (2 * ROWS)) * nkv * seqs;
    int sms = 148, device = 0;
    if (cudaGetDevice(&device) == cudaSuccess)
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (variant == 2 || (variant == 0 && ctas2 >= sms)) {
        static bool configured2 = false;
        if (!configured2) {
            const cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc2_kernel,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATC2_SMEM);
            if (e != cudaSuccess)
                return (int)e;
            configured2 = true;
        }
        const dim3 grid2((unsigned)((rows + 2 * ROWS - 1) / (2 * ROWS)), nkv, seqs);
        launch(attn_prefill_tc2_kernel, grid2, dim3(ATC2_THREADS), ATC2_SMEM, stream, mk, mv, p);
        return launch_status();
    }
    if (kv_splits > 1) {
        // key ranges: only this kernel (one query tile per CTA) has them
        if (kv_splits > 64 || !scratch || tokens <= 0 || scratch_floats < tokens * nq * kv_splits * (long long)(D + 2)
            || (long long)seqs * kv_splits > 65535)
            return CHIBI_ERR_ARGUMENT;
        p.kv_splits = kv_splits;
        p.part_o = scratch;
        p.part_ml = scratch + (size_t)tokens * nq * kv_splits * D;
    }
    const dim3 grid((unsigned)((rows + ROWS - 1) / ROWS), nkv, seqs * p.kv_splits);
    launch(attn_prefill_tc_kernel, grid, dim3(ATC_THREADS), ATC_SMEM, stream, mk, mv, p);
    int st = launch_status();
    if (st == CHIBI_OK && p.kv_splits > 1) {
        launch(attn_prefill_merge_kernel, dim3(nq, max_q_len, seqs), dim3(D), 0, stream, p);
        st = launch_status();
    }
    return st;
}
