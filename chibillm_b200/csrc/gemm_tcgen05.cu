// out[M, N] = x[M, K] * w[N, K]^T (+ residual) in bfloat16 on the 5th-generation
// tensor cores: TMA brings 128-byte-swizzled K-major tiles of both operands into
// shared memory, one elected thread issues tcgen05.mma (128 x BN x 16 per
// instruction) into a TMEM accumulator, four warps read the accumulator back
// with tcgen05.ld and write the result.
//
// The operand with 128 rows per tile ("A") is x for large M and w for small M
// (decode: the weights fill the 128-row side, the few tokens are the N side of
// the instruction, so no tensor-core work is wasted on padding rows and each
// CTA streams a 128-row slab of the weights).  For small M the K range can be
// split over several CTAs; partial sums go to a 32-bit scratch array and a
// second kernel adds them in a fixed order.
//
// Warp roles (192 threads): warp 0 loads, warp 1 owns TMEM and issues the MMAs,
// warps 2..5 are the epilogue (warp w reads TMEM lanes 32 * (w % 4) ..).
#include <mutex>
#include <unordered_map>

#define CHIBI_UNIT gemm_tcgen05
#define CHIBI_UNIT_ID 3
#include "common.cuh"
#include "sm100.cuh"
#include "tensor_map.cuh"

namespace chibi {

using namespace sm100;

constexpr int TILE_A = 128;   // rows of the A operand per tile = UMMA M
constexpr int TILE_K = 64;    // bf16 per row of a tile = one 128-byte swizzle atom
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;

struct GemmParams {
    int rows_a, rows_b, K;
    int k_blocks_total, k_blocks_per_split;
    int swap;              // 0: A = x (lane = token m, column = feature n); 1: A = w
    int M, N;              // logical sizes of out
    void* out;
    int out_type;
    long long out_stride;
    const float* residual;
    long long res_stride;
    float* partial;        // [splits][M][N] when the K range is split through global memory, else null
    int swiglu;            // the rows of w come in blocks of 64 gate rows then 64 up rows; out[M, N / 2] =
                           // silu(gate) * up
    int* error;
    // Many rows (the persistent kernel): the last sk_tiles output tiles do not fill a round of all
    // CTAs, so the other CTAs help with them.  CTA i < sk_tiles takes the first sk_head K blocks of
    // tile i (these CTAs walk K together, as a round of whole tiles does, and share what they load);
    // the rest of those tiles' K blocks, end to end, is dealt out in runs of sk_per to the next
    // sk_helpers CTAs.  A helper writes the sums of each piece to a slot of sk_scratch and counts
    // itself in; the tile's first CTA adds those slots to its own sums, in K order, and writes the tile.
    int sk_tiles, sk_head, sk_helpers, sk_per, sk_slots_per_helper;
    float* sk_scratch;     // [helpers][slots per helper][128 x BN]
    int* sk_counters;      // [sk_tiles][4], zero between launches
    // Many rows, RMSNorm folded into the products around it.  The per-row factor of the norm commutes
    // with a product: RMSNorm(h) W^T = inv[m] * ((h * w_norm) W^T).  The product that completes the
    // residual (out = residual + x W^T, 32-bit) also writes normed_out = bf16(out * (norm_w + offset))
    // and, per row and column tile, the sum of the squares of out (ssq_out[m][tile]); the product that
    // reads normed_out multiplies its sums by inv[m] = rsqrt(sum of row_ssq[m][0 .. parts) / n + eps)
    // before what follows (conversion to bfloat16, SwiGLU).
    const void* norm_w;    // [N], null: no norm output
    int norm_w_type;
    float norm_offset;
    __nv_bfloat16* normed_out;
    long long normed_stride;
    float* ssq_out;        // [M][ssq_out_parts]
    int ssq_out_parts;
    const float* row_ssq;  // [M][row_ssq_parts], null: no factor
    int row_ssq_parts;
    float row_eps;
    int row_n;
    // Many rows, the q | k | v product finished head by head (head size 128: a 256-column tile is two
    // heads, and a thread of the epilogue holds a token's whole head).  Query and key heads get their
    // RMSNorm (weights may be null) and the split-half rotation with the token's cosines and sines;
    // query heads go to q_out [M][nq * 128], key and value heads to the token's slot of the paged
    // caches.  Nothing is written to `out`.
    const float* h_cos_sin;        // [M][128]: 64 cosines then 64 sines of each token; null: not this mode
    const long long* h_slots;      // [M]: element offset of the token's slot for kv head 0, or -1 (no write)
    __nv_bfloat16* h_q_out;
    __nv_bfloat16* h_k_cache;
    __nv_bfloat16* h_v_cache;
    const void* h_q_norm_w;
    const void* h_k_norm_w;
    int h_w_type, h_nq, h_nkv, h_page_size;
    float h_eps, h_offset;
};

template <int BN>
struct GemmSmem {
    static constexpr int A_BYTES = TILE_A * TILE_K * 2;
    static constexpr int B_BYTES = BN * TILE_K * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
};

__device__ __forceinline__ void store_value(const GemmParams& p, int m, int n, float v)
{
    if (m >= p.M || n >= p.N)
        return;
    if (p.residual)
        v = p.residual[(size_t)m * p.res_stride + n] + v;
    if (p.out_type == CHIBI_F32)
        static_cast<float*>(p.out)[(size_t)m * p.out_stride + n] = v;
    else
        static_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.out_stride + n] = __float2bfloat16_rn(v);
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b, const GemmParams p)
{
    pdl_trigger();
    using S = GemmSmem<BN>;
    extern __shared__ uint8_t smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * S::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tmem_full_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_a = blockIdx.x, tile_b = blockIdx.y, split = blockIdx.z;
    const int kb_begin = split * p.k_blocks_per_split;
    int kb_end = kb_begin + p.k_blocks_per_split;
    if (kb_end > p.k_blocks_total)
        kb_end = p.k_blocks_total;
    const int kb_count = kb_end > kb_begin ? kb_end - kb_begin : 0;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(tmem_full_bar, 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            tma_prefetch_descriptor(&map_a);
            tma_prefetch_descriptor(&map_b);
            // The weights do not depend on the kernel before this one: their first
            // tiles are on their way before we wait for it.  (Weights are the A
            // operand when the operands are swapped, else the B operand.)
            const int early = kb_count < STAGES ? kb_count : STAGES;
            for (int i = 0; i < early; ++i) {
                uint8_t* a_dst = smem + i * S::STAGE_BYTES;
                mbar_arrive_expect_tx(&full_bar[i], S::STAGE_BYTES);
                const int k = (kb_begin + i) * TILE_K;
                if (p.swap)
                    tma_load_2d(a_dst, &map_a, &full_bar[i], k, tile_a * TILE_A);
                else
                    tma_load_2d(a_dst + S::A_BYTES, &map_b, &full_bar[i], k, tile_b * BN);
            }
            pdl_wait();
            for (int i = 0; i < early; ++i) {
                uint8_t* a_dst = smem + i * S::STAGE_BYTES;
                const int k = (kb_begin + i) * TILE_K;
                if (p.swap)
                    tma_load_2d(a_dst + S::A_BYTES, &map_b, &full_bar[i], k, tile_b * BN);
                else
                    tma_load_2d(a_dst, &map_a, &full_bar[i], k, tile_a * TILE_A);
            }
            for (int i = early; i < kb_count; ++i) {
                const int s = i % STAGES;
                const uint32_t round = i / STAGES;
                mbar_wait(&empty_bar[s], (round - 1) & 1, p.error, 11);
                uint8_t* a_dst = smem + s * S::STAGE_BYTES;
                uint8_t* b_dst = a_dst + S::A_BYTES;
                mbar_arrive_expect_tx(&full_bar[s], S::STAGE_BYTES);
                const int k = (kb_begin + i) * TILE_K;
                tma_load_2d(a_dst, &map_a, &full_bar[s], k, tile_a * TILE_A);
                tma_load_2d(b_dst, &map_b, &full_bar[s], k, tile_b * BN);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = make_idesc_bf16_f32(TILE_A, BN);
            for (int i = 0; i < kb_count; ++i) {
                const int s = i % STAGES;
                const uint32_t round = i / STAGES;
                mbar_wait(&full_bar[s], round & 1, p.error, 12);
                tcgen05_fence_after();
                const uint32_t a_addr = smem_addr(smem + s * S::STAGE_BYTES);
                const uint32_t b_addr = a_addr + S::A_BYTES;
#pragma unroll
                for (int k = 0; k < TILE_K / UMMA_K; ++k) {
                    const uint64_t a_desc = make_kmajor_sw128_desc(a_addr + k * UMMA_K * 2);
                    const uint64_t b_desc = make_kmajor_sw128_desc(b_addr + k * UMMA_K * 2);
                    tcgen05_mma_bf16(tmem_base, a_desc, b_desc, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                tcgen05_commit(&empty_bar[s]);   // the stage is free once these MMAs have read it
            }
            tcgen05_commit(tmem_full_bar);
        }
    } else {
        // epilogue: lane quarter of this warp
        const int quarter = warp & 3;
        const int a_row = tile_a * TILE_A + quarter * 32 + lane;
        bool ok = true;
        pdl_wait();        // before this warp reads or writes global memory
        if (kb_count > 0)
            ok = mbar_wait(tmem_full_bar, 0, p.error, 13);
        tcgen05_fence_after();
        timeline_mark(0);              // the accumulator is complete
        constexpr int CHUNK = BN < 32 ? 16 : 32;
        if (p.swiglu) {
            // x is the A operand: this thread has row m and the BN columns of w's rows, which come
            // as [64 gate | 64 up] blocks
            const int m = a_row;
            if constexpr (BN >= 128) {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    if ((c0 & 64) != 0)
                        continue;                       // the up halves are read with their gate halves
                    uint32_t g[32], u[32];
                    if (kb_count > 0 && ok) {
                        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c0;
                        tmem_load_32x32(taddr, g);
                        tmem_load_32x32(taddr + 64, u);
                        tmem_load_wait();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            g[j] = u[j] = 0;
                    }
                    // w rows tile_b * BN + c0 .. are gate rows of feature (tile_b * BN + c0) / 2 + (c0 % 64)
                    const int w_row = tile_b * BN + c0;
                    const int feat0 = (w_row >> 7) * 64 + (w_row & 63);
                    const int inter = p.N >> 1;
                    if (m < p.M) {
                        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.out_stride + feat0;
                        if (feat0 + 32 <= inter && p.out_stride % 8 == 0) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                __nv_bfloat162 h[4];
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    const float g0 = __uint_as_float(g[8 * j + 2 * q]), g1 = __uint_as_float(g[8 * j + 2 * q + 1]);
                                    const float u0 = __uint_as_float(u[8 * j + 2 * q]), u1 = __uint_as_float(u[8 * j + 2 * q + 1]);
                                    h[q] = __floats2bfloat162_rn((g0 / (1.f + expf(-g0))) * u0, (g1 / (1.f + expf(-g1))) * u1);
                                }
                                reinterpret_cast<uint4*>(dst)[j] = *reinterpret_cast<uint4*>(h);
                            }
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (feat0 + j < inter) {
                                    const float gv = __uint_as_float(g[j]), uv = __uint_as_float(u[j]);
                                    dst[j] = __float2bfloat16_rn((gv / (1.f + expf(-gv))) * uv);
                                }
                        }
                    }
                }
            }
        } else
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += CHUNK) {
            uint32_t r[CHUNK];
            if (kb_count > 0 && ok) {
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c0;
                if constexpr (CHUNK == 32)
                    tmem_load_32x32(taddr, r);
                else
                    tmem_load_32x16(taddr, r);
                tmem_load_wait();
            } else {
#pragma unroll
                for (int j = 0; j < CHUNK; ++j)
                    r[j] = 0;
            }
            const int b_row0 = tile_b * BN + c0;
            if (p.partial) {
                float* base = p.partial + (size_t)split * p.M * p.N;
#pragma unroll
                for (int j = 0; j < CHUNK; ++j) {
                    const int m = p.swap ? b_row0 + j : a_row;
                    const int n = p.swap ? a_row : b_row0 + j;
                    if (m < p.M && n < p.N)
                        base[(size_t)m * p.N + n] = __uint_as_float(r[j]);
                }
            } else if (p.swap) {
#pragma unroll
                for (int j = 0; j < CHUNK; ++j)
                    store_value(p, b_row0 + j, a_row, __uint_as_float(r[j]));
            } else {
                const int m = a_row;
                const bool vec = m < p.M && b_row0 + CHUNK <= p.N && (p.out_stride % 8 == 0)
                    && (!p.residual || p.res_stride % 4 == 0);
                if (vec && p.out_type == CHIBI_F32) {
                    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.out) + (size_t)m * p.out_stride + b_row0);
                    const float4* res = p.residual
                        ? reinterpret_cast<const float4*>(p.residual + (size_t)m * p.res_stride + b_row0)
                        : nullptr;
#pragma unroll
                    for (int j = 0; j < CHUNK / 4; ++j) {
                        float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                               __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                        if (res) {
                            const float4 q = res[j];
                            v.x = q.x + v.x; v.y = q.y + v.y; v.z = q.z + v.z; v.w = q.w + v.w;
                        }
                        dst[j] = v;
                    }
                } else if (vec && p.out_type == CHIBI_BF16 && !p.residual) {
                    uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.out_stride + b_row0);
#pragma unroll
                    for (int j = 0; j < CHUNK / 8; ++j) {
                        __nv_bfloat162 h[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            h[q] = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * q]),
                                                         __uint_as_float(r[8 * j + 2 * q + 1]));
                        dst[j] = *reinterpret_cast<uint4*>(h);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < CHUNK; ++j)
                        store_value(p, m, b_row0 + j, __uint_as_float(r[j]));
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------ many rows: one CTA per SM
// The epilogue of one 128 x BN tile whose rows are tokens (x is the A operand).
// tcgen05.ld gives a thread one row of the tile; written out like that, every
// store instruction of a warp would touch 32 rows with 16 bytes each.  So a warp
// passes each 32 x 128-byte piece through a staging buffer in shared memory
// (16-byte units, XOR-swizzled by row so that neither side has bank conflicts)
// and writes it with eight lanes per row: four whole 128-byte lines per
// instruction.  `taddr` is the TMEM address of this thread's lane at the tile's
// first column, `m0` the matrix row of the warp's first lane.
constexpr int EPILOGUE_STAGE_BYTES = 32 * 128;     // per epilogue warp

__device__ __forceinline__ uint4* stage_unit(uint8_t* stage, int row, int unit)
{
    return reinterpret_cast<uint4*>(stage + row * 128 + ((unit ^ (row & 7)) << 4));
}

__device__ __forceinline__ float silu_mul(float g, float u)
{
    return __fdividef(g, 1.f + __expf(-g)) * u;
}

// One 128-row tile of the q | k | v product as one or two heads (see GemmParams): this thread's token is
// row m0 + lane, `inv` the factor that the row of x lacked.  The rotation pairs column j with column
// j + 64 of the same row, so the head is read in pairs of 32-column pieces; the results pass
// through the staging buffer as two lines of 64 columns, as everywhere in this epilogue.
__device__ __forceinline__ float head_weight(const void* w, int type, int col, float offset)
{
    return (type == CHIBI_F32 ? static_cast<const float*>(w)[col]
                              : __bfloat162float(static_cast<const __nv_bfloat16*>(w)[col])) + offset;
}

__device__ __forceinline__ void write_staged_line(uint8_t* stage, __nv_bfloat16* dst, int lane)
{
    const int sub = lane >> 3, unit = lane & 7;
    const unsigned long long mine = reinterpret_cast<unsigned long long>(dst);
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = 4 * i + sub;
        const uint4 v = *stage_unit(stage, r, unit);
        const unsigned long long d = __shfl_sync(0xffffffffu, mine, r);        // row r's destination
        if (d)
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(d) + unit * 8) = v;
    }
    __syncwarp();
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b)
{
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// head_w: [2][128] floats in shared memory, the norm weights (+ offset) of query and key heads
// (ones without a norm).
__device__ __forceinline__ void epilogue_heads(const GemmParams& p, uint32_t taddr, int m0, int lane, int tile_b,
                                               int heads_per_tile, uint8_t* stage, float inv, const float* head_w)
{
    const int m = m0 + lane;
    const bool row_ok = m < p.M;
    const long long slot = (row_ok && p.h_slots) ? p.h_slots[m] : -1;
    const float* cs = p.h_cos_sin + (size_t)(row_ok ? m : 0) * 128;
#pragma unroll 1
    for (int hh = 0; hh < heads_per_tile; ++hh) {
        const int head = tile_b * heads_per_tile + hh;            // the same for the whole warp
        const uint32_t t0 = taddr + hh * 128;
        const int kind = head < p.h_nq ? 0 : (head < p.h_nq + p.h_nkv ? 1 : 2);
        __nv_bfloat16* dst = nullptr;                             // this thread's row of the head
        if (row_ok) {
            if (kind == 0)
                dst = p.h_q_out + ((size_t)m * p.h_nq + head) * 128;
            else if (slot >= 0 && kind == 1)
                dst = p.h_k_cache + slot + (size_t)(head - p.h_nq) * p.h_page_size * 128;
            else if (slot >= 0)
                dst = p.h_v_cache + slot + (size_t)(head - p.h_nq - p.h_nkv) * p.h_page_size * 128;
        }
        if (kind == 2) {
            // a value head: the sums as they are
#pragma unroll 1
            for (int c0 = 0; c0 < 128; c0 += 64) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t r32[32];
                    tmem_load_32x32(t0 + c0 + 32 * h, r32);
                    tmem_load_wait();
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        *stage_unit(stage, lane, 4 * h + j) =
                            make_uint4(pack_bf16(inv * __uint_as_float(r32[8 * j]), inv * __uint_as_float(r32[8 * j + 1])),
                                       pack_bf16(inv * __uint_as_float(r32[8 * j + 2]), inv * __uint_as_float(r32[8 * j + 3])),
                                       pack_bf16(inv * __uint_as_float(r32[8 * j + 4]), inv * __uint_as_float(r32[8 * j + 5])),
                                       pack_bf16(inv * __uint_as_float(r32[8 * j + 6]), inv * __uint_as_float(r32[8 * j + 7])));
                }
                write_staged_line(stage, dst ? dst + c0 : nullptr, lane);
            }
            continue;
        }
        const bool normed = (kind == 0 ? p.h_q_norm_w : p.h_k_norm_w) != nullptr;
        const float* w = head_w + kind * 128;
        // the row's cosines and sines of the first columns are on their way while the sum of
        // squares is taken
        float4 cv[4], sv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            cv[u] = *reinterpret_cast<const float4*>(cs + 4 * u);
            sv[u] = *reinterpret_cast<const float4*>(cs + 64 + 4 * u);
        }
        float scale = inv;                                        // the row's factor times the head's
        if (normed) {
            float ss = 0.f;
#pragma unroll 1
            for (int c0 = 0; c0 < 128; c0 += 32) {
                uint32_t r32[32];
                tmem_load_32x32(t0 + c0, r32);
                tmem_load_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float x = inv * __uint_as_float(r32[j]);
                    ss = fmaf(x, x, ss);
                }
            }
            scale = inv * rsqrtf(ss / 128.f + p.h_eps);
        }
        uint32_t lo[32], hi[32];                                  // columns 0..63 and 64..127 as bfloat16 pairs
#pragma unroll
        for (int c = 0; c < 64; c += 16) {
            uint32_t a[16], b[16];
            tmem_load_32x16(t0 + c, a);
            tmem_load_32x16(t0 + 64 + c, b);
            float4 cn[4], sn[4];                                  // the next columns' angles
            if (c + 16 < 64) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    cn[u] = *reinterpret_cast<const float4*>(cs + c + 16 + 4 * u);
                    sn[u] = *reinterpret_cast<const float4*>(cs + 64 + c + 16 + 4 * u);
                }
            }
            tmem_load_wait();
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float cosv[4] = { cv[u].x, cv[u].y, cv[u].z, cv[u].w };
                const float sinv[4] = { sv[u].x, sv[u].y, sv[u].z, sv[u].w };
                float ol[4], oh[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = 4 * u + e;
                    const float x = (scale * __uint_as_float(a[j])) * w[c + j];
                    const float y = (scale * __uint_as_float(b[j])) * w[64 + c + j];
                    ol[e] = x * cosv[e] - y * sinv[e];
                    oh[e] = y * cosv[e] + x * sinv[e];
                }
                lo[(c >> 1) + 2 * u] = pack_bf16(ol[0], ol[1]);
                lo[(c >> 1) + 2 * u + 1] = pack_bf16(ol[2], ol[3]);
                hi[(c >> 1) + 2 * u] = pack_bf16(oh[0], oh[1]);
                hi[(c >> 1) + 2 * u + 1] = pack_bf16(oh[2], oh[3]);
            }
            if (c + 16 < 64) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    cv[u] = cn[u];
                    sv[u] = sn[u];
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
            *stage_unit(stage, lane, j) = make_uint4(lo[4 * j], lo[4 * j + 1], lo[4 * j + 2], lo[4 * j + 3]);
        write_staged_line(stage, dst, lane);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            *stage_unit(stage, lane, j) = make_uint4(hi[4 * j], hi[4 * j + 1], hi[4 * j + 2], hi[4 * j + 3]);
        write_staged_line(stage, dst ? dst + 64 : nullptr, lane);
    }
}

template <int BN>
__device__ __forceinline__ void epilogue_token_rows(const GemmParams& p, uint32_t taddr, int m0, int lane,
                                                    int tile_b, uint8_t* stage, const float* head_w = nullptr)
{
    const int m = m0 + lane;
    const int sub = lane >> 3, unit = lane & 7;      // the write-out: rows 4 * i + sub, 16-byte unit `unit`
    const bool inside = (tile_b + 1) * BN <= p.N && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
    // the factor of the norm that was left out of x (this thread's row; 1 without one)
    float inv = 1.f;
    if (p.row_ssq && m < p.M) {
        float ss = 0.f;
        for (int j = 0; j < p.row_ssq_parts; ++j)
            ss += __ldg(p.row_ssq + (size_t)m * p.row_ssq_parts + j);
        inv = rsqrtf(ss / (float)p.row_n + p.row_eps);
    }
    // every branch below is taken by whole warps: tcgen05.ld is a warp-wide instruction
    if constexpr (BN % 128 == 0) {
        if (p.h_cos_sin) {
            epilogue_heads(p, taddr, m0, lane, tile_b, BN / 128, stage, inv, head_w);
            return;
        }
    }
    if (p.swiglu && inside && p.out_stride % 8 == 0) {
        // the BN columns are rows of w, which come as [64 gate | 64 up] blocks
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 128) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t g[32], u[32];
                tmem_load_32x32(taddr + c0 + 32 * h, g);
                tmem_load_32x32(taddr + c0 + 64 + 32 * h, u);
                tmem_load_wait();
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 v[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        v[q] = __floats2bfloat162_rn(
                            silu_mul(inv * __uint_as_float(g[8 * j + 2 * q]), inv * __uint_as_float(u[8 * j + 2 * q])),
                            silu_mul(inv * __uint_as_float(g[8 * j + 2 * q + 1]),
                                     inv * __uint_as_float(u[8 * j + 2 * q + 1])));
                    *stage_unit(stage, lane, 4 * h + j) = *reinterpret_cast<uint4*>(v);
                }
            }
            __syncwarp();
            const int feat0 = (tile_b * BN + c0) >> 1;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = 4 * i + sub;
                const uint4 v = *stage_unit(stage, r, unit);
                if (m0 + r < p.M)
                    *reinterpret_cast<uint4*>(out + (size_t)(m0 + r) * p.out_stride + feat0 + unit * 8) = v;
            }
            __syncwarp();
        }
        return;
    }
    if (p.swiglu) {
        const int inter = p.N >> 1;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
            if ((c0 & 64) != 0)
                continue;                           // the up halves are read with their gate halves
            uint32_t g[32], u[32];
            tmem_load_32x32(taddr + c0, g);
            tmem_load_32x32(taddr + c0 + 64, u);
            tmem_load_wait();
            const int w_row = tile_b * BN + c0;
            const int feat0 = (w_row >> 7) * 64 + (w_row & 63);
            if (m < p.M) {
                __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.out_stride + feat0;
                for (int j = 0; j < 32; ++j)
                    if (feat0 + j < inter) {
                        const float gv = __uint_as_float(g[j]), uv = __uint_as_float(u[j]);
                        dst[j] = __float2bfloat16_rn((gv / (1.f + expf(-gv))) * uv);
                    }
            }
            __syncwarp();
        }
        return;
    }
    if (p.out_type == CHIBI_F32 && inside && p.out_stride % 4 == 0
        && (!p.residual || (p.res_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0))) {
        // out may be the residual itself: the residual of the next 32 columns is
        // fetched before this piece is stored (the compiler may not move it up)
        float* out = static_cast<float*>(p.out);
        const float* res = p.residual;
        const int n_tile = tile_b * BN;
        float4 q[8], qn[8];
        float ssq[8];                   // with a norm output: squares of this lane's columns of rows 4 i + sub
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = m0 + 4 * i + sub;
            q[i] = (res && r < p.M) ? *reinterpret_cast<const float4*>(res + (size_t)r * p.res_stride + n_tile + unit * 4)
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
            ssq[i] = 0.f;
        }
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t r32[32];
            tmem_load_32x32(taddr + c0, r32);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = m0 + 4 * i + sub;
                qn[i] = (res && r < p.M && c0 + 32 < BN)
                    ? *reinterpret_cast<const float4*>(res + (size_t)r * p.res_stride + n_tile + c0 + 32 + unit * 4)
                    : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            tmem_load_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j)
                *stage_unit(stage, lane, j) = make_uint4(r32[4 * j], r32[4 * j + 1], r32[4 * j + 2], r32[4 * j + 3]);
            __syncwarp();
            float w4[4] = { 0.f, 0.f, 0.f, 0.f };
            if (p.norm_w) {
                const int col = n_tile + c0 + unit * 4;
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    w4[e] = (p.norm_w_type == CHIBI_F32 ? static_cast<const float*>(p.norm_w)[col + e]
                                                        : __bfloat162float(static_cast<const __nv_bfloat16*>(p.norm_w)[col + e]))
                        + p.norm_offset;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = 4 * i + sub;
                const uint4 v = *stage_unit(stage, r, unit);
                const float4 h = make_float4(q[i].x + __uint_as_float(v.x), q[i].y + __uint_as_float(v.y),
                                             q[i].z + __uint_as_float(v.z), q[i].w + __uint_as_float(v.w));
                if (m0 + r < p.M) {
                    *reinterpret_cast<float4*>(out + (size_t)(m0 + r) * p.out_stride + n_tile + c0 + unit * 4) = h;
                    if (p.norm_w) {
                        ssq[i] = fmaf(h.x, h.x, fmaf(h.y, h.y, fmaf(h.z, h.z, fmaf(h.w, h.w, ssq[i]))));
                        const __nv_bfloat162 lo = __floats2bfloat162_rn(h.x * w4[0], h.y * w4[1]);
                        const __nv_bfloat162 hi = __floats2bfloat162_rn(h.z * w4[2], h.w * w4[3]);
                        uint2 packed;
                        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
                        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(p.normed_out + (size_t)(m0 + r) * p.normed_stride + n_tile + c0 + unit * 4) =
                            packed;
                    }
                }
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i)
                q[i] = qn[i];
        }
        if (p.norm_w) {
            // a row's eight lanes (the units) add up, always in the same order
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float s = ssq[i];
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                const int r = m0 + 4 * i + sub;
                if (unit == 0 && r < p.M)
                    p.ssq_out[(size_t)r * p.ssq_out_parts + tile_b] = s;
            }
        }
        return;
    }
    if (p.out_type == CHIBI_BF16 && !p.residual && inside && p.out_stride % 8 == 0) {
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t r32[32];
                tmem_load_32x32(taddr + c0 + 32 * h, r32);
                tmem_load_wait();
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 v[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        v[q] = __floats2bfloat162_rn(inv * __uint_as_float(r32[8 * j + 2 * q]),
                                                     inv * __uint_as_float(r32[8 * j + 2 * q + 1]));
                    *stage_unit(stage, lane, 4 * h + j) = *reinterpret_cast<uint4*>(v);
                }
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = 4 * i + sub;
                const uint4 v = *stage_unit(stage, r, unit);
                if (m0 + r < p.M)
                    *reinterpret_cast<uint4*>(out + (size_t)(m0 + r) * p.out_stride + tile_b * BN + c0 + unit * 8) = v;
            }
            __syncwarp();
        }
        return;
    }
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_load_32x32(taddr + c0, r);
        tmem_load_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j)
            store_value(p, m, tile_b * BN + c0 + j, __uint_as_float(r[j]));
        __syncwarp();
    }
}

// The pieces of work of one CTA of the persistent kernel, in the order in which its three roles
// take them: whole tiles (tile t, t + CTAs, ...), then either the head of one shared tile or a
// helper's run over the tails of shared tiles (see GemmParams).
struct WorkWalk {
    int t, step, whole_tiles, kb, head, own_tile, tail, pos, end, slot;
    __device__ WorkWalk(const GemmParams& p, int tiles_total)
    {
        whole_tiles = tiles_total - p.sk_tiles;
        kb = p.k_blocks_total;
        t = blockIdx.x;
        step = gridDim.x;
        head = p.sk_head;
        tail = kb - head;
        own_tile = (int)blockIdx.x < p.sk_tiles ? whole_tiles + (int)blockIdx.x : -1;
        const int helper = (int)blockIdx.x - p.sk_tiles;
        pos = end = 0;
        slot = 0;
        if (helper >= 0 && helper < p.sk_helpers) {
            const int all = p.sk_tiles * tail;
            const long long b = (long long)helper * p.sk_per;
            pos = b < all ? (int)b : all;
            end = b + p.sk_per < all ? (int)(b + p.sk_per) : all;
            slot = helper * p.sk_slots_per_helper;
        }
    }
    // kind: 0 a whole tile, 1 the head of a shared tile (collect the rest), 2 a helper's piece (-> slot)
    __device__ bool next(int& tile, int& k0, int& k1, int& kind, int& piece_slot)
    {
        piece_slot = 0;
        if (t < whole_tiles) {
            tile = t;
            k0 = 0;
            k1 = kb;
            kind = 0;
            t += step;
            return true;
        }
        if (own_tile >= 0) {
            tile = own_tile;
            k0 = 0;
            k1 = head;
            kind = head < kb ? 1 : 0;
            own_tile = -1;
            return true;
        }
        if (pos < end) {
            const int ti = pos / tail;
            k0 = head + (pos - ti * tail);
            k1 = k0 + (end - pos) < kb ? k0 + (end - pos) : kb;
            tile = whole_tiles + ti;
            kind = 2;
            piece_slot = slot++;
            pos += k1 - k0;
            return true;
        }
        return false;
    }
};

__device__ __forceinline__ int load_acquire(const int* p)
{
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// A CTA that has K blocks from the middle of a tile: its sums go to its slot and the warp counts
// itself in for its quarter of the rows.  A slot is [quarter][half of the columns][column / 4][row][4],
// so that what one warp of the collecting CTA needs is one run of 16 KB per half.
constexpr int SK_HALF_FLOATS = 32 * 32 * 4;         // 128 columns of 32 rows
template <int BN>
__device__ __forceinline__ void contribute_partial_tile(const GemmParams& p, uint32_t taddr, int quarter, int lane,
                                                        int shared_tile, int piece_slot)
{
    static_assert(BN == 256, "the slot layout is written for tiles of 256 columns");
    float4* slot = reinterpret_cast<float4*>(p.sk_scratch + (size_t)piece_slot * (TILE_A * BN)
                                             + (size_t)quarter * 2 * SK_HALF_FLOATS) + lane;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_load_32x32(taddr + c0, r);
        tmem_load_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j)
            slot[(c0 / 4 + j) * 32] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                  __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
    }
    __threadfence();
    __syncwarp();
    if (lane == 0)
        atomicAdd(p.sk_counters + shared_tile * 4 + quarter, 1);
}

// The CTA with a tile's first K blocks: waits (with a limit) until the helpers that share the
// tile's other K blocks have left their sums, adds them to its own in TMEM in K order, and clears
// the counter for the next launch.  The sums come through shared memory by bulk copies, 16 KB at a
// time into three buffers (`buffers`: 48 KB of this warp's own, free because this is the CTA's last
// piece of work).
template <int BN>
__device__ __forceinline__ void collect_partial_tiles(const GemmParams& p, uint32_t taddr, int quarter, int lane,
                                                      int shared_tile, uint8_t* buffers, uint64_t* bars)
{
    static_assert(BN == 256, "the slot layout is written for tiles of 256 columns");
    // the tile's tail is [shared_tile * tail, + tail) of the helpers' range; helper j's piece of it is
    // the (shared_tile - first tile of j)-th slot of j
    const int tail = p.k_blocks_total - p.sk_head;
    const int helper0 = (shared_tile * tail) / p.sk_per;
    const int others = ((shared_tile + 1) * tail - 1) / p.sk_per - helper0 + 1;
    const auto slot_of = [&](int c) {
        const int j = helper0 + c;
        return j * p.sk_slots_per_helper + shared_tile - (j * p.sk_per) / tail;
    };
    int* counter = p.sk_counters + shared_tile * 4 + quarter;
    int ok = 1;
    if (lane == 0 && load_acquire(counter) < others) {
        const long long start = clock64();
        while (load_acquire(counter) < others) {
            if (clock64() - start > WAIT_LIMIT_CYCLES) {
                if (p.error)
                    atomicExch(p.error, 15);
                ok = 0;
                break;
            }
            __nanosleep(40);
        }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    if (!ok)
        return;
    if (lane == 0)
        *counter = 0;
    const float* mine = p.sk_scratch + (size_t)quarter * 2 * SK_HALF_FLOATS;
    const int items = 2 * others;               // (CTA, half of the columns), in that order
    constexpr uint32_t BYTES = SK_HALF_FLOATS * 4;
    const auto fetch = [&](int n) {             // item n -> buffer n % 3 (lane 0 only)
        mbar_arrive_expect_tx(&bars[n % 3], BYTES);
        bulk_load(buffers + (n % 3) * BYTES, mine + (size_t)slot_of(n >> 1) * (TILE_A * BN) + (n & 1) * SK_HALF_FLOATS,
                  BYTES, &bars[n % 3]);
    };
    if (lane == 0) {
        fetch(0);
        fetch(1);
    }
#pragma unroll 1
    for (int i = 0; i < items; ++i) {
        if (i + 2 < items) {
            __syncwarp();                        // every lane has read what item i - 1 left in that buffer
            if (lane == 0) {
                fence_proxy_async();
                fetch(i + 2);
            }
        }
        if (!__all_sync(0xffffffffu, mbar_wait(&bars[i % 3], (i / 3) & 1, p.error, 16)))
            return;                              // (the whole warp: what follows is warp-wide)
        const float4* src = reinterpret_cast<const float4*>(buffers + (i % 3) * BYTES) + lane;
        const uint32_t col0 = (i & 1) * 128;
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 32) {
            uint32_t r[32];
            tmem_load_32x32(taddr + col0 + c0, r);
            tmem_load_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 q = src[(c0 / 4 + j) * 32];
                r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + q.x);
                r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + q.y);
                r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + q.z);
                r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + q.w);
            }
            tmem_store_32x32(taddr + col0 + c0, r);
        }
        tmem_store_wait();
    }
}

// Tile t of the many-row kernel -> (row block, column block).  The row blocks are taken in bands
// of 16 (2,048 rows): within a band the row block runs fastest, so the CTAs that work at the same
// time share a few blocks of w and the band's rows of x (16 x 128 x K values) stay in L2 while
// the column blocks go by; without bands, with 64 row blocks and K = 8,192, x (134 MB) was
// fetched from memory again for every pair of column blocks.
constexpr int TILE_BAND = 16;
template <int BAND = TILE_BAND>
__device__ __forceinline__ void tile_of(int t, int tiles_m, int tiles_total, int& tile_a, int& tile_b)
{
    const int tiles_n = tiles_total / tiles_m;
    const int per_band = BAND * tiles_n;
    const int band = t / per_band, within = t - band * per_band;
    const int rows = min(BAND, tiles_m - band * BAND);
    tile_b = within / rows;
    tile_a = band * BAND + (within - tile_b * rows);
}

// x is the A operand (many rows).  One CTA per SM walks over the output tiles (tile_of above).
// Two accumulators in TMEM: while the four epilogue warps read one tile out, the MMA thread
// already fills the other.
template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                               const __grid_constant__ CUtensorMap map_b, const GemmParams p,
                               int tiles_m, int tiles_total)
{
    pdl_trigger();
    using S = GemmSmem<BN>;
    static_assert(2 * BN <= 512, "two accumulators must fit the 512 TMEM columns");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * S::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tmem_full_bar = empty_bar + STAGES;     // [2]
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;     // [2]
    uint64_t* collect_bar = tmem_empty_bar + 2;       // [4][3]: the bulk copies of a shared-out tile's other sums
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(collect_bar + 12);
    uint8_t* stage_base = reinterpret_cast<uint8_t*>(tmem_slot + 4);      // 16-byte aligned
    float* head_w = reinterpret_cast<float*>(stage_base + 4 * EPILOGUE_STAGE_BYTES);   // [2][128]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t TMEM_COLS = 2 * BN;
    if (p.h_cos_sin && threadIdx.x < 128) {
        // the norm weights of query and key heads (weights: nothing of this step writes them)
        head_w[threadIdx.x] = p.h_q_norm_w ? head_weight(p.h_q_norm_w, p.h_w_type, threadIdx.x, p.h_offset) : 1.f;
        head_w[128 + threadIdx.x] = p.h_k_norm_w ? head_weight(p.h_k_norm_w, p.h_w_type, threadIdx.x, p.h_offset) : 1.f;
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full_bar[b], 1);
            mbar_init(&tmem_empty_bar[b], 128);       // every epilogue thread arrives
        }
        for (int b = 0; b < 12; ++b)
            mbar_init(&collect_bar[b], 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            tma_prefetch_descriptor(&map_a);
            tma_prefetch_descriptor(&map_b);
            uint32_t it = 0;
            bool waited = false;
            WorkWalk walk(p, tiles_total);
            int t, k0, k1, kind, piece_slot;
            while (walk.next(t, k0, k1, kind, piece_slot)) {
                int tile_a, tile_b;
                tile_of(t, tiles_m, tiles_total, tile_a, tile_b);
                for (int kb = k0; kb < k1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (round > 0)
                        mbar_wait(&empty_bar[s], (round - 1) & 1, p.error, 11);
                    uint8_t* a_dst = smem + s * S::STAGE_BYTES;
                    mbar_arrive_expect_tx(&full_bar[s], S::STAGE_BYTES);
                    // w does not depend on the kernel before this one; x does
                    tma_load_2d(a_dst + S::A_BYTES, &map_b, &full_bar[s], kb * TILE_K, tile_b * BN);
                    if (!waited) {
                        pdl_wait();
                        waited = true;
                    }
                    tma_load_2d(a_dst, &map_a, &full_bar[s], kb * TILE_K, tile_a * TILE_A);
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = make_idesc_bf16_f32(TILE_A, BN);
            uint32_t it = 0, lt = 0;
            WorkWalk walk(p, tiles_total);
            int t, k0, k1, kind, piece_slot;
            for (; walk.next(t, k0, k1, kind, piece_slot); ++lt) {
                const uint32_t buf = lt & 1, use = lt >> 1;
                if (use > 0)
                    mbar_wait(&tmem_empty_bar[buf], (use - 1) & 1, p.error, 14);
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = k0; kb < k1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    mbar_wait(&full_bar[s], round & 1, p.error, 12);
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_addr(smem + s * S::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + S::A_BYTES;
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; ++k) {
                        const uint64_t a_desc = make_kmajor_sw128_desc(a_addr + k * UMMA_K * 2);
                        const uint64_t b_desc = make_kmajor_sw128_desc(b_addr + k * UMMA_K * 2);
                        tcgen05_mma_bf16(d_tmem, a_desc, b_desc, idesc, (kb > k0 || k > 0) ? 1u : 0u);
                    }
                    tcgen05_commit(&empty_bar[s]);
                }
                tcgen05_commit(&tmem_full_bar[buf]);
            }
        }
    } else {
        const int quarter = warp & 3;
        pdl_wait();
        uint32_t lt = 0;
        WorkWalk walk(p, tiles_total);
        int t, k0, k1, kind, piece_slot;
        for (; walk.next(t, k0, k1, kind, piece_slot); ++lt) {
            int tile_a, tile_b;
            tile_of(t, tiles_m, tiles_total, tile_a, tile_b);
            const uint32_t buf = lt & 1, use = lt >> 1;
            mbar_wait(&tmem_full_bar[buf], use & 1, p.error, 13);
            tcgen05_fence_after();
            const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(quarter * 32) << 16);
            const int shared_tile = t - walk.whole_tiles;
            bool piece = false;
            if constexpr (BN == 256) {              // only tiles of 256 columns are ever shared out
                if (kind == 2) {
                    contribute_partial_tile<BN>(p, taddr, quarter, lane, shared_tile, piece_slot);
                    piece = true;
                } else if (kind == 1) {
                    // (this is the CTA's last piece of work and its products are done: the stages are free)
                    static_assert(STAGES >= 4 && S::STAGE_BYTES >= 3 * SK_HALF_FLOATS * 4, "a stage per epilogue warp");
                    collect_partial_tiles<BN>(p, taddr, quarter, lane, shared_tile, smem + quarter * S::STAGE_BYTES,
                                              collect_bar + 3 * quarter);
                }
            }
            if (!piece)
                epilogue_token_rows<BN>(p, taddr, tile_a * TILE_A + quarter * 32, lane, tile_b,
                                        stage_base + quarter * EPILOGUE_STAGE_BYTES, head_w);
            tcgen05_fence_before();
            mbar_arrive(&tmem_empty_bar[buf]);
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// The same walk over output tiles by pairs of CTAs (a cluster of two, on the SMs of one TPC): a
// tile is 256 rows x BN columns (256 or 128), computed by tcgen05.mma of 256 rows that the even CTA
// issues for both.  Each CTA fetches its 128 rows of x and its half of the tile's BN rows of w (with
// BN = 256: 32 KB per K block for as many sums as a CTA on its own gets from 48 KB), holds its 128
// rows of the accumulator in its own TMEM and runs the epilogue of those rows.  The barriers that count a
// stage's bytes and the accumulators' release are the even CTA's; its commits arrive in both CTAs.
// A wait that runs out ends the role's loop; every thread of both CTAs reaches the cluster
// barrier at the end.
template <int BN>
struct PairSmem {
    static constexpr int A_BYTES = TILE_A * TILE_K * 2;
    static constexpr int B_BYTES = (BN / 2) * TILE_K * 2;       // this CTA's half of the tile's rows of w
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
};
template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const GemmParams p, int tiles_m, int tiles_total)
{
    pdl_trigger();
    using S = PairSmem<BN>;
    constexpr int PAIR_STAGE_BYTES = S::STAGE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * PAIR_STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tmem_full_bar = empty_bar + STAGES;     // [2]
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;     // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
    uint8_t* stage_base = reinterpret_cast<uint8_t*>(tmem_slot + 4);      // 16-byte aligned
    float* head_w = reinterpret_cast<float*>(stage_base + 4 * EPILOGUE_STAGE_BYTES);   // [2][128]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    constexpr uint32_t TMEM_COLS = 2 * BN;
    if (p.h_cos_sin && threadIdx.x < 128) {
        head_w[threadIdx.x] = p.h_q_norm_w ? head_weight(p.h_q_norm_w, p.h_w_type, threadIdx.x, p.h_offset) : 1.f;
        head_w[128 + threadIdx.x] = p.h_k_norm_w ? head_weight(p.h_k_norm_w, p.h_w_type, threadIdx.x, p.h_offset) : 1.f;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);               // the even CTA's arrival with both CTAs' bytes
            mbar_init(&empty_bar[s], 1);              // a commit, in both CTAs
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full_bar[b], 1);          // a commit, in both CTAs
            mbar_init(&tmem_empty_bar[b], 256);       // every epilogue thread of both CTAs, at the even CTA
        }
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, TMEM_COLS);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before();
    cluster_sync();                                   // both CTAs' barriers exist before either is signalled
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            tma_prefetch_descriptor(&map_a);
            tma_prefetch_descriptor(&map_b);
            uint32_t it = 0;
            bool waited = false, ok = true;
            for (int t = pair; t < tiles_total && ok; t += pairs) {
                int tile_a, tile_b;
                tile_of<TILE_BAND / 2>(t, tiles_m, tiles_total, tile_a, tile_b);   // bands of 2,048 rows here too
                for (int kb = 0; kb < p.k_blocks_total; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1, p.error, 17)) {
                        ok = false;
                        break;
                    }
                    uint8_t* a_dst = smem + s * PAIR_STAGE_BYTES;
                    if (rank == 0)
                        mbar_arrive_expect_tx(&full_bar[s], 2 * PAIR_STAGE_BYTES);
                    const uint32_t bar = peer_smem_addr(smem_addr(&full_bar[s]), 0);
                    tma_load_2d_pair(a_dst + S::A_BYTES, &map_b, bar, kb * TILE_K,
                                     tile_b * BN + (int)rank * (BN / 2));
                    if (!waited) {
                        pdl_wait();
                        waited = true;
                    }
                    tma_load_2d_pair(a_dst, &map_a, bar, kb * TILE_K, (tile_a * 2 + (int)rank) * TILE_A);
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0 && elect_one()) {
            constexpr uint32_t idesc = make_idesc_bf16_f32(2 * TILE_A, BN);
            uint32_t it = 0, lt = 0;
            bool ok = true;
            for (int t = pair; t < tiles_total && ok; t += pairs, ++lt) {
                const uint32_t buf = lt & 1, use = lt >> 1;
                if (use > 0 && !mbar_wait(&tmem_empty_bar[buf], (use - 1) & 1, p.error, 20))
                    break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < p.k_blocks_total; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (!mbar_wait(&full_bar[s], round & 1, p.error, 18)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_addr(smem + s * PAIR_STAGE_BYTES);
                    const uint32_t b_addr = a_addr + S::A_BYTES;
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; ++k) {
                        const uint64_t a_desc = make_kmajor_sw128_desc(a_addr + k * UMMA_K * 2);
                        const uint64_t b_desc = make_kmajor_sw128_desc(b_addr + k * UMMA_K * 2);
                        tcgen05_mma_bf16_pair(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    tcgen05_commit_pair(&empty_bar[s], 3);
                }
                if (ok)
                    tcgen05_commit_pair(&tmem_full_bar[buf], 3);
            }
        }
    } else {
        const int quarter = warp & 3;
        pdl_wait();
        uint32_t lt = 0;
        for (int t = pair; t < tiles_total; t += pairs, ++lt) {
            int tile_a, tile_b;
            tile_of<TILE_BAND / 2>(t, tiles_m, tiles_total, tile_a, tile_b);   // bands of 2,048 rows here too
            const uint32_t buf = lt & 1, use = lt >> 1;
            if (!mbar_wait(&tmem_full_bar[buf], use & 1, p.error, 19))
                break;
            tcgen05_fence_after();
            const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(quarter * 32) << 16);
            epilogue_token_rows<BN>(p, taddr, (tile_a * 2 + (int)rank) * TILE_A + quarter * 32, lane, tile_b,
                                    stage_base + quarter * EPILOGUE_STAGE_BYTES, head_w);
            tcgen05_fence_before();
            mbar_arrive_cluster(peer_smem_addr(smem_addr(&tmem_empty_bar[buf]), 0));     // the even CTA's
        }
    }
    tcgen05_fence_before();
    cluster_sync();                                   // nobody signals a CTA that has left
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// out = (residual +) sum over splits, in split order.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, void* out,
                                     int out_type, long long out_stride, const float* residual,
                                     long long res_stride, int M, int N)
{
    pdl_enter();
    const long long total = (long long)M * N;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int m = (int)(i / N), n = (int)(i - (long long)m * N);
        float v = 0.f;
        for (int s = 0; s < splits; ++s)
            v += partial[(size_t)s * total + i];
        if (residual)
            v = residual[(size_t)m * res_stride + n] + v;
        if (out_type == CHIBI_F32)
            static_cast<float*>(out)[(size_t)m * out_stride + n] = v;
        else
            static_cast<__nv_bfloat16*>(out)[(size_t)m * out_stride + n] = __float2bfloat16_rn(v);
    }
}

// ------------------------------------------------------------------ host side
constexpr int STREAM_K_COUNTERS = 4096;
// zero when loaded; every use that ends well leaves them zero (chibi_gemm_reset_stream_counters after one that did not)
__device__ int stream_k_counters[STREAM_K_COUNTERS];
static struct { float* scratch; long long floats; int fill_divisor; int* counters; } stream_k = { nullptr, 0, 4, nullptr };

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid,
                       cudaStream_t stream)
{
    constexpr size_t smem = STAGES * GemmSmem<BN>::STAGE_BYTES + (2 * STAGES + 1) * 8 + 16 + 1024;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess)
            return (int)e;
        configured = true;
    }
    launch(gemm_tcgen05_kernel<BN, STAGES>, dim3(grid), dim3(GEMM_THREADS), smem, stream, ma, mb, p);
    return launch_status();
}

template <int BN, int STAGES>
static int launch_gemm_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p,
                                  int tiles_m, int tiles_n, cudaStream_t stream, bool share_last_round = true)
{
    constexpr size_t smem = STAGES * GemmSmem<BN>::STAGE_BYTES + (2 * STAGES + 4 + 12) * 8 + 16
        + 4 * EPILOGUE_STAGE_BYTES + 2 * 128 * sizeof(float) + 1024;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<BN, STAGES>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess)
            return (int)e;
        configured = true;
    }
    const int tiles = tiles_m * tiles_n;
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess)
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    int ctas = tiles < sms ? tiles : sms;
    GemmParams q = p;
    // A last round that would leave most SMs idle is shared out by K blocks instead.  Measured at
    // 2,048 rows: a round that fills a quarter of the SMs or less gains (5120 x 17408: 333 -> 274 us;
    // 7168 x 5120: 120 -> 116), a fuller one does not (under the power cap the busy SMs of a partly
    // filled round run faster, and adding up the partial sums costs 15 to 20 us: 4096 x 4096 with
    // 108 tiles left, 56 -> 63 us).
    const int rest = tiles % sms, kb = p.k_blocks_total;
    if (share_last_round && stream_k.scratch && stream_k.counters && rest > 0
        && rest * stream_k.fill_divisor <= sms && kb >= 16
        && rest * 4 <= STREAM_K_COUNTERS) {
        // CTAs to a tile: what the idle SMs allow, at most eight (the first CTA adds the others' sums
        // one after the other); head and helpers' runs of about the same length
        const double share = (double)sms / rest < 8.0 ? (double)sms / rest : 8.0;
        int head = (int)((kb + share - 1e-9) / share);
        if (head < 1)
            head = 1;
        const int tail = kb - head;
        int helpers = sms - rest < rest * 7 ? sms - rest : rest * 7;
        if (tail > 0 && helpers > 0) {
            const int per = (rest * tail + helpers - 1) / helpers;
            helpers = (rest * tail + per - 1) / per;
            const int slots_per = (per + tail - 1) / tail + 1;
            if ((long long)helpers * slots_per * TILE_A * BN <= stream_k.floats) {
                ctas = sms;
                q.sk_tiles = rest;
                q.sk_head = head;
                q.sk_helpers = helpers;
                q.sk_per = per;
                q.sk_slots_per_helper = slots_per;
                q.sk_scratch = stream_k.scratch;
                q.sk_counters = stream_k.counters;
            }
        }
    }
    launch(gemm_tcgen05_persistent_kernel<BN, STAGES>, dim3(ctas), dim3(GEMM_THREADS), smem, stream, ma, mb, q,
           tiles_m, tiles);
    return launch_status();
}

// Pairs of CTAs on tiles of 256 rows x BN columns (gemm_tcgen05_pair_kernel); tiles_m counts blocks of 256 rows.
template <int BN, int STAGES>
static int launch_gemm_pairs(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int tiles_m,
                             int tiles_n, cudaStream_t stream)
{
    constexpr size_t smem = STAGES * PairSmem<BN>::STAGE_BYTES + (2 * STAGES + 4) * 8 + 16 + 4 * EPILOGUE_STAGE_BYTES
        + 2 * 128 * sizeof(float) + 1024;
    static_assert(smem <= 227 * 1024, "the stages must fit the shared memory of an SM");
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<BN, STAGES>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess)
            return (int)e;
        configured = true;
    }
    const int tiles = tiles_m * tiles_n;
    // as many pairs as are resident at once (74 on 148 SMs: every TPC one), asked of the driver once
    static int resident_pairs = 0;
    if (resident_pairs == 0) {
        int device = 0, sms = 148, clusters = 0;
        if (cudaGetDevice(&device) == cudaSuccess)
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (sms / 2));
        cfg.blockDim = dim3(GEMM_THREADS);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tcgen05_pair_kernel<BN, STAGES>, &cfg) != cudaSuccess
            || clusters < 1) {
            cudaGetLastError();
            clusters = sms / 2;
        }
        resident_pairs = clusters < sms / 2 ? clusters : sms / 2;
    }
    const int pairs = tiles < resident_pairs ? tiles : resident_pairs;
    launch_cluster_x(gemm_tcgen05_pair_kernel<BN, STAGES>, dim3(2 * pairs), dim3(GEMM_THREADS), smem, stream, 2, ma,
                     mb, p, tiles_m, tiles);
    return launch_status();
}

// x [M, K], w [N, K] -> the tensor maps of the pair kernel and its launch.
static int launch_pairs(const void* x, const void* w, const GemmParams& p, int M, int N, int K, long long x_stride,
                        long long w_stride, int bn, cudaStream_t stream)
{
    CUtensorMap ma, mb;
    if (!tensor_map_2d(x, M, K, x_stride, TILE_A, &ma) || !tensor_map_2d(w, N, K, w_stride, bn / 2, &mb))
        return CHIBI_ERR_UNSUPPORTED;
    const int tiles_m = (M + 2 * TILE_A - 1) / (2 * TILE_A);
    if (bn == 128)
        return launch_gemm_pairs<128, 8>(ma, mb, p, tiles_m, N / 128, stream);
    return launch_gemm_pairs<256, 6>(ma, mb, p, tiles_m, N / 256, stream);
}

} // namespace chibi

using namespace chibi;


// How many K splits chibi_gemm_bf16 would use (0: it does not take the shape),
// so that a caller can size the scratch array: splits * M * N floats.
static int sm_count()
{
    static int count = 0;
    if (count == 0) {
        int device = 0, n = 0;
        if (cudaGetDevice(&device) == cudaSuccess
            && cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && n > 0)
            count = n;
        else
            return 148;
    }
    return count;
}

// How the kernel for many rows cuts the output.  Tiles of 256 columns by one CTA each (128 rows);
// the same by pairs of CTAs (256 rows a tile: a tenth to a seventh faster where the rounds are
// filled alike, measured at 448 to 8,192 rows of the Qwen3-8B products; from 256 rows on, with
// what their last block of 256 rows leaves empty counted against them); or
// tiles of 128 columns where those fill the rounds of one CTA per SM so much better that it makes
// up for their lower efficiency (about a tenth below single tiles of 256, the rows of x being fetched
// for half as many columns): 512 rows x 4,096 columns are 64 tiles of 256 (64 of 148 SMs busy)
// or 128 of 128; or those by pairs of CTAs (256 rows x 128 columns).  Where single tiles of 256 columns
// leave a last round that is shared out by K blocks (a quarter of the SMs or less), that competes
// with the cost of adding its partial sums up.
static bool pair_tiles = true;
static int pair_force = 0;        // 128 or 256: that tile width in pairs wherever the shape allows
static int pair_min_rows = 256;
struct ManyRowsPlan {
    int bn;        // 0: N is no multiple of 128
    bool pairs;
};
static ManyRowsPlan many_rows_plan(int M, int N, int K)
{
    if (N % 256 != 0)
        return { N % 128 == 0 ? 128 : 0, false };
    if (pair_force && M >= 2 * TILE_A)
        return { pair_force, true };
    const int sms = sm_count();
    const long long t256 = (long long)((M + TILE_A - 1) / TILE_A) * (N / 256);
    const long long rest = t256 % sms;
    // (a lone round of so few tiles is shared out only where K is long: with 64 K blocks, whole
    // tiles of 128 columns are faster: o of Qwen3-8B at 160 / 192 / 256 rows 240 -> 372, 286 -> 445,
    // 375 -> 590 TFLOP/s; down, 192 K blocks, 373 -> 361, 435 -> 425, 564 -> 558)
    const bool shared = rest > 0 && rest * 4 <= sms && (t256 > sms || (K + TILE_K - 1) / TILE_K >= 128);
    auto fill = [](long long tiles, long long slots) {
        return (double)tiles / (double)(((tiles + slots - 1) / slots) * slots);
    };
    // Worth of each way against single tiles of 256 columns in full rounds (time = tiles / SMs / worth).
    // A shared-out last round fills the SMs but adds the partial sums up: about 25 us, which is
    // 62 K blocks of a tile (0.4 us each).  Pairs gain 1.12 (measured 1.07 to 1.15) on their own
    // rounds of 74; pairs on tiles of 128 columns work like single CTAs on 256.  Measured: 4,096 x
    // 6,144 x 4,096 takes 152 us shared out and 137 in pairs (six rounds, the last a fifth full);
    // 2,048 x 5,120 with K = 17,408 258 shared out and 285 in pairs (three rounds, the last a
    // sixth full), with K = 5,120 94 and 88.
    const double k_blocks = (double)((K + TILE_K - 1) / TILE_K);
    const double single = shared ? 1.0 / (1.0 + 62.5 * sms / (k_blocks * (double)t256)) : fill(t256, sms);
    const double narrow = fill(2 * t256, sms) * 0.9;
    double paired = 0.0, paired_narrow = 0.0;
    if (pair_tiles && M >= 2 * TILE_A) {
        const long long row_blocks = (M + 2 * TILE_A - 1) / (2 * TILE_A);
        // rows past the end in a pair's last block of 256 against those in a single CTA's last 128:
        // 384 rows are three full blocks of 128 or two of 256 a quarter empty (gate|up 73.8 us by
        // single CTAs, 80.0 by pairs), 448 rows fill both alike (92.2 and 79.9)
        const double rows_used = (double)(((M + TILE_A - 1) / TILE_A) * TILE_A) / (double)(row_blocks * 2 * TILE_A);
        if (M >= pair_min_rows)
            paired = fill(row_blocks * (N / 256), sms / 2) * 1.12 * rows_used;
        paired_narrow = fill(row_blocks * (N / 128), sms / 2) * rows_used;
    }
    if (paired >= single && paired >= narrow && paired >= paired_narrow)
        return { 256, true };
    if (paired_narrow > single && paired_narrow > narrow)
        return { 128, true };
    return { narrow > single ? 128 : 256, false };
}

static int many_rows_tile_width(int M, int N, int K) { return many_rows_plan(M, N, K).bn; }

static bool many_rows_in_pairs(int M, int N, int K) { return many_rows_plan(M, N, K).pairs; }

// The cut of a product of many rows: the tile's columns (0: not taken), + 1 if pairs of CTAs compute it.
CHIBI_API int chibi_gemm_many_rows_plan(int M, int N, int K)
{
    const ManyRowsPlan plan = many_rows_plan(M, N, K);
    return plan.bn + (plan.pairs ? 1 : 0);
}

// How the product of many rows uses pairs of CTAs: 0 never, 1 where the plan above prefers them
// (the default; tiles of 256 x 256 from `min_rows` rows on, 256 unless given), 2 / 3 tiles of
// 256 x 256 / 256 x 128 wherever the columns come in whole tiles and there are 256 rows or more
// (for tests and measurements).
CHIBI_API int chibi_gemm_set_pair_tiles(int enabled, int min_rows)
{
    pair_tiles = enabled != 0;
    pair_force = enabled == 2 ? 256 : (enabled == 3 ? 128 : 0);
    if (min_rows > 0)
        pair_min_rows = min_rows;
    return CHIBI_OK;
}

// 33 to 64 rows and so few tiles that two or more splits fit the SMs once: one CTA per SM with
// eight stages in flight instead of three CTAs with three.  Measured at 64 rows (q|k|v 6144 x 4096,
// o 4096 x 4096, down 4096 x 12288): 12.7, 10.0 and 20.8 us against 14.2, 12.4 and 21.6, and the
// partial sums that the next kernel has to add shrink from 4, 4 and 13 splits to 3, 4 and 4.
static bool few_deep_ctas(int M, int N)
{
    if (M > 64)
        return true;       // tiles of 128 or 256 tokens: one CTA per SM is all that fits
    return M > 32 && ((N + TILE_A - 1) / TILE_A) * 2 <= sm_count();
}

// Up to so many rows the weights may be the operand on the 128-row side with the rows as the
// columns of the instruction (16 to 128 of them): every weight is fetched once by N / 128 x splits
// CTAs that do little but stream it.  A CTA also fetches its K range of all the rows, though: with
// 128 rows that is as many bytes again as its weights, with 256 rows twice as many, and what an
// SM can take in bounds the product (measured: 256-row tiles lose to the kernel for many rows).
// (Before, this ended at 64 rows, and a decode step of 65 sequences took 22 % longer than one of 64.)
constexpr int FEW_ROWS_MAX = 128;
CHIBI_API int chibi_gemm_few_rows_max() { return FEW_ROWS_MAX; }

// 65 to FEW_ROWS_MAX rows: the weights stay the streamed operand only where the K range is split
// at least in two (N / 128 tiles fill half the SMs or less: q|k|v, o, down of the usual shapes);
// a wide product (gate | up) has CTAs enough without and is faster in the kernel for many rows.
static bool few_rows_kernel(int M, int N)
{
    return M <= 64 || (M <= FEW_ROWS_MAX && ((N + TILE_A - 1) / TILE_A) * 2 <= sm_count());
}

// For few rows (M <= FEW_ROWS_MAX) the K range is split so that the CTAs of one launch
// fill the SMs once, evenly: with three stages four CTAs of the 16-token variant
// (three of the wider ones) fit an SM.  The partial sums are written and read
// once, 8 bytes per value against 2 N K bytes of weights: they may reach 0.3 of
// the weights' bytes (they mostly stay in L2; measured at 64 rows, 0.15 left a
// product of 64 CTAs that could not keep the memory busy: 105 against 97 us per
// layer), and a split has at least two K blocks.
// `max_splits` > 0: no more splits than that (a consumer that has only so many loads in flight).
CHIBI_API int chibi_gemm_bf16_splits_capped(int M, int N, int K, int max_splits)
{
    if (M <= 0 || N <= 0 || K <= 0 || K % 8 != 0)
        return 0;
    if (!few_rows_kernel(M, N))
        return 1;
    const int tiles = (N + TILE_A - 1) / TILE_A;
    const int k_blocks = (K + TILE_K - 1) / TILE_K;
    if (few_deep_ctas(M, N)) {
        // one CTA per SM with eight stages: as many splits as fill the SMs once
        int splits = sm_count() / tiles;
        if (splits > k_blocks / 2)
            splits = k_blocks / 2;
        if (splits < 1)
            splits = 1;
        const int per = (k_blocks + splits - 1) / splits;
        return (k_blocks + per - 1) / per;
    }
    const int resident = sm_count() * (M <= 16 ? 4 : 3);
    int splits = tiles >= resident ? 1 : resident / tiles;
    const int traffic_cap = (int)(0.3 * K / (4.0 * M));
    if (splits > traffic_cap)
        splits = traffic_cap;
    if (splits > k_blocks / 2)
        splits = k_blocks / 2;
    // Whoever adds the partial sums up has the loads of sixteen splits in flight at once; a
    // seventeenth costs a second trip to L2 on the critical path of a decode step (measured:
    // 18 -> 16 splits of the down product of Qwen3-8B, 1.5 us a layer).  And a CTA should have
    // at least five K blocks to stream, or its three stages are most of its work.
    if (splits > 16)
        splits = 16;
    if (k_blocks >= 20 && splits > k_blocks / 5)
        splits = k_blocks / 5;
    if (max_splits > 0 && splits > max_splits)
        splits = max_splits;
    if (splits < 1)
        splits = 1;
    const int per = (k_blocks + splits - 1) / splits;
    return (k_blocks + per - 1) / per;
}

CHIBI_API int chibi_gemm_bf16_splits(int M, int N, int K) { return chibi_gemm_bf16_splits_capped(M, N, K, 0); }

// Returns CHIBI_ERR_UNSUPPORTED for shapes or alignments it does not take; the
// caller then uses the plain kernel.
static int gemm_bf16_impl(const void* x, const void* w, void* out, int out_type,
                         const float* residual, int M, int N, int K, long long x_stride,
                         long long w_stride, long long out_stride, long long res_stride,
                         float* scratch, long long scratch_floats, int* error, cudaStream_t stream,
                         bool reduce, bool share_last_round = true, int max_splits = 0)
{
    if (M <= 0 || N <= 0)
        return CHIBI_OK;
    if (K <= 0 || K % 8 != 0 || x_stride % 8 != 0 || w_stride % 8 != 0
        || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
        return CHIBI_ERR_UNSUPPORTED;
    if (out_type != CHIBI_F32 && out_type != CHIBI_BF16)
        return CHIBI_ERR_ARGUMENT;
    if (out_type == CHIBI_F32 && (reinterpret_cast<uintptr_t>(out) & 15))
        return CHIBI_ERR_UNSUPPORTED;
    if (out_type == CHIBI_BF16 && (reinterpret_cast<uintptr_t>(out) & 15))
        return CHIBI_ERR_UNSUPPORTED;
    if (residual && (reinterpret_cast<uintptr_t>(residual) & 15))
        return CHIBI_ERR_UNSUPPORTED;

    GemmParams p {};
    p.K = K;
    p.M = M;
    p.N = N;
    p.out = out;
    p.out_type = out_type;
    p.out_stride = out_stride;
    p.residual = residual;
    p.res_stride = res_stride;
    p.error = error;
    p.k_blocks_total = (K + TILE_K - 1) / TILE_K;
    const int splits = chibi_gemm_bf16_splits_capped(M, N, K, max_splits);
    if (splits <= 0)
        return CHIBI_ERR_UNSUPPORTED;
    p.k_blocks_per_split = (p.k_blocks_total + splits - 1) / splits;
    if (splits > 1) {
        if (!scratch || scratch_floats < (long long)splits * M * N)
            return CHIBI_ERR_ARGUMENT;
        p.partial = scratch;
    }
    CUtensorMap ma, mb;
    int status;
    if (few_rows_kernel(M, N)) {
        const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
        p.swap = 1;
        p.rows_a = N;
        p.rows_b = M;
        if (!tensor_map_2d(w, N, K, w_stride, TILE_A, &ma) || !tensor_map_2d(x, M, K, x_stride, bn, &mb))
            return CHIBI_ERR_UNSUPPORTED;
        const dim3 grid((N + TILE_A - 1) / TILE_A, 1, splits);
        if (bn == 16)
            status = launch_gemm<16, 3>(ma, mb, p, grid, stream);
        else if (bn == 32)
            status = launch_gemm<32, 3>(ma, mb, p, grid, stream);
        else if (bn == 128)
            status = launch_gemm<128, 6>(ma, mb, p, grid, stream);      // 6 x 32 KB, one CTA per SM
        else if (few_deep_ctas(M, N))
            status = launch_gemm<64, 8>(ma, mb, p, grid, stream);
        else
            status = launch_gemm<64, 3>(ma, mb, p, grid, stream);
    } else {
        p.swap = 0;
        p.rows_a = M;
        p.rows_b = N;
        const int chosen = many_rows_tile_width(M, N, K);    // 0: N is no multiple of 128
        const int bn = chosen ? chosen : (N >= 256 ? 256 : (N > 64 ? 128 : 64));
        if (!tensor_map_2d(x, M, K, x_stride, TILE_A, &ma) || !tensor_map_2d(w, N, K, w_stride, bn, &mb))
            return CHIBI_ERR_UNSUPPORTED;
        const dim3 grid((M + TILE_A - 1) / TILE_A, (N + bn - 1) / bn, 1);
        if (grid.y > 65535)
            return CHIBI_ERR_UNSUPPORTED;
        if (many_rows_in_pairs(M, N, K)) {
            status = launch_pairs(x, w, p, M, N, K, x_stride, w_stride, bn, stream);
        } else if (bn == 256)
            status = launch_gemm_persistent<256, 4>(ma, mb, p, grid.x, grid.y, stream, share_last_round);
        else if (bn == 128 && chosen == 128)
            status = launch_gemm_persistent<128, 6>(ma, mb, p, grid.x, grid.y, stream, false);
        else if (bn == 128)
            status = launch_gemm<128, 4>(ma, mb, p, grid, stream);
        else
            status = launch_gemm<64, 4>(ma, mb, p, grid, stream);
    }
    if (status != CHIBI_OK)
        return status;
    if (splits > 1 && reduce) {
        const long long total = (long long)M * N;
        int blocks = (int)((total + 255) / 256);
        if (blocks > 148 * 8)
            blocks = 148 * 8;
        launch(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream, scratch, splits, out, out_type, out_stride,
                                                         residual, res_stride, M, N);
        return launch_status();
    }
    return CHIBI_OK;
}

CHIBI_API int chibi_gemm_bf16(const void* x, const void* w, void* out, int out_type,
                              const float* residual, int M, int N, int K, long long x_stride,
                              long long w_stride, long long out_stride, long long res_stride,
                              float* scratch, long long scratch_floats, int* error,
                              cudaStream_t stream)
{
    return gemm_bf16_impl(x, w, out, out_type, residual, M, N, K, x_stride, w_stride, out_stride,
                          res_stride, scratch, scratch_floats, error, stream, true);
}

// Scratch for the many-row kernel's shared-out last round: up to 2 * multiProcessorCount slots of
// 128 * 256 floats, 16-byte aligned, used by one stream at a time.  Without it (null) every tile is computed whole.
CHIBI_API int chibi_gemm_set_stream_scratch(float* scratch, long long floats)
{
    if (scratch && (reinterpret_cast<uintptr_t>(scratch) & 15))
        return CHIBI_ERR_ARGUMENT;
    if (scratch && !stream_k.counters) {
        // looked up here, once, and not at a launch (which may be part of a stream capture)
        void* counters = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&counters, stream_k_counters);
        if (e != cudaSuccess)
            return (int)e;
        stream_k.counters = static_cast<int*>(counters);
    }
    stream_k.scratch = scratch;
    stream_k.floats = scratch ? floats : 0;
    return CHIBI_OK;
}

// After a wait of the shared-out last round ran out (error word 15 or 16) its counters may be left
// non-zero, and the next launch that shares out the same tiles would add sums that are not written
// yet.  This puts them back to zero, in stream order.
CHIBI_API int chibi_gemm_reset_stream_counters(cudaStream_t stream)
{
    if (!stream_k.counters)
        return CHIBI_OK;
    return (int)cudaMemsetAsync(stream_k.counters, 0, sizeof(int) * STREAM_K_COUNTERS, stream);
}

// out = x * w^T of more than 64 rows with what follows it done in the same kernel: + residual, or
// (epilogue 1) SwiGLU over w's rows arranged as blocks of 64 gate rows followed by their 64 up
// rows (out is then [M, N / 2], bfloat16).  Few rows split their K range instead
// (chibi_gemm_bf16_partial and the kernels that finish a split product).
CHIBI_API int chibi_gemm_bf16_fused(const void* x, const void* w, void* out, int out_type,
                                    const float* residual, int M, int N, int K, long long x_stride,
                                    long long w_stride, long long out_stride, long long res_stride,
                                    int epilogue, int* error, cudaStream_t stream)
{
    if (M <= 0 || N <= 0)
        return CHIBI_OK;
    if (K <= 0 || K % 8 != 0 || x_stride % 8 != 0 || w_stride % 8 != 0
        || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)
        || (reinterpret_cast<uintptr_t>(out) & 15) || (residual && (reinterpret_cast<uintptr_t>(residual) & 15)))
        return CHIBI_ERR_UNSUPPORTED;
    if (out_type != CHIBI_F32 && out_type != CHIBI_BF16)
        return CHIBI_ERR_ARGUMENT;
    if (epilogue == 1 && (N % 128 != 0 || out_type != CHIBI_BF16 || residual))
        return CHIBI_ERR_UNSUPPORTED;
    GemmParams p {};
    p.K = K;
    p.M = M;
    p.N = N;
    p.out = out;
    p.out_type = out_type;
    p.out_stride = out_stride;
    p.residual = residual;
    p.res_stride = res_stride;
    p.error = error;
    p.swiglu = epilogue == 1 ? 1 : 0;
    p.k_blocks_total = (K + TILE_K - 1) / TILE_K;
    CUtensorMap ma, mb;
    if (M <= 64)
        return CHIBI_ERR_UNSUPPORTED;
    p.k_blocks_per_split = p.k_blocks_total;
    p.swap = 0;
    p.rows_a = M;
    p.rows_b = N;
    const int chosen = many_rows_tile_width(M, N, K);
    const int bn = chosen ? chosen : (N >= 256 ? 256 : (N > 64 || p.swiglu ? 128 : 64));
    if (!tensor_map_2d(x, M, K, x_stride, TILE_A, &ma) || !tensor_map_2d(w, N, K, w_stride, bn, &mb))
        return CHIBI_ERR_UNSUPPORTED;
    const dim3 grid((M + TILE_A - 1) / TILE_A, (N + bn - 1) / bn, 1);
    if (grid.y > 65535)
        return CHIBI_ERR_UNSUPPORTED;
    if (many_rows_in_pairs(M, N, K))
        return launch_pairs(x, w, p, M, N, K, x_stride, w_stride, bn, stream);
    if (bn == 256)
        return launch_gemm_persistent<256, 4>(ma, mb, p, grid.x, grid.y, stream);
    if (bn == 128 && chosen == 128)
        return launch_gemm_persistent<128, 6>(ma, mb, p, grid.x, grid.y, stream, false);
    if (bn == 128)
        return launch_gemm<128, 4>(ma, mb, p, grid, stream);
    return launch_gemm<64, 4>(ma, mb, p, grid, stream);
}

// Many rows with an RMSNorm folded into the products around it (see GemmParams).  `scale`
// (may be null) describes the factor that x lacks; `norm` (may be null) asks for the norm output of
// the completed residual.  epilogue 1: SwiGLU as in chibi_gemm_bf16_fused.  Only the kernel for more
// than FEW_ROWS_MAX rows with whole tiles of 128 or 256 columns does this: CHIBI_ERR_UNSUPPORTED
// otherwise, and the caller applies the norm or the factor with kernels of their own.
struct ChibiRowScale {
    const float* ssq;      // [M][parts] sums of squares
    int parts;
    float eps;
    int n;                 // width of the normalised rows
};
struct ChibiNormOut {
    const void* w;         // [N] norm weight
    int w_type;
    float offset;
    void* out;             // [M][N] bfloat16: (residual + x W^T) * (w + offset), without the row's factor
    long long out_stride;
    float* ssq;            // [M][parts], parts = chibi_gemm_bf16_norm_parts(N)
    long long ssq_floats;
};

// Sums of squares per row that a product of M rows with a norm output writes: one for each of its
// column tiles (0: the kernel does not take the width).
CHIBI_API int chibi_gemm_bf16_norm_parts(int M, int N, int K)
{
    const int bn = M > FEW_ROWS_MAX && N > 0 ? many_rows_tile_width(M, N, K) : 0;
    return bn ? N / bn : 0;
}

// `heads` (may be null; then `out` is not written and may be null): the product is q | k | v of
// head size 128 (N = (nq + 2 nkv) * 128, or nq * 128 without caches) and every head is finished in
// the epilogue: per-head RMSNorm for query and key heads (weights may be null), rotation of the whole
// head with the token's cosines and sines, query heads to q_out, key and value heads to the token's
// cache slot.
struct ChibiHeadsOut {
    const float* cos_sin;      // [M][128] from chibi_rope_table
    const long long* slots;    // [M] from chibi_cache_slots; null without caches
    void* q_out;               // [M][nq * 128] bfloat16
    void* k_cache;             // [pages][nkv][page_size][128] bfloat16, or null
    void* v_cache;
    const void* q_norm_w;      // [128] or null
    const void* k_norm_w;
    int w_type, nq, nkv, page_size;
    float eps, offset;
};

CHIBI_API int chibi_gemm_bf16_rows(const void* x, const void* w, void* out, int out_type, const float* residual,
                                   int M, int N, int K, long long x_stride, long long w_stride, long long out_stride,
                                   long long res_stride, int epilogue, const ChibiRowScale* scale,
                                   const ChibiNormOut* norm, const ChibiHeadsOut* heads, int* error,
                                   cudaStream_t stream)
{
    if (M <= FEW_ROWS_MAX || N <= 0 || N % 128 != 0 || K <= 0 || K % 8 != 0 || x_stride % 8 != 0 || w_stride % 8 != 0
        || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)
        || (reinterpret_cast<uintptr_t>(out) & 15) || (residual && (reinterpret_cast<uintptr_t>(residual) & 15)))
        return CHIBI_ERR_UNSUPPORTED;
    const int bn = many_rows_tile_width(M, N, K);
    if (heads) {
        const bool caches = heads->k_cache != nullptr;
        if (epilogue != 0 || norm || residual)
            return CHIBI_ERR_ARGUMENT;
        if (!heads->cos_sin || !heads->q_out || heads->nq < 1 || heads->nkv < 0 || (caches && (!heads->v_cache || !heads->slots || heads->nkv < 1 || heads->page_size < 1))
            || ((heads->q_norm_w || heads->k_norm_w) && heads->w_type != CHIBI_F32 && heads->w_type != CHIBI_BF16))
            return CHIBI_ERR_ARGUMENT;
        if ((long long)N != (long long)(heads->nq + (caches ? 2 * heads->nkv : 0)) * 128
            || (reinterpret_cast<uintptr_t>(heads->q_out) & 15) || (reinterpret_cast<uintptr_t>(heads->cos_sin) & 15)
            || (caches && ((reinterpret_cast<uintptr_t>(heads->k_cache) & 15) || (reinterpret_cast<uintptr_t>(heads->v_cache) & 15))))
            return CHIBI_ERR_UNSUPPORTED;
    }
    GemmParams p {};
    p.K = K;
    p.M = M;
    p.N = N;
    p.out = out;
    p.out_type = out_type;
    p.out_stride = out_stride;
    p.residual = residual;
    p.res_stride = res_stride;
    p.error = error;
    p.swiglu = epilogue == 1 ? 1 : 0;
    p.k_blocks_total = (K + TILE_K - 1) / TILE_K;
    p.k_blocks_per_split = p.k_blocks_total;
    p.swap = 0;
    p.rows_a = M;
    p.rows_b = N;
    if (p.swiglu) {
        if (out_type != CHIBI_BF16 || residual || out_stride % 8 != 0 || norm)
            return CHIBI_ERR_UNSUPPORTED;
    } else if (norm) {
        // the path that adds the residual in 32-bit, whole tiles only
        if (out_type != CHIBI_F32 || !residual || out_stride % 4 != 0 || res_stride % 4 != 0 || scale)
            return CHIBI_ERR_UNSUPPORTED;
    } else if (heads) {
        p.h_cos_sin = heads->cos_sin;
        p.h_slots = heads->k_cache ? heads->slots : nullptr;
        p.h_q_out = static_cast<__nv_bfloat16*>(heads->q_out);
        p.h_k_cache = static_cast<__nv_bfloat16*>(heads->k_cache);
        p.h_v_cache = static_cast<__nv_bfloat16*>(heads->v_cache);
        p.h_q_norm_w = heads->q_norm_w;
        p.h_k_norm_w = heads->k_norm_w;
        p.h_w_type = heads->w_type;
        p.h_nq = heads->nq;
        p.h_nkv = heads->k_cache ? heads->nkv : 0;
        p.h_page_size = heads->page_size;
        p.h_eps = heads->eps;
        p.h_offset = heads->offset;
    } else if (out_type != CHIBI_BF16 || residual || out_stride % 8 != 0) {
        return CHIBI_ERR_UNSUPPORTED;      // a factor is applied where the sums become bfloat16
    }
    if (scale) {
        if (!scale->ssq || scale->parts < 1 || scale->n < 1)
            return CHIBI_ERR_ARGUMENT;
        p.row_ssq = scale->ssq;
        p.row_ssq_parts = scale->parts;
        p.row_eps = scale->eps;
        p.row_n = scale->n;
    }
    if (norm) {
        const int parts = N / bn;
        if (!norm->w || !norm->out || !norm->ssq || norm->ssq_floats < (long long)M * parts
            || (norm->w_type != CHIBI_F32 && norm->w_type != CHIBI_BF16) || norm->out_stride % 4 != 0
            || (reinterpret_cast<uintptr_t>(norm->out) & 7))
            return CHIBI_ERR_ARGUMENT;
        p.norm_w = norm->w;
        p.norm_w_type = norm->w_type;
        p.norm_offset = norm->offset;
        p.normed_out = static_cast<__nv_bfloat16*>(norm->out);
        p.normed_stride = norm->out_stride;
        p.ssq_out = norm->ssq;
        p.ssq_out_parts = parts;
    }
    CUtensorMap ma, mb;
    if (many_rows_in_pairs(M, N, K))
        return launch_pairs(x, w, p, M, N, K, x_stride, w_stride, bn, stream);
    if (!tensor_map_2d(x, M, K, x_stride, TILE_A, &ma) || !tensor_map_2d(w, N, K, w_stride, bn, &mb))
        return CHIBI_ERR_UNSUPPORTED;
    if (bn == 128)
        return launch_gemm_persistent<128, 6>(ma, mb, p, (M + TILE_A - 1) / TILE_A, N / 128, stream, false);
    return launch_gemm_persistent<256, 4>(ma, mb, p, (M + TILE_A - 1) / TILE_A, N / 256, stream);
}

// The first half only, for shapes that chibi_gemm_bf16_splits_capped splits (> 1): the
// partial sums [splits][M][N] stay in `scratch` for a kernel that adds them up
// together with what follows the product (chibi_reduce_* below and elsewhere).
// `max_splits` > 0: at most so many splits (what the adding kernel fetches in one go).
CHIBI_API int chibi_gemm_bf16_partial(const void* x, const void* w, int M, int N, int K,
                                      long long x_stride, long long w_stride, float* scratch,
                                      long long scratch_floats, int max_splits, int* error, cudaStream_t stream)
{
    if (chibi_gemm_bf16_splits_capped(M, N, K, max_splits) <= 1 || (reinterpret_cast<uintptr_t>(scratch) & 15))
        return CHIBI_ERR_UNSUPPORTED;
    return gemm_bf16_impl(x, w, scratch, CHIBI_F32, nullptr, M, N, K, x_stride, w_stride, N, 0, scratch,
                          scratch_floats, error, stream, false, true, max_splits);
}

// ------------------------------------------------------------------ kernels that finish a split product
namespace chibi {

// residual[m, :] += sum over splits (in split order); then, if a norm weight is
// given, normed[m, :] = RMSNorm(residual[m, :]).  One block per row; the row
// stays in registers (N <= 16 * blockDim.x, N a multiple of 4).
template <typename TW, typename TO>
__global__ void __launch_bounds__(512)
reduce_residual_rmsnorm_kernel(const float* __restrict__ partial, int splits, int M, int N,
                               float* residual, long long res_stride, const TW* __restrict__ w,
                               TO* __restrict__ normed, long long normed_stride, float eps, float offset)
{
    pdl_enter();
    __shared__ float scratch[33];
    const int m = blockIdx.x;
    const int n4 = N >> 2;
    const size_t total4 = ((size_t)M * N) >> 2;
    float4* res = reinterpret_cast<float4*>(residual + (size_t)m * res_stride);
    const float4* part = reinterpret_cast<const float4*>(partial) + (size_t)m * n4;
    float4 v[4];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int j = threadIdx.x + i * blockDim.x;
        if (j < n4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int sp = 0; sp < splits; ++sp) {
                const float4 q = part[(size_t)sp * total4 + j];
                acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
            }
            const float4 r = res[j];
            acc.x = r.x + acc.x; acc.y = r.y + acc.y; acc.z = r.z + acc.z; acc.w = r.w + acc.w;
            res[j] = acc;
            v[i] = acc;
            s = fmaf(acc.x, acc.x, s);
            s = fmaf(acc.y, acc.y, s);
            s = fmaf(acc.z, acc.z, s);
            s = fmaf(acc.w, acc.w, s);
        } else {
            v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if (!w)
        return;
    s = block_sum(s, scratch);
    const float inv = rsqrtf(s / (float)N + eps);
    TO* dst = normed + (size_t)m * normed_stride;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int j = threadIdx.x + i * blockDim.x;
        if (j < n4) {
            const float o0 = (v[i].x * inv) * (to_f32(w[4 * j]) + offset);
            const float o1 = (v[i].y * inv) * (to_f32(w[4 * j + 1]) + offset);
            const float o2 = (v[i].z * inv) * (to_f32(w[4 * j + 2]) + offset);
            const float o3 = (v[i].w * inv) * (to_f32(w[4 * j + 3]) + offset);
            dst[4 * j] = from_f32<TO>(o0);
            dst[4 * j + 1] = from_f32<TO>(o1);
            dst[4 * j + 2] = from_f32<TO>(o2);
            dst[4 * j + 3] = from_f32<TO>(o3);
        }
    }
}

// The same with a cluster of CTAs per row, each taking a run of columns (one
// float4 per thread, all of a thread's loads in flight together); the CTAs push
// their sums of squares into one another's shared memory and meet at one
// cluster barrier.
template <typename TW, typename TO>
__global__ void __launch_bounds__(1024)
reduce_residual_rmsnorm_cluster_kernel(const float* __restrict__ partial, int splits, int M, int N,
                                       float* residual, long long res_stride, const TW* __restrict__ w,
                                       TO* __restrict__ normed, long long normed_stride, float eps,
                                       float offset)
{
    pdl_trigger();
    __shared__ float scratch[33];
    __shared__ float sums[8];                        // sums[r]: the sum of squares of CTA r's columns
    const int m = blockIdx.y;
    const int parts = gridDim.x;                     // CTAs per row = cluster size (<= 8)
    const int n4 = N >> 2;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;   // float4 index within the row
    const size_t total4 = ((size_t)M * N) >> 2;
    if (j < n4) {
        // while the product before this kernel still runs
        const float4* part = reinterpret_cast<const float4*>(partial) + (size_t)m * n4 + j;
        prefetch_l2(part);
        prefetch_l2(part + (size_t)(splits - 1) * total4);
        prefetch_l2(residual + (size_t)m * res_stride + 4 * j);
        if (w) {
            prefetch_l2(w + 4 * j);
            prefetch_l2(normed + (size_t)m * normed_stride + 4 * j);
        }
    }
    pdl_wait();
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float wv[4] = { 0.f, 0.f, 0.f, 0.f };
    float s = 0.f;
    if (j < n4) {
        // everything this thread reads is on its way at once: its column of up to 16 splits, the
        // residual and the norm weights
        const float4* part = reinterpret_cast<const float4*>(partial) + (size_t)m * n4 + j;
        float4* res = reinterpret_cast<float4*>(residual + (size_t)m * res_stride) + j;
        const float4 r = *res;
        if (w) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
                wv[u] = to_f32(w[4 * j + u]) + offset;
        }
        for (int sp0 = 0; sp0 < splits; sp0 += 16) {
            float4 q[16];
#pragma unroll
            for (int u = 0; u < 16; ++u)
                q[u] = sp0 + u < splits ? part[(size_t)(sp0 + u) * total4] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                acc.x += q[u].x; acc.y += q[u].y; acc.z += q[u].z; acc.w += q[u].w;
            }
        }
        acc.x = r.x + acc.x; acc.y = r.y + acc.y; acc.z = r.z + acc.z; acc.w = r.w + acc.w;
        *res = acc;
        s = acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    }
    timeline_mark(0);                  // the sums are added up
    if (!w)
        return;
    s = block_sum(s, scratch);
    // every CTA puts its sum into slot `rank` of every CTA of the cluster; after one cluster
    // barrier each CTA adds the slots of its own copy, in rank order
    if ((int)threadIdx.x < parts)
        st_peer_shared_f32(smem_addr(&sums[cluster_cta_rank()]), threadIdx.x, s);
    cluster_sync();
    timeline_mark(1);                  // the row's sum of squares is known
    float total = 0.f;
    for (int r = 0; r < parts; ++r)
        total += sums[r];
    const float inv = rsqrtf(total / (float)N + eps);
    if (j < n4) {
        TO* dst = normed + (size_t)m * normed_stride + 4 * j;
        dst[0] = from_f32<TO>((acc.x * inv) * wv[0]);
        dst[1] = from_f32<TO>((acc.y * inv) * wv[1]);
        dst[2] = from_f32<TO>((acc.z * inv) * wv[2]);
        dst[3] = from_f32<TO>((acc.w * inv) * wv[3]);
    }
}

// act[m, c] = silu(gate) * up with gate = sum of partial[s][m][c] and up = sum of
// partial[s][m][I + c], in split order.  Two columns per thread.
template <typename TO>
__global__ void reduce_swiglu_kernel(const float* __restrict__ partial, int splits, int M, int inter,
                                     TO* __restrict__ out, int interleaved)
{
    pdl_enter();
    const int half = inter >> 1;
    const int c2 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c2 >= half)
        return;
    const int m = blockIdx.y;
    const size_t total = (size_t)M * 2 * inter;
    const float* row = partial + (size_t)m * 2 * inter;
    // columns of gate and up for features 2 c2, 2 c2 + 1: [gate | up], or blocks of 64 gate
    // columns each followed by its 64 up columns
    const int f = 2 * c2;
    const int g_col = interleaved ? ((f >> 6) << 7) + (f & 63) : f;
    const int u_col = interleaved ? g_col + 64 : inter + f;
    float2 g = make_float2(0.f, 0.f), u = make_float2(0.f, 0.f);
    for (int sp0 = 0; sp0 < splits; sp0 += 4) {
        float2 gq[4], uq[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const bool on = sp0 + k < splits;
            gq[k] = on ? *reinterpret_cast<const float2*>(row + (sp0 + k) * total + g_col) : make_float2(0.f, 0.f);
            uq[k] = on ? *reinterpret_cast<const float2*>(row + (sp0 + k) * total + u_col) : make_float2(0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            g.x += gq[k].x; g.y += gq[k].y; u.x += uq[k].x; u.y += uq[k].y;
        }
    }
    out[(size_t)m * inter + 2 * c2] = from_f32<TO>((g.x / (1.f + expf(-g.x))) * u.x);
    out[(size_t)m * inter + 2 * c2 + 1] = from_f32<TO>((g.y / (1.f + expf(-g.y))) * u.y);
}

} // namespace chibi

CHIBI_API int chibi_reduce_residual_rmsnorm(const float* partial, int splits, int M, int N,
                                            float* residual, long long res_stride, const void* w,
                                            int w_type, void* normed, int normed_type,
                                            long long normed_stride, float eps, float offset,
                                            cudaStream_t stream)
{
    if (M <= 0)
        return CHIBI_OK;
    if (N % 4 != 0 || N > 16 * 512 || res_stride % 4 != 0 || splits < 1
        || (reinterpret_cast<uintptr_t>(partial) & 15) || (reinterpret_cast<uintptr_t>(residual) & 15))
        return CHIBI_ERR_UNSUPPORTED;
    // a cluster of CTAs per row when the row divides evenly into runs of 128..1024 columns
    int parts = 0;
    for (int cand = 8; cand >= 2; --cand)
        if ((N / 4) % cand == 0 && N / 4 / cand >= 32 && N / 4 / cand <= 256 && (N / 4 / cand) % 32 == 0) {
            parts = cand;
            break;
        }
    if (parts > 0 && M <= 65535) {
        const dim3 grid(parts, M);
        const int threads = N / 4 / parts;
        if (!w) {
            // no norm, nothing to exchange: the same grid without the cluster
            launch(reduce_residual_rmsnorm_cluster_kernel<float, float>, grid, dim3(threads), 0, stream,
                   partial, splits, M, N, residual, res_stride, (const float*)nullptr, (float*)nullptr,
                   (long long)0, eps, offset);
            return launch_status();
        }
        CHIBI_DISPATCH_TYPE(w_type, TW, CHIBI_DISPATCH_TYPE(normed_type, TO, {
            launch_cluster_x(reduce_residual_rmsnorm_cluster_kernel<TW, TO>, grid, dim3(threads), 0, stream, parts,
                             partial, splits, M, N, residual, res_stride, (const TW*)w, (TO*)normed,
                             normed_stride, eps, offset);
        }));
        return launch_status();
    }
    int block = 32;
    while (block * 16 < N)
        block <<= 1;
    if (block < 128 && N >= 512)
        block = 128;
    if (!w) {
        launch(reduce_residual_rmsnorm_kernel<float, float>, dim3(M), dim3(block), 0, stream, 
            partial, splits, M, N, residual, res_stride, nullptr, nullptr, 0, eps, offset);
        return launch_status();
    }
    CHIBI_DISPATCH_TYPE(w_type, TW, CHIBI_DISPATCH_TYPE(normed_type, TO, {
        launch(reduce_residual_rmsnorm_kernel<TW, TO>, dim3(M), dim3(block), 0, stream, 
            partial, splits, M, N, residual, res_stride, (const TW*)w, (TO*)normed, normed_stride, eps,
            offset);
    }));
    return launch_status();
}

CHIBI_API int chibi_reduce_swiglu(const float* partial, int splits, int M, int inter, void* out,
                                  int out_type, int interleaved, cudaStream_t stream)
{
    if (M <= 0)
        return CHIBI_OK;
    if (inter % 2 != 0 || M > 65535 || splits < 1 || (reinterpret_cast<uintptr_t>(partial) & 7)
        || (interleaved && inter % 64 != 0))
        return CHIBI_ERR_UNSUPPORTED;
    const dim3 grid((inter / 2 + 255) / 256, M);
    CHIBI_DISPATCH_TYPE(out_type, TO, {
        launch(reduce_swiglu_kernel<TO>, dim3(grid), dim3(256), 0, stream, partial, splits, M, inter, (TO*)out,
               interleaved);
    });
    return launch_status();
}

// ------------------------------------------------------------------ no-allocation entry point
#include "no_alloc_api.h"

// Scratch for the split-K partial sums of chibi_gemm_bf16_noalloc.  In host code
// this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_noalloc_scratch[CHIBI_NOALLOC_SCRATCH_FLOATS];

CHIBI_API const char* chibi_error_string(int code)
{
    switch (code) {
    case CHIBI_OK: return "ok";
    case CHIBI_ERR_ARGUMENT: return "invalid argument";
    case CHIBI_ERR_UNSUPPORTED: return "shape or alignment that this kernel does not take";
    case CHIBI_ERR_DEVICE_CHECK: return "a device-side check failed";
    case CHIBI_ERR_SCRATCH_LIMIT:
        return "the product needs more scratch than the library's built-in array holds "
               "(splits * M * N > CHIBI_NOALLOC_SCRATCH_FLOATS)";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown error code";
    }
}

CHIBI_API int chibi_gemm_bf16_noalloc(const void* x, const void* w, void* out, int out_type,
                                      const float* residual, int M, int N, int K,
                                      long long x_stride, long long w_stride, long long out_stride,
                                      long long res_stride, int* error, cudaStream_t stream)
{
    constexpr int MAX_DEVICES = 64;
    static float* device_ptr[MAX_DEVICES] = {};
    static std::mutex mutex;
    const int splits = chibi_gemm_bf16_splits(M, N, K);
    if (M > 0 && N > 0 && splits <= 0)
        return CHIBI_ERR_UNSUPPORTED;
    if (splits > 1 && (long long)splits * M * N > (long long)CHIBI_NOALLOC_SCRATCH_FLOATS)
        return CHIBI_ERR_SCRATCH_LIMIT;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess)
        return (int)e;
    if (device < 0 || device >= MAX_DEVICES)
        return CHIBI_ERR_ARGUMENT;
    float* scratch;
    {
        std::lock_guard<std::mutex> lock(mutex);
        if (!device_ptr[device]) {
            // once per device, with that device current: the array's address on this device
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess)
                return (int)e;
            device_ptr[device] = static_cast<float*>(p);
        }
        scratch = device_ptr[device];
    }
    // every tile of a many-row product is computed whole here: the scratch and the counters that
    // share out a last round of tiles belong to the engine's stream
    return gemm_bf16_impl(x, w, out, out_type, residual, M, N, K, x_stride, w_stride, out_stride,
                          res_stride, scratch, CHIBI_NOALLOC_SCRATCH_FLOATS, error, stream, true, false);
}
