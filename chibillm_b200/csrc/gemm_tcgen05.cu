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

#include "common.cuh"
#include "sm100.cuh"

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
    float* partial;        // [splits][M][N] when the K range is split, else null
    int* error;
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
            for (int i = 0; i < kb_count; ++i) {
                const int s = i % STAGES;
                const uint32_t round = i / STAGES;
                if (round > 0)
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
        if (kb_count > 0)
            ok = mbar_wait(tmem_full_bar, 0, p.error, 13);
        tcgen05_fence_after();
        constexpr int CHUNK = BN < 32 ? 16 : 32;
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

// out = (residual +) sum over splits, in split order.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, void* out,
                                     int out_type, long long out_stride, const float* residual,
                                     long long res_stride, int M, int N)
{
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
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess
            && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

struct MapKey {
    const void* ptr;
    long long rows, cols, stride;
    int box_rows;
    bool operator==(const MapKey& o) const
    {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && stride == o.stride && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const
    {
        size_t h = reinterpret_cast<size_t>(k.ptr);
        h = h * 1000003u ^ (size_t)k.rows;
        h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.stride;
        h = h * 1000003u ^ (size_t)k.box_rows;
        return h;
    }
};

// A map over a row-major bf16 matrix [rows, cols] with `stride` elements between
// rows; boxes of 64 columns x box_rows rows, 128-byte swizzle, zeros outside.
static bool tensor_map_2d(const void* ptr, long long rows, long long cols, long long stride,
                          int box_rows, CUtensorMap* out)
{
    static std::mutex mutex;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key { ptr, rows, cols, stride, box_rows };
    std::lock_guard<std::mutex> lock(mutex);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn fn = encode_tiled();
    if (!fn)
        return false;
    const cuuint64_t dims[2] = { (cuuint64_t)cols, (cuuint64_t)rows };
    const cuuint64_t strides[1] = { (cuuint64_t)stride * 2 };
    const cuuint32_t box[2] = { (cuuint32_t)TILE_K, (cuuint32_t)box_rows };
    const cuuint32_t elem[2] = { 1, 1 };
    CUtensorMap map;
    const CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                          box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return false;
    if (cache.size() > 8192)
        cache.clear();
    cache.emplace(key, map);
    *out = map;
    return true;
}

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
    gemm_tcgen05_kernel<BN, STAGES><<<grid, GEMM_THREADS, smem, stream>>>(ma, mb, p);
    return launch_status();
}

} // namespace chibi

using namespace chibi;

// How many K splits chibi_gemm_bf16 would use (0: it does not take the shape),
// so that a caller can size the scratch array: splits * M * N floats.
CHIBI_API int chibi_gemm_bf16_splits(int M, int N, int K)
{
    if (M <= 0 || N <= 0 || K <= 0 || K % 8 != 0)
        return 0;
    if (M > 64)
        return 1;
    const int tiles = (N + TILE_A - 1) / TILE_A;
    const int k_blocks = (K + TILE_K - 1) / TILE_K;
    int splits = (2 * 148 + tiles - 1) / tiles;
    const int most = k_blocks / 4 > 0 ? k_blocks / 4 : 1;
    if (splits > most)
        splits = most;
    if (splits > 16)
        splits = 16;
    if (splits < 1)
        splits = 1;
    const int per = (k_blocks + splits - 1) / splits;
    return (k_blocks + per - 1) / per;
}

// Returns CHIBI_ERR_UNSUPPORTED for shapes or alignments it does not take; the
// caller then uses the plain kernel.
CHIBI_API int chibi_gemm_bf16(const void* x, const void* w, void* out, int out_type,
                              const float* residual, int M, int N, int K, long long x_stride,
                              long long w_stride, long long out_stride, long long res_stride,
                              float* scratch, long long scratch_floats, int* error,
                              cudaStream_t stream)
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
    const int splits = chibi_gemm_bf16_splits(M, N, K);
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
    if (M <= 64) {
        const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
        p.swap = 1;
        p.rows_a = N;
        p.rows_b = M;
        if (!tensor_map_2d(w, N, K, w_stride, TILE_A, &ma) || !tensor_map_2d(x, M, K, x_stride, bn, &mb))
            return CHIBI_ERR_UNSUPPORTED;
        const dim3 grid((N + TILE_A - 1) / TILE_A, 1, splits);
        if (bn == 16)
            status = launch_gemm<16, 6>(ma, mb, p, grid, stream);
        else if (bn == 32)
            status = launch_gemm<32, 5>(ma, mb, p, grid, stream);
        else
            status = launch_gemm<64, 4>(ma, mb, p, grid, stream);
    } else {
        p.swap = 0;
        p.rows_a = M;
        p.rows_b = N;
        const int bn = N >= 256 ? 256 : (N > 64 ? 128 : 64);
        if (!tensor_map_2d(x, M, K, x_stride, TILE_A, &ma) || !tensor_map_2d(w, N, K, w_stride, bn, &mb))
            return CHIBI_ERR_UNSUPPORTED;
        const dim3 grid((M + TILE_A - 1) / TILE_A, (N + bn - 1) / bn, 1);
        if (grid.y > 65535)
            return CHIBI_ERR_UNSUPPORTED;
        if (bn == 256)
            status = launch_gemm<256, 4>(ma, mb, p, grid, stream);
        else if (bn == 128)
            status = launch_gemm<128, 4>(ma, mb, p, grid, stream);
        else
            status = launch_gemm<64, 4>(ma, mb, p, grid, stream);
    }
    if (status != CHIBI_OK)
        return status;
    if (splits > 1) {
        const long long total = (long long)M * N;
        int blocks = (int)((total + 255) / 256);
        if (blocks > 148 * 8)
            blocks = 148 * 8;
        splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(scratch, splits, out, out_type, out_stride,
                                                         residual, res_stride, M, N);
        return launch_status();
    }
    return CHIBI_OK;
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
    return chibi_gemm_bf16(x, w, out, out_type, residual, M, N, K, x_stride, w_stride, out_stride,
                           res_stride, scratch, CHIBI_NOALLOC_SCRATCH_FLOATS, error, stream);
}
