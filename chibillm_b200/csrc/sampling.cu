// Token selection from 32-bit logits: argmax (ties go to the lowest id, as in
// the reference's reduction, src/metal/kernels/sampling.metal:55-60,145-149)
// and temperature sampling by inverse CDF with one given uniform per row.
#define CHIBI_UNIT sampling
#define CHIBI_UNIT_ID 5
#include "common.cuh"

namespace chibi {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_WARPS = SAMPLE_THREADS / 32;
constexpr int ARGMAX_THREADS = 256;
constexpr int ARGMAX_MAX_SLICES = 64;

__device__ __forceinline__ void better(float& bv, int& bi, float v, int i)
{
    if (v > bv || (v == bv && i < bi)) {
        bv = v;
        bi = i;
    }
}

__device__ __forceinline__ void warp_better(float& bv, int& bi)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        better(bv, bi, ov, oi);
    }
}

// Best (value, id) of a block's threads; every thread gets it.
template <int WARPS>
__device__ __forceinline__ void block_better(float& bv, int& bi, float* sv, int* si)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    warp_better(bv, bi);
    if (lane == 0) {
        sv[warp] = bv;
        si[warp] = bi;
    }
    __syncthreads();
    bv = lane < WARPS ? sv[lane] : -INFINITY;
    bi = lane < WARPS ? si[lane] : 0x7fffffff;
    warp_better(bv, bi);
    __syncthreads();
}

// ------------------------------------------------------------------ greedy, two stages
// Stage 1: grid (slices, rows); a block finds the best id of its slice of the
// vocabulary.  Stage 2: one block per row picks the best slice.
__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_slices_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int slice,
                     float* __restrict__ part_v, int* __restrict__ part_i)
{
    pdl_enter();
    __shared__ float sv[32];
    __shared__ int si[32];
    const int row = blockIdx.y;
    const float* x = logits + (size_t)row * row_stride;
    const int begin = blockIdx.x * slice;
    const int end = begin + slice < vocab ? begin + slice : vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += ARGMAX_THREADS) {
        const float v = x[i];
        if (v == v)                                  // NaN never wins
            better(bv, bi, v, i);
    }
    block_better<ARGMAX_THREADS / 32>(bv, bi, sv, si);
    if (threadIdx.x == 0) {
        part_v[row * gridDim.x + blockIdx.x] = bv;
        part_i[row * gridDim.x + blockIdx.x] = bi;
    }
}

__global__ void argmax_pick_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                                   int slices, int* __restrict__ out)
{
    pdl_enter();
    const int row = blockIdx.x, lane = threadIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int s = lane; s < slices; s += 32)
        better(bv, bi, part_v[row * slices + s], part_i[row * slices + s]);
    warp_better(bv, bi);
    if (lane == 0)
        out[row] = bi == 0x7fffffff ? 0 : bi;
}

// ------------------------------------------------------------------ temperature
// One block per row.  Rows with temperature <= 0 (or a null temperature array)
// are greedy.  Otherwise p_i = exp((x_i - max) / T); the chosen id is the first
// i whose running sum of p (in id order) exceeds u * sum(p).  Warp w owns the
// ids [w * span, (w + 1) * span): the warps' totals locate the warp that holds
// the target, and that warp walks its ids 32 at a time with a shuffle scan.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
              const float* __restrict__ temperature, const float* __restrict__ uniform,
              int* __restrict__ out)
{
    pdl_enter();
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float totals[SAMPLE_WARPS];
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)row * row_stride;
    const float T = temperature ? temperature[row] : 0.f;

    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float v = x[i];
        if (v == v)
            better(bv, bi, v, i);
    }
    block_better<SAMPLE_WARPS>(bv, bi, sv, si);
    const float maxv = bv;
    const int argmax = bi == 0x7fffffff ? 0 : bi;
    if (!(T > 0.f)) {
        if (tid == 0)
            out[row] = argmax;
        return;
    }
    const float invT = 1.f / T;
    const int span = (((vocab + SAMPLE_WARPS - 1) / SAMPLE_WARPS) + 31) & ~31;   // a multiple of 32
    const int begin = warp * span;
    const int end = begin + span < vocab ? begin + span : vocab;
    // total of this warp's ids, formed tile by tile in the order of the walk below
    float run = 0.f;
    for (int base = begin; base < end; base += 32) {
        const int i = base + lane;
        float p = i < end ? expf((x[i] - maxv) * invT) : 0.f;
        p = warp_sum(p);
        run += p;
    }
    if (lane == 0)
        totals[warp] = run;
    __syncthreads();
    float before = 0.f, total = 0.f;
    for (int w = 0; w < SAMPLE_WARPS; ++w) {
        if (w < warp)
            before += totals[w];
        total += totals[w];
    }
    const float target = uniform[row] * total;
    const float after = before + totals[warp];
    // the last warp that holds any id also takes a target that rounding pushed to the total
    const bool last = end == vocab && begin < end;
    if (begin < end && target >= before && (target < after || last)) {
        float acc = before;
        int pick = end - 1;
        bool found = false;
        for (int base = begin; base < end && !found; base += 32) {
            const int i = base + lane;
            const float p = i < end ? expf((x[i] - maxv) * invT) : 0.f;
            float scan = p;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float n = __shfl_up_sync(0xffffffffu, scan, o);
                if (lane >= o)
                    scan += n;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, i < end && acc + scan > target);
            if (hit) {
                pick = base + __ffs(hit) - 1;
                found = true;
            }
            acc += __shfl_sync(0xffffffffu, scan, 31);
        }
        if (lane == 0)
            out[row] = pick;
    }
}

} // namespace chibi

using namespace chibi;

// Scratch floats that chibi_sample needs for `rows` all-greedy rows.
CHIBI_API long long chibi_sample_scratch_floats(long long rows) { return rows * ARGMAX_MAX_SLICES * 2; }

CHIBI_API int chibi_sample(const float* logits, long long row_stride, long long rows, int vocab,
                           const float* temperature, const float* uniform, int* out, float* scratch,
                           long long scratch_floats, cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (vocab <= 0 || (temperature && !uniform) || rows > 65535)
        return CHIBI_ERR_ARGUMENT;
    if (!temperature && scratch && scratch_floats >= chibi_sample_scratch_floats(rows)) {
        int slices = (vocab + 4095) / 4096;
        if (slices > ARGMAX_MAX_SLICES)
            slices = ARGMAX_MAX_SLICES;
        const int slice = (vocab + slices - 1) / slices;
        slices = (vocab + slice - 1) / slice;
        float* part_v = scratch;
        int* part_i = reinterpret_cast<int*>(scratch + rows * ARGMAX_MAX_SLICES);
        launch(argmax_slices_kernel, dim3(dim3(slices, (unsigned)rows)), dim3(ARGMAX_THREADS), 0, stream, 
            logits, row_stride, vocab, slice, part_v, part_i);
        launch(argmax_pick_kernel, dim3((unsigned)rows), dim3(32), 0, stream, part_v, part_i, slices, out);
        return launch_status();
    }
    launch(sample_kernel, dim3((unsigned)rows), dim3(SAMPLE_THREADS), 0, stream, logits, row_stride, vocab,
                                                                 temperature, uniform, out);
    return launch_status();
}
