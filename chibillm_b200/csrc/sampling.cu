// Token selection from 32-bit logits: argmax (ties go to the lowest id, as in
// the reference's reduction, src/metal/kernels/sampling.metal:55-60,145-149)
// and temperature sampling by inverse CDF with one given uniform per row.
#include "common.cuh"

namespace chibi {

constexpr int SAMPLE_THREADS = 256;

__device__ __forceinline__ void better(float& bv, int& bi, float v, int i)
{
    if (v > bv || (v == bv && i < bi)) {
        bv = v;
        bi = i;
    }
}

// One block per row.  Rows with temperature <= 0 (or a null temperature
// array) are greedy.  Otherwise p_i = exp((x_i - max) / T); the chosen id is
// the first i whose running sum of p (in id order) exceeds u * sum(p).  Each
// thread owns one contiguous segment of ids, so the running sum is formed in a
// fixed order that depends on the vocabulary size only.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
              const float* __restrict__ temperature, const float* __restrict__ uniform,
              int* __restrict__ out)
{
    __shared__ float sv[SAMPLE_THREADS];
    __shared__ int si[SAMPLE_THREADS];
    __shared__ float scratch[33];
    __shared__ int chosen;
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * row_stride;
    const float T = temperature ? temperature[row] : 0.f;

    const int seg = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = tid * seg;
    const int end = begin + seg < vocab ? begin + seg : vocab;

    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = begin; i < end; ++i) {
        const float v = x[i];
        if (v == v) // NaN never wins
            better(bv, bi, v, i);
    }
    sv[tid] = bv;
    si[tid] = bi;
    __syncthreads();
    for (int o = SAMPLE_THREADS / 2; o > 0; o >>= 1) {
        if (tid < o) {
            float v = sv[tid];
            int i = si[tid];
            better(v, i, sv[tid + o], si[tid + o]);
            sv[tid] = v;
            si[tid] = i;
        }
        __syncthreads();
    }
    const float maxv = sv[0];
    const int argmax = si[0] == 0x7fffffff ? 0 : si[0];
    if (!(T > 0.f)) {
        if (tid == 0)
            out[row] = argmax;
        return;
    }
    __syncthreads();
    const float invT = 1.f / T;
    float part = 0.f;
    for (int i = begin; i < end; ++i)
        part += expf((x[i] - maxv) * invT);
    sv[tid] = part;
    if (tid == 0)
        chosen = argmax;
    __syncthreads();
    // Exclusive prefix over the segments, in segment order, by one thread.
    if (tid == 0) {
        float run = 0.f;
        for (int i = 0; i < SAMPLE_THREADS; ++i) {
            const float p = sv[i];
            sv[i] = run;
            run += p;
        }
        scratch[0] = run;
    }
    __syncthreads();
    const float total = scratch[0];
    const float target = uniform[row] * total;
    const float before = sv[tid];
    const float after = (tid + 1 < SAMPLE_THREADS) ? sv[tid + 1] : total;
    if (begin < end && target >= before && (target < after || tid == SAMPLE_THREADS - 1 || end == vocab)) {
        float run = before;
        int pick = end - 1;
        for (int i = begin; i < end; ++i) {
            run += expf((x[i] - maxv) * invT);
            if (run > target) {
                pick = i;
                break;
            }
        }
        chosen = pick;
    }
    __syncthreads();
    if (tid == 0)
        out[row] = chosen;
}

} // namespace chibi

using namespace chibi;

CHIBI_API int chibi_sample(const float* logits, long long row_stride, long long rows, int vocab,
                           const float* temperature, const float* uniform, int* out,
                           cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (vocab <= 0 || (temperature && !uniform))
        return CHIBI_ERR_ARGUMENT;
    sample_kernel<<<(unsigned)rows, SAMPLE_THREADS, 0, stream>>>(logits, row_stride, vocab,
                                                                 temperature, uniform, out);
    return launch_status();
}
