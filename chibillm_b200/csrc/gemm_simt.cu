// out[M, N] = x[M, K] * w[N, K]^T (+ residual[M, N]) with plain 32-bit FMAs.
//
// This is the matrix product of the true 32-bit path (no tensor-core mode, so
// no reduced-precision inputs or accumulators) and the fall-back of the
// bfloat16 path for shapes the tensor-core kernel refuses.  Every output
// element is one thread's sequential sum over k = 0..K-1, so the result of a
// row does not depend on how many rows the call has.
#define CHIBI_UNIT gemm_simt
#define CHIBI_UNIT_ID 2
#include "common.cuh"

namespace chibi {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                 const float* __restrict__ residual, int M, int N, int K, long long x_stride,
                 long long w_stride, long long out_stride, long long res_stride)
{
    pdl_enter();
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4; // 16 x 16 threads, each TM x TN outputs
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j)
            acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int r = e >> 4, kk = e & 15;
            const int k = k0 + kk;
            float xv = 0.f, wv = 0.f;
            if (k < K) {
                if (m0 + r < M)
                    xv = to_f32(x[(size_t)(m0 + r) * x_stride + k]);
                if (n0 + r < N)
                    wv = to_f32(w[(size_t)(n0 + r) * w_stride + k]);
            }
            xs[kk][r] = xv;
            ws[kk][r] = wv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i)
                a[i] = xs[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j)
                b[j] = ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j)
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M)
            continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N)
                continue;
            float v = acc[i][j];
            if (residual)
                v = residual[(size_t)m * res_stride + n] + v;
            out[(size_t)m * out_stride + n] = from_f32<TO>(v);
        }
    }
}

} // namespace chibi

using namespace chibi;

CHIBI_API int chibi_gemm_simt(const void* x, int x_type, const void* w, int w_type, void* out,
                              int out_type, const float* residual, int M, int N, int K,
                              long long x_stride, long long w_stride, long long out_stride,
                              long long res_stride, cudaStream_t stream)
{
    if (M <= 0 || N <= 0)
        return CHIBI_OK;
    if (K < 0)
        return CHIBI_ERR_ARGUMENT;
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535)
        return CHIBI_ERR_UNSUPPORTED;
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(w_type, TW, CHIBI_DISPATCH_TYPE(out_type, TO, {
        launch(gemm_simt_kernel<TX, TW, TO>, dim3(grid), dim3(256), 0, stream, 
            (const TX*)x, (const TW*)w, (TO*)out, residual, M, N, K, x_stride, w_stride,
            out_stride, res_stride);
    })));
    return launch_status();
}
