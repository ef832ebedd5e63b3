// An entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference (nireo/chibillm allocates through its
// Metal context for every operation); it is an addition of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits -- a plug-in
// inside a host application that owns the whole device heap and hands out none
// of it, a real-time or safety-reviewed loop in which an allocation (which may
// synchronise the device or fail) is not allowed after start-up, or a caller
// that lives inside someone else's memory pool and cannot grow it.  Such a
// caller owns its inputs and outputs already, but has nowhere to put the
// scratch array that the matrix product needs when it splits the K range over
// several CTAs (few rows, as in decoding).
//
// What it does: the same kernels as chibi_gemm_bf16 -- out[M, N] = x[M, K] *
// w[N, K]^T (+ residual), bfloat16 inputs, 32-bit accumulation -- with the
// partial sums kept in an array that is part of the library's image:
// CHIBI_NOALLOC_SCRATCH_FLOATS 32-bit values (4 MiB) of device memory per GPU
// that loads the library, held until the process exits.  The call allocates
// nothing: no cudaMalloc, no cudaFree, no allocating library routine.
//
// Limits and rules:
//  * splits * M * N (splits = chibi_gemm_bf16_splits(M, N, K)) must not exceed
//    CHIBI_NOALLOC_SCRATCH_FLOATS; a larger product is refused with
//    CHIBI_ERR_SCRATCH_LIMIT and nothing is launched.  chibi_error_string()
//    turns a code into a sentence.
//  * A product that chibi_gemm_bf16_splits() does not split (more than 128 rows;
//    65 to 128 rows of a wide one) uses no scratch at
//    all; each of its tiles is computed whole by one CTA (the library's other
//    entry points may share a last, sparse round of tiles among idle CTAs
//    through scratch and counters that belong to the engine's stream; this
//    entry point never touches those).
//  * The first call on a device looks up the array's device address (once per
//    device, with that device current).  Make that first call before any stream
//    capture begins.
//  * Every call on a device shares the one array, and the array keeps what the
//    last call left in it.  Nothing in it has to start at zero: every value that
//    the second kernel adds up is written by the first kernel of the same call.
//    Two calls that may run on the GPU at the same time (different streams, or
//    different host threads) race on the array and give wrong sums; order them.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CHIBI_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define CHIBI_ERR_SCRATCH_LIMIT (-4)

// Returns 0, a positive cudaError_t, or a negative code of this library
// (-1 bad argument, -2 shape or alignment the tensor-core kernel does not take,
// CHIBI_ERR_SCRATCH_LIMIT).  Arguments as chibi_gemm_bf16: strides in elements,
// out_type 0 = float32, 1 = bfloat16, residual may be null or alias out, error
// may be null or point to a device int that a kernel sets when a wait runs out.
int chibi_gemm_bf16_noalloc(const void* x, const void* w, void* out, int out_type,
                            const float* residual, int M, int N, int K, long long x_stride,
                            long long w_stride, long long out_stride, long long res_stride,
                            int* error, cudaStream_t stream);

// A sentence for a return code of this library's entry points.
const char* chibi_error_string(int code);

#ifdef __cplusplus
}
#endif
