// Shared helpers of the sm_100a kernels: element types, loads and stores in
// 32-bit arithmetic, warp and block reductions, launch checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

// Element type codes used by every C entry point.
#define CHIBI_F32 0
#define CHIBI_BF16 1

// Return codes of the C entry points (0 = ok, >0 = cudaError_t, <0 = ours).
#define CHIBI_OK 0
#define CHIBI_ERR_ARGUMENT (-1)
#define CHIBI_ERR_UNSUPPORTED (-2)
#define CHIBI_ERR_DEVICE_CHECK (-3)

#define CHIBI_API extern "C" __attribute__((visibility("default")))

namespace chibi {

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v)
{
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds at least 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0)
        scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0)
            scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0)
        scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0)
            scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Programmatic dependent launch: a kernel lets the next kernel of its stream be
// scheduled as soon as all of its own CTAs run (pdl_trigger), and the next
// kernel waits (pdl_wait) for this one to finish, with its writes visible,
// before it touches global memory.  That hides the launch latency between the
// many short kernels of a decode step.  Both instructions do nothing in a kernel
// that was launched without the attribute.
__device__ __forceinline__ void pdl_trigger_now() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_now() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#ifndef CHIBI_TIMELINE
__device__ __forceinline__ void timeline_mark(int) {}
__device__ __forceinline__ void pdl_trigger() { pdl_trigger_now(); }
__device__ __forceinline__ void pdl_wait() { pdl_wait_now(); }
__device__ __forceinline__ void pdl_enter()
{
    pdl_trigger();
    pdl_wait();
}
#else
// A build with -DCHIBI_TIMELINE records, for every CTA of every kernel, when it started, when its
// wait for the kernel before it ended and when its last warp left, with the SM it ran on
// (%globaltimer, nanoseconds), into an array that the host hands over with
// chibi_timeline_set_<file>.  The first statement of every kernel is pdl_trigger() or pdl_enter():
// in this build they also open the record, and a local object closes it on every way out.  The
// libraries of the product are built without the flag and contain none of this.
struct TimelineRecord {
    unsigned int unit, line, block, blocks, sm, pad;
    unsigned long long start, waited, end;
    unsigned long long marks[4];       // points inside a kernel (timeline_mark), latest arrival
};
static __device__ TimelineRecord* g_timeline_records;
static __device__ unsigned int* g_timeline_count;
static __device__ unsigned int g_timeline_capacity;

__device__ __forceinline__ unsigned long long global_timer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned int& timeline_slot()
{
    __shared__ unsigned int slot;
    return slot;
}
struct TimelineScope {
    __device__ __forceinline__ TimelineScope(unsigned int line)
    {
        if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
            unsigned int s = 0xffffffffu;
            if (g_timeline_records) {
                s = atomicAdd(g_timeline_count, 1u);
                if (s >= g_timeline_capacity) {
                    s = 0xffffffffu;
                } else {
                    TimelineRecord& r = g_timeline_records[s];
                    unsigned int sm;
                    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
                    r.unit = CHIBI_UNIT_ID;
                    r.line = line;
                    r.block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
                    r.blocks = gridDim.x * gridDim.y * gridDim.z;
                    r.sm = sm;
                    r.waited = 0;
                    r.end = 0;
                    r.marks[0] = r.marks[1] = r.marks[2] = r.marks[3] = 0;
                    r.start = global_timer();
                }
            }
            timeline_slot() = s;
        }
        __syncthreads();
    }
    __device__ __forceinline__ ~TimelineScope()
    {
        const unsigned int s = timeline_slot();
        if (s != 0xffffffffu && (threadIdx.x & 31) == 0)
            atomicMax(&g_timeline_records[s].end, global_timer());
    }
};
__device__ __forceinline__ void timeline_waited()
{
    const unsigned int s = timeline_slot();
    if (s != 0xffffffffu && (threadIdx.x & 31) == 0)
        atomicCAS(&g_timeline_records[s].waited, 0ull, global_timer());
}
__device__ __forceinline__ void timeline_mark(int i)
{
    const unsigned int s = timeline_slot();
    if (s != 0xffffffffu && (threadIdx.x & 31) == 0)
        atomicMax(&g_timeline_records[s].marks[i], global_timer());
}
#define pdl_trigger() TimelineScope timeline_scope(__LINE__); pdl_trigger_now()
#define pdl_wait() do { pdl_wait_now(); timeline_waited(); } while (0)
#define pdl_enter() TimelineScope timeline_scope(__LINE__); pdl_trigger_now(); pdl_wait_now(); timeline_waited()
#endif

// Asks for the line at p in L2, and with it for the translation of its page.  A
// kernel that was launched early does this for the addresses it will touch
// before pdl_wait(): after a product has streamed hundreds of megabytes of
// weights, the first access to a page otherwise waits for a page-table walk.
// (L2 is where the GPU's memory is coherent, so a line fetched before its
// producer wrote it is not stale.)
__device__ __forceinline__ void prefetch_l2(const void* p)
{
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// Programmatic dependent launch is how every kernel but a step's first is launched.
inline bool pdl_enabled() { return true; }

// Launches with a thread-block cluster of (1, 1, cluster_z) CTAs when cluster_z > 1.
// `ordered`: an ordinary launch, which starts only after everything before it in
// the stream has completed.
template <typename... KArgs, typename... Args>
inline void launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                           cudaStream_t stream, int cluster_z, Args&&... args);

template <bool ORDERED, typename... KArgs, typename... Args>
inline void launch_with(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                        cudaStream_t stream, int cluster_z, Args&&... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (!ORDERED && pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = (unsigned)cluster_z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline void launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                           cudaStream_t stream, int cluster_z, Args&&... args)
{
    launch_with<false>(kernel, grid, block, smem, stream, cluster_z, static_cast<Args&&>(args)...);
}

// The step's first kernel (the embedding) is launched this way.  Every kernel
// after it, however early programmatic dependent launch lets it start, therefore
// runs after all that was written before the embedding: the step's index arrays
// (positions, sequence of each token, lengths, block tables) and the cache
// entries of earlier steps.  Kernels may read those before their pdl_wait().
template <typename... KArgs, typename... Args>
inline void launch_ordered(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                           Args&&... args)
{
    launch_with<true>(kernel, grid, block, smem, stream, 1, static_cast<Args&&>(args)...);
}

// Launches with a thread-block cluster of (cluster_x, 1, 1) CTAs.
template <typename... KArgs, typename... Args>
inline void launch_cluster_x(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, int cluster_x, Args&&... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline void launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                   Args&&... args)
{
    launch_cluster(kernel, grid, block, smem, stream, 1, static_cast<Args&&>(args)...);
}

inline int launch_status()
{
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? CHIBI_OK : static_cast<int>(e);
}

} // namespace chibi

// Calls `body` with `T` bound to the element type that `code` names.
#define CHIBI_DISPATCH_TYPE(code, T, ...)                                                          \
    do {                                                                                           \
        if ((code) == CHIBI_F32) {                                                                 \
            using T = float;                                                                       \
            __VA_ARGS__;                                                                           \
        } else if ((code) == CHIBI_BF16) {                                                         \
            using T = __nv_bfloat16;                                                               \
            __VA_ARGS__;                                                                           \
        } else {                                                                                   \
            return CHIBI_ERR_ARGUMENT;                                                             \
        }                                                                                          \
    } while (0)

#ifdef CHIBI_TIMELINE
#define CHIBI_TIMELINE_CAT2(a, b) a##b
#define CHIBI_TIMELINE_CAT(a, b) CHIBI_TIMELINE_CAT2(a, b)
// Where this file's kernels write their records (null: nowhere).  `count` is shared by all files
// of all libraries, so the records of a step form one list.
CHIBI_API int CHIBI_TIMELINE_CAT(chibi_timeline_set_, CHIBI_UNIT)(void* records, unsigned int* count,
                                                                 unsigned int capacity)
{
    cudaError_t e = cudaMemcpyToSymbol(chibi::g_timeline_records, &records, sizeof(records));
    if (e == cudaSuccess)
        e = cudaMemcpyToSymbol(chibi::g_timeline_count, &count, sizeof(count));
    if (e == cudaSuccess)
        e = cudaMemcpyToSymbol(chibi::g_timeline_capacity, &capacity, sizeof(capacity));
    return (int)e;
}
#endif
