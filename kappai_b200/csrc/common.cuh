// Shared helpers of the kernel libraries: element types, conversions,
// reductions and the launcher conventions.
//
// Conventions of every launcher (extern "C"):
//   * pointers are raw device pointers, sizes are in elements, `stream` is a
//     cudaStream_t passed as void*;
//   * `dtype` selects the storage type of activations / weights / cache:
//     0 = float32 (the true 32-bit path), 1 = bfloat16;
//   * the return value is 0 or a cudaError_t / a negative argument error;
//   * statistics (norm sums, softmax, conv sums, rotation) are float32 in both
//     modes; only storage and matrix operands differ.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define KP_DTYPE_F32 0
#define KP_DTYPE_BF16 1

#define KP_ERR_BAD_ARG (-22)
#define KP_ERR_UNSUPPORTED (-95)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum with a fixed tree (the same for every launch shape, so a
// row's statistic does not depend on what else is in the batch).  `smem` holds
// at least 32 floats.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = (lane < nwarp) ? smem[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = (lane < nwarp) ? smem[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

// Programmatic dependent launch.  Every kernel of this package is launched with the attribute that lets
// it start while the kernel before it in the stream is still running, and begins with kp_pdl_begin():
// it waits until that kernel has finished and its writes are visible, then lets the kernel after it
// start in turn.  So launch latency and a kernel's ramp-up hide under its predecessor.  Only work that
// depends on nothing written by earlier kernels (loading weights) may come before kp_pdl_begin().
// Device timeline (built only with -DKP_TRACE=<library number>, as the second build that
// kappai_b200.ops.timeline asks for): thread 0 of every CTA notes the global timer when it enters a kernel
// (mark 0) and when its wait on the kernel before is over (mark 1); the matrix-product kernels also note the end of
// a CTA's work (2) and of its producer's (3).  The records show how the kernels of a step overlap inside a
// captured graph, which no per-kernel timing does.  The marks cost an atomic each: the traced step runs 10 to
// 15 % slower, so read shares and gaps, not absolutes.
#ifdef KP_TRACE
struct KpTraceRec { unsigned long long t; unsigned tag; unsigned info; };
#define KP_TRACE_CAP (1 << 18)
__device__ KpTraceRec g_kp_trace[KP_TRACE_CAP];
__device__ unsigned g_kp_trace_n;
__device__ __forceinline__ void kp_trace_mark(unsigned phase) {
    unsigned i = atomicAdd(&g_kp_trace_n, 1u);
    if (i < KP_TRACE_CAP) {
        unsigned smid; asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        unsigned b = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        unsigned g = gridDim.x * gridDim.y * gridDim.z;
        g_kp_trace[i] = {t, ((unsigned)KP_TRACE << 24) | (phase << 16) | smid, (min(g, 65535u) << 16) | min(b, 65535u)};
    }
}
extern "C" int kp_trace_dump(void* out, int max_recs) {
    unsigned n = 0, zero = 0;
    cudaDeviceSynchronize();
    if (cudaMemcpyFromSymbol(&n, g_kp_trace_n, sizeof(n)) != cudaSuccess) return -1;
    if (n > KP_TRACE_CAP) n = KP_TRACE_CAP;
    if ((int)n > max_recs) n = max_recs;
    if (n && cudaMemcpyFromSymbol(out, g_kp_trace, (size_t)n * sizeof(KpTraceRec)) != cudaSuccess) return -2;
    cudaMemcpyToSymbol(g_kp_trace_n, &zero, sizeof(zero));
    return (int)n;
}
#define KP_TRACE_MARK(ph) do { if (threadIdx.x == 0) kp_trace_mark(ph); } while (0)
#define KP_TRACE_MARK_LANE(ph) kp_trace_mark(ph)
#else
#define KP_TRACE_MARK(ph)
#define KP_TRACE_MARK_LANE(ph)
#endif
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void kp_pdl_begin() { KP_TRACE_MARK(0); pdl_wait(); KP_TRACE_MARK(1); pdl_launch_dependents(); }
// The same with the kernel after this one let in first: it may then become resident, and run what it has
// before its own wait (a product's producers fill their rings with weights), while this kernel still waits
// for the one before it.  For the small kernels of a decode step that stand between two products.
__device__ __forceinline__ void kp_pdl_begin_early() { KP_TRACE_MARK(0); pdl_launch_dependents(); pdl_wait(); KP_TRACE_MARK(1); }
// Early only for a step of several rows: with a single row (batch 1) the early form measured 2 % slower.
__device__ __forceinline__ void kp_pdl_begin_early_if(bool several_rows) {
    if (several_rows) kp_pdl_begin_early(); else kp_pdl_begin();
}

template <typename... KArgs, typename... Args>
static inline cudaError_t kp_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                        Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

static inline int kp_launch_status() {
    cudaError_t e = cudaGetLastError();
    return (int)e;
}

#define KP_DISPATCH_DTYPE(dtype, T, ...)                 \
    do {                                                 \
        if ((dtype) == KP_DTYPE_F32) {                   \
            typedef float T;                             \
            __VA_ARGS__;                                 \
        } else if ((dtype) == KP_DTYPE_BF16) {           \
            typedef bf16 T;                              \
            __VA_ARGS__;                                 \
        } else {                                         \
            return KP_ERR_BAD_ARG;                       \
        }                                                \
    } while (0)
