// Tensor-map (TMA) loads and mbarriers: the pieces that kernels with a TMA producer share.
//
// The driver's cuTensorMapEncodeTiled is reached through the runtime (cudaGetDriverEntryPoint), so nothing
// links against the driver library.  Every wait on an mbarrier is bounded by the clock: a wait that gives
// up returns false and the caller decides (kernels here set a status word and return).
#pragma once
#include <cuda.h>

#include "common.cuh"

#define KP_TMA_WAIT_NS 1000000000ull        // one second: far beyond any legitimate wait

__device__ __forceinline__ uint32_t kp_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void kp_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(kp_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void kp_mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void kp_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(kp_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void kp_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(kp_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool kp_mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(kp_smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long kp_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// false if the barrier did not flip within limit_ns
__device__ __forceinline__ bool kp_mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                     unsigned long long limit_ns = KP_TMA_WAIT_NS) {
    if (kp_mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = kp_now_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++)
            if (kp_mbar_try_wait(bar, parity)) return true;
        if (kp_now_ns() - t0 > limit_ns) return false;
    }
}
// A CTA that gave up a wait must not leave while bulk copies into its shared memory may still be under way
// (the memory could be handed to the next CTA meanwhile): it lingers for a moment that is far longer than any
// copy takes.  Only the failure path comes here.
__device__ __forceinline__ void kp_linger_after_failure() {
    const unsigned long long t0 = kp_now_ns();
    while (kp_now_ns() - t0 < 200000ull) __nanosleep(1000);
}

// The status word of a library whose kernels wait with a limit: 0, or 1 once a wait has given up.
//   kp_<name>_status()          reads and clears it (synchronises the device);
//   kp_<name>_status_address()  its device address, for a kernel that collects the status words of a step.
#define KP_STATUS_WORD(var, name)                                                                     \
    __device__ int var = 0;                                                                           \
    extern "C" int kp_##name##_status(void) {                                                         \
        int v = 0, zero = 0;                                                                          \
        if (cudaMemcpyFromSymbol(&v, var, sizeof(int)) != cudaSuccess) return -1;                     \
        if (v) cudaMemcpyToSymbol(var, &zero, sizeof(int));                                           \
        return v;                                                                                     \
    }                                                                                                 \
    extern "C" void* kp_##name##_status_address(void) {                                               \
        void* p = nullptr;                                                                            \
        return cudaGetSymbolAddress(&p, var) == cudaSuccess ? p : nullptr;                            \
    }
// box of the 2-D tensor at (x, y) -> shared memory; x * element size must be a multiple of 16 bytes
__device__ __forceinline__ void kp_tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(kp_smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(kp_smem_u32(bar)) : "memory");
}

typedef CUresult (*KpEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline KpEncodeTiledFn kp_encode_tiled_fn() {
    static KpEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (KpEncodeTiledFn)p;
    }
    return fn;
}

// rows x cols bf16 with row stride ld elements; box box_cols (at most 64: one 128-byte swizzle span) x box_rows,
// 128-byte swizzle, zero fill out of bounds
static inline int kp_make_map_bf16_2d(CUtensorMap* map, const void* base, unsigned long long rows, int cols, long long ld,
                                      int box_cols, int box_rows) {
    KpEncodeTiledFn fn = kp_encode_tiled_fn();
    if (!fn) return KP_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : KP_ERR_UNSUPPORTED;
}
