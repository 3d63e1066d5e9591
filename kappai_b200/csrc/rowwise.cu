// Row-wise kernels: embedding gather, RMSNorm, SwiGLU, casts.
// One row's result never depends on the other rows of the launch.
#include "common.cuh"

// x[r,:] = float(table[ids[r],:])            (src/backend/cpu/common.c:1774-1782)
// `scale` multiplies the row (1.0 = none; the architecture decides).
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                  float* __restrict__ x, int d, float scale) {
    const int r = blockIdx.x;
    const T* src = table + (size_t)ids[r] * d;
    float* dst = x + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = to_f32(src[i]) * scale;
}

// y[r,:] = (x[row,:] * rsqrt(mean(x^2) + eps)) * w     (src/backend/cpu/scalar/quants.c:1489-1512)
// row = rows ? rows[r] : r.  The sum of squares is float32 with a fixed tree.
template <typename T>
__global__ void rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                    T* __restrict__ y, const int* __restrict__ rows, int d, float eps) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* src = x + (size_t)(rows ? rows[r] : r) * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = src[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    T* dst = y + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = from_f32<T>((src[i] * scale) * w[i]);
}

// act = silu(gate) * up,  silu(g) = g / (1 + exp(-g))     (src/backend/cpu/scalar/core.c:774-800)
// gate_up rows hold [gate(ff) | up(ff)].
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, int n, int ff) {
    const size_t total = (size_t)n * ff;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / ff, c = i % ff;
        const float g = to_f32(gu[r * 2 * ff + c]);
        const float u = to_f32(gu[r * 2 * ff + ff + c]);
        act[i] = from_f32<T>((g / (1.0f + expf(-g))) * u);
    }
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(to_f32(in[i]));
}

static inline int grid_for(size_t total, int block) {
    size_t g = (total + block - 1) / block;
    if (g > 148 * 16) g = 148 * 16;
    if (g < 1) g = 1;
    return (int)g;
}

extern "C" {

int kp_embed_rows(const void* table, const int* ids, float* x, int n, int d, float scale, int dtype, void* stream) {
    if (n <= 0) return 0;
    KP_DISPATCH_DTYPE(dtype, T, (embed_rows_kernel<T><<<n, 256, 0, (cudaStream_t)stream>>>((const T*)table, ids, x, d, scale)));
    return kp_launch_status();
}

int kp_rmsnorm_rows(const float* x, const float* w, void* y, const int* rows, int n, int d, float eps, int dtype,
                    void* stream) {
    if (n <= 0) return 0;
    KP_DISPATCH_DTYPE(dtype, T, (rmsnorm_rows_kernel<T><<<n, 256, 0, (cudaStream_t)stream>>>(x, w, (T*)y, rows, d, eps)));
    return kp_launch_status();
}

int kp_swiglu(const void* gate_up, void* act, int n, int ff, int dtype, void* stream) {
    if (n <= 0) return 0;
    const int g = grid_for((size_t)n * ff, 256);
    KP_DISPATCH_DTYPE(dtype, T, (swiglu_kernel<T><<<g, 256, 0, (cudaStream_t)stream>>>((const T*)gate_up, (T*)act, n, ff)));
    return kp_launch_status();
}

// dtype_in/out: 0 f32, 1 bf16
int kp_cast(const void* in, void* out, long long n, int dtype_in, int dtype_out, void* stream) {
    if (n <= 0) return 0;
    const int g = grid_for((size_t)n, 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype_in == KP_DTYPE_F32 && dtype_out == KP_DTYPE_BF16)
        cast_kernel<float, bf16><<<g, 256, 0, s>>>((const float*)in, (bf16*)out, (size_t)n);
    else if (dtype_in == KP_DTYPE_BF16 && dtype_out == KP_DTYPE_F32)
        cast_kernel<bf16, float><<<g, 256, 0, s>>>((const bf16*)in, (float*)out, (size_t)n);
    else
        return KP_ERR_BAD_ARG;
    return kp_launch_status();
}

}  // extern "C"
