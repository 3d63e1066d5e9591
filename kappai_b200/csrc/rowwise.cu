// Row-wise kernels: embedding gather, RMSNorm, SwiGLU, casts.
// One row's result never depends on the other rows of the launch.
#include "common.cuh"

// x[r,:] = float(table[ids[r],:])            (src/backend/cpu/common.c:1774-1782)
// `scale` multiplies the row (1.0 = none; the architecture decides).
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                  float* __restrict__ x, int d, float scale) {
    kp_pdl_begin();
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
    kp_pdl_begin();
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

// four consecutive outputs in one store (the destination is 8- or 16-byte aligned: d % 4 == 0)
__device__ __forceinline__ void store4(float* dst, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(bf16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = o;
}

// The same for rows of at most 8192 floats that are 16-byte aligned: each thread keeps its 8 float4 of the
// row in registers, so the row is read once.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_rows_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                        const int* __restrict__ rows, int d, float eps) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * d);
    const int n4 = d >> 2;
    float4 v[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int i = threadIdx.x + j * 256;
        v[j] = i < n4 ? __ldg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
        ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    T* dst = y + (size_t)r * d;
    const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            const float4 ww = __ldg(w4 + i);
            store4(dst + 4 * i, (v[j].x * scale) * ww.x, (v[j].y * scale) * ww.y, (v[j].z * scale) * ww.z,
                   (v[j].w * scale) * ww.w);
        }
    }
}

// Rows of at most 2048 elements (a multiple of 4), two kernels with ONE arithmetic, so that which of them runs
// (it depends on the number of rows) changes no bit of the result.  The row is 16 groups of 32 float4; "lane" l
// of "part" g (0..7) sums the squares of float4 l of group g, then of group g + 8, in element order; a lane's
// eight parts are added in order of g; the 32 lane sums are added by the warp butterfly.
//  * warp kernel (many rows): one warp a row, the row in registers (all loads in flight at once), no
//    block-wide barrier, eight rows a block.
//  * block kernel (few rows): 256 threads a row (thread = (part, lane)), so that a row's loads are spread
//    over more threads and the rows over more SMs.
__device__ __forceinline__ float sumsq8(const float4& a, const float4& b) {
    float ss = 0.f;
    ss = fmaf(a.x, a.x, ss); ss = fmaf(a.y, a.y, ss); ss = fmaf(a.z, a.z, ss); ss = fmaf(a.w, a.w, ss);
    ss = fmaf(b.x, b.x, ss); ss = fmaf(b.y, b.y, ss); ss = fmaf(b.z, b.z, ss); ss = fmaf(b.w, b.w, ss);
    return ss;
}

template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_rows_warp_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                         const int* __restrict__ rows, int n, int d, float eps) {
    kp_pdl_begin();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= n) return;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * d);
    const int n4 = d >> 2;
    float4 v[16];
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int i = lane + j * 32;
        v[j] = i < n4 ? __ldg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float ss = sumsq8(v[0], v[8]);
#pragma unroll
    for (int g = 1; g < 8; g++) ss += sumsq8(v[g], v[g + 8]);
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    T* dst = y + (size_t)r * d;
    const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int i = lane + j * 32;
        if (i < n4) {
            const float4 ww = __ldg(w4 + i);
            store4(dst + 4 * i, (v[j].x * scale) * ww.x, (v[j].y * scale) * ww.y, (v[j].z * scale) * ww.z,
                   (v[j].w * scale) * ww.w);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_rows_blk_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                        const int* __restrict__ rows, int d, float eps) {
    kp_pdl_begin_early();       // (measured with one row as well: a decode step 609 -> 601 us)
    __shared__ float part[8][32];
    __shared__ float scale_s;
    const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int r = blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * d);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    const int n4 = d >> 2;
    const int ia = lane + 32 * g, ib = lane + 32 * (g + 8);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 a = ia < n4 ? __ldg(src + ia) : zero, b = ib < n4 ? __ldg(src + ib) : zero;
    const float4 wa = ia < n4 ? __ldg(w4 + ia) : zero, wb = ib < n4 ? __ldg(w4 + ib) : zero;
    part[g][lane] = sumsq8(a, b);
    __syncthreads();
    if (g == 0) {
        float ss = part[0][lane];
#pragma unroll
        for (int k = 1; k < 8; k++) ss += part[k][lane];
        ss = warp_sum(ss);
        if (lane == 0) scale_s = 1.0f / sqrtf(ss / (float)d + eps);
    }
    __syncthreads();
    const float scale = scale_s;
    T* dst = y + (size_t)r * d;
    if (ia < n4) store4(dst + 4 * ia, (a.x * scale) * wa.x, (a.y * scale) * wa.y, (a.z * scale) * wa.z, (a.w * scale) * wa.w);
    if (ib < n4) store4(dst + 4 * ib, (b.x * scale) * wb.x, (b.y * scale) * wb.y, (b.z * scale) * wb.z, (b.w * scale) * wb.w);
}

// act = silu(gate) * up,  silu(g) = g / (1 + exp(-g))     (src/backend/cpu/scalar/core.c:774-800)
// gate_up rows hold [gate(ff) | up(ff)].
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, int n, int ff) {
    kp_pdl_begin();
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
    kp_pdl_begin();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(to_f32(in[i]));
}

static inline int grid_for(size_t total, int block) {
    size_t g = (total + block - 1) / block;
    if (g > 148 * 16) g = 148 * 16;
    if (g < 1) g = 1;
    return (int)g;
}

// The tables of a captured decode step, brought to the device by a kernel instead of a copy engine: `src` is the
// step's staging buffer in pinned host memory (the device reads it over the bus), `dst` the static buffer that the
// graph's kernels read; and, in the same launch, the step's token ids from where the sampler left them.  (A
// 2 KB cudaMemcpyAsync between two graph launches costs about 10 us of stream time, this about 3.)
__global__ void step_tables_kernel(const int4* src, int4* __restrict__ dst, int n4, const int* __restrict__ tok_src,
                                   int tok_off, int n_tok) {
    kp_pdl_begin();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    // with tokens given, their place in the tables (words tok_off ..., whole int4s) is theirs alone
    const bool toks = tok_src != nullptr && i * 4 >= tok_off && i * 4 < tok_off + (n_tok + 3) / 4 * 4;
    if (i < n4 && !toks) {
        int4 v;                                   // (a volatile load: host memory, rewritten between launches)
        asm volatile("ld.volatile.global.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src + i));
        dst[i] = v;
    }
    if (toks) {
        int* d = reinterpret_cast<int*>(dst) + i * 4;
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (i * 4 + j - tok_off < n_tok) d[j] = tok_src[i * 4 + j - tok_off];
    }
}

// The status words of a step's kernels brought together: out[0] = OR of the words at the given device
// addresses.  Launched behind a step; its one word travels to the host with the step's sampled tokens, so the
// host learns without any further synchronisation whether a kernel's bounded wait gave up.
__global__ void gather_status_kernel(const unsigned long long* __restrict__ addrs, int n, int* __restrict__ out) {
    kp_pdl_begin();
    if (threadIdx.x == 0) {
        int v = 0;
        for (int i = 0; i < n; i++) v |= *reinterpret_cast<const volatile int*>(addrs[i]);
        out[0] = v;
    }
}

extern "C" {

int kp_embed_rows(const void* table, const int* ids, float* x, int n, int d, float scale, int dtype, void* stream) {
    if (n <= 0) return 0;
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(embed_rows_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, (const T*)table, ids, x, d, scale)));
    return kp_launch_status();
}

int kp_rmsnorm_rows(const float* x, const float* w, void* y, const int* rows, int n, int d, float eps, int dtype,
                    void* stream) {
    if (n <= 0) return 0;
    if ((d & 3) == 0 && d <= 8192 && (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) == 0) {
        // which kernel runs depends on the row's size and alignment only, never on the batch
        if (d <= 2048) {
            if (n <= 256) {
                KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(rmsnorm_rows_blk_kernel<T>, dim3(n), dim3(256), 0,
                                                           (cudaStream_t)stream, x, w, (T*)y, rows, d, eps)));
            } else {
                KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(rmsnorm_rows_warp_kernel<T>, dim3((n + 7) / 8), dim3(256), 0,
                                                           (cudaStream_t)stream, x, w, (T*)y, rows, n, d, eps)));
            }
            return kp_launch_status();
        }
        KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(rmsnorm_rows_vec_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, x, w, (T*)y, rows, d, eps)));
        return kp_launch_status();
    }
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(rmsnorm_rows_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, x, w, (T*)y, rows, d, eps)));
    return kp_launch_status();
}

int kp_swiglu(const void* gate_up, void* act, int n, int ff, int dtype, void* stream) {
    if (n <= 0) return 0;
    const int g = grid_for((size_t)n * ff, 256);
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(swiglu_kernel<T>, dim3(g), dim3(256), 0, (cudaStream_t)stream, (const T*)gate_up, (T*)act, n, ff)));
    return kp_launch_status();
}

// dtype_in/out: 0 f32, 1 bf16
int kp_cast(const void* in, void* out, long long n, int dtype_in, int dtype_out, void* stream) {
    if (n <= 0) return 0;
    const int g = grid_for((size_t)n, 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype_in == KP_DTYPE_F32 && dtype_out == KP_DTYPE_BF16)
        kp_launch_pdl(cast_kernel<float, bf16>, dim3(g), dim3(256), 0, s, (const float*)in, (bf16*)out, (size_t)n);
    else if (dtype_in == KP_DTYPE_BF16 && dtype_out == KP_DTYPE_F32)
        kp_launch_pdl(cast_kernel<bf16, float>, dim3(g), dim3(256), 0, s, (const bf16*)in, (float*)out, (size_t)n);
    else
        return KP_ERR_BAD_ARG;
    return kp_launch_status();
}

// n_words a multiple of 4, both buffers 16-byte aligned.  tok_src (may be null): n_tok token ids on the device that
// go to words tok_off ... of dst (tok_off a multiple of 4) instead of what src holds there.
int kp_step_tables(const void* src, void* dst, int n_words, const int* tok_src, int tok_off, int n_tok, void* stream) {
    if (n_words <= 0 || (n_words & 3) || (tok_off & 3) || ((uintptr_t)src & 15) || ((uintptr_t)dst & 15)) return KP_ERR_BAD_ARG;
    if (tok_src != nullptr && (tok_off < 0 || n_tok < 0 || tok_off + n_tok > n_words)) return KP_ERR_BAD_ARG;
    const int n4 = n_words / 4;
    kp_launch_pdl(step_tables_kernel, dim3((n4 + 255) / 256), dim3(256), 0, (cudaStream_t)stream, (const int4*)src, (int4*)dst,
                  n4, tok_src, tok_off, n_tok);
    return kp_launch_status();
}

int kp_gather_status(const unsigned long long* addrs, int n, int* out, void* stream) {
    if (n < 0 || !out) return KP_ERR_BAD_ARG;
    kp_launch_pdl(gather_status_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, addrs, n, out);
    return kp_launch_status();
}

}  // extern "C"
