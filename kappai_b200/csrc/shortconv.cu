// Gated causal depthwise short convolution with per-request state, for a
// batch of segments (prompt portions and single decoded tokens alike).
//
// Per channel c and row t of a segment (src/backend/cpu/common.c:2393-2431):
//   bx_t  = B[t,c] * X[t,c]
//   y_t   = sum_{k<K-1} hist[k] * w[c,k] + bx_t * w[c,K-1]  (+ bias[c])
//   out_t = C[t,c] * y_t ;  hist <- (hist[1:], bx_t)
// with p = [B | C | X] the in_proj output (3*d wide) and hist the previous
// K-1 values of bx of this request, oldest first, zero at a sequence's start.
//
// The sum is a finite filter, so rows are independent given the K-1 values
// before them: those come from earlier rows of the same segment or, at the
// segment's head, from the request's state slot (nothing if the segment
// starts at position 0, which is why a reused slot needs no clearing).
// State layout: state[slot][K-1][d] float32.  The forward kernel only reads
// the state; the update kernel, launched after it, writes the new history, one
// thread per (segment, channel) so that a shift by fewer than K-1 rows reads
// every old value before it is overwritten.
#include "common.cuh"

#define KP_CONV_MAX_K 16

template <typename T>
__device__ __forceinline__ float bx_of(const T* __restrict__ p, size_t row, int ldp, int d, int c) {
    const T* r = p + row * ldp;
    return __fmul_rn(to_f32(r[c]), to_f32(r[2 * (size_t)d + c]));
}

// One arithmetic for every kernel of this file: each product and each sum is rounded on its own (no fused
// multiply-add, which the compiler would place differently from kernel to kernel), so that which kernel runs
// -- it depends on the shape of the step -- changes no bit of a row's result.
__device__ __forceinline__ float tap(float h, float w) { return __fmul_rn(h, w); }
__device__ __forceinline__ float add_tap(float sum, float h, float w) { return __fadd_rn(sum, __fmul_rn(h, w)); }
// K == 3: (h0 w0 + h1 w1) + bx w2 (src/backend/cpu/common.c:2411)
__device__ __forceinline__ float conv_sum3(float h0, float h1, float bx, float w0, float w1, float w2) {
    return __fadd_rn(__fadd_rn(__fmul_rn(h0, w0), __fmul_rn(h1, w1)), __fmul_rn(bx, w2));
}
__device__ __forceinline__ float gate_out(float c, float sum, bool has_bias, float b) {
    return __fmul_rn(c, has_bias ? __fadd_rn(sum, b) : sum);
}

template <typename T>
__global__ void shortconv_fwd_kernel(const T* __restrict__ p, int ldp, const float* __restrict__ w,
                                     const float* __restrict__ bias, const float* __restrict__ state,
                                     const int* __restrict__ row_seg, const int* __restrict__ cu_rows,
                                     const int* __restrict__ seg_pos, const int* __restrict__ seg_slot,
                                     T* __restrict__ out, int ldo, int n, int d, int K) {
    kp_pdl_begin();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int row = blockIdx.y;
    if (c >= d || row >= n) return;
    const int seg = row_seg[row];
    const int t = row - cu_rows[seg];                 // row index inside the segment
    const bool fresh = seg_pos[seg] == 0;             // a sequence's first portion: history is zero
    const float* st = state + (size_t)seg_slot[seg] * (K - 1) * d;
    const float* wc = w + (size_t)c * K;
    const float bx = bx_of(p, row, ldp, d, c);

    float hist[KP_CONV_MAX_K - 1];
    for (int k = 0; k < K - 1; k++) {
        const int st_t = t - (K - 1) + k;             // time of hist[k] relative to the segment's start
        float h;
        if (st_t >= 0) h = bx_of(p, (size_t)(row - (K - 1) + k), ldp, d, c);
        else h = fresh ? 0.f : st[(size_t)(K - 1 + st_t) * d + c];
        hist[k] = h;
    }
    float sum;
    if (K == 3) {
        sum = conv_sum3(hist[0], hist[1], bx, wc[0], wc[1], wc[2]);
    } else {
        sum = tap(bx, wc[K - 1]);                                  // src/backend/cpu/common.c:2422-2424
        for (int k = 0; k < K - 1; k++) sum = add_tap(sum, hist[k], wc[k]);
    }
    out[(size_t)row * ldo + c] = from_f32<T>(gate_out(to_f32(p[(size_t)row * ldp + d + c]), sum, bias != nullptr,
                                                      bias ? bias[c] : 0.f));
}

template <typename T>
__global__ void shortconv_state_kernel(const T* __restrict__ p, int ldp, float* __restrict__ state,
                                       const int* __restrict__ cu_rows, const int* __restrict__ seg_pos,
                                       const int* __restrict__ seg_slot, int n_seg, int d, int K) {
    kp_pdl_begin();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int seg = blockIdx.y;
    if (c >= d || seg >= n_seg) return;
    const int r0 = cu_rows[seg], nr = cu_rows[seg + 1] - r0;
    if (nr <= 0) return;
    const bool fresh = seg_pos[seg] == 0;
    float* st = state + (size_t)seg_slot[seg] * (K - 1) * d;
    for (int j = 0; j < K - 1; j++) {                 // ascending: old[j + nr] is read before it is written
        const int t = nr - (K - 1) + j;               // time of the new hist[j] relative to the segment's start
        float v;
        if (t >= 0) v = bx_of(p, (size_t)(r0 + t), ldp, d, c);
        else v = fresh ? 0.f : st[(size_t)(K - 1 + t) * d + c];
        st[(size_t)j * d + c] = v;
    }
}

// The forward kernel with 16-byte accesses: a thread computes VEC consecutive channels of one row
// (VEC = 8 bfloat16 or 4 float32).  Needs d % VEC == 0 and 16-byte aligned rows.
template <typename T> struct ConvVec;
template <> struct ConvVec<bf16> { static constexpr int N = 8; };
template <> struct ConvVec<float> { static constexpr int N = 4; };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float* f);
template <>
__device__ __forceinline__ void load_vec<bf16>(const bf16* p, float* f) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void load_vec<float>(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
__device__ __forceinline__ void store_vec(bf16* p, const float* f) {
    uint4 o;
    uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&t);
    }
    *reinterpret_cast<uint4*>(p) = o;
}
__device__ __forceinline__ void store_vec(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}

template <typename T>
__global__ void __launch_bounds__(128)
shortconv_fwd_vec_kernel(const T* __restrict__ p, int ldp, const float* __restrict__ w,
                         const float* __restrict__ bias, const float* __restrict__ state,
                         const int* __restrict__ row_seg, const int* __restrict__ cu_rows,
                         const int* __restrict__ seg_pos, const int* __restrict__ seg_slot,
                         T* __restrict__ out, int ldo, int n, int d, int K) {
    kp_pdl_begin();
    constexpr int V = ConvVec<T>::N;
    const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    const int row = blockIdx.y;
    if (c0 >= d || row >= n) return;
    const int seg = row_seg[row];
    const int t = row - cu_rows[seg];
    const bool fresh = seg_pos[seg] == 0;
    const float* st = state + (size_t)seg_slot[seg] * (K - 1) * d;
    const T* pr = p + (size_t)row * ldp;
    float bv[V], cv[V], xv[V], bx[V], sum[V];
    load_vec<T>(pr + c0, bv);
    load_vec<T>(pr + d + c0, cv);
    load_vec<T>(pr + 2 * (size_t)d + c0, xv);
#pragma unroll
    for (int i = 0; i < V; i++) bx[i] = __fmul_rn(bv[i], xv[i]);
    // same order of summation as the scalar kernel: K == 3: (h0 w0 + h1 w1) + bx w2; else bx w[K-1] + h0 w0 + ...
    if (K != 3) {
#pragma unroll
        for (int i = 0; i < V; i++) sum[i] = tap(bx[i], w[(size_t)(c0 + i) * K + K - 1]);
    }
    for (int k = 0; k < K - 1; k++) {
        const int st_t = t - (K - 1) + k;
        float h[V];
        if (st_t >= 0) {
            float hb[V], hx[V];
            const T* ph = p + (size_t)(row - (K - 1) + k) * ldp;
            load_vec<T>(ph + c0, hb);
            load_vec<T>(ph + 2 * (size_t)d + c0, hx);
#pragma unroll
            for (int i = 0; i < V; i++) h[i] = __fmul_rn(hb[i], hx[i]);
        } else {
#pragma unroll
            for (int i = 0; i < V; i++) h[i] = fresh ? 0.f : st[(size_t)(K - 1 + st_t) * d + c0 + i];
        }
        if (K == 3) {
#pragma unroll
            for (int i = 0; i < V; i++) {
                const float term = tap(h[i], w[(size_t)(c0 + i) * K + k]);
                sum[i] = k == 0 ? term : __fadd_rn(sum[i], term);
            }
        } else {
#pragma unroll
            for (int i = 0; i < V; i++) sum[i] = add_tap(sum[i], h[i], w[(size_t)(c0 + i) * K + k]);
        }
    }
    float o[V];
#pragma unroll
    for (int i = 0; i < V; i++) {
        float s2 = sum[i];
        if (K == 3) s2 = add_tap(s2, bx[i], w[(size_t)(c0 + i) * K + 2]);
        o[i] = gate_out(cv[i], s2, bias != nullptr, bias ? bias[c0 + i] : 0.f);
    }
    store_vec(out + (size_t)row * ldo + c0, o);
}

// Many rows (prompt portions), conv length KK <= 4: a thread takes its V channels through CONV_ROWS consecutive
// rows, keeping the last KK-1 products B*X and the channel weights in registers, so every input is read once
// (the kernel above reads each row KK times).  The history of a chunk's first rows comes from the rows before
// it or, at the head of a segment, from the state; the order of summation is that of the kernels above.
#define CONV_ROWS 8
template <typename T, int KK>
__global__ void __launch_bounds__(128)
shortconv_fwd_rows_kernel(const T* __restrict__ p, int ldp, const float* __restrict__ w,
                          const float* __restrict__ bias, const float* __restrict__ state,
                          const int* __restrict__ row_seg, const int* __restrict__ cu_rows,
                          const int* __restrict__ seg_pos, const int* __restrict__ seg_slot,
                          T* __restrict__ out, int ldo, int n, int d) {
    kp_pdl_begin();
    constexpr int V = ConvVec<T>::N;
    const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    const int row_lo = blockIdx.y * CONV_ROWS;
    if (c0 >= d || row_lo >= n) return;
    const int row_hi = min(n, row_lo + CONV_ROWS);
    float wk[KK][V], bs[V];
#pragma unroll
    for (int i = 0; i < V; i++) {
#pragma unroll
        for (int k = 0; k < KK; k++) wk[k][i] = w[(size_t)(c0 + i) * KK + k];
        bs[i] = bias ? bias[c0 + i] : 0.f;
    }
    float hist[KK - 1][V];                              // B*X of the KK-1 rows before the current one (oldest first)
#pragma unroll
    for (int k = 0; k < KK - 1; k++) {
        const int r = row_lo - (KK - 1) + k;
        if (r >= 0) {
            float hb[V], hx[V];
            load_vec<T>(p + (size_t)r * ldp + c0, hb);
            load_vec<T>(p + (size_t)r * ldp + 2 * (size_t)d + c0, hx);
#pragma unroll
            for (int i = 0; i < V; i++) hist[k][i] = __fmul_rn(hb[i], hx[i]);
        } else {
#pragma unroll
            for (int i = 0; i < V; i++) hist[k][i] = 0.f;
        }
    }
#pragma unroll 2
    for (int row = row_lo; row < row_hi; row++) {
        const int seg = row_seg[row];
        const int t = row - cu_rows[seg];
        const T* pr = p + (size_t)row * ldp;
        float bv[V], cv[V], xv[V], bx[V], sum[V];
        load_vec<T>(pr + c0, bv);
        load_vec<T>(pr + d + c0, cv);
        load_vec<T>(pr + 2 * (size_t)d + c0, xv);
#pragma unroll
        for (int i = 0; i < V; i++) bx[i] = __fmul_rn(bv[i], xv[i]);
        if (t < KK - 1) {
            // the head of a segment: rows before it belong to another request; the history is the state (or zero)
            const bool fresh = seg_pos[seg] == 0;
            const float* st = state + (size_t)seg_slot[seg] * (KK - 1) * d;
#pragma unroll
            for (int k = 0; k < KK - 1; k++) {
                const int st_t = t - (KK - 1) + k;
                if (st_t < 0) {
#pragma unroll
                    for (int i = 0; i < V; i++) hist[k][i] = fresh ? 0.f : st[(size_t)(KK - 1 + st_t) * d + c0 + i];
                }
            }
        }
        if (KK != 3) {
#pragma unroll
            for (int i = 0; i < V; i++) sum[i] = tap(bx[i], wk[KK - 1][i]);
#pragma unroll
            for (int k = 0; k < KK - 1; k++)
#pragma unroll
                for (int i = 0; i < V; i++) sum[i] = add_tap(sum[i], hist[k][i], wk[k][i]);
        } else {
#pragma unroll
            for (int i = 0; i < V; i++) sum[i] = conv_sum3(hist[0][i], hist[1][i], bx[i], wk[0][i], wk[1][i], wk[2][i]);
        }
        float o[V];
#pragma unroll
        for (int i = 0; i < V; i++) o[i] = gate_out(cv[i], sum[i], bias != nullptr, bs[i]);
        store_vec(out + (size_t)row * ldo + c0, o);
#pragma unroll
        for (int k = 0; k + 1 < KK - 1; k++)
#pragma unroll
            for (int i = 0; i < V; i++) hist[k][i] = hist[k + 1][i];
#pragma unroll
        for (int i = 0; i < V; i++) hist[KK - 2][i] = bx[i];
    }
}

// Every segment is one row (a decode step): output and new state by the same
// thread, so one launch does both.  Row r belongs to segment r.
template <typename T>
__global__ void shortconv_decode_kernel(const T* __restrict__ p, int ldp, const float* __restrict__ w,
                                        const float* __restrict__ bias, float* __restrict__ state,
                                        const int* __restrict__ seg_pos, const int* __restrict__ seg_slot,
                                        T* __restrict__ out, int ldo, int n, int d, int K) {
    kp_pdl_begin_early_if(n > 1);
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int row = blockIdx.y;
    if (c >= d || row >= n) return;
    const bool fresh = seg_pos[row] == 0;
    float* st = state + (size_t)seg_slot[row] * (K - 1) * d;
    const float* wc = w + (size_t)c * K;
    const float bx = bx_of(p, row, ldp, d, c);
    float hist[KP_CONV_MAX_K - 1];
    for (int k = 0; k < K - 1; k++) hist[k] = fresh ? 0.f : st[(size_t)k * d + c];
    float sum;
    if (K == 3) {
        sum = conv_sum3(hist[0], hist[1], bx, wc[0], wc[1], wc[2]);
    } else {
        sum = tap(bx, wc[K - 1]);
        for (int k = 0; k < K - 1; k++) sum = add_tap(sum, hist[k], wc[k]);
    }
    out[(size_t)row * ldo + c] = from_f32<T>(gate_out(to_f32(p[(size_t)row * ldp + d + c]), sum, bias != nullptr,
                                                      bias ? bias[c] : 0.f));
    for (int k = 0; k + 1 < K - 1; k++) st[(size_t)k * d + c] = hist[k + 1];
    st[(size_t)(K - 2) * d + c] = bx;
}

extern "C" {

int kp_shortconv_decode(const void* p, int ldp, const float* w, const float* bias, float* state, const int* seg_pos,
                        const int* seg_slot, void* out, int ldo, int n, int d, int K, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (K < 2 || K > KP_CONV_MAX_K || n > 65535) return KP_ERR_UNSUPPORTED;
    dim3 grid((d + 127) / 128, n);
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(shortconv_decode_kernel<T>, dim3(grid), dim3(128), 0, (cudaStream_t)stream, 
        (const T*)p, ldp, w, bias, state, seg_pos, seg_slot, (T*)out, ldo, n, d, K)));
    return kp_launch_status();
}

int kp_shortconv_forward(const void* p, int ldp, const float* w, const float* bias, const float* state,
                         const int* row_seg, const int* cu_rows, const int* seg_pos, const int* seg_slot,
                         void* out, int ldo, int n, int d, int K, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (K < 2 || K > KP_CONV_MAX_K) return KP_ERR_UNSUPPORTED;
    if (n > 65535 * 32) return KP_ERR_UNSUPPORTED;
    if (n > 65535) return KP_ERR_UNSUPPORTED;
    {
        // 16-byte path: which kernel runs depends on sizes and alignment only, and both sum in the same order
        const int vec = dtype == KP_DTYPE_BF16 ? 8 : 4;
        const size_t esz = dtype == KP_DTYPE_BF16 ? 2 : 4;
        if (d % vec == 0 && ldp % vec == 0 && ldo % vec == 0 && (((uintptr_t)p | (uintptr_t)out) & 15) == 0 && esz) {
            if (K <= 4) {
                // which kernel runs depends on the layer's sizes and alignment only, never on the batch
                dim3 rgrid((d / vec + 127) / 128, (n + CONV_ROWS - 1) / CONV_ROWS);
#define CONV_ROWS_LAUNCH(KK)                                                                                       \
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(shortconv_fwd_rows_kernel<T, KK>, dim3(rgrid), dim3(128), 0,         \
        (cudaStream_t)stream, (const T*)p, ldp, w, bias, state, row_seg, cu_rows, seg_pos, seg_slot, (T*)out, ldo, n, d)))
                if (K == 2) { CONV_ROWS_LAUNCH(2); } else if (K == 3) { CONV_ROWS_LAUNCH(3); } else { CONV_ROWS_LAUNCH(4); }
#undef CONV_ROWS_LAUNCH
                return kp_launch_status();
            }
            dim3 vgrid((d / vec + 127) / 128, n);
            KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(shortconv_fwd_vec_kernel<T>, dim3(vgrid), dim3(128), 0, (cudaStream_t)stream,
                (const T*)p, ldp, w, bias, state, row_seg, cu_rows, seg_pos, seg_slot, (T*)out, ldo, n, d, K)));
            return kp_launch_status();
        }
    }
    dim3 grid((d + 127) / 128, n);
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(shortconv_fwd_kernel<T>, dim3(grid), dim3(128), 0, (cudaStream_t)stream, 
        (const T*)p, ldp, w, bias, state, row_seg, cu_rows, seg_pos, seg_slot, (T*)out, ldo, n, d, K)));
    return kp_launch_status();
}

int kp_shortconv_update_state(const void* p, int ldp, float* state, const int* cu_rows, const int* seg_pos,
                              const int* seg_slot, int n_seg, int d, int K, int dtype, void* stream) {
    if (n_seg <= 0) return 0;
    if (K < 2 || K > KP_CONV_MAX_K || n_seg > 65535) return KP_ERR_UNSUPPORTED;
    dim3 grid((d + 127) / 128, n_seg);
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(shortconv_state_kernel<T>, dim3(grid), dim3(128), 0, (cudaStream_t)stream, 
        (const T*)p, ldp, state, cu_rows, seg_pos, seg_slot, n_seg, d, K)));
    return kp_launch_status();
}

}  // extern "C"
