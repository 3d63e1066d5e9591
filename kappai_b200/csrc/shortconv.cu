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
    return to_f32(r[c]) * to_f32(r[2 * (size_t)d + c]);
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
        sum = hist[0] * wc[0] + hist[1] * wc[1] + bx * wc[2];      // src/backend/cpu/common.c:2411
    } else {
        sum = bx * wc[K - 1];                                      // src/backend/cpu/common.c:2422-2424
        for (int k = 0; k < K - 1; k++) sum += hist[k] * wc[k];
    }
    if (bias) sum += bias[c];
    out[(size_t)row * ldo + c] = from_f32<T>(to_f32(p[(size_t)row * ldp + d + c]) * sum);
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

// Every segment is one row (a decode step): output and new state by the same
// thread, so one launch does both.  Row r belongs to segment r.
template <typename T>
__global__ void shortconv_decode_kernel(const T* __restrict__ p, int ldp, const float* __restrict__ w,
                                        const float* __restrict__ bias, float* __restrict__ state,
                                        const int* __restrict__ seg_pos, const int* __restrict__ seg_slot,
                                        T* __restrict__ out, int ldo, int n, int d, int K) {
    kp_pdl_begin();
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
        sum = hist[0] * wc[0] + hist[1] * wc[1] + bx * wc[2];
    } else {
        sum = bx * wc[K - 1];
        for (int k = 0; k < K - 1; k++) sum += hist[k] * wc[k];
    }
    if (bias) sum += bias[c];
    out[(size_t)row * ldo + c] = from_f32<T>(to_f32(p[(size_t)row * ldp + d + c]) * sum);
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
    dim3 grid((d + 127) / 128, n);
    if (n > 65535) return KP_ERR_UNSUPPORTED;
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
