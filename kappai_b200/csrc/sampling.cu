// Sampling on the device: repeat penalty, greedy argmax, temperature sampling
// over the full vocabulary, and top-k / top-p / min-p filtered sampling.
//
// Semantics follow the reference's sampler (src/sampler.c:205-352):
//   penalty -> greedy if temperature <= 0 or top_k == 1 (:345-346)
//   -> no filter active: softmax(logits / T) over the whole vocabulary with the
//      sum in double, inverse CDF in index order (:234-258)
//   -> else keep the top_k largest (or the 1024 largest when only top_p /
//      min_p filter, :218-232), sorted descending; v_i = exp(l_i/T - max);
//      top-p: cut after the candidate whose cumulative probability first
//      exceeds p (:271-281); min-p: keep p_i >= min_p * p_0, at least one
//      (:283-291); draw by inverse CDF over the kept ones (:293-310).
//   argmax ties go to the lowest index (:125-136).
// The uniform number of each row is made on the host from (seed, request,
// step) and passed in, so a draw does not depend on the batch.
#include "common.cuh"

#define SAMPLE_THREADS 1024
#define SAMPLE_MAX_CAND 1024

__device__ __forceinline__ unsigned int order_key(float f) {
    unsigned int u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // ascending in the float order
}

// ---- repeat penalty: each occurrence of a token among `recent` divides a
// positive logit by the penalty or multiplies a non-positive one (:205-216)
__global__ void repeat_penalty_kernel(float* __restrict__ logits, int V, const int* __restrict__ recent,
                                      int max_recent, const float* __restrict__ penalty) {
    kp_pdl_begin();
    const int row = blockIdx.x;
    const float pen = penalty[row];
    if (pen == 1.0f) return;
    float* l = logits + (size_t)row * V;
    const int* r = recent + (size_t)row * max_recent;
    for (int i = threadIdx.x; i < max_recent; i += blockDim.x) {
        const int tok = r[i];
        if (tok < 0 || tok >= V) continue;
        bool first = true;
        for (int j = 0; j < i; j++)
            if (r[j] == tok) { first = false; break; }
        if (!first) continue;
        int m = 0;
        for (int j = i; j < max_recent; j++) m += (r[j] == tok);
        float v = l[tok];
        for (int k = 0; k < m; k++) v = v > 0.f ? v / pen : v * pen;
        l[tok] = v;
    }
}

// ---- block argmax with lowest index on ties
__device__ int block_argmax(const float* __restrict__ l, int V, float scale, float* s_val, int* s_idx,
                            float* out_max) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = l[i] * scale;
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        bv = lane < nw ? s_val[lane] : -INFINITY;
        bi = lane < nw ? s_idx[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { s_val[0] = bv; s_idx[0] = bi; }
    }
    __syncthreads();
    const int r = s_idx[0];
    if (out_max) *out_max = s_val[0];
    __syncthreads();
    return r == 0x7fffffff ? 0 : r;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                   const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
                   const float* __restrict__ uniform, int* __restrict__ out) {
    kp_pdl_begin();
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ double s_pref[SAMPLE_THREADS];
    __shared__ unsigned int s_hist[256];
    __shared__ float c_val[SAMPLE_MAX_CAND];
    __shared__ int c_idx[SAMPLE_MAX_CAND];
    __shared__ int s_cnt[SAMPLE_THREADS];
    __shared__ int s_cnt2[SAMPLE_THREADS];
    __shared__ unsigned int s_prefix, s_kleft;
    __shared__ int s_result;
    __shared__ double s_total;

    const int row = blockIdx.x, tid = threadIdx.x;
    const float* l = logits + (size_t)row * V;
    const float T = temperature[row];
    const int k_in = top_k[row];
    const float tp = top_p[row], mp = min_p[row];

    if (T <= 0.f || k_in == 1) {
        const int r = block_argmax(l, V, 1.0f, s_val, s_idx, nullptr);
        if (tid == 0) out[row] = r;
        return;
    }
    const float inv_t = 1.0f / T;
    const bool k_active = k_in > 0 && k_in < V;

    if (!k_active && tp >= 1.0f && mp <= 0.0f) {
        // full vocabulary
        float mx;
        block_argmax(l, V, inv_t, s_val, s_idx, &mx);
        const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
        const int b = tid * chunk, e = min(b + chunk, V);
        double loc = 0.0;
        for (int i = b; i < e; i++) loc += (double)expf(l[i] * inv_t - mx);
        s_pref[tid] = loc;
        __syncthreads();
        if (tid == 0) {
            double acc = 0.0;
            for (int t = 0; t < SAMPLE_THREADS; t++) { const double v = s_pref[t]; s_pref[t] = acc; acc += v; }
            s_result = -1;
            s_total = acc;         // s_pref now holds exclusive prefixes
        }
        __syncthreads();
        const double total = s_total;
        const double rnd = (double)uniform[row] * total;
        const double lo = s_pref[tid], hi = lo + loc;
        if (b < e && rnd >= lo && rnd < hi) {
            double acc = lo;
            int pick = e - 1;
            for (int i = b; i < e; i++) {
                acc += (double)expf(l[i] * inv_t - mx);
                if (rnd < acc) { pick = i; break; }
            }
            s_result = pick;      // intervals are disjoint: at most one thread gets here
        }
        __syncthreads();
        if (tid == 0) out[row] = s_result >= 0 ? s_result : V - 1;
        return;
    }

    // ---- candidates: the k largest, k = top_k or min(V, 1024)
    const int k = k_active ? k_in : min(V, SAMPLE_MAX_CAND);
    // radix select of the k-th largest key, one byte at a time from the top
    if (tid == 0) { s_prefix = 0; s_kleft = (unsigned)k; }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = tid; i < 256; i += blockDim.x) s_hist[i] = 0;
        __syncthreads();
        const unsigned int prefix = s_prefix;
        const unsigned int mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = tid; i < V; i += blockDim.x) {
            const unsigned int key = order_key(l[i]);
            if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            unsigned int left = s_kleft;
            int b = 255;
            for (; b > 0; b--) {
                if (s_hist[b] >= left) break;
                left -= s_hist[b];
            }
            s_prefix = prefix | ((unsigned)b << shift);
            s_kleft = left;
        }
        __syncthreads();
    }
    const unsigned int thr = s_prefix;      // key of the k-th largest; s_kleft of the keys equal to it are kept
    const int n_eq_keep = (int)s_kleft;
    // ordered compaction: keys > thr, then the first n_eq_keep keys == thr, both in index order
    {
        const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
        const int b = tid * chunk, e = min(b + chunk, V);
        int ng = 0, ne = 0;
        for (int i = b; i < e; i++) {
            const unsigned int key = order_key(l[i]);
            ng += key > thr;
            ne += key == thr;
        }
        s_cnt[tid] = ng;
        s_cnt2[tid] = ne;
        __syncthreads();
        if (tid == 0) {
            int a = 0, c = 0;
            for (int t = 0; t < SAMPLE_THREADS; t++) {
                const int x = s_cnt[t], y = s_cnt2[t];
                s_cnt[t] = a; s_cnt2[t] = c;
                a += x; c += y;
            }
            s_result = a;          // number of keys > thr
        }
        __syncthreads();
        const int n_gt = s_result;
        int pg = s_cnt[tid], pe = s_cnt2[tid];
        for (int i = b; i < e; i++) {
            const float v = l[i];
            const unsigned int key = order_key(v);
            if (key > thr) { c_val[pg] = v; c_idx[pg] = i; pg++; }
            else if (key == thr) {
                if (pe < n_eq_keep) { c_val[n_gt + pe] = v; c_idx[n_gt + pe] = i; }
                pe++;
            }
        }
        for (int i = k + tid; i < SAMPLE_MAX_CAND; i += blockDim.x) { c_val[i] = -INFINITY; c_idx[i] = 0x7fffffff; }
        __syncthreads();
    }
    // bitonic sort, descending by value, ascending index on ties
    for (int size = 2; size <= SAMPLE_MAX_CAND; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const int i = tid;
            const int j = i ^ stride;
            if (j > i) {
                const bool desc = (i & size) == 0;
                const float vi = c_val[i], vj = c_val[j];
                const int ii = c_idx[i], ij = c_idx[j];
                const bool i_before_j = vi > vj || (vi == vj && ii < ij);
                if (desc ? !i_before_j : i_before_j) {
                    c_val[i] = vj; c_val[j] = vi; c_idx[i] = ij; c_idx[j] = ii;
                }
            }
            __syncthreads();
        }
    }
    // the sequential tail of the reference, by one thread (at most 1024 candidates)
    if (tid == 0) {
        int kept = k;
        const float mx = c_val[0] * inv_t;
        float sum = 0.f;
        for (int i = 0; i < kept; i++) { c_val[i] = expf(c_val[i] * inv_t - mx); sum += c_val[i]; }
        if (tp < 1.0f) {
            float cum = 0.f;
            for (int i = 0; i < kept; i++) {
                cum += c_val[i] / sum;
                if (cum > tp) { kept = i + 1; break; }
            }
        }
        if (mp > 0.0f) {
            const float min_prob = mp * (c_val[0] / sum);
            int n = 0;
            while (n < kept && (c_val[n] / sum) >= min_prob) n++;
            kept = n > 0 ? n : 1;
        }
        float psum = 0.f;
        for (int i = 0; i < kept; i++) psum += c_val[i];
        const float rnd = uniform[row] * psum;
        float acc = 0.f;
        int pick = kept - 1;
        for (int i = 0; i < kept; i++) {
            acc += c_val[i];
            if (rnd < acc) { pick = i; break; }
        }
        out[row] = c_idx[pick];
    }
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_rows_kernel(const float* __restrict__ logits, int V, int* __restrict__ out) {
    kp_pdl_begin();
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    const int r = block_argmax(logits + (size_t)blockIdx.x * V, V, 1.0f, s_val, s_idx, nullptr);
    if (threadIdx.x == 0) out[blockIdx.x] = r;
}

// Two stages for large vocabularies: ARGMAX_SLICES blocks a row each find the best of their slice
// (lowest index on ties), then one warp a row picks the best slice (lowest slice on ties).
#define ARGMAX_SLICES 32
__global__ void __launch_bounds__(256)
argmax_slices_kernel(const float* __restrict__ logits, int V, float* __restrict__ part_val, int* __restrict__ part_idx) {
    kp_pdl_begin();
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    const int row = blockIdx.y, sl = blockIdx.x;
    const int per = (V + ARGMAX_SLICES - 1) / ARGMAX_SLICES;
    const int b = sl * per, e = min(b + per, V);
    float mx;
    int r = 0x7fffffff;
    if (b < e) r = b + block_argmax(logits + (size_t)row * V + b, e - b, 1.0f, s_val, s_idx, &mx);
    if (threadIdx.x == 0) {
        part_val[row * ARGMAX_SLICES + sl] = b < e ? mx : -INFINITY;
        part_idx[row * ARGMAX_SLICES + sl] = r;
    }
}
__global__ void argmax_final_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx,
                                    int* __restrict__ out) {
    kp_pdl_begin();
    const int row = blockIdx.x, lane = threadIdx.x;
    float bv = part_val[row * ARGMAX_SLICES + lane];
    int bi = part_idx[row * ARGMAX_SLICES + lane];
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

extern "C" {

// scratch: n * 32 floats then n * 32 ints, or null (one block a row; for small vocabularies)
int kp_argmax_rows(const float* logits, int n, int V, int* out, void* scratch, void* stream) {
    if (n <= 0) return 0;
    if (V < 1) return KP_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (scratch == nullptr || V < 8192 || n > 65535) {
        kp_launch_pdl(argmax_rows_kernel, dim3(n), dim3(SAMPLE_THREADS), 0, s, logits, V, out);
    } else {
        float* pv = (float*)scratch;
        int* pi = (int*)(pv + (size_t)n * ARGMAX_SLICES);
        kp_launch_pdl(argmax_slices_kernel, dim3(dim3(ARGMAX_SLICES, n)), dim3(256), 0, s, logits, V, pv, pi);
        kp_launch_pdl(argmax_final_kernel, dim3(n), dim3(32), 0, s, pv, pi, out);
    }
    return kp_launch_status();
}

int kp_repeat_penalty(float* logits, int n, int V, const int* recent, int max_recent, const float* penalty,
                      void* stream) {
    if (n <= 0 || max_recent <= 0) return 0;
    kp_launch_pdl(repeat_penalty_kernel, dim3(n), dim3(128), 0, (cudaStream_t)stream, logits, V, recent, max_recent, penalty);
    return kp_launch_status();
}

// top_k > 1024 (and < V) is refused.  The host checks it per row before the call.
int kp_sample_rows(const float* logits, int n, int V, const float* temperature, const int* top_k, const float* top_p,
                   const float* min_p, const float* uniform, int* out, void* stream) {
    if (n <= 0) return 0;
    if (V < 1) return KP_ERR_BAD_ARG;
    kp_launch_pdl(sample_rows_kernel, dim3(n), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, logits, V, temperature, top_k, top_p, min_p,
                                                                       uniform, out);
    return kp_launch_status();
}

}  // extern "C"
