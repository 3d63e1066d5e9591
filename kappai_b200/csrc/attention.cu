// Causal GQA attention of a batch of rows over the paged cache.
//
// For the row at position p of a request, head h reads kv head g = h / (H/G)
// and the keys t in [max(0, p - window + 1), p] (window <= 0: all keys):
//   s_t = (q . K_t) * scale ;  out = sum_t softmax(s)_t V_t
// (src/backend/cpu/scalar/core.c:383-433: online softmax with running max M,
// sum S and rescaled accumulator).  Keys are found through the request's
// block table: key t lies in page table[t / page_size] at offset t % page_size
// of the layer's cache [page][K|V][G][page_size][hd].  The keys of the rows of
// this very step were written before this kernel runs, so a prompt portion
// sees the earlier pages and its own rows alike.
//
// General kernel (any head_dim that is a multiple of 2 up to 256, any H, G,
// page size, window): one block per (head, row), 128 keys per tile, float32
// statistics.  Tiles start at multiples of 128 of the absolute key index, so
// the order of summation does not depend on how a prompt was cut.
#include "common.cuh"

#define ATT_THREADS 128
#define KP_MAX_HEAD_DIM 256

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
attention_rows_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ cache,
                      const int* __restrict__ block_table, int max_blocks, const int* __restrict__ row_seg,
                      const int* __restrict__ positions, T* __restrict__ out, int ldo, float scale, int window,
                      int page_size, int H, int G, int hd) {
    kp_pdl_begin();
    __shared__ float qs[KP_MAX_HEAD_DIM];
    __shared__ float ps[ATT_THREADS];
    __shared__ float red[32];
    const int tid = threadIdx.x;
    const int h = blockIdx.x, row = blockIdx.y;
    const int g = h / (H / G);
    const int pos = positions[row];
    const int* bt = block_table + (size_t)row_seg[row] * max_blocks;
    const int k_lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int k_hi = pos;
    const size_t page_stride = (size_t)2 * G * page_size * hd;   // elements per page (K and V)
    const size_t k_off = (size_t)g * page_size * hd;
    const size_t v_off = ((size_t)G + g) * page_size * hd;

    for (int i = tid; i < hd; i += ATT_THREADS) qs[i] = to_f32(q[(size_t)row * ldq + (size_t)h * hd + i]);
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc0 = 0.f, acc1 = 0.f;
    for (int tile0 = (k_lo / ATT_THREADS) * ATT_THREADS; tile0 <= k_hi; tile0 += ATT_THREADS) {
        const int key = tile0 + tid;
        const bool valid = key >= k_lo && key <= k_hi;
        float s = -INFINITY;
        if (valid) {
            const T* kp = cache + (size_t)bt[key / page_size] * page_stride + k_off + (size_t)(key % page_size) * hd;
            float dot = 0.f;
            for (int i = 0; i < hd; i++) dot = fmaf(qs[i], to_f32(kp[i]), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, block_max(s, red));
        const float pe = valid ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float tsum = block_sum(pe, red);
        l = l * corr + tsum;
        __syncthreads();
        ps[tid] = pe;
        __syncthreads();
        acc0 *= corr;
        acc1 *= corr;
        const int kk_lo = max(k_lo - tile0, 0);
        const int kk_hi = min(k_hi - tile0, ATT_THREADS - 1);
        for (int kk = kk_lo; kk <= kk_hi; kk++) {
            const int key2 = tile0 + kk;
            const T* vp = cache + (size_t)bt[key2 / page_size] * page_stride + v_off + (size_t)(key2 % page_size) * hd;
            const float pv = ps[kk];
            if (tid < hd) acc0 = fmaf(pv, to_f32(vp[tid]), acc0);
            if (tid + ATT_THREADS < hd) acc1 = fmaf(pv, to_f32(vp[tid + ATT_THREADS]), acc1);
        }
        m = m_new;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T* o = out + (size_t)row * ldo + (size_t)h * hd;
    if (tid < hd) o[tid] = from_f32<T>(acc0 * inv);
    if (tid + ATT_THREADS < hd) o[tid + ATT_THREADS] = from_f32<T>(acc1 * inv);
}

extern "C" int kp_attention_rows(const void* q, int ldq, const void* cache, const int* block_table, int max_blocks,
                                 const int* row_seg, const int* positions, void* out, int ldo, float scale,
                                 int window, int page_size, int n, int H, int G, int hd, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (hd < 2 || hd > KP_MAX_HEAD_DIM) return KP_ERR_UNSUPPORTED;
    if (G < 1 || H % G != 0 || page_size < 1) return KP_ERR_BAD_ARG;
    if (n > 65535) return KP_ERR_UNSUPPORTED;
    dim3 grid(H, n);
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(attention_rows_kernel<T>, dim3(grid), dim3(ATT_THREADS), 0, (cudaStream_t)stream, 
        (const T*)q, ldq, (const T*)cache, block_table, max_blocks, row_seg, positions, (T*)out, ldo, scale, window,
        page_size, H, G, hd)));
    return kp_launch_status();
}
