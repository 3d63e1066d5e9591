// Split-KV attention for rows that each read a long cache (decode steps and
// very short portions): the keys of one (row, kv head) are cut into chunks of
// 256 at multiples of 256 of the absolute key index; one CTA per (chunk, kv
// head, row) computes, for all R = H/G query heads that share the kv head, the
// chunk's scores, its maximum m, its sum l of exp(s - m) and the unnormalised
// sum of exp(s - m) V; a second kernel merges the chunks of a row in order.
// Same formulas as attention.cu (src/backend/cpu/scalar/core.c:383-433); the
// chunk grid does not depend on the batch, so neither does the result.
//
// Scratch (global memory beyond inputs and outputs, given by the caller):
//   part_acc [n_rows][H][n_chunks][hd] float, part_ml [n_rows][H][n_chunks][2] float.
// Only the chunks that intersect a row's key range are written and read.
#include "common.cuh"

#define AD_CHUNK 256
#define AD_THREADS 256
#define AD_RMAX 8
#define KP_MAX_HEAD_DIM 256

template <typename T> struct Vec16;
template <> struct Vec16<bf16> { static constexpr int N = 8; };
template <> struct Vec16<float> { static constexpr int N = 4; };

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& v, float* f);
template <>
__device__ __forceinline__ void unpack16<bf16>(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void unpack16<float>(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}

__device__ __forceinline__ void key_range(int pos, int window, int& k_lo, int& k_hi) {
    k_lo = window > 0 ? max(0, pos - window + 1) : 0;
    k_hi = pos;
}

// HD, RR: head size and query heads per kv head fixed at compile time (loops unroll, loads overlap);
// 0 means "taken from the arguments".
template <typename T, int HD, int RR>
__global__ void __launch_bounds__(AD_THREADS)
attn_split_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ cache, const int* __restrict__ block_table,
                  int max_blocks, const int* __restrict__ row_seg, const int* __restrict__ positions,
                  float* __restrict__ part_acc, float* __restrict__ part_ml, int n_chunks, float scale, int window,
                  int page_size, int H, int G, int hd_rt) {
    kp_pdl_begin();
    extern __shared__ float smem[];
    const int hd = HD ? HD : hd_rt;
    const int R = RR ? RR : H / G;
    float* qs = smem;                              // [R][hd]
    float* ps = qs + R * hd;                       // [R][AD_CHUNK]
    float* red = ps + R * AD_CHUNK;                // [n_slices][R][hd]  (also used for the small reductions)
    __shared__ float wred[AD_THREADS / 32][AD_RMAX];
    __shared__ float stat_m[AD_RMAX], stat_l[AD_RMAX];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk = blockIdx.x, g = blockIdx.y, row = blockIdx.z;
    int k_lo, k_hi;
    key_range(positions[row], window, k_lo, k_hi);
    const int c0 = chunk * AD_CHUNK;
    if (c0 > k_hi || c0 + AD_CHUNK - 1 < k_lo) return;          // the chunk holds none of this row's keys
    const int* bt = block_table + (size_t)row_seg[row] * max_blocks;
    const size_t page_stride = (size_t)2 * G * page_size * hd;
    const size_t k_off = (size_t)g * page_size * hd, v_off = ((size_t)G + g) * page_size * hd;

    for (int i = tid; i < R * hd; i += AD_THREADS)
        qs[i] = to_f32(q[(size_t)row * ldq + (size_t)(g * R) * hd + i]);
    __syncthreads();

    // (head size 64, 16-bit cache) the values this thread multiplies later are fetched now, so that their
    // latency passes under the scores and the softmax: thread = (pair of dims, slice of 32 keys)
    constexpr bool PREFETCH_V = (HD == 64) && (sizeof(T) == 2);
    uint32_t vpre[PREFETCH_V ? 32 : 1];
    if (PREFETCH_V) {
        const int pair_p = tid & 31, slice_p = tid >> 5;
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const int key2 = c0 + slice_p * 32 + j;
            uint32_t v = 0;
            if (key2 >= k_lo && key2 <= k_hi)
                v = *reinterpret_cast<const uint32_t*>(cache + (size_t)bt[key2 / page_size] * page_stride + v_off +
                                                       (size_t)(key2 % page_size) * hd + 2 * pair_p);
            vpre[j] = v;
        }
    }

    // scores: one key a thread, all R heads
    const int key = c0 + tid;
    const bool valid = key >= k_lo && key <= k_hi;
    float s[AD_RMAX];
#pragma unroll
    for (int r = 0; r < AD_RMAX; r++) s[r] = 0.f;
    if (valid) {
        const T* kp = cache + (size_t)bt[key / page_size] * page_stride + k_off + (size_t)(key % page_size) * hd;
        constexpr int VN = Vec16<T>::N;
#pragma unroll
        for (int i = 0; i < hd; i += VN) {
            float kf[VN];
            unpack16<T>(*reinterpret_cast<const uint4*>(kp + i), kf);
#pragma unroll
            for (int r = 0; r < AD_RMAX; r++) {
                if (r < R) {
                    const float* qr = qs + r * hd + i;
#pragma unroll
                    for (int j = 0; j < VN; j++) s[r] = fmaf(qr[j], kf[j], s[r]);
                }
            }
        }
    }
    // per head: chunk maximum, exp, chunk sum
#pragma unroll
    for (int r = 0; r < AD_RMAX; r++) {
        if (r < R) {
            s[r] = valid ? s[r] * scale : -INFINITY;
            const float m = warp_max(s[r]);
            if (lane == 0) wred[warp][r] = m;
        }
    }
    __syncthreads();
    if (tid < R) {
        float m = wred[0][tid];
        for (int w = 1; w < AD_THREADS / 32; w++) m = fmaxf(m, wred[w][tid]);
        stat_m[tid] = m;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < AD_RMAX; r++) {
        if (r < R) {
            const float p = valid ? expf(s[r] - stat_m[r]) : 0.f;
            ps[r * AD_CHUNK + tid] = p;
            const float l = warp_sum(p);
            if (lane == 0) wred[warp][r] = l;
        }
    }
    __syncthreads();
    if (tid < R) {
        float l = 0.f;
        for (int w = 0; w < AD_THREADS / 32; w++) l += wred[w][tid];
        stat_l[tid] = l;
    }

    // P V: thread = (pair of dims, slice of keys); slices are summed in order afterwards
    const int pairs = hd >> 1;
    const int n_slices = AD_THREADS / pairs;
    const int per = (AD_CHUNK + n_slices - 1) / n_slices;
    const int pair = tid % pairs, slice = tid / pairs;
    float acc[AD_RMAX][2];
#pragma unroll
    for (int r = 0; r < AD_RMAX; r++) acc[r][0] = acc[r][1] = 0.f;
    if (PREFETCH_V) {
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const int kk = slice * 32 + j;                       // keys outside the row's range have p = 0
            const float v0 = __uint_as_float(vpre[j] << 16), v1 = __uint_as_float(vpre[j] & 0xffff0000u);
#pragma unroll
            for (int r = 0; r < AD_RMAX; r++) {
                if (r < R) {
                    const float p = ps[r * AD_CHUNK + kk];
                    acc[r][0] = fmaf(p, v0, acc[r][0]);
                    acc[r][1] = fmaf(p, v1, acc[r][1]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < AD_RMAX; r++) {
            if (r < R) {
                red[((size_t)slice * R + r) * hd + 2 * pair] = acc[r][0];
                red[((size_t)slice * R + r) * hd + 2 * pair + 1] = acc[r][1];
            }
        }
    } else if (slice < n_slices) {
        const int kk_lo = max(slice * per, k_lo - c0), kk_hi = min(min((slice + 1) * per, AD_CHUNK) - 1, k_hi - c0);
#pragma unroll 8
        for (int kk = kk_lo; kk <= kk_hi; kk++) {
            const int key2 = c0 + kk;
            const T* vp = cache + (size_t)bt[key2 / page_size] * page_stride + v_off +
                          (size_t)(key2 % page_size) * hd + 2 * pair;
            const float v0 = to_f32(vp[0]), v1 = to_f32(vp[1]);
#pragma unroll
            for (int r = 0; r < AD_RMAX; r++) {
                if (r < R) {
                    const float p = ps[r * AD_CHUNK + kk];
                    acc[r][0] = fmaf(p, v0, acc[r][0]);
                    acc[r][1] = fmaf(p, v1, acc[r][1]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < AD_RMAX; r++) {
            if (r < R) {
                red[((size_t)slice * R + r) * hd + 2 * pair] = acc[r][0];
                red[((size_t)slice * R + r) * hd + 2 * pair + 1] = acc[r][1];
            }
        }
    }
    __syncthreads();
    for (int e = tid; e < R * hd; e += AD_THREADS) {
        const int r = e / hd, d = e % hd;
        float v = 0.f;
        for (int sl = 0; sl < n_slices; sl++) v += red[((size_t)sl * R + r) * hd + d];
        part_acc[(((size_t)row * H + g * R + r) * n_chunks + chunk) * hd + d] = v;
    }
    if (tid < R) {
        float* ml = part_ml + (((size_t)row * H + g * R + tid) * n_chunks + chunk) * 2;
        ml[0] = stat_m[tid];
        ml[1] = stat_l[tid];
    }
}

#define MERGE_THREADS 256
#define MERGE_BATCH 4096                                    // floats of accumulators in shared memory at a time

// The chunks of a row and head put together: out = sum_c acc_c * exp(m_c - m) / sum_c l_c * exp(m_c - m), the
// sums in chunk order.  One CTA a (head, row).  The statistics of the row's chunks and the weights
// exp(m_c - m) are brought into shared memory once by all threads together; only the sums themselves run
// chunk by chunk (a context of 32k tokens has 128 chunks: with every thread walking global memory three times
// for them the merge took longer than half of the attention itself).
template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                  const int* __restrict__ positions, T* __restrict__ out, int ldo, int n_chunks,
                                  int chunk_keys, int window, int H, int hd) {
    kp_pdl_begin_early_if(gridDim.y > 1);
    extern __shared__ __align__(16) float merge_sm[];       // [MERGE_BATCH], [n_chunks] l_c, [n_chunks] exp(m_c - m), [32]
    const int h = blockIdx.x, row = blockIdx.y, tid = threadIdx.x, nt = blockDim.x;
    int k_lo, k_hi;
    key_range(positions[row], window, k_lo, k_hi);
    // (a position beyond the chunks the caller gave is the caller's fault; the clamp keeps the reads inside
    // the scratch and the shared arrays all the same)
    const int c_hi = min(k_hi / chunk_keys, n_chunks - 1), c_lo = min(k_lo / chunk_keys, c_hi), n = c_hi - c_lo + 1;
    float* s_acc = merge_sm;
    float* s_l = merge_sm + MERGE_BATCH;
    float* s_w = s_l + n_chunks;
    float* s_red = s_w + n_chunks;
    // the accumulators: brought in batches of MERGE_BATCH floats by all threads (every load of a batch in
    // flight at once), then added chunk by chunk by the thread of each dimension
    const float* pa = part_acc + (((size_t)row * H + h) * n_chunks + c_lo) * hd;
    const int mb = MERGE_BATCH / hd;                        // chunks a batch
    constexpr int PER = MERGE_BATCH / 4 / MERGE_THREADS;    // float4 a thread and batch
    float4 reg[PER];
    auto fetch = [&](int c0) {                              // the batch from chunk c0 on, into registers
        const int nb = min(mb, n - c0);
#pragma unroll
        for (int k = 0; k < PER; k++) {
            const int i = (k * MERGE_THREADS + tid) * 4;
            if (i < nb * hd) reg[k] = *reinterpret_cast<const float4*>(pa + (size_t)c0 * hd + i);
        }
    };
    fetch(0);                                               // under way while the statistics are worked out
    const float* ml = part_ml + (((size_t)row * H + h) * n_chunks + c_lo) * 2;
    float m = -INFINITY;
    for (int c = tid; c < n; c += nt) {
        const float2 v = *reinterpret_cast<const float2*>(ml + 2 * c);
        s_w[c] = v.x;                                       // m_c for now
        s_l[c] = v.y;
        m = fmaxf(m, v.x);
    }
    m = warp_max(m);
    if ((tid & 31) == 0) s_red[tid >> 5] = m;
    __syncthreads();
    m = -INFINITY;
    for (int w = 0; w < (nt + 31) / 32; w++) m = fmaxf(m, s_red[w]);
    for (int c = tid; c < n; c += nt) s_w[c] = expf(s_w[c] - m);
    __syncthreads();
    float l = 0.f;
    for (int c = 0; c < n; c++) l = __fmaf_rn(s_l[c], s_w[c], l);
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    float v = 0.f;
    for (int c0 = 0; c0 < n; c0 += mb) {
        const int nb = min(mb, n - c0);
#pragma unroll
        for (int k = 0; k < PER; k++) {
            const int i = (k * MERGE_THREADS + tid) * 4;
            if (i < nb * hd) *reinterpret_cast<float4*>(s_acc + i) = reg[k];
        }
        __syncthreads();
        if (c0 + mb < n) fetch(c0 + mb);                    // the next batch is under way while this one is added
        if (tid < hd)
            for (int j = 0; j < nb; j++) v = fmaf(s_acc[j * hd + tid], s_w[c0 + j], v);
        __syncthreads();
    }
    if (tid < hd) out[(size_t)row * ldo + (size_t)h * hd + tid] = from_f32<T>(v * inv);
}

// The same for rows of at most 64 chunks (16k keys), one warp a (head, row) and no shared memory: the lanes
// hold the chunks' statistics and weights and pass them round, every lane sums its dimensions (lane, lane + 32,
// ...) chunk by chunk.  The arithmetic is that of the kernel above, so a row's result does not depend on which
// of the two ran.  (With 64 rows the kernel above took 10.7 us for 2048 small CTAs of 256 threads.)
#define MERGE_WARP_CHUNKS 64
#define MERGE_WARP_BLOCK 16                               // chunks whose sums a warp fetches at a time
template <typename T>
__global__ void attn_merge_warp_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                       const int* __restrict__ positions, T* __restrict__ out, int ldo, int n_chunks,
                                       int chunk_keys, int window, int H, int hd, int n_rows) {
    kp_pdl_begin_early_if(n_rows > 1);
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);          // (row, head)
    if (item >= n_rows * H) return;
    const int row = item / H, h = item - row * H;
    int k_lo, k_hi;
    key_range(positions[row], window, k_lo, k_hi);
    const int c_hi = min(k_hi / chunk_keys, n_chunks - 1), c_lo = min(k_lo / chunk_keys, c_hi), n = c_hi - c_lo + 1;
    const float* pa = part_acc + (((size_t)row * H + h) * n_chunks + c_lo) * hd;
    const float* ml = part_ml + (((size_t)row * H + h) * n_chunks + c_lo) * 2;
    // the sums of the first MERGE_WARP_BLOCK chunks are on their way while the statistics are worked out
    constexpr int B = MERGE_WARP_BLOCK;
    float a[B][4];
    auto fetch = [&](int c0) {
#pragma unroll
        for (int j = 0; j < B; j++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int d = lane + 32 * i;
                a[j][i] = (c0 + j < n && d < hd) ? pa[(size_t)(c0 + j) * hd + d] : 0.f;
            }
    };
    fetch(0);
    float m0 = -INFINITY, l0 = 0.f, m1 = -INFINITY, l1 = 0.f;                       // chunks lane and lane + 32
    if (lane < n) { const float2 v = *reinterpret_cast<const float2*>(ml + 2 * lane); m0 = v.x; l0 = v.y; }
    if (lane + 32 < n) { const float2 v = *reinterpret_cast<const float2*>(ml + 2 * (lane + 32)); m1 = v.x; l1 = v.y; }
    const float m = warp_max(fmaxf(m0, m1));
    const float w0 = lane < n ? expf(m0 - m) : 0.f, w1 = lane + 32 < n ? expf(m1 - m) : 0.f;
    float l = 0.f, v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c0 = 0; c0 < n; c0 += B) {
        if (c0) fetch(c0);
#pragma unroll
        for (int j = 0; j < B; j++) {
            const int c = c0 + j;
            if (c < n) {                                                            // (the same for all lanes)
                const float wc = __shfl_sync(0xffffffffu, c < 32 ? w0 : w1, c & 31);
                const float lc = __shfl_sync(0xffffffffu, c < 32 ? l0 : l1, c & 31);
                l = __fmaf_rn(lc, wc, l);
#pragma unroll
                for (int i = 0; i < 4; i++) v[i] = fmaf(a[j][i], wc, v[i]);
            }
        }
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int d = lane + 32 * i;
        if (d < hd) out[(size_t)row * ldo + (size_t)h * hd + d] = from_f32<T>(v[i] * inv);
    }
}

static size_t merge_smem_bytes(int n_chunks) { return sizeof(float) * ((size_t)2 * n_chunks + 32 + MERGE_BATCH); }

template <typename T>
static int launch_merge(const float* part_acc, const float* part_ml, const int* positions, void* out, int ldo,
                        int n_chunks, int chunk_keys, int window, int n, int H, int hd, cudaStream_t s) {
    if (n_chunks <= MERGE_WARP_CHUNKS && hd <= 128) {
        const int warps = 8;
        kp_launch_pdl(attn_merge_warp_kernel<T>, dim3((n * H + warps - 1) / warps), dim3(warps * 32), 0, s, part_acc, part_ml,
                      positions, (T*)out, ldo, n_chunks, chunk_keys, window, H, hd, n);
        return kp_launch_status();
    }
    const size_t smem = merge_smem_bytes(n_chunks);
    if (smem > 200 * 1024) return KP_ERR_UNSUPPORTED;       // (25,000 chunks: 6.5 million keys)
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attn_merge_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (hd > MERGE_THREADS || (hd & 3)) return KP_ERR_UNSUPPORTED;
    kp_launch_pdl(attn_merge_kernel<T>, dim3(H, n), dim3(MERGE_THREADS), smem, s, part_acc, part_ml, positions, (T*)out, ldo,
                  n_chunks, chunk_keys, window, H, hd);
    return kp_launch_status();
}

static size_t split_smem_bytes(int R, int hd) {
    const int pairs = hd / 2;
    const int n_slices = AD_THREADS / pairs;
    return sizeof(float) * ((size_t)R * hd + (size_t)R * AD_CHUNK + (size_t)n_slices * R * hd);
}

extern "C" {

// Elements of float scratch the split kernel needs for these sizes (part_acc then part_ml).
long long kp_attention_split_scratch(int n_rows, int H, int hd, int n_chunks) {
    return (long long)n_rows * H * n_chunks * (hd + 2);
}

// n_chunks: chunks of 256 keys the grid covers; must reach the largest position in the batch.
int kp_attention_split(const void* q, int ldq, const void* cache, const int* block_table, int max_blocks,
                       const int* row_seg, const int* positions, void* out, int ldo, float* scratch, int n_chunks,
                       float scale, int window, int page_size, int n, int H, int G, int hd, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (hd < 16 || hd > KP_MAX_HEAD_DIM || (hd & 15)) return KP_ERR_UNSUPPORTED;
    if (G < 1 || H % G != 0 || H / G > AD_RMAX || page_size < 1 || n_chunks < 1) return KP_ERR_UNSUPPORTED;
    if (n > 65535 || G > 65535) return KP_ERR_UNSUPPORTED;
    const int R = H / G;
    const size_t smem = split_smem_bytes(R, hd);
    float* part_acc = scratch;
    float* part_ml = scratch + (size_t)n * H * n_chunks * hd;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_chunks, G, n);
#define AD_LAUNCH(T, HD, RR)                                                                                      \
    kp_launch_pdl(attn_split_kernel<T, HD, RR>, dim3(grid), dim3(AD_THREADS), smem, s, (const T*)q, ldq, (const T*)cache, block_table,       \
                                                                max_blocks, row_seg, positions, part_acc, part_ml,    \
                                                                n_chunks, scale, window, page_size, H, G, hd)
    KP_DISPATCH_DTYPE(dtype, T, {
        cudaError_t e0;
        if (hd == 64 && R == 4) e0 = AD_LAUNCH(T, 64, 4);
        else if (hd == 64) e0 = AD_LAUNCH(T, 64, 0);
        else if (hd == 128) e0 = AD_LAUNCH(T, 128, 0);
        else e0 = AD_LAUNCH(T, 0, 0);
        if (e0 != cudaSuccess) { cudaGetLastError(); return (int)e0; }      // the first launch that failed
        return launch_merge<T>(part_acc, part_ml, positions, out, ldo, n_chunks, AD_CHUNK, window, n, H, hd, s);
    });
#undef AD_LAUNCH
    return kp_launch_status();
}

// The merge alone, for partials of chunks of `chunk_keys` keys that another kernel wrote into `scratch` in the
// same format.
int kp_attention_merge(const int* positions, void* out, int ldo, const float* scratch, int n_chunks, int chunk_keys,
                       int window, int n, int H, int hd, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (hd < 16 || hd > KP_MAX_HEAD_DIM || n > 65535 || chunk_keys < 1) return KP_ERR_UNSUPPORTED;
    const float* part_acc = scratch;
    const float* part_ml = scratch + (size_t)n * H * n_chunks * hd;
    KP_DISPATCH_DTYPE(dtype, T, return launch_merge<T>(part_acc, part_ml, positions, out, ldo, n_chunks, chunk_keys, window,
                                                       n, H, hd, (cudaStream_t)stream));
    return kp_launch_status();
}

}  // extern "C"
