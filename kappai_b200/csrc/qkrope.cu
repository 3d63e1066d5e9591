// Fused per-head RMSNorm of q and k, rotary position encoding, and the write
// of k and v into the paged cache.
//
// Input rows hold [q: H*hd | k: G*hd | v: G*hd].  For each q and k head
//   x <- (x * rsqrt(mean(x^2) + eps)) * w          (src/backend/cpu/scalar/quants.c:1521-1531)
// then, for j < rot/2 with c,s = cos,sin(pos * theta^(-2j/rot)) from a table
// built in double precision (src/compute.c:22-65):
//   neox pairing (j, j + rot/2), interleaved pairing (2j, 2j+1):
//   (a, b) <- (a c - b s, a s + b c)               (src/backend/cpu/quants.h:395-409)
// q goes to q_out; k and v go to the page and offset given by slot_map
// (cache layout [page][K|V][G][page_size][hd]; src/backend/cpu/common.c:1603-1694
// stores the same rows at [layer][kv head][pos][hd]).
// Norm (w == nullptr) and rotation (cos_tab == nullptr) can each be left out.
// With q_out == nullptr, q and k are normed/rotated in place and nothing is
// written to the cache (for a position encoding applied between two calls).
#include "common.cuh"

#define KP_MAX_HEAD_DIM 256

template <typename T>
__global__ void __launch_bounds__(128)
qk_norm_rope_kv_kernel(const T* qkv, int ld, const float* __restrict__ q_w,
                       const float* __restrict__ k_w, float eps, const float* __restrict__ cos_tab,
                       const float* __restrict__ sin_tab, int rot, int interleaved,
                       const int* __restrict__ positions, const int* __restrict__ slot_map,
                       T* q_out, int ldq, T* __restrict__ cache, int page_size,
                       int H, int G, int hd, int write_kv) {
    kp_pdl_begin();
    __shared__ float buf[4][KP_MAX_HEAD_DIM];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x * 4 + warp;          // 0..H-1 q, H..H+G-1 k, H+G..H+2G-1 v
    const int row = blockIdx.y;
    if (head >= H + 2 * G) return;
    const int kind = head < H ? 0 : (head < H + G ? 1 : 2);
    const bool in_place = q_out == nullptr;            // norm/rotate q and k where they are; no cache write
    if (kind != 0 && !write_kv && !(in_place && kind == 1)) return;
    const T* src = qkv + (size_t)row * ld + (size_t)head * hd;
    float* x = buf[warp];

    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) {
        const float v = to_f32(src[i]);
        x[i] = v;
        ss = fmaf(v, v, ss);
    }
    const float* w = kind == 0 ? q_w : (kind == 1 ? k_w : nullptr);
    if (w) {
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)hd + eps);
        for (int i = lane; i < hd; i += 32) x[i] = (x[i] * scale) * w[i];
    }
    __syncwarp();
    if (kind != 2 && cos_tab) {
        const int half = rot >> 1;
        const size_t tb = (size_t)positions[row] * half;
        for (int j = lane; j < half; j += 32) {
            const int ia = interleaved ? 2 * j : j;
            const int ib = interleaved ? 2 * j + 1 : j + half;
            const float c = cos_tab[tb + j], s = sin_tab[tb + j];
            const float a = x[ia], b = x[ib];
            x[ia] = a * c - b * s;
            x[ib] = a * s + b * c;
        }
        __syncwarp();
    }
    T* dst;
    if (in_place) {
        dst = const_cast<T*>(src);
    } else if (kind == 0) {
        dst = q_out + (size_t)row * ldq + (size_t)head * hd;
    } else {
        const int slot = slot_map[row];
        if (slot < 0) return;
        const int page = slot / page_size, off = slot % page_size;
        const int g = kind == 1 ? head - H : head - H - G;
        dst = cache + ((((size_t)page * 2 + (kind - 1)) * G + g) * page_size + off) * hd;
    }
    for (int i = lane; i < hd; i += 32) dst[i] = from_f32<T>(x[i]);
}

extern "C" int kp_qk_norm_rope_kv(const void* qkv, int ld, const float* q_w, const float* k_w, float eps,
                                  const float* cos_tab, const float* sin_tab, int rot, int interleaved,
                                  const int* positions, const int* slot_map, void* q_out, int ldq, void* cache,
                                  int page_size, int n, int H, int G, int hd, int write_kv, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (hd < 2 || hd > KP_MAX_HEAD_DIM || (hd & 1)) return KP_ERR_UNSUPPORTED;
    if (cos_tab && (rot < 2 || rot > hd || (rot & 1))) return KP_ERR_BAD_ARG;
    if (n > 65535) return KP_ERR_UNSUPPORTED;
    dim3 grid((H + 2 * G + 3) / 4, n);
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(qk_norm_rope_kv_kernel<T>, dim3(grid), dim3(128), 0, (cudaStream_t)stream, 
        (const T*)qkv, ld, q_w, k_w, eps, cos_tab, sin_tab, rot, interleaved, positions, slot_map, (T*)q_out, ldq,
        (T*)cache, page_size, H, G, hd, write_kv)));
    return kp_launch_status();
}
