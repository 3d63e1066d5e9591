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

// The same for bfloat16 with head size 64 or 128, full NeoX rotation (or none) and 16-byte aligned rows: a
// thread holds 8 consecutive elements of a head (one 16-byte load and one 16-byte store), hd / 8 lanes share
// a head; the sum of squares and the rotation partner (element i + hd/2: the lane hd/16 further on) come by
// warp shuffles.  Same arithmetic in the same order as the general kernel.
template <int HD>
__global__ void __launch_bounds__(128)
qk_norm_rope_kv_vec_kernel(const bf16* __restrict__ qkv, int ld, const float* __restrict__ q_w,
                           const float* __restrict__ k_w, float eps, const float* __restrict__ cos_tab,
                           const float* __restrict__ sin_tab, const int* __restrict__ positions,
                           const int* __restrict__ slot_map, bf16* __restrict__ q_out, int ldq,
                           bf16* __restrict__ cache, int page_size, int H, int G, int write_kv) {
    kp_pdl_begin_early();
    constexpr int L = HD / 8;                          // lanes a head
    constexpr int HPB = 128 / L;                       // heads a block
    const int lane_in = threadIdx.x % L;
    const int head = blockIdx.x * HPB + threadIdx.x / L;
    const int row = blockIdx.y;
    const bool live = head < H + 2 * G;
    const int hh = live ? head : 0;
    const int kind = hh < H ? 0 : (hh < H + G ? 1 : 2);
    const uint4 raw = *reinterpret_cast<const uint4*>(qkv + (size_t)row * ld + (size_t)hh * HD + lane_in * 8);
    float x[8];
    {
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; i++) { const float2 f = __bfloat1622float2(p2[i]); x[2 * i] = f.x; x[2 * i + 1] = f.y; }
    }
    const float* w = kind == 0 ? q_w : (kind == 1 ? k_w : nullptr);
    if (w) {                                            // (uniform over the lanes of a head)
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) ss = fmaf(x[i], x[i], ss);
#pragma unroll
        for (int o = L / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float scale = 1.0f / sqrtf(ss / (float)HD + eps);
        const float4 w0 = __ldg(reinterpret_cast<const float4*>(w + lane_in * 8));
        const float4 w1 = __ldg(reinterpret_cast<const float4*>(w + lane_in * 8) + 1);
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] = (x[i] * scale) * ww[i];
    }
    if (cos_tab != nullptr) {                          // every lane takes part in the shuffles
        const bool lower = lane_in < L / 2;            // holds the `a` of its pairs; the partner holds `b`
        const size_t tb = (size_t)positions[row] * (HD / 2) + (size_t)(lane_in % (L / 2)) * 8;
        const float4 c0 = __ldg(reinterpret_cast<const float4*>(cos_tab + tb)), c1 = __ldg(reinterpret_cast<const float4*>(cos_tab + tb) + 1);
        const float4 s0 = __ldg(reinterpret_cast<const float4*>(sin_tab + tb)), s1 = __ldg(reinterpret_cast<const float4*>(sin_tab + tb) + 1);
        const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float other = __shfl_xor_sync(0xffffffffu, x[i], L / 2);
            if (kind != 2) x[i] = lower ? x[i] * cc[i] - other * sn[i] : other * sn[i] + x[i] * cc[i];
        }
    }
    if (!live || (kind != 0 && !write_kv)) return;
    uint4 o;
    {
        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; i++) p2[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    }
    bf16* dst;
    if (kind == 0) {
        dst = q_out + (size_t)row * ldq + (size_t)head * HD;
    } else {
        const int slot = slot_map[row];
        if (slot < 0) return;
        const int page = slot / page_size, off = slot % page_size;
        const int g = kind == 1 ? head - H : head - H - G;
        dst = cache + ((((size_t)page * 2 + (kind - 1)) * G + g) * page_size + off) * HD;
    }
    *reinterpret_cast<uint4*>(dst + lane_in * 8) = o;
}

extern "C" int kp_qk_norm_rope_kv(const void* qkv, int ld, const float* q_w, const float* k_w, float eps,
                                  const float* cos_tab, const float* sin_tab, int rot, int interleaved,
                                  const int* positions, const int* slot_map, void* q_out, int ldq, void* cache,
                                  int page_size, int n, int H, int G, int hd, int write_kv, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (hd < 2 || hd > KP_MAX_HEAD_DIM || (hd & 1)) return KP_ERR_UNSUPPORTED;
    if (cos_tab && (rot < 2 || rot > hd || (rot & 1))) return KP_ERR_BAD_ARG;
    if (n > 65535) return KP_ERR_UNSUPPORTED;
    // the 16-byte form: bfloat16, head size 64 or 128, whole-head NeoX rotation or none, aligned rows
    if (dtype == KP_DTYPE_BF16 && (hd == 64 || hd == 128) && q_out != nullptr && (!cos_tab || (rot == hd && !interleaved)) &&
        (ld % 8 == 0) && (ldq % 8 == 0) && !((uintptr_t)qkv & 15) && !((uintptr_t)q_out & 15) && !((uintptr_t)cache & 15) &&
        (!q_w || !((uintptr_t)q_w & 15)) && (!k_w || !((uintptr_t)k_w & 15)) &&
        (!cos_tab || (!((uintptr_t)cos_tab & 15) && !((uintptr_t)sin_tab & 15)))) {
        const int hpb = 128 / (hd / 8);
        dim3 vgrid((H + 2 * G + hpb - 1) / hpb, n);
        if (hd == 64)
            kp_launch_pdl(qk_norm_rope_kv_vec_kernel<64>, dim3(vgrid), dim3(128), 0, (cudaStream_t)stream, (const bf16*)qkv, ld, q_w,
                          k_w, eps, cos_tab, sin_tab, positions, slot_map, (bf16*)q_out, ldq, (bf16*)cache, page_size, H, G, write_kv);
        else
            kp_launch_pdl(qk_norm_rope_kv_vec_kernel<128>, dim3(vgrid), dim3(128), 0, (cudaStream_t)stream, (const bf16*)qkv, ld, q_w,
                          k_w, eps, cos_tab, sin_tab, positions, slot_map, (bf16*)q_out, ldq, (bf16*)cache, page_size, H, G, write_kv);
        return kp_launch_status();
    }
    dim3 grid((H + 2 * G + 3) / 4, n);
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(qk_norm_rope_kv_kernel<T>, dim3(grid), dim3(128), 0, (cudaStream_t)stream, 
        (const T*)qkv, ld, q_w, k_w, eps, cos_tab, sin_tab, rot, interleaved, positions, slot_map, (T*)q_out, ldq,
        (T*)cache, page_size, H, G, hd, write_kv)));
    return kp_launch_status();
}
