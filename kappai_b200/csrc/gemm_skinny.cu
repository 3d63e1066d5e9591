// C[M,N] = A[M,K] * W[N,K]^T for few rows (M <= 64): the decode-step product.
//
// The work is reading W once from HBM, so the kernel is a weight streamer:
// a CTA owns 8 rows of W (one n8 tile of mma.m16n8k16 with the batch rows as
// the m side) and its 8 warps split K in interleaved blocks of 32; every
// thread loads 16 contiguous bytes of its W row and of its activation rows
// straight into the mma fragment layout (the k order inside a block of 32 is
// permuted identically for both operands, which a dot product does not see),
// with several blocks in flight.  The 8 partial sums of a CTA are added in warp
// order, so an output depends on its own activation row only, whatever M is.
//
// Epilogues: bias; store bf16 / store fp32 / accumulate into fp32 (residual);
// SwiGLU (W holds gate rows then up rows, ff apart; the CTA streams both and
// writes silu(g)*u).  K must be a multiple of 32 and rows 16-byte aligned.
#include "common.cuh"

#define EPI_STORE 0
#define EPI_STORE_F32 1
#define EPI_ACCUM_F32 2
#define EPI_SWIGLU 3

#define SK_WARPS 8
#define SK_UNROLL 4

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_cached(const uint4* p) { return __ldg(p); }

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT: m16 tiles of batch rows; HALF: only rows 0..7 of the single tile exist (M <= 8)
template <int MT, bool HALF, int EPI>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const bf16* __restrict__ A, int lda, const bf16* __restrict__ W, int ldw,
                   const float* __restrict__ bias, void* __restrict__ Cv, int ldc, int M, int N, int K, int ff) {
    constexpr int NW = (EPI == EPI_SWIGLU) ? 2 : 1;          // weight streams
    __shared__ float red[SK_WARPS][NW][MT][4][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 8;
    const int n_out = (EPI == EPI_SWIGLU) ? ff : N;          // output columns
    const int wrow = min(n0 + g, n_out - 1);
    const uint4* wp[NW];
    wp[0] = reinterpret_cast<const uint4*>(W + (size_t)wrow * ldw) + t;
    if (NW == 2) wp[1] = reinterpret_cast<const uint4*>(W + (size_t)(ff + wrow) * ldw) + t;
    const uint4* ap[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        const int r0 = min(mt * 16 + g, M - 1), r1 = min(mt * 16 + g + 8, M - 1);
        ap[mt][0] = reinterpret_cast<const uint4*>(A + (size_t)r0 * lda) + t;
        ap[mt][1] = reinterpret_cast<const uint4*>(A + (size_t)r1 * lda) + t;
    }
    float acc[NW][MT][4];
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[w][mt][i] = 0.f;

    const int nkb = K >> 5;
    for (int kb0 = warp; kb0 < nkb; kb0 += SK_WARPS * SK_UNROLL) {
        uint4 wv[SK_UNROLL][NW];
#pragma unroll
        for (int u = 0; u < SK_UNROLL; u++) {
            const int kb = kb0 + u * SK_WARPS;
            if (kb < nkb) {
#pragma unroll
                for (int w = 0; w < NW; w++) wv[u][w] = ld_stream(wp[w] + (size_t)kb * 4);
            }
        }
#pragma unroll
        for (int u = 0; u < SK_UNROLL; u++) {
            const int kb = kb0 + u * SK_WARPS;
            if (kb < nkb) {
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const uint4 lo = ld_cached(ap[mt][0] + (size_t)kb * 4);
                    uint4 hi = make_uint4(0, 0, 0, 0);
                    if (!HALF) hi = ld_cached(ap[mt][1] + (size_t)kb * 4);
#pragma unroll
                    for (int w = 0; w < NW; w++) {
                        mma_bf16(acc[w][mt], lo.x, hi.x, lo.y, hi.y, wv[u][w].x, wv[u][w].y);
                        mma_bf16(acc[w][mt], lo.z, hi.z, lo.w, hi.w, wv[u][w].z, wv[u][w].w);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) red[warp][w][mt][i][lane] = acc[w][mt][i];
    __syncthreads();
    // sum the warps' partials in order and write: thread (mt, i, lane) <- element i of tile mt of lane's fragment
    for (int e = threadIdx.x; e < MT * 4 * 32; e += SK_WARPS * 32) {
        const int l = e & 31, i = (e >> 5) & 3, mt = e >> 7;
        const int m = mt * 16 + (l >> 2) + ((i & 2) ? 8 : 0);
        const int n = n0 + (l & 3) * 2 + (i & 1);
        if (m >= M || n >= n_out) continue;
        float v = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < SK_WARPS; w8++) v += red[w8][0][mt][i][l];
        if (bias) v += bias[n];
        const size_t o = (size_t)m * ldc + n;
        if (EPI == EPI_SWIGLU) {
            float u = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < SK_WARPS; w8++) u += red[w8][NW - 1][mt][i][l];
            if (bias) u += bias[ff + n];
            // gate and up are rounded to the storage type before the activation, as the unfused path stores them
            const float gq = to_f32(from_f32<bf16>(v)), uq = to_f32(from_f32<bf16>(u));
            ((bf16*)Cv)[o] = from_f32<bf16>((gq / (1.0f + expf(-gq))) * uq);
        } else if (EPI == EPI_STORE) {
            ((bf16*)Cv)[o] = from_f32<bf16>(v);
        } else if (EPI == EPI_STORE_F32) {
            ((float*)Cv)[o] = v;
        } else {
            ((float*)Cv)[o] += v;
        }
    }
}

template <int MT, bool HALF>
static int launch_epi(const bf16* A, int lda, const bf16* W, int ldw, const float* bias, void* C, int ldc, int M,
                      int N, int K, int ff, int epi, cudaStream_t s) {
    const int n_out = epi == EPI_SWIGLU ? ff : N;
    dim3 grid((n_out + 7) / 8);
    switch (epi) {
        case EPI_STORE:
            gemm_skinny_kernel<MT, HALF, EPI_STORE><<<grid, SK_WARPS * 32, 0, s>>>(A, lda, W, ldw, bias, C, ldc, M, N, K, ff);
            break;
        case EPI_STORE_F32:
            gemm_skinny_kernel<MT, HALF, EPI_STORE_F32><<<grid, SK_WARPS * 32, 0, s>>>(A, lda, W, ldw, bias, C, ldc, M, N, K, ff);
            break;
        case EPI_ACCUM_F32:
            gemm_skinny_kernel<MT, HALF, EPI_ACCUM_F32><<<grid, SK_WARPS * 32, 0, s>>>(A, lda, W, ldw, bias, C, ldc, M, N, K, ff);
            break;
        case EPI_SWIGLU:
            gemm_skinny_kernel<MT, HALF, EPI_SWIGLU><<<grid, SK_WARPS * 32, 0, s>>>(A, lda, W, ldw, bias, C, ldc, M, N, K, ff);
            break;
        default:
            return KP_ERR_BAD_ARG;
    }
    return kp_launch_status();
}

// epi: 0 store bf16, 1 store f32, 2 accumulate f32, 3 SwiGLU (N = 2*ff rows of W, output [M, ff] bf16)
extern "C" int kp_gemm_skinny(const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc,
                              int M, int N, int K, int epi, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K < 32 || (K & 31) || (lda & 7) || (ldw & 7)) return KP_ERR_UNSUPPORTED;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return KP_ERR_UNSUPPORTED;
    int ff = 0;
    if (epi == EPI_SWIGLU) {
        if (N & 1) return KP_ERR_BAD_ARG;
        ff = N / 2;
    }
    const bf16* a = (const bf16*)A;
    const bf16* w = (const bf16*)W;
    cudaStream_t s = (cudaStream_t)stream;
    if (M <= 8) return launch_epi<1, true>(a, lda, w, ldw, bias, C, ldc, M, N, K, ff, epi, s);
    if (M <= 16) return launch_epi<1, false>(a, lda, w, ldw, bias, C, ldc, M, N, K, ff, epi, s);
    if (M <= 32) return launch_epi<2, false>(a, lda, w, ldw, bias, C, ldc, M, N, K, ff, epi, s);
    if (M <= 48) return launch_epi<3, false>(a, lda, w, ldw, bias, C, ldc, M, N, K, ff, epi, s);
    return launch_epi<4, false>(a, lda, w, ldw, bias, C, ldc, M, N, K, ff, epi, s);
}
