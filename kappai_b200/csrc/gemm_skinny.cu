// C[M,N] = A[M,K] * W[N,K]^T for few rows (M <= 64): the decode-step product.
//
// The work is reading W once from HBM, so the kernel is a weight streamer:
// a CTA owns 8 rows of W (one n8 tile of mma.m16n8k16 with the batch rows as
// the m side) and its 8 warps split K in interleaved blocks of 32; every
// thread loads 16 contiguous bytes of its W row and of its activation rows
// straight into the mma fragment layout (the k order inside a block of 32 is
// permuted identically for both operands, which a dot product does not see),
// with several blocks in flight.  The partial sums of a CTA's warps are added
// in warp order, so an output depends on its own activation row only, whatever
// M is.
//
// Epilogues: bias; store bf16 / store fp32 / accumulate into fp32 (residual);
// SwiGLU (W holds gate rows then up rows, ff apart; the CTA streams both and
// writes silu(g)*u).  K must be a multiple of 32 and rows 16-byte aligned.
//
// The kernels are launched with programmatic dependent launch: the weight
// loads of the first iteration do not depend on the kernel before, so they are
// issued before griddepcontrol.wait and overlap that kernel's tail.
#include "common.cuh"

#define EPI_STORE 0
#define EPI_STORE_F32 1
#define EPI_ACCUM_F32 2
#define EPI_SWIGLU 3

#define SK_WARPS 8
#define SK_U 4                 // k-blocks of 32 a warp has in flight per stage
#define SK_THREADS (SK_WARPS * 32)

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}


struct SkinnyArgs {
    const bf16* A; int lda;              // bf16 activations
    const bf16* W; int ldw;
    const float* bias;
    void* C; int ldc;
    int M, N, K, ff;
};

// MT: m16 tiles of batch rows; HALF: only rows 0..7 of the single tile exist (M <= 8).
// Each warp walks its k-blocks in stages of SK_U blocks, two stages in flight: the loads of the next
// stage are issued before the products of the current one.
template <int MT, bool HALF, int EPI>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const SkinnyArgs p) {
    constexpr int NW = (EPI == EPI_SWIGLU) ? 2 : 1;          // weight streams
    constexpr int U = SK_U;
    constexpr int STEP = SK_WARPS * U;
    __shared__ float red[SK_WARPS][NW][MT][4][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int M = p.M, K = p.K;
    const int n0 = blockIdx.x * 8;
    const int n_out = (EPI == EPI_SWIGLU) ? p.ff : p.N;      // output columns
    const int wrow = min(n0 + g, n_out - 1);
    const uint4* wp[NW];
    wp[0] = reinterpret_cast<const uint4*>(p.W + (size_t)wrow * p.ldw) + t;
    if (NW == 2) wp[1] = reinterpret_cast<const uint4*>(p.W + (size_t)(p.ff + wrow) * p.ldw) + t;
    const int nkb = K >> 5;

    uint4 wa[U][NW], wb[U][NW];
    auto load_stage = [&](uint4 (&wv)[U][NW], int kb0) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int kb = kb0 + u * SK_WARPS;
            if (kb < nkb) {
#pragma unroll
                for (int w = 0; w < NW; w++) wv[u][w] = ld_stream(wp[w] + (size_t)kb * 4);
            }
        }
    };
    // weights of the first stage: independent of everything that ran before
    load_stage(wa, warp);
    KP_TRACE_MARK(0);
    pdl_wait();                                               // now the activations are there
    KP_TRACE_MARK(1);
    pdl_launch_dependents();

    int r0[MT], r1[MT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        r0[mt] = min(mt * 16 + g, M - 1);
        r1[mt] = min(mt * 16 + g + 8, M - 1);
    }
    float acc[NW][MT][4];
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[w][mt][i] = 0.f;

    auto compute_stage = [&](const uint4 (&wv)[U][NW], int kb0) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int kb = kb0 + u * SK_WARPS;
            if (kb < nkb) {
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    uint4 lo, hi = make_uint4(0, 0, 0, 0);
                    lo = __ldg(reinterpret_cast<const uint4*>(p.A + (size_t)r0[mt] * p.lda) + kb * 4 + t);
                    if (!HALF) hi = __ldg(reinterpret_cast<const uint4*>(p.A + (size_t)r1[mt] * p.lda) + kb * 4 + t);
#pragma unroll
                    for (int w = 0; w < NW; w++) {
                        mma_bf16(acc[w][mt], lo.x, hi.x, lo.y, hi.y, wv[u][w].x, wv[u][w].y);
                        mma_bf16(acc[w][mt], lo.z, hi.z, lo.w, hi.w, wv[u][w].z, wv[u][w].w);
                    }
                }
            }
        }
    };
    for (int kb0 = warp; kb0 < nkb; kb0 += 2 * STEP) {
        if (kb0 + STEP < nkb) load_stage(wb, kb0 + STEP);
        compute_stage(wa, kb0);
        if (kb0 + STEP < nkb) {
            if (kb0 + 2 * STEP < nkb) load_stage(wa, kb0 + 2 * STEP);
            compute_stage(wb, kb0 + STEP);
        }
    }
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) red[warp][w][mt][i][lane] = acc[w][mt][i];
    __syncthreads();
    // sum the warps' partials in warp order and write: element i of tile mt of lane l's fragment
    for (int e = threadIdx.x; e < MT * 4 * 32; e += SK_THREADS) {
        const int l = e & 31, i = (e >> 5) & 3, mt = e >> 7;
        const int m = mt * 16 + (l >> 2) + ((i & 2) ? 8 : 0);
        const int n = n0 + (l & 3) * 2 + (i & 1);
        if (m >= M || n >= n_out) continue;
        float v = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < SK_WARPS; w8++) v += red[w8][0][mt][i][l];
        if (p.bias) v += p.bias[n];
        const size_t o = (size_t)m * p.ldc + n;
        if (EPI == EPI_SWIGLU) {
            float u = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < SK_WARPS; w8++) u += red[w8][NW - 1][mt][i][l];
            if (p.bias) u += p.bias[p.ff + n];
            // gate and up are rounded to the storage type before the activation, as the unfused path stores them
            const float gq = to_f32(from_f32<bf16>(v)), uq = to_f32(from_f32<bf16>(u));
            ((bf16*)p.C)[o] = from_f32<bf16>((gq / (1.0f + expf(-gq))) * uq);
        } else if (EPI == EPI_STORE) {
            ((bf16*)p.C)[o] = from_f32<bf16>(v);
        } else if (EPI == EPI_STORE_F32) {
            ((float*)p.C)[o] = v;
        } else {
            ((float*)p.C)[o] += v;
        }
    }
}

template <typename Kern>
static int launch_pdl(Kern kern, dim3 grid, cudaStream_t s, const SkinnyArgs& a) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(SK_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
    return (int)e;
}

template <int MT, bool HALF>
static int launch_epi(const SkinnyArgs& a, int epi, cudaStream_t s) {
    const int n_out = epi == EPI_SWIGLU ? a.ff : a.N;
    dim3 grid((n_out + 7) / 8);
    switch (epi) {
        case EPI_STORE: return launch_pdl(gemm_skinny_kernel<MT, HALF, EPI_STORE>, grid, s, a);
        case EPI_STORE_F32: return launch_pdl(gemm_skinny_kernel<MT, HALF, EPI_STORE_F32>, grid, s, a);
        case EPI_ACCUM_F32: return launch_pdl(gemm_skinny_kernel<MT, HALF, EPI_ACCUM_F32>, grid, s, a);
        case EPI_SWIGLU: return launch_pdl(gemm_skinny_kernel<MT, HALF, EPI_SWIGLU>, grid, s, a);
        default: return KP_ERR_BAD_ARG;
    }
}

static int launch_m(const SkinnyArgs& a, int epi, cudaStream_t s) {
    if (a.M <= 8) return launch_epi<1, true>(a, epi, s);
    if (a.M <= 16) return launch_epi<1, false>(a, epi, s);
    if (a.M <= 32) return launch_epi<2, false>(a, epi, s);
    if (a.M <= 48) return launch_epi<3, false>(a, epi, s);
    return launch_epi<4, false>(a, epi, s);
}

static int check_common(int M, int N, int K, int ldw, const void* W, int epi, int* ff) {
    if (M > 64 || K < 32 || (K & 31) || (ldw & 7) || ((uintptr_t)W & 15)) return KP_ERR_UNSUPPORTED;
    *ff = 0;
    if (epi == EPI_SWIGLU) {
        if (N & 1) return KP_ERR_BAD_ARG;
        *ff = N / 2;
    }
    return 0;
}

extern "C" {

// epi: 0 store bf16, 1 store f32, 2 accumulate f32, 3 SwiGLU (N = 2*ff rows of W, output [M, ff] bf16)
int kp_gemm_skinny(const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc, int M, int N,
                   int K, int epi, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    SkinnyArgs a = {};
    int st = check_common(M, N, K, ldw, W, epi, &a.ff);
    if (st) return st;
    if ((lda & 7) || ((uintptr_t)A & 15)) return KP_ERR_UNSUPPORTED;
    a.A = (const bf16*)A; a.lda = lda; a.W = (const bf16*)W; a.ldw = ldw; a.bias = bias; a.C = C; a.ldc = ldc;
    a.M = M; a.N = N; a.K = K;
    return launch_m(a, epi, (cudaStream_t)stream);
}

}  // extern "C"
