// C[M,N] = A[M,K] * W[N,K]^T for few rows (M <= 64), weights streamed by the
// bulk-copy engine: the decode-step product for the usual layer shapes.
//
// A CTA owns 8 rows of W (one n8 tile of mma.m16n8k16, batch rows on the m
// side; 2 x 8 rows for the SwiGLU epilogue).  At its start, before anything
// that depends on the kernel before it, it issues cp.async.bulk copies of its
// whole slab of W (8 rows x K) into shared memory, chunk by chunk of 256
// columns, each chunk signalling an mbarrier.  So the bytes in flight per SM
// are the slabs of its resident CTAs (tens of KB each), not what registers can
// hold.  The four warps then take the k-blocks of 32 of each chunk as it lands
// (block b of a chunk goes to warp b % 4), read W fragments from shared memory
// (rows padded so that the 16-byte fragment reads do not collide in banks) and
// activation fragments from global memory, which L1 serves after the first CTA
// of an SM.  The warps' partial sums are added in warp order: an output depends
// on its own activation row only, whatever M is.
//
// Fused in front (NORM, M <= 16): A = bf16((x * rsqrt(mean(x^2)+eps)) * w) of
// the float32 residual rows (src/backend/cpu/scalar/quants.c:1489-1512).
// Epilogues: bias; store bf16 / fp32; accumulate into fp32; SwiGLU.
//
// Every mbarrier wait is bounded; a wait that gives up sets a status word that
// the host can read (kp_stream_status), and the CTA still waits (bounded) for
// its remaining copies before it returns.
//
// Limits: K a multiple of 256; the slab (8 or 16 rows of K bf16 plus padding)
// must fit in 96 KB.  Other shapes take the register-streaming kernel.
#include "common.cuh"

#define EPI_STORE 0
#define EPI_STORE_F32 1
#define EPI_ACCUM_F32 2
#define EPI_SWIGLU 3

#define ST_WARPS 4
#define ST_THREADS (ST_WARPS * 32)
#define ST_CHUNK 256                         // columns a chunk (one mbarrier each)
#define ST_MAX_CHUNKS 32
#define ST_MAX_SLAB (96 * 1024)
#define ST_WAIT_NS 1000000000ull             // one second: far beyond any legitimate wait

__device__ int g_stream_status = 0;          // 0 ok; 1: a bounded wait gave up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// false if the barrier did not flip within ST_WAIT_NS
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = now_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (now_ns() - t0 > ST_WAIT_NS) return false;
    }
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
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

__device__ __forceinline__ uint4 normed8(const float* __restrict__ x, const float* __restrict__ nw, float scale) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(x)), b = __ldg(reinterpret_cast<const float4*>(x) + 1);
    const float4 wa = __ldg(reinterpret_cast<const float4*>(nw)), wb = __ldg(reinterpret_cast<const float4*>(nw) + 1);
    uint4 r;
    r.x = pack_bf16((a.x * scale) * wa.x, (a.y * scale) * wa.y);
    r.y = pack_bf16((a.z * scale) * wa.z, (a.w * scale) * wa.w);
    r.z = pack_bf16((b.x * scale) * wb.x, (b.y * scale) * wb.y);
    r.w = pack_bf16((b.z * scale) * wb.z, (b.w * scale) * wb.w);
    return r;
}

struct StreamArgs {
    const bf16* A; int lda;              // bf16 activations (NORM = false)
    const float* X; int ldx;             // float32 residual (NORM = true)
    const float* norm_w; float eps;
    const int* rows;                     // optional gather of the rows of X
    const bf16* W; int ldw;
    const float* bias;
    void* C; int ldc;
    int M, N, K, ff;
    int pitch;                           // bytes between rows of the slab in shared memory
};

// shared memory: [slab: NW*8 rows of `pitch` bytes][barriers: n_chunks x 8 B][red: ST_WARPS*NW*MT*128 floats][scales]
template <int MT, bool HALF, int EPI, bool NORM>
__global__ void __launch_bounds__(ST_THREADS)
gemm_stream_kernel(const StreamArgs p) {
    constexpr int NW = (EPI == EPI_SWIGLU) ? 2 : 1;
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int M = p.M, K = p.K, pitch = p.pitch;
    const int n_chunks = K / ST_CHUNK;
    unsigned char* slab = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)NW * 8 * pitch);
    float* red = reinterpret_cast<float*>(bars + ST_MAX_CHUNKS);
    float* scales = red + ST_WARPS * NW * MT * 128;
    const int n0 = blockIdx.x * 8;
    const int n_out = (EPI == EPI_SWIGLU) ? p.ff : p.N;

    if (threadIdx.x == 0) {
        for (int c = 0; c < n_chunks; c++) mbar_init(&bars[c], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0) {
        // the whole slab: chunk c of row r is one copy of 512 bytes; lanes share the copies out
        if (lane == 0)
            for (int c = 0; c < n_chunks; c++) mbar_expect_tx(&bars[c], NW * 8 * ST_CHUNK * 2);
        __syncwarp();
        const int n_copies = NW * 8 * n_chunks;
        for (int i = lane; i < n_copies; i += 32) {
            const int r = i % (NW * 8), c = i / (NW * 8);            // consecutive lanes: the rows of one chunk
            const int wrow = (r < 8 ? 0 : p.ff) + min(n0 + (r & 7), n_out - 1);
            bulk_g2s(slab + (size_t)r * pitch + (size_t)c * ST_CHUNK * 2,
                     p.W + (size_t)wrow * p.ldw + (size_t)c * ST_CHUNK, ST_CHUNK * 2, &bars[c]);
        }
    }
    pdl_wait();                                               // from here on the activations may be read
    pdl_launch_dependents();

    int r0[MT], r1[MT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        r0[mt] = min(mt * 16 + g, M - 1);
        r1[mt] = min(mt * 16 + g + 8, M - 1);
        if (NORM && p.rows) { r0[mt] = p.rows[r0[mt]]; r1[mt] = p.rows[r1[mt]]; }
    }
    if (NORM) {
        for (int row = warp; row < M; row += ST_WARPS) {
            const int xr = p.rows ? p.rows[row] : row;
            const float4* xp = reinterpret_cast<const float4*>(p.X + (size_t)xr * p.ldx);
            float ss = 0.f;
            for (int i = lane; i < (K >> 2); i += 32) {
                const float4 v = __ldg(xp + i);
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            }
            ss = warp_sum(ss);
            if (lane == 0) scales[row] = 1.0f / sqrtf(ss / (float)K + p.eps);
        }
        __syncthreads();
    }
    float sc0 = 0.f, sc1 = 0.f;
    if (NORM) { sc0 = scales[min(g, M - 1)]; sc1 = scales[min(g + 8, M - 1)]; }

    float acc[NW][MT][4];
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[w][mt][i] = 0.f;

    auto load_acts = [&](uint4 (&lo)[MT], uint4 (&hi)[MT], int kb) {
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            hi[mt] = make_uint4(0, 0, 0, 0);
            if (NORM) {
                const int k = kb * 32 + 8 * t;
                lo[mt] = normed8(p.X + (size_t)r0[mt] * p.ldx + k, p.norm_w + k, sc0);
                if (!HALF) hi[mt] = normed8(p.X + (size_t)r1[mt] * p.ldx + k, p.norm_w + k, sc1);
            } else {
                lo[mt] = __ldg(reinterpret_cast<const uint4*>(p.A + (size_t)r0[mt] * p.lda) + kb * 4 + t);
                if (!HALF) hi[mt] = __ldg(reinterpret_cast<const uint4*>(p.A + (size_t)r1[mt] * p.lda) + kb * 4 + t);
            }
        }
    };

    // a chunk holds 8 k-blocks of 32: warp w takes blocks w and w + 4
    const unsigned char* wrow_s[NW];
#pragma unroll
    for (int w = 0; w < NW; w++) wrow_s[w] = slab + (size_t)(w * 8 + g) * pitch + 16 * t;
    bool timed_out = false;
    uint4 lo[2][MT], hi[2][MT];
    load_acts(lo[0], hi[0], warp);
    load_acts(lo[1], hi[1], warp + ST_WARPS);
    for (int c = 0; c < n_chunks; c++) {
        if (!mbar_wait_bounded(&bars[c], 0)) timed_out = true;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int kb = c * 8 + warp + j * ST_WARPS;
            uint4 wv[NW];
#pragma unroll
            for (int w = 0; w < NW; w++) wv[w] = *reinterpret_cast<const uint4*>(wrow_s[w] + (size_t)kb * 64);
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int w = 0; w < NW; w++) {
                    mma_bf16(acc[w][mt], lo[j][mt].x, hi[j][mt].x, lo[j][mt].y, hi[j][mt].y, wv[w].x, wv[w].y);
                    mma_bf16(acc[w][mt], lo[j][mt].z, hi[j][mt].z, lo[j][mt].w, hi[j][mt].w, wv[w].z, wv[w].w);
                }
            if (c + 1 < n_chunks) load_acts(lo[j], hi[j], kb + 8);       // the same block of the next chunk
        }
    }
    if (timed_out) atomicExch(&g_stream_status, 1);

#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) red[(((warp * NW + w) * MT + mt) * 4 + i) * 32 + lane] = acc[w][mt][i];
    __syncthreads();
    for (int e = threadIdx.x; e < MT * 4 * 32; e += ST_THREADS) {
        const int l = e & 31, i = (e >> 5) & 3, mt = e >> 7;
        const int m = mt * 16 + (l >> 2) + ((i & 2) ? 8 : 0);
        const int n = n0 + (l & 3) * 2 + (i & 1);
        if (m >= M || n >= n_out) continue;
        float v = 0.f;
#pragma unroll
        for (int w4 = 0; w4 < ST_WARPS; w4++) v += red[(((w4 * NW + 0) * MT + mt) * 4 + i) * 32 + l];
        if (p.bias) v += p.bias[n];
        const size_t o = (size_t)m * p.ldc + n;
        if (EPI == EPI_SWIGLU) {
            float u = 0.f;
#pragma unroll
            for (int w4 = 0; w4 < ST_WARPS; w4++) u += red[(((w4 * NW + NW - 1) * MT + mt) * 4 + i) * 32 + l];
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

static int slab_pitch(int K) {
    const int row = K * 2;
    return (row % 128 == 0) ? row + 64 : row;          // pitch = 64 mod 128: 16-byte reads of 8 rows spread over all banks
}

static size_t smem_bytes(int NW, int MT, int pitch) {
    return (size_t)NW * 8 * pitch + ST_MAX_CHUNKS * 8 + sizeof(float) * (ST_WARPS * NW * MT * 128 + 16);
}

template <typename Kern>
static int launch_pdl(Kern kern, dim3 grid, size_t smem, cudaStream_t s, const StreamArgs& a) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(ST_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kern, a);
}

template <int MT, bool HALF, bool NORM>
static int launch_epi(const StreamArgs& a, int epi, cudaStream_t s) {
    const int n_out = epi == EPI_SWIGLU ? a.ff : a.N;
    dim3 grid((n_out + 7) / 8);
    const size_t sm = smem_bytes(epi == EPI_SWIGLU ? 2 : 1, MT, a.pitch);
    switch (epi) {
        case EPI_STORE: return launch_pdl(gemm_stream_kernel<MT, HALF, EPI_STORE, NORM>, grid, sm, s, a);
        case EPI_STORE_F32: return launch_pdl(gemm_stream_kernel<MT, HALF, EPI_STORE_F32, NORM>, grid, sm, s, a);
        case EPI_ACCUM_F32: return launch_pdl(gemm_stream_kernel<MT, HALF, EPI_ACCUM_F32, NORM>, grid, sm, s, a);
        case EPI_SWIGLU: return launch_pdl(gemm_stream_kernel<MT, HALF, EPI_SWIGLU, NORM>, grid, sm, s, a);
        default: return KP_ERR_BAD_ARG;
    }
}

template <bool NORM>
static int launch_m(const StreamArgs& a, int epi, cudaStream_t s) {
    if (a.M <= 8) return launch_epi<1, true, NORM>(a, epi, s);
    if (a.M <= 16) return launch_epi<1, false, NORM>(a, epi, s);
    if (NORM) return KP_ERR_UNSUPPORTED;
    if (a.M <= 32) return launch_epi<2, false, false>(a, epi, s);
    if (a.M <= 48) return launch_epi<3, false, false>(a, epi, s);
    return launch_epi<4, false, false>(a, epi, s);
}

static int check_common(StreamArgs& a, int M, int N, int K, int ldw, const void* W, int epi) {
    if (M > 64 || K < ST_CHUNK || (K % ST_CHUNK) || K / ST_CHUNK > ST_MAX_CHUNKS || (ldw & 7) || ((uintptr_t)W & 15))
        return KP_ERR_UNSUPPORTED;
    a.ff = 0;
    if (epi == EPI_SWIGLU) {
        if (N & 1) return KP_ERR_BAD_ARG;
        a.ff = N / 2;
    }
    a.pitch = slab_pitch(K);
    if ((size_t)(epi == EPI_SWIGLU ? 2 : 1) * 8 * a.pitch > ST_MAX_SLAB) return KP_ERR_UNSUPPORTED;
    return 0;
}

extern "C" {

// 1 if this product fits the kernel's limits (K a multiple of 256, slab within 96 KB), else 0
int kp_gemm_stream_fits(int M, int N, int K, int epi) {
    StreamArgs a = {};
    static const int dummy_aligned = 0;
    (void)dummy_aligned;
    return check_common(a, M, N, K, 8, (const void*)16, epi) == 0;
}

int kp_gemm_stream(const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc, int M, int N,
                   int K, int epi, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    StreamArgs a = {};
    int st = check_common(a, M, N, K, ldw, W, epi);
    if (st) return st;
    if ((lda & 7) || ((uintptr_t)A & 15)) return KP_ERR_UNSUPPORTED;
    a.A = (const bf16*)A; a.lda = lda; a.W = (const bf16*)W; a.ldw = ldw; a.bias = bias; a.C = C; a.ldc = ldc;
    a.M = M; a.N = N; a.K = K;
    return launch_m<false>(a, epi, (cudaStream_t)stream);
}

int kp_gemm_stream_norm(const float* X, int ldx, const float* norm_w, float eps, const int* rows, const void* W,
                        int ldw, const float* bias, void* C, int ldc, int M, int N, int K, int epi, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    StreamArgs a = {};
    int st = check_common(a, M, N, K, ldw, W, epi);
    if (st) return st;
    if (M > 16 || (ldx & 3) || ((uintptr_t)X & 15) || ((uintptr_t)norm_w & 15)) return KP_ERR_UNSUPPORTED;
    a.X = X; a.ldx = ldx; a.norm_w = norm_w; a.eps = eps; a.rows = rows;
    a.W = (const bf16*)W; a.ldw = ldw; a.bias = bias; a.C = C; a.ldc = ldc; a.M = M; a.N = N; a.K = K;
    return launch_m<true>(a, epi, (cudaStream_t)stream);
}

// Reads (and clears) the status word: 0 ok, 1 if a bounded wait gave up since the last call.  Synchronises.
int kp_stream_status(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_stream_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int));
    return v;
}

}  // extern "C"
