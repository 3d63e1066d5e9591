// C[M,N] = A[M,K] * W[N,K]^T for few rows (M <= 64), weights streamed by the bulk-copy engine through a
// ring in shared memory: the decode-step product for the usual layer shapes.
//
// The work is reading W once from HBM, and a decode step is a chain of such products, each only a few
// microseconds long.  So the kernel is built to keep HBM busy across kernel boundaries:
//
//  * Persistent CTAs, two or three an SM.  A CTA walks the 8-row tiles of W it owns (tile t, t + grid, ...); for the
//    SwiGLU epilogue a tile is 8 gate rows and the 8 matching up rows.
//  * A producer warp streams the tiles' rows in chunks of 512 columns (one cp.async.bulk of 1 KB a row and
//    chunk) into a ring of stages in shared memory; each stage has a "full" mbarrier (armed with the byte
//    count) and an "empty" mbarrier (the consumer warps arrive when they have read it).  The producer
//    runs ahead of the consumers, also across tile boundaries, so the stream never drains inside a kernel.
//  * The ring is 64 KB a CTA with three CTAs an SM, 88 KB with two (products of few tiles), and the kernel
//    is launched with programmatic dependent launch: the next product's CTAs become resident as soon as this
//    one's leave and their producers fill their rings before griddepcontrol.wait (weights depend on no
//    earlier kernel).
//  * Eight consumer warps take the k-blocks of 32 of a stage (block b to warp b % 8), read W fragments from
//    shared memory (rows padded: 16-byte reads of 8 rows hit all banks) and activation fragments from
//    global memory (L1 serves them), and issue mma.m16n8k16 with the batch rows on the m side.  At a tile's
//    end their partial sums are added in warp order, so an output depends on its own activation row only.
//
// Epilogues: bias; store bf16 / fp32; accumulate into fp32; SwiGLU; the conv step of a decode step (a tile holds
// the 8 matching rows of B, C and X, as the SwiGLU tile holds gate and up: B, C, X are rounded to bfloat16 as the
// separate kernels store them, then the arithmetic of shortconv.cu's decode kernel, state update included).  Every mbarrier wait is bounded; a wait that gives up sets a status word (kp_stream_status) and
// the warp stops waiting for further stages.
//
// Limits: K a multiple of 512.  Other shapes take the register-streaming kernel.
#include <type_traits>

#include "tma.cuh"

#define EPI_STORE 0
#define EPI_STORE_F32 1
#define EPI_ACCUM_F32 2
#define EPI_SWIGLU 3
#define EPI_CONV_STEP 4                      // W = [B; C; X] rows (in_proj of the gated short convolution): the conv step of
                                             // one-row segments runs in the epilogue, with the state update

#define ST_CONSUMERS 8                       // consumer warps
#define ST_THREADS ((ST_CONSUMERS + 1) * 32) // plus the producer warp
#define ST_COLS 512                          // columns of a stage: 16 k-blocks of 32, 2 a consumer warp
#define ST_ROW_BYTES (ST_COLS * 2 + 64)      // a stage row in shared memory: 1 KB of data, pitch = 64 mod 128
#define ST_RING_BYTES (64 * 1024)            // the ring with three CTAs an SM: 7 stages of 8 rows, 3 of 2 x 8
#define ST_RING_BYTES_FEW (88 * 1024)        // with two CTAs an SM (products with few tiles): 10 stages of 8 rows

KP_STATUS_WORD(g_stream_status, stream)          // 0 ok; 1: a bounded wait gave up

// Built with -DKP_TEST_HOOKS (a library of its own that only the tests load), the kernel can be told to
// leave one stage of its ring unfilled and to give up its waits after a shorter time, so that a test sees
// a wait run out, the kernel return and the status word rise, with nothing faulting or hanging.
#ifdef KP_TEST_HOOKS
__device__ int g_test_skip_stage = -1;                     // the producer of CTA 0 never fills this stage (-1: none)
__device__ unsigned long long g_test_wait_ns = KP_TMA_WAIT_NS;
#define ST_WAIT_NS g_test_wait_ns
extern "C" int kp_gemm_stream_test_fault(int skip_stage, unsigned long long wait_ns) {
    if (cudaMemcpyToSymbol(g_test_skip_stage, &skip_stage, sizeof(int)) != cudaSuccess) return -1;
    if (wait_ns == 0) wait_ns = KP_TMA_WAIT_NS;
    return cudaMemcpyToSymbol(g_test_wait_ns, &wait_ns, sizeof(wait_ns)) == cudaSuccess ? 0 : -1;
}
#else
#define ST_WAIT_NS KP_TMA_WAIT_NS
#endif

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(kp_smem_u32(dst)), "l"(src), "r"(bytes), "r"(kp_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(ST_CONSUMERS * 32) : "memory"); }

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

struct StreamArgs {
    const bf16* A; int lda;              // bf16 activations
    const bf16* W; int ldw;
    const float* bias;
    void* C; int ldc;
    int M, N, K, ff;                     // ff: output columns of an epilogue that joins rows of W (SwiGLU: N / 2; conv step: N / 3)
    int n_stages;                        // stages of the ring
    // the conv step (EPI_CONV_STEP): taps [ff][conv_k], optional bias [ff], state [slots][conv_k - 1][ff], and for
    // every row its position (0: the state counts as zero) and its state slot
    const float* conv_w; const float* conv_bias; float* conv_state;
    const int* seg_pos; const int* seg_slot;
    int conv_k;
};

// shared memory: [ring: n_stages x NW*8 rows x ST_ROW_BYTES][full[n_stages]][empty[n_stages]][red]
// WIDE (more than 16 batch rows, no SwiGLU): a tile is 16 rows of W, so that an activation fragment, whose
// loads weigh more than the weights' once there are several m-tiles, serves two n-tiles.
template <int MT, bool HALF, int EPI, bool WIDE>
__global__ void __launch_bounds__(ST_THREADS)
gemm_stream_kernel(const StreamArgs p) {
    constexpr int NW = EPI == EPI_CONV_STEP ? 3 : ((EPI == EPI_SWIGLU || WIDE) ? 2 : 1);
    constexpr int ROWS = NW * 8;
    constexpr int TROWS = WIDE ? 16 : 8;                                 // output columns a tile
    constexpr int STAGE_BYTES = ROWS * ST_ROW_BYTES;
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int M = p.M, K = p.K, S = p.n_stages;
    unsigned char* ring = smem;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)S * STAGE_BYTES);
    uint64_t* empty = full + S;
    float* red = reinterpret_cast<float*>(empty + S);                    // [ST_CONSUMERS][NW][MT][4][32]
    const int n_out = (EPI == EPI_SWIGLU || EPI == EPI_CONV_STEP) ? p.ff : p.N;
    const int n_tiles = (n_out + TROWS - 1) / TROWS;
    const int n_chunks = K / ST_COLS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) { kp_mbar_init(&full[s], 1); kp_mbar_init(&empty[s], ST_CONSUMERS); }
        kp_mbar_init_fence();
    }
    __syncthreads();

    if (warp == ST_CONSUMERS) {
        // ---- producer: the weights depend on no earlier kernel, so it starts at once (no wait on the kernel before)
        pdl_launch_dependents();
        if (lane == 0) KP_TRACE_MARK_LANE(0);
        int it = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
            const int n0 = tile * TROWS;
            const bf16* src = nullptr;
            if (lane < ROWS) {
                const int wrow = WIDE ? min(n0 + lane, n_out - 1) : (lane >> 3) * p.ff + min(n0 + (lane & 7), n_out - 1);
                src = p.W + (size_t)wrow * p.ldw;
            }
            for (int c = 0; c < n_chunks; c++, it++) {
                const int s = it % S;
                int ok = 1;
                if (lane == 0) {
                    ok = kp_mbar_wait_bounded(&empty[s], ((it / S) & 1) ^ 1, ST_WAIT_NS) ? 1 : 0;
#ifdef KP_TEST_HOOKS
                    if (ok && blockIdx.x == 0 && it == g_test_skip_stage) ok = 2;      // stage left unfilled
#endif
                    if (ok == 1) kp_mbar_expect_tx(&full[s], ROWS * ST_COLS * 2);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { alive = false; break; }
#ifdef KP_TEST_HOOKS
                if (ok == 2) continue;
#endif
                if (lane < ROWS)
                    bulk_g2s(ring + (size_t)s * STAGE_BYTES + (size_t)lane * ST_ROW_BYTES, src + (size_t)c * ST_COLS,
                             ST_COLS * 2, &full[s]);
            }
        }
        if (!alive && lane == 0) atomicExch(&g_stream_status, 1);
        if (lane == 0) KP_TRACE_MARK_LANE(3);
        return;
    }

    // ---- consumers
    const int g = lane >> 2, t = lane & 3;
    pdl_wait();                                               // from here on the activations may be read
    KP_TRACE_MARK(1);
    pdl_launch_dependents();
    int r0[MT], r1[MT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        r0[mt] = min(mt * 16 + g, M - 1);
        r1[mt] = min(mt * 16 + g + 8, M - 1);
    }
    auto load_acts = [&](uint4 (&lo)[MT], uint4 (&hi)[MT], int kb) {
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            hi[mt] = make_uint4(0, 0, 0, 0);
            lo[mt] = __ldg(reinterpret_cast<const uint4*>(p.A + (size_t)r0[mt] * p.lda) + kb * 4 + t);
            if (!HALF) hi[mt] = __ldg(reinterpret_cast<const uint4*>(p.A + (size_t)r1[mt] * p.lda) + kb * 4 + t);
        }
    };

    int it = 0;
    bool alive = true;
    const int nkb = K >> 5;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int n0 = tile * TROWS;
        float acc[NW][MT][4];
#pragma unroll
        for (int w = 0; w < NW; w++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[w][mt][i] = 0.f;
        // What the epilogue needs beside the sums and that is there already (the old value of an accumulated
        // output; the conv step's position, state and taps) is fetched now, so that its trips to L2 run under
        // the main loop instead of behind it.  (One output a thread: a tile of one m-tile and 8 columns.)
        constexpr bool PRE = MT == 1 && !WIDE && (EPI == EPI_ACCUM_F32 || EPI == EPI_CONV_STEP);
        float pre_c = 0.f, pre_hist[3] = {0.f, 0.f, 0.f}, pre_cw[4] = {0.f, 0.f, 0.f, 0.f};
        bool pre_conv = false;
        if (PRE && threadIdx.x < 128) {
            const int l = threadIdx.x & 31, i = (threadIdx.x >> 5) & 3;
            const int m = (l >> 2) + ((i & 2) ? 8 : 0), n = n0 + (l & 3) * 2 + (i & 1);
            if (m < M && n < n_out) {
                if (EPI == EPI_ACCUM_F32) pre_c = ((const float*)p.C)[(size_t)m * p.ldc + n];
                if (EPI == EPI_CONV_STEP && p.conv_k <= 4) {
                    pre_conv = true;
                    const int Kc = p.conv_k;
                    const bool fresh = p.seg_pos[m] == 0;
                    const float* st = p.conv_state + (size_t)p.seg_slot[m] * (Kc - 1) * p.ff;
                    const float* cw = p.conv_w + (size_t)n * Kc;
#pragma unroll
                    for (int k = 0; k < 3; k++)
                        if (k < Kc - 1) pre_hist[k] = fresh ? 0.f : st[(size_t)k * p.ff + n];
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        if (k < Kc) pre_cw[k] = cw[k];
                }
            }
        }
        // this warp's k-blocks: warp, warp + 8, ... (two a stage); their activations are fetched PF blocks
        // (one stage) ahead.  Fetching two stages ahead was measured and gained nothing.
        constexpr int PF = 2;
        uint4 lo[PF][MT], hi[PF][MT];
#pragma unroll
        for (int i = 0; i < PF; i++)
            if (warp + i * ST_CONSUMERS < nkb) load_acts(lo[i], hi[i], warp + i * ST_CONSUMERS);
        auto run_stage = [&](int c, auto slot0) {
            constexpr int SLOT0 = decltype(slot0)::value;
            const int s = it % S;
            if (alive && !kp_mbar_wait_bounded(&full[s], (it / S) & 1, ST_WAIT_NS)) alive = false;
            const unsigned char* stage = ring + (size_t)s * STAGE_BYTES + 16 * t;
#pragma unroll
            for (int j = 0; j < 2; j++) {
                constexpr int dummy = 0; (void)dummy;
                const int kbs = warp + j * ST_CONSUMERS;                  // block inside the stage
                const int kb = c * 16 + kbs;
                uint4 wv[NW];
#pragma unroll
                for (int w = 0; w < NW; w++)
                    wv[w] = *reinterpret_cast<const uint4*>(stage + (size_t)(w * 8 + g) * ST_ROW_BYTES + kbs * 64);
                const int sl = SLOT0 + j;
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int w = 0; w < NW; w++) {
                        mma_bf16(acc[w][mt], lo[sl][mt].x, hi[sl][mt].x, lo[sl][mt].y, hi[sl][mt].y, wv[w].x, wv[w].y);
                        mma_bf16(acc[w][mt], lo[sl][mt].z, hi[sl][mt].z, lo[sl][mt].w, hi[sl][mt].w, wv[w].z, wv[w].w);
                    }
                if (kb + PF * ST_CONSUMERS < nkb) load_acts(lo[sl], hi[sl], kb + PF * ST_CONSUMERS);
            }
            __syncwarp();
            if (lane == 0) kp_mbar_arrive(&empty[s]);                       // this warp has read the stage
            it++;
        };
        for (int c = 0; c < n_chunks; c += PF / 2) {
            run_stage(c, std::integral_constant<int, 0>{});
            if (PF == 4 && c + 1 < n_chunks) run_stage(c + 1, std::integral_constant<int, (PF == 4 ? 2 : 0)>{});
        }
        // the tile's result: the warps' partial sums, added in warp order
#pragma unroll
        for (int w = 0; w < NW; w++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) red[(((warp * NW + w) * MT + mt) * 4 + i) * 32 + lane] = acc[w][mt][i];
        consumer_sync();
        for (int e = threadIdx.x; e < (WIDE ? 2 : 1) * MT * 4 * 32; e += ST_CONSUMERS * 32) {
            const int l = e & 31, i = (e >> 5) & 3, mt = (e >> 7) % MT, wsel = WIDE ? e / (MT * 128) : 0;
            const int m = mt * 16 + (l >> 2) + ((i & 2) ? 8 : 0);
            const int n = n0 + wsel * 8 + (l & 3) * 2 + (i & 1);
            if (m >= M || n >= n_out) continue;
            float v = 0.f;
#pragma unroll
            for (int w4 = 0; w4 < ST_CONSUMERS; w4++) v += red[(((w4 * NW + wsel) * MT + mt) * 4 + i) * 32 + l];
            if (p.bias) v += p.bias[n];
            const size_t o = (size_t)m * p.ldc + n;
            if (EPI == EPI_CONV_STEP) {
                float cg = 0.f, xv = 0.f;
#pragma unroll
                for (int w4 = 0; w4 < ST_CONSUMERS; w4++) {
                    cg += red[(((w4 * NW + 1) * MT + mt) * 4 + i) * 32 + l];
                    xv += red[(((w4 * NW + NW - 1) * MT + mt) * 4 + i) * 32 + l];
                }
                if (p.bias) { cg += p.bias[p.ff + n]; xv += p.bias[2 * p.ff + n]; }
                // B, C and X as the separate product stores them, then shortconv.cu's decode step: every product and
                // sum rounded on its own (src/backend/cpu/common.c:2393-2431)
                const float b = to_f32(from_f32<bf16>(v)), cq = to_f32(from_f32<bf16>(cg)), xq = to_f32(from_f32<bf16>(xv));
                const int d = p.ff, Kc = p.conv_k;
                const float* cw = p.conv_w + (size_t)n * Kc;
                const bool fresh = p.seg_pos[m] == 0;
                float* st = p.conv_state + (size_t)p.seg_slot[m] * (Kc - 1) * d;
                const float bx = __fmul_rn(b, xq);
                float hist[15], tap[16];
                if (pre_conv) {
#pragma unroll
                    for (int k = 0; k < 3; k++) hist[k] = pre_hist[k];
#pragma unroll
                    for (int k = 0; k < 4; k++) tap[k] = pre_cw[k];
                } else {
                    for (int k = 0; k < Kc - 1; k++) hist[k] = fresh ? 0.f : st[(size_t)k * d + n];
                    for (int k = 0; k < Kc; k++) tap[k] = cw[k];
                }
                float sum;
                if (Kc == 3) {
                    sum = __fadd_rn(__fadd_rn(__fmul_rn(hist[0], tap[0]), __fmul_rn(hist[1], tap[1])), __fmul_rn(bx, tap[2]));
                } else {
                    sum = __fmul_rn(bx, tap[Kc - 1]);
                    for (int k = 0; k < Kc - 1; k++) sum = __fadd_rn(sum, __fmul_rn(hist[k], tap[k]));
                }
                if (p.conv_bias) sum = __fadd_rn(sum, p.conv_bias[n]);
                ((bf16*)p.C)[o] = from_f32<bf16>(__fmul_rn(cq, sum));
                for (int k = 0; k + 1 < Kc - 1; k++) st[(size_t)k * d + n] = hist[k + 1];
                st[(size_t)(Kc - 2) * d + n] = bx;
            } else if (EPI == EPI_SWIGLU) {
                float u = 0.f;
#pragma unroll
                for (int w4 = 0; w4 < ST_CONSUMERS; w4++) u += red[(((w4 * NW + NW - 1) * MT + mt) * 4 + i) * 32 + l];
                if (p.bias) u += p.bias[p.ff + n];
                // gate and up are rounded to the storage type before the activation, as the unfused path stores them
                const float gq = to_f32(from_f32<bf16>(v)), uq = to_f32(from_f32<bf16>(u));
                ((bf16*)p.C)[o] = from_f32<bf16>((gq / (1.0f + expf(-gq))) * uq);
            } else if (EPI == EPI_STORE) {
                ((bf16*)p.C)[o] = from_f32<bf16>(v);
            } else if (EPI == EPI_STORE_F32) {
                ((float*)p.C)[o] = v;
            } else {
                ((float*)p.C)[o] = (PRE ? pre_c : ((float*)p.C)[o]) + v;
            }
        }
        consumer_sync();                                                 // red is free for the next tile
    }
    KP_TRACE_MARK(2);
    if (!alive) {
        if (lane == 0) atomicExch(&g_stream_status, 1);
        kp_linger_after_failure();
    }
}

static size_t smem_bytes(int NW, int MT, int n_stages) {
    return (size_t)n_stages * NW * 8 * ST_ROW_BYTES + (size_t)2 * n_stages * 8 +
           sizeof(float) * (ST_CONSUMERS * NW * MT * 128);
}

static int n_sm() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}


template <typename Kern>
static int launch_pdl(Kern kern, dim3 grid, size_t smem, cudaStream_t s, const StreamArgs& a) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return (int)kp_launch_pdl(kern, grid, dim3(ST_THREADS), smem, s, a);
}

template <int MT, bool HALF>
static int launch_epi(StreamArgs a, int epi, cudaStream_t s) {
    // tiles of 16 rows of W from three m-tiles on (see the kernel; measured at 64 batch rows: 2048 x 5632 15.5 us
    // against 23.7, 2048 x 2048 8.0 against 12.2; at 32 rows the narrow tile is as fast or faster)
    constexpr bool WIDE = MT >= 3;
    const bool joins = epi == EPI_SWIGLU || epi == EPI_CONV_STEP;        // a tile joins rows of W that lie ff apart
    const int NW = epi == EPI_CONV_STEP ? 3 : ((epi == EPI_SWIGLU || WIDE) ? 2 : 1);
    const int n_out = joins ? a.ff : a.N;
    const int n_tiles = (n_out + (WIDE && !joins ? 15 : 7)) / (WIDE && !joins ? 16 : 8);
    // Measured on B200 (8 and 16 rows): three CTAs an SM with a 64 KB ring is best or tied for products with
    // many tiles (6144 x 2048: 6.9 us against 8.1 with 53 KB); a product with at most two tiles an SM (2048
    // rows) does better with two CTAs an SM and more of its long rows in flight (2048 x 5632: 8.3 against 10.3).
    const bool few = n_tiles <= 2 * n_sm();
    const int per_sm = few ? 2 : 3;
    const int ring = few ? ST_RING_BYTES_FEW : ST_RING_BYTES;
    a.n_stages = ring / (NW * 8 * ST_ROW_BYTES);
    if (a.n_stages < 2) a.n_stages = 2;
    int g = n_sm() * per_sm;
    if (g > n_tiles) g = n_tiles;
    dim3 grid(g);
    const size_t sm = smem_bytes(NW, MT, a.n_stages);
    switch (epi) {
        case EPI_STORE: return launch_pdl(gemm_stream_kernel<MT, HALF, EPI_STORE, WIDE>, grid, sm, s, a);
        case EPI_STORE_F32: return launch_pdl(gemm_stream_kernel<MT, HALF, EPI_STORE_F32, WIDE>, grid, sm, s, a);
        case EPI_ACCUM_F32: return launch_pdl(gemm_stream_kernel<MT, HALF, EPI_ACCUM_F32, WIDE>, grid, sm, s, a);
        case EPI_SWIGLU: return launch_pdl(gemm_stream_kernel<MT, HALF, EPI_SWIGLU, false>, grid, sm, s, a);
        case EPI_CONV_STEP:
            // at most 16 rows: from 32 rows on the tensor-core kernel and the separate conv kernel are faster (measured)
            if constexpr (MT == 1) return launch_pdl(gemm_stream_kernel<MT, HALF, EPI_CONV_STEP, false>, grid, sm, s, a);
            else return KP_ERR_UNSUPPORTED;
        default: return KP_ERR_BAD_ARG;
    }
}

static int launch_m(const StreamArgs& a, int epi, cudaStream_t s) {
    if (a.M <= 8) return launch_epi<1, true>(a, epi, s);
    if (a.M <= 16) return launch_epi<1, false>(a, epi, s);
    if (a.M <= 32) return launch_epi<2, false>(a, epi, s);
    if (a.M <= 48) return launch_epi<3, false>(a, epi, s);
    return launch_epi<4, false>(a, epi, s);
}

static int check_common(StreamArgs& a, int M, int N, int K, int ldw, const void* W, int epi) {
    if (M > 64 || K < ST_COLS || (K % ST_COLS) || (ldw & 7) || ((uintptr_t)W & 15)) return KP_ERR_UNSUPPORTED;
    a.ff = 0;
    if (epi == EPI_SWIGLU) {
        if (N & 1) return KP_ERR_BAD_ARG;
        a.ff = N / 2;
    }
    if (epi == EPI_CONV_STEP) {
        if (N % 3) return KP_ERR_BAD_ARG;
        a.ff = N / 3;
    }
    return 0;
}

extern "C" {

int kp_gemm_stream(const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc, int M, int N,
                   int K, int epi, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    StreamArgs a = {};
    int st = check_common(a, M, N, K, ldw, W, epi);
    if (st) return st;
    if ((lda & 7) || ((uintptr_t)A & 15)) return KP_ERR_UNSUPPORTED;
    a.A = (const bf16*)A; a.lda = lda; a.W = (const bf16*)W; a.ldw = ldw; a.bias = bias; a.C = C; a.ldc = ldc;
    a.M = M; a.N = N; a.K = K;
    return launch_m(a, epi, (cudaStream_t)stream);
}

// The in_proj of the gated short convolution with the conv step of a decode step in its epilogue: W = [B; C; X]
// ([3 d, K]), C = [M, d] bfloat16; conv_w [d][conv_k], conv_bias [d] or null, state [slots][conv_k - 1][d], and
// for each of the M <= 16 rows its position (seg_pos) and state slot (seg_slot).  Rows are one-row segments.
int kp_gemm_stream_conv_step(const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc, int M,
                             int N, int K, const float* conv_w, const float* conv_bias, float* conv_state,
                             const int* seg_pos, const int* seg_slot, int conv_k, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    StreamArgs a = {};
    int st = check_common(a, M, N, K, ldw, W, EPI_CONV_STEP);
    if (st) return st;
    if (M > 16 || (lda & 7) || ((uintptr_t)A & 15) || conv_k < 2 || conv_k > 16 || !conv_w || !conv_state || !seg_pos ||
        !seg_slot)
        return KP_ERR_UNSUPPORTED;
    a.A = (const bf16*)A; a.lda = lda; a.W = (const bf16*)W; a.ldw = ldw; a.bias = bias; a.C = C; a.ldc = ldc;
    a.M = M; a.N = N; a.K = K;
    a.conv_w = conv_w; a.conv_bias = conv_bias; a.conv_state = conv_state; a.seg_pos = seg_pos; a.seg_slot = seg_slot;
    a.conv_k = conv_k;
    return launch_m(a, EPI_CONV_STEP, (cudaStream_t)stream);
}

}  // extern "C"
