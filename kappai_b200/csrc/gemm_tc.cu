// C[M,N] = A[M,K] * W[N,K]^T (bfloat16 in, float32 accumulation) on the 5th-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory, operands brought to shared memory by TMA.
// The product of prompt portions, and of few-row steps where it was measured faster than weight streaming.
//
// Persistent CTAs, one an SM; a CTA computes tiles of 128 x BN of C (tile b, b + grid, ...; m runs fastest so
// that the CTAs that run together share W tiles in L2).  BN is 256 or 128 for products of many rows (chosen by
// a cost model of rounds over the SMs), and for at most 128 rows the narrowest of 256..32 that still runs in
// one round, so that as many CTAs as possible pull on the memory.  Roles by warp:
//   warp 0   : TMA producer.  For every k-block of 64 it waits for a free stage, arms the stage's "full"
//              mbarrier with the byte count and issues the tiled loads of the A box (128 rows x 64, or only
//              the rows there are, rounded up to 8, when M < 128) and the W box (BN rows x 64), both with
//              the 128-byte swizzle, no multicast.  The ring has as many stages as fit shared memory.
//   warp 1   : allocates 2 x BN columns of tensor memory (two accumulators: the epilogue of a tile runs under
//              the main loop of the next), then one lane issues the MMAs: four tcgen05.mma (128 x BN x 16) per
//              stage, descriptors advanced by 32 bytes inside the swizzled rows; tcgen05.commit frees the
//              stage ("empty" mbarrier) and, after the last k-block, signals "accumulator full".
//   the rest : epilogue, two warps for each quarter of the 128 lanes of tensor memory (a warp may only read
//              the lanes 32 * (warp % 4) ...), taking the 32-column pieces in turn so that more loads and
//              stores are in flight.  Each reads its lanes with tcgen05.ld (32 columns at a time), applies
//              bias / residual accumulation / SwiGLU, writes its rows of C and hands the accumulator back.
// Rows of A beyond M and rows of W beyond N are zero-filled by TMA (out-of-bounds fill) and masked at the
// store; K needs no padding (the tail of the last k-block is zero-filled too) but K % 8 == 0 (16-byte rows).
// Each output row sums its k-blocks in order, so a row's result does not depend on M.
//
// SwiGLU epilogue: W holds gate rows then up rows (ff apart).  The CTA's W tile is BN/2 gate rows and the
// matching BN/2 up rows (two TMA boxes into one tile), so accumulator columns c and BN/2 + c are the gate and
// up of one output column: the epilogue writes silu(gate) * up.
//
// Split over K (17 to 1024 rows: up to eight rows of tiles, where that brings fewer bytes into the busiest SM): the
// product is cut along K into `splits` parts, the unit of
// work being (tile, part), all units in one round over the SMs and the parts of a tile one thread-block cluster.
// Every CTA leaves the float32 sums of its unit in its own shared memory (the ring is free by then); after the
// cluster's barrier each adds up its share of the tile, reading the other CTAs' sums over the cluster's shared
// memory, the parts in order of their number -- so the result does not depend on timing -- then the epilogue.
// With it every SM brings in a part of A only, and wide tiles still keep all SMs streaming.
//
// Every wait on an mbarrier is bounded.  A wait that gives up sets a status word (kp_tc_status), the CTA
// stops issuing work, still frees its tensor memory and returns.
#include "tcgen05.cuh"

#define EPI_STORE 0
#define EPI_STORE_F32 1
#define EPI_ACCUM_F32 2
#define EPI_SWIGLU 3

#define TC_BM 128
#define TC_BK 64
#define TC_EPI_PER_Q 2                       // epilogue warps for each quarter of the tensor-memory lanes
#define TC_THREADS (64 + TC_EPI_PER_Q * 128) // the producer warp, the MMA warp and the epilogue warps

KP_STATUS_WORD(g_tc_status, tc)          // 0 ok; 1: a bounded wait gave up

struct TcArgs {
    const float* bias;
    void* C; int ldc;
    int M, N, K, ff;
    int vec_ok;                             // rows of C are 16-byte aligned: whole pieces go out in 16-byte stores
    int a_rows;                             // rows of the A box: 128, fewer (a multiple of 8) when M < 128
    int n_stages;                           // stages of the ring
    int splits;                             // parts along K (1: none); only with one row of tiles; the cluster's size
    int kb_per_split;                       // k-blocks a part
};

// all threads of all CTAs of the cluster; what they wrote to shared memory before is visible to the others after
__device__ __forceinline__ void kp_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 16 bytes of the shared memory of the cluster's CTA `rank`, at the place that `addr` has in this CTA's
__device__ __forceinline__ float4 kp_ld_cluster_f4(uint32_t addr, int rank) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(addr), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(ra) : "memory");
    return v;
}

// the epilogue warps (threads 64 ...) among themselves
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_PER_Q * 128) : "memory"); }

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
}

// A piece of W output columns (32, or 4 in the split's reduction) of row m, from its sums g (and u: the up half,
// SwiGLU), to C: bias, SwiGLU or accumulation, and the store (vector stores where rows of C are 16-byte aligned).
template <int EPI, int W>
__device__ __forceinline__ void tc_finish(const TcArgs& p, int n_lim, const float (&g)[W], const float (&u)[W], int m,
                                          int n_base) {
    float v[W];
#pragma unroll
    for (int j = 0; j < W; j++) {
        float x = g[j];
        if (p.bias && n_base + j < n_lim) x += p.bias[n_base + j];
        if (EPI == EPI_SWIGLU) {
            float up = u[j];
            if (p.bias && n_base + j < n_lim) up += p.bias[p.ff + n_base + j];
            // gate and up are rounded to the storage type first, as the unfused path stores them
            const float gq = to_f32(from_f32<bf16>(x)), uq = to_f32(from_f32<bf16>(up));
            x = (gq / (1.0f + expf(-gq))) * uq;
        }
        v[j] = x;
    }
    const bool whole = p.vec_ok && n_base + W <= n_lim;                  // vector stores of the whole piece
    if (EPI == EPI_STORE || EPI == EPI_SWIGLU) {
        bf16* dst = (bf16*)p.C + (size_t)m * p.ldc + n_base;
        if (whole && W >= 8) {
#pragma unroll
            for (int j = 0; j + 8 <= W; j += 8) {
                uint4 o;
                o.x = pack2(v[j], v[j + 1]); o.y = pack2(v[j + 2], v[j + 3]);
                o.z = pack2(v[j + 4], v[j + 5]); o.w = pack2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(dst + j) = o;
            }
        } else if (whole && W == 4) {
            *reinterpret_cast<uint2*>(dst) = make_uint2(pack2(v[0], v[1]), pack2(v[2], v[3]));
        } else {
#pragma unroll
            for (int j = 0; j < W; j++)
                if (n_base + j < n_lim) dst[j] = from_f32<bf16>(v[j]);
        }
    } else {
        float* dst = (float*)p.C + (size_t)m * p.ldc + n_base;
        if (whole) {
#pragma unroll
            for (int j = 0; j < W; j += 4) {
                float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                if (EPI == EPI_ACCUM_F32) {
                    const float4 c4 = *reinterpret_cast<const float4*>(dst + j);
                    o.x += c4.x; o.y += c4.y; o.z += c4.z; o.w += c4.w;
                }
                *reinterpret_cast<float4*>(dst + j) = o;
            }
        } else {
#pragma unroll
            for (int j = 0; j < W; j++) {
                if (n_base + j < n_lim) {
                    float x = v[j];
                    if (EPI == EPI_ACCUM_F32) x += dst[j];
                    dst[j] = x;
                }
            }
        }
    }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, const TcArgs p) {
    constexpr int B_BYTES = BN * TC_BK * 2;
    constexpr int N_OUT_TILE = (EPI == EPI_SWIGLU) ? BN / 2 : BN;       // output columns of the tile
    const int A_BYTES = p.a_rows * TC_BK * 2;                            // the rows of A that are brought in
    const int STAGES = p.n_stages;
    extern __shared__ unsigned char smem[];
    // STAGES x (A tile | B tile); the swizzled tiles must start on 1024-byte boundaries.  With fewer than 128
    // rows of A a stage is smaller and the ring has more of them; the MMA still reads 128 rows from the
    // stage's start (on into the W tile and beyond: the host leaves room after the last stage), and what it
    // makes of the rest lands in accumulator rows that nobody reads.
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * (A_BYTES + B_BYTES) + (TC_BM * TC_BK * 2 - A_BYTES));
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;                                  // [2]: accumulator b holds a finished tile
    uint64_t* acc_empty = acc_full + 2;                                   // [2]: accumulator b has been read out
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = (p.K + TC_BK - 1) / TC_BK;
    const int n_out = (EPI == EPI_SWIGLU) ? p.ff : p.N;
    const int tiles_m = (p.M + TC_BM - 1) / TC_BM, tiles_n = (n_out + N_OUT_TILE - 1) / N_OUT_TILE;
    const int n_tiles = tiles_m * tiles_n;
    const int S = p.splits;                                              // parts along K; a unit of work is (tile, part)
    const int n_units = n_tiles * S;
    // the CTA is persistent: it takes tiles blockIdx.x, blockIdx.x + gridDim.x, ... ; consecutive tiles
    // share the W tile (m runs fastest), so the CTAs that run together read the same few W tiles from L2

    // set-up that depends on no earlier kernel comes before the wait on it
    if (threadIdx.x == 0) {
        // (the tensor maps are fetched now: the first TMA load through a map that has not been used waits for it)
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmA)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmW)) : "memory");
        for (int s = 0; s < STAGES; s++) { kp_mbar_init(&full[s], 1); kp_mbar_init(&empty[s], 1); }
        for (int b2 = 0; b2 < 2; b2++) { kp_mbar_init(&acc_full[b2], 1); kp_mbar_init(&acc_empty[b2], 4 * TC_EPI_PER_Q); }
        *abort_flag = 0;
        kp_mbar_init_fence();
    }
    if (warp == 1) kp_tmem_alloc(tmem_slot, 2 * BN);                         // two accumulators of BN columns
    kp_tc_fence_before();
    __syncthreads();
    kp_tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool parts_ok = false;                                                // (epilogue warps) this CTA's sums are in shared memory

    if (warp == 0) {
        if (lane == 0) {
            auto load_w = [&](int s, int kb, int n0) {
                unsigned char* b_dst = tiles + (size_t)s * (A_BYTES + B_BYTES) + A_BYTES;
                if (EPI == EPI_SWIGLU) {
                    kp_tma_load_2d(b_dst, &tmW, kb * TC_BK, n0, &full[s]);                       // gate rows
                    kp_tma_load_2d(b_dst + B_BYTES / 2, &tmW, kb * TC_BK, p.ff + n0, &full[s]);  // up rows
                } else {
                    kp_tma_load_2d(b_dst, &tmW, kb * TC_BK, n0, &full[s]);
                }
            };
            // The weights depend on no earlier kernel: the W tiles of the first unit's first k-blocks (as many as
            // the ring has stages) are on their way before the wait on the kernel before; their A tiles follow it.
            int pre = 0;
            if ((int)blockIdx.x < n_units) {
                const int tile = blockIdx.x / S, part = blockIdx.x - tile * S;
                const int n0 = (tile / tiles_m) * N_OUT_TILE;
                const int kb_lo = part * p.kb_per_split, kb_hi = min(n_kb, kb_lo + p.kb_per_split);
                pre = min(STAGES, kb_hi - kb_lo);
                for (int i = 0; i < pre; i++) {
                    kp_mbar_expect_tx(&full[i], A_BYTES + B_BYTES);
                    load_w(i, kb_lo + i, n0);
                }
            }
            KP_TRACE_MARK_LANE(0);
            pdl_wait();
            KP_TRACE_MARK_LANE(1);
            pdl_launch_dependents();
            int s = 0;                                                    // stage, and the parity of its round
            uint32_t ph = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
                const int tile = unit / S, part = unit - tile * S;
                const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * N_OUT_TILE;
                const int kb_lo = part * p.kb_per_split, kb_hi = min(n_kb, kb_lo + p.kb_per_split);
                for (int kb = kb_lo; kb < kb_hi; kb++) {
                    unsigned char* a_dst = tiles + (size_t)s * (A_BYTES + B_BYTES);
                    if (pre > 0) {
                        pre--;                                            // armed, W on its way: only A is missing
                    } else {
                        if (*abort_flag || !kp_mbar_wait_bounded(&empty[s], ph ^ 1)) { *abort_flag = 1; ok = false; break; }
                        kp_mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                        load_w(s, kb, n0);
                    }
                    kp_tma_load_2d(a_dst, &tmA, kb * TC_BK, m0, &full[s]);
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        kp_pdl_begin();
        if (lane == 0) {
            constexpr uint32_t idesc = kp_umma_idesc(TC_BM, BN);
            int s = 0, ti = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x, ti++) {
                const int b2 = ti & 1;                                    // accumulator of this unit
                if (*abort_flag || !kp_mbar_wait_bounded(&acc_empty[b2], ((ti >> 1) & 1) ^ 1)) { *abort_flag = 1; break; }
                kp_tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(b2 * BN);
                const int part = unit % S;
                const int kb_lo = part * p.kb_per_split, kb_hi = min(n_kb, kb_lo + p.kb_per_split);
                for (int kb = kb_lo; kb < kb_hi; kb++) {
                    if (!kp_mbar_wait_bounded(&full[s], ph)) { *abort_flag = 1; ok = false; break; }
                    kp_tc_fence_after();
                    const uint32_t a_addr = kp_smem_u32(tiles + (size_t)s * (A_BYTES + B_BYTES));
                    const uint64_t adesc = kp_umma_desc(a_addr), bdesc = kp_umma_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; k++)      // 32 bytes along K inside the swizzled row: +2 in the address field
                        kp_umma_bf16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, ((kb - kb_lo) | k) ? 1u : 0u);
                    kp_umma_commit(&empty[s]);                    // the stage is free when these MMAs have read it
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (ok) kp_umma_commit(&acc_full[b2]);            // arrives when every MMA of the tile has completed
            }
        }
    } else {
        kp_pdl_begin();
        // epilogue: warp w reads the 32 lanes (w % 4) * 32 ... of tensor memory; it works on unit i while the
        // MMA warp already fills the other accumulator with unit i + 1
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;                                 // which of the quarter's warps
        int ti = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x, ti++) {
            const int b2 = ti & 1;
            const int tile = unit / S;
            const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * N_OUT_TILE;
            if (!kp_mbar_wait_bounded(&acc_full[b2], (ti >> 1) & 1) || *abort_flag) { ok = false; break; }
            kp_tc_fence_after();
            const int m = m0 + q * 32 + lane;
            const uint32_t lane_base = tmem_base + (uint32_t)(b2 * BN) + ((uint32_t)(q * 32) << 16);
            if (S == 1) {
#pragma unroll 1
                for (int c = half * 32; c < N_OUT_TILE; c += 32 * TC_EPI_PER_Q) {
                    uint32_t r[32], u[32];
                    kp_tmem_ld32(lane_base + c, r);
                    if (EPI == EPI_SWIGLU) kp_tmem_ld32(lane_base + BN / 2 + c, u);
                    if (m < p.M) {
                        float g[32], up[32];
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            g[j] = __uint_as_float(r[j]);
                            up[j] = EPI == EPI_SWIGLU ? __uint_as_float(u[j]) : 0.f;
                        }
                        tc_finish<EPI, 32>(p, n_out, g, up, m, n0 + c);
                    }
                }
                // this warp has read the accumulator out: hand it back to the MMA warp
                kp_tc_fence_before();
                __syncwarp();
                if (lane == 0) kp_mbar_arrive(&acc_empty[b2]);
                continue;
            }
            // split over K: this part's sums of the whole accumulator (BN columns) go to this CTA's shared memory
            // (the ring is free: every MMA of the unit has completed), laid out [piece of 32 columns][float4 of
            // the piece][row of the tile][4] so that a warp's rows lie one behind the other; the tile's CTAs -- a cluster --
            // add them up below
            float4* mine = reinterpret_cast<float4*>(tiles);
            const int R = min(TC_BM, p.M - m0);                          // rows of this tile
#pragma unroll 1
            for (int c = half * 32; c < BN; c += 32 * TC_EPI_PER_Q) {
                uint32_t r[32];
                kp_tmem_ld32(lane_base + c, r);
                if (m < p.M) {
                    float4* dst = mine + (size_t)(c >> 5) * 8 * R + (m - m0);
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        dst[(size_t)j * R] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                           __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                }
            }
            kp_tc_fence_before();
            __syncwarp();
            if (lane == 0) kp_mbar_arrive(&acc_empty[b2]);
            parts_ok = true;
        }
        if (!ok && lane == 0) atomicExch(&g_tc_status, 1);
    }
    kp_tc_fence_before();
    __syncthreads();
    if (S > 1) {
        // Split over K: the CTAs of a tile are a cluster (rank = part).  When all of them have their sums in
        // shared memory, each adds up its share of the tile, reading the others' over the cluster's shared
        // memory: the parts in the order of their numbers, so the result does not depend on timing; then the
        // epilogue.  Every thread of every CTA comes here, also after a wait that gave up, so the cluster's
        // barriers always complete; no CTA leaves before the others have read its sums.
        kp_cluster_sync();
        if (warp >= 2 && parts_ok) {
            const int tile = blockIdx.x / S, part = blockIdx.x - tile * S;
            const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * N_OUT_TILE;
            const int R = min(TC_BM, p.M - m0);                           // rows of this tile
            const int n_vec = N_OUT_TILE / 32 * R * 8;                    // float4s of the tile's output
            const int lo = (int)((long long)n_vec * part / S), hi = (int)((long long)n_vec * (part + 1) / S);
            const uint32_t mine = kp_smem_u32(tiles);
            const uint32_t up_off = (uint32_t)(BN / 64) * 8 * R * 16;     // bytes from a gate piece to its up piece
            constexpr int NT = TC_EPI_PER_Q * 128;
            // VI float4s a thread at a time, the parts four by four: the loads of a round are all in flight
            // together (each is a trip to another SM), the sums still run in the order of the parts
            constexpr int VI = EPI == EPI_SWIGLU ? 2 : 4;
            for (int i0 = lo + (int)threadIdx.x - 64; i0 < hi; i0 += VI * NT) {
                float4 g[VI], up[VI];
#pragma unroll
                for (int v = 0; v < VI; v++) g[v] = up[v] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int sp0 = 0; sp0 < S; sp0 += 4) {
                    float4 t[VI][4], t2[VI][4];
#pragma unroll
                    for (int v = 0; v < VI; v++)
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int idx = i0 + v * NT;
                            t[v][u] = t2[v][u] = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (idx < hi && sp0 + u < S) {
                                t[v][u] = kp_ld_cluster_f4(mine + (uint32_t)idx * 16, sp0 + u);
                                if (EPI == EPI_SWIGLU) t2[v][u] = kp_ld_cluster_f4(mine + (uint32_t)idx * 16 + up_off, sp0 + u);
                            }
                        }
#pragma unroll
                    for (int v = 0; v < VI; v++)
#pragma unroll
                        for (int u = 0; u < 4; u++)
                            if (sp0 + u < S) {
                                g[v].x += t[v][u].x; g[v].y += t[v][u].y; g[v].z += t[v][u].z; g[v].w += t[v][u].w;
                                up[v].x += t2[v][u].x; up[v].y += t2[v][u].y; up[v].z += t2[v][u].z; up[v].w += t2[v][u].w;
                            }
                }
#pragma unroll
                for (int v = 0; v < VI; v++) {
                    const int idx = i0 + v * NT;
                    if (idx < hi) {
                        const float g4[4] = {g[v].x, g[v].y, g[v].z, g[v].w}, u4[4] = {up[v].x, up[v].y, up[v].z, up[v].w};
                        const int piece = idx / (R * 8), rem = idx - piece * (R * 8);
                        const int j4 = rem / R, row = rem - j4 * R;
                        tc_finish<EPI, 4>(p, n_out, g4, u4, m0 + row, n0 + piece * 32 + j4 * 4);
                    }
                }
            }
        }
        kp_cluster_sync();
    }
    if (threadIdx.x == 64) KP_TRACE_MARK_LANE(2);
    if (warp == 1) kp_tmem_dealloc(tmem_base, 2 * BN);
}

// ------------------------------------------------------------------------------------------ host side
#define TC_SMEM_KB 208                       // shared memory for the ring
#ifndef TC_SPLIT_MAX_M_TILES
#define TC_SPLIT_MAX_M_TILES 8               // rows of tiles up to which a product may be cut along K
#endif
#ifndef TC_SPLIT_COST_KB
#define TC_SPLIT_COST_KB 64                  // what a split over K costs beside the operand reads, as KB brought into an SM
#endif

// SMs of the current device (asked once)
static int tc_n_sm() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    return sms;
}

// Shared memory of a launch: `stages` ring stages, the slack behind a short last stage, barriers, alignment.
static size_t tc_smem(int a_rows, int bn, int* stages_out) {
    const int stage = a_rows * TC_BK * 2 + bn * TC_BK * 2;
    const int slack = (TC_BM - a_rows) * TC_BK * 2;            // the MMA's reads past a short last stage
    int stages = (TC_SMEM_KB * 1024 - slack) / stage;
    if (stages > 24) stages = 24;
    if (stages < 2) stages = 2;
    *stages_out = stages;
    return (size_t)stages * stage + slack + (size_t)(2 * stages + 4) * 8 + 16 + 1024;
}

template <int BN, int EPI>
static int prepare(size_t smem) {
    auto kern = gemm_tc_kernel<BN, EPI>;
    static size_t attr_smem = 0;
    if (smem > attr_smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_smem = smem;
    }
    return 0;
}

// Clusters of `cluster` CTAs of this kernel that the device runs at once (asked once for each size; 0 if it cannot
// be said): a split over K wants all its tiles' clusters in one round.
template <int BN, int EPI>
static int max_clusters(int cluster, size_t smem) {
    static int known[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    if (cluster < 2 || cluster > 8) return 0;
    if (known[cluster] == 0) {
        known[cluster] = -1;
        if (prepare<BN, EPI>(smem) == 0) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(cluster * 64); cfg.blockDim = dim3(TC_THREADS); cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr; cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<BN, EPI>, &cfg) == cudaSuccess && n > 0) known[cluster] = n;
            else cudaGetLastError();
        }
    }
    return known[cluster] > 0 ? known[cluster] : 0;
}

template <int BN, int EPI>
static int launch(const CUtensorMap& ta, const CUtensorMap& tw, TcArgs a, cudaStream_t s) {
    int stages = 0;
    const size_t smem = tc_smem(a.a_rows, BN, &stages);
    a.n_stages = stages;
    int st = prepare<BN, EPI>(smem);
    if (st) return st;
    const int n_out = (EPI == EPI_SWIGLU) ? a.ff : a.N;
    const int n_tile = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
    const int n_units = ((n_out + n_tile - 1) / n_tile) * ((a.M + TC_BM - 1) / TC_BM) * a.splits;
    const int sms = tc_n_sm();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.splits > 1 ? n_units : (n_units < sms ? n_units : sms));   // persistent: one CTA an SM
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 1;
    if (a.splits > 1) {                                        // the parts of a tile: one cluster
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = a.splits; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    cfg.attrs = attr;
    cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, EPI>, ta, tw, a);
    return kp_launch_status();
}

// Clusters of `cluster` CTAs that run at once, for the tile width and epilogue of a launch.
static int tc_max_clusters(int bn, int epi, int cluster, int a_rows) {
    int stages = 0;
    const size_t smem = tc_smem(a_rows, bn, &stages);
#define TC_MC(BN_, EPI_) return max_clusters<BN_, EPI_>(cluster, smem);
#define TC_MC_BN(EPI_)                                             \
    switch (bn) {                                                  \
        case 256: TC_MC(256, EPI_)                                 \
        case 128: TC_MC(128, EPI_)                                 \
        case 64: TC_MC(64, EPI_)                                   \
        default: return 0;                                         \
    }
    switch (epi) {
        case EPI_STORE: TC_MC_BN(EPI_STORE)
        case EPI_STORE_F32: TC_MC_BN(EPI_STORE_F32)
        case EPI_ACCUM_F32: TC_MC_BN(EPI_ACCUM_F32)
        case EPI_SWIGLU: TC_MC_BN(EPI_SWIGLU)
        default: return 0;
    }
#undef TC_MC_BN
#undef TC_MC
}

extern "C" {

// epi: 0 store bf16, 1 store f32, 2 accumulate into f32, 3 SwiGLU (W = [gate; up], N = 2*ff, output [M, ff] bf16).
// split: products of 17 to 1024 rows may be cut along K (0: never).
int kp_gemm_tc_split(const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc, int M, int N,
                     int K, int epi, int split, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K < 8 || (K & 7) || (lda & 7) || (ldw & 7) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return KP_ERR_UNSUPPORTED;
    if ((long long)((M + TC_BM - 1) / TC_BM) > 65535) return KP_ERR_UNSUPPORTED;
    TcArgs a = {};
    a.bias = bias; a.C = C; a.ldc = ldc; a.M = M; a.N = N; a.K = K; a.ff = 0;
    {
        const int esz = (epi == EPI_STORE || epi == EPI_SWIGLU) ? 2 : 4;
        a.vec_ok = (((uintptr_t)C & 15) == 0 && ((size_t)ldc * esz) % 16 == 0) ? 1 : 0;
    }
    if (epi == EPI_SWIGLU) {
        if (N & 1) return KP_ERR_BAD_ARG;
        a.ff = N / 2;
    }
    const int n_out = epi == EPI_SWIGLU ? a.ff : N;
    // Tile width.  Many rows: by a small cost model: a CTA's main loop is bound by the bytes that it brings
    // into shared memory for each k-block (128 rows of A and BN rows of W), so a narrow tile costs about 2/3
    // of a wide one and does half the work; the number of rounds over the SMs decides between them.
    // At most 128 rows (one row of tiles, W streamed once): see below.
    const long long m_tiles = (M + TC_BM - 1) / TC_BM;
    const int sms = tc_n_sm();
    const int lowest = epi == EPI_SWIGLU ? 64 : 32;                      // the narrowest tile
    auto tiles_at = [&](int w) { const int cols = epi == EPI_SWIGLU ? w / 2 : w; return (n_out + cols - 1) / cols; };
    int bn;
    if (m_tiles > 1) {
        const long long rounds_wide = (((n_out + 255) / 256) * m_tiles + sms - 1) / sms;
        const long long rounds_narrow = (((n_out + 127) / 128) * m_tiles + sms - 1) / sms;
        bn = (epi == EPI_SWIGLU || rounds_wide * 3 <= rounds_narrow * 2) ? 256 : 128;
    } else {
        // the narrowest tile that still runs in one round over the SMs (as many CTAs as possible pull on the
        // memory, none waits for a second round); products too wide for that take the widest tile
        bn = 256;
        while (bn > lowest && tiles_at(bn / 2) <= sms) bn /= 2;
    }
    // 17 to 128 rows (one row of tiles; for more see below): what bounds the product is the bytes that the busiest SM brings in, about
    // 45 GB/s an SM whatever the source -- its share of W and, for every tile, all the rows of A.  Unsplit, a
    // narrow tile reads A once for a few rows of W (64 rows by 2048 x 5632 in 32-row tiles: 720 KB of A for 360 KB
    // of W) and wide tiles leave SMs idle.  So the product is cut along K as well: (tile width, parts) is chosen
    // so that the units fill one round over the SMs and a unit brings in the fewest bytes; the price of the split
    // (partial sums out and in, the wait for the other parts) is counted as TC_SPLIT_COST_KB of traffic.
    a.splits = 1;
    a.kb_per_split = (K + TC_BK - 1) / TC_BK;
    a.a_rows = M >= TC_BM ? TC_BM : (M + 7) / 8 * 8;
    if (m_tiles <= TC_SPLIT_MAX_M_TILES && M > 16 && split) {
        // (the same holds for a few rows of tiles -- a prompt portion or decoded tokens beside one, 129 to 1024
        // rows -- where the product has few tiles and a long K: 264 rows by 2048 x 5632 are 48 tiles of 88 k-blocks)
        const int rows = M < TC_BM ? M : TC_BM;                          // rows of a tile
        const int n_kb = (K + TC_BK - 1) / TC_BK;
        long long best = -1;
        int best_bn = bn, best_sp = 1;
        for (int w = 256; w >= (lowest < 64 ? 64 : lowest); w /= 2) {
            const int tiles = tiles_at(w) * (int)m_tiles;
            const long long rounds = (tiles + sms - 1) / sms;
            int stages = 0;
            const size_t ring = tc_smem(a.a_rows, w, &stages) - 2048;
            for (int sp = 1; sp <= 8; sp++) {
                if (sp > 1) {
                    if (tiles * sp > sms || sp * 2 > n_kb || (size_t)rows * w * 4 > ring) break;
                    if (tiles > tc_max_clusters(w, epi, sp, a.a_rows)) continue;  // the clusters would not all run at once
                }
                const int kbs = (n_kb + sp - 1) / sp;
                if (sp > 1 && (n_kb + kbs - 1) / kbs != sp) continue;            // a part would be empty
                long long cost = (sp == 1 ? rounds * n_kb : kbs) * (long long)(TC_BK * 2) * (w + a.a_rows);
                if (sp > 1) {
                    // the sums that a CTA reads from the others come in over the same port
                    cost += TC_SPLIT_COST_KB * 1024 + (long long)rows * w * 4 * (sp - 1) / sp;
                }
                if (best < 0 || cost < best) { best = cost; best_bn = w; best_sp = sp; }
            }
        }
        if (best_sp > 1) {
            bn = best_bn;
            a.splits = best_sp;
            a.kb_per_split = (n_kb + best_sp - 1) / best_sp;
        }
    }
    alignas(64) CUtensorMap ta, tw;
    int st = kp_make_map_bf16_2d(&ta, A, (unsigned long long)M, K, lda, TC_BK, a.a_rows);
    if (st) return st;
    st = kp_make_map_bf16_2d(&tw, W, (unsigned long long)N, K, ldw, TC_BK, epi == EPI_SWIGLU ? bn / 2 : bn);
    if (st) return st;
    cudaStream_t s = (cudaStream_t)stream;
#define TC_PICK(EPI)                                               \
    switch (bn) {                                                  \
        case 256: return launch<256, EPI>(ta, tw, a, s);           \
        case 128: return launch<128, EPI>(ta, tw, a, s);           \
        case 64: return launch<64, EPI>(ta, tw, a, s);             \
        default: return launch<32, EPI>(ta, tw, a, s);             \
    }
    switch (epi) {
        case EPI_STORE: TC_PICK(EPI_STORE)
        case EPI_STORE_F32: TC_PICK(EPI_STORE_F32)
        case EPI_ACCUM_F32: TC_PICK(EPI_ACCUM_F32)
        case EPI_SWIGLU:
            switch (bn) {
                case 256: return launch<256, EPI_SWIGLU>(ta, tw, a, s);
                case 128: return launch<128, EPI_SWIGLU>(ta, tw, a, s);
                default: return launch<64, EPI_SWIGLU>(ta, tw, a, s);
            }
        default: return KP_ERR_BAD_ARG;
    }
#undef TC_PICK
}

int kp_gemm_tc(const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc, int M, int N,
               int K, int epi, void* stream) {
    return kp_gemm_tc_split(A, lda, W, ldw, bias, C, ldc, M, N, K, epi, 0, stream);
}

}  // extern "C"
