// Tensor-core attention over the paged cache (bfloat16, head size 64 or 128).
//
// Two kernels share the tile machinery (K/V tiles of 64 keys brought into
// shared memory with cp.async through the block table, swizzled so that
// ldmatrix reads do not collide; S = Q K^T and O = P V with mma.m16n8k16;
// softmax statistics in float32; P rounded to bfloat16 as a matrix operand):
//
//  * attn_split_mma: rows that each read a long cache (decode).  One CTA per
//    (chunk of 256 keys, kv head, row); the R = H/G query heads that share the
//    kv head are the rows of the m16 tile; each of the 4 warps takes one 64-key
//    tile of the chunk; the warps' partial results are combined in warp order
//    and written as the chunk's (m, l, unnormalised O) to scratch, in the format
//    of attention_decode.cu, whose merge kernel finishes the row.
//  * attn_prefill_mma: segments of many rows.  One CTA per (64 query rows of a
//    segment, head): 4 warps x 16 rows, looping over the KV tiles up to the
//    causal limit, double-buffered.
//
// Formulas as in attention.cu (src/backend/cpu/scalar/core.c:383-433).  Tiles
// start at multiples of 64 of the absolute key index, chunks at multiples of
// 256, so the order of summation does not depend on how a prompt was cut or
// what else is in the batch.
#include "tma.cuh"

#define AM_TILE 64
#define AM_CHUNK 256
#define AM_RMAX 8

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int sz = valid ? 16 : 0;                  // size 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// `bytes` (a multiple of 16, both addresses 16-byte aligned) from global to shared memory; completes on `bar`
__device__ __forceinline__ void kp_bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(kp_smem_u32(dst)), "l"(src), "r"(bytes), "r"(kp_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// A tile in shared memory: 64 rows (keys) of HD bf16, as HD / 64 halves of 64 rows x 128 bytes; in a half the
// 16-byte chunk c of row r lies at chunk c ^ (r & 7).  This is what a TMA box of 64 columns with the 128-byte
// swizzle writes (tile on a 1024-byte boundary), so both ways of loading a tile give the same layout.
template <int HD>
__device__ __forceinline__ bf16* tile_chunk(bf16* tile, int r, int c) {
    return tile + (size_t)(c >> 3) * (AM_TILE * 64) + (size_t)r * 64 + (((c & 7) ^ (r & 7)) << 3);
}

// Bring keys [k0, k0+64) of one kv head into a K tile and a V tile.  Keys outside [k_lo, k_hi] are zero-filled.
template <int HD>
__device__ __forceinline__ void load_kv_tile(bf16* Kt, bf16* Vt, const bf16* __restrict__ cache, const int* __restrict__ bt,
                                             size_t page_stride, size_t k_off, size_t v_off, int page_size, int k0,
                                             int k_lo, int k_hi, int tid, int nthreads) {
    constexpr int CPR = HD / 8;                      // 16-byte chunks a row
    for (int i = tid; i < AM_TILE * CPR; i += nthreads) {
        const int r = i / CPR, c = i % CPR;
        const int key = k0 + r;
        const bool valid = key >= k_lo && key <= k_hi;
        const bf16* src = cache;
        if (valid) src = cache + (size_t)bt[key / page_size] * page_stride + (size_t)(key % page_size) * HD + c * 8;
        cp_async16(tile_chunk<HD>(Kt, r, c), src + (valid ? k_off : 0), valid);
        cp_async16(tile_chunk<HD>(Vt, r, c), src + (valid ? v_off : 0), valid);
    }
}

// S[16 x 64] = Q[16 x HD] K^T for one warp; qf: the A fragments of Q (4 registers a k-step)
template <int HD>
__device__ __forceinline__ void qk_tile(float (&s)[8][4], const uint32_t (&qf)[HD / 16][4], bf16* Kt, int lane) {
#pragma unroll
    for (int nt = 0; nt < 8; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) s[nt][i] = 0.f;
    const int j = lane >> 3, r = lane & 7;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) {
#pragma unroll
        for (int nt = 0; nt < 8; nt += 2) {
            uint32_t b[4];
            ldmatrix_x4(b, tile_chunk<HD>(Kt, (nt + (j >> 1)) * 8 + r, ks * 2 + (j & 1)));
            mma_bf16(s[nt], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b[0], b[1]);
            mma_bf16(s[nt + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b[2], b[3]);
        }
    }
}

// O[16 x HD] += P[16 x 64] V for one warp; pf: P as A fragments (4 registers a k-step of 16 keys)
template <int HD>
__device__ __forceinline__ void pv_tile(float (&o)[HD / 8][4], const uint32_t (&pf)[4][4], bf16* Vt, int lane) {
    const int j = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
#pragma unroll
        for (int dn = 0; dn < HD / 8; dn += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, tile_chunk<HD>(Vt, kk * 16 + (j & 1) * 8 + r, dn + (j >> 1)));
            mma_bf16(o[dn], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b[0], b[1]);
            mma_bf16(o[dn + 1], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b[2], b[3]);
        }
    }
}

// ------------------------------------------------------------------ decode (split over chunks)
// NW warps a CTA, one tile of 64 keys each: a chunk is NW * 64 keys.  Small chunks (NW = 1) give many short CTAs,
// which fill the SMs evenly and keep many loads in flight; the merge then has more partial results to add.
//
// TMA = true: the tiles come by tiled TMA loads from the cache seen as one 2-D tensor (rows = page, K|V, kv
// head, key of the page; HD columns), one box of min(page size, 64) keys x 64 columns each, issued by one
// thread: no address arithmetic in the other threads.  Needs a page size that divides 64 or is a multiple of
// it, and a multiple of 8.  Boxes wholly outside the row's keys are not loaded; V rows outside them are zeroed.
KP_STATUS_WORD(g_attn_status, attention_mma)          // 0 ok; 1: a bounded wait gave up

template <int HD, int NW, bool TMA>
__global__ void __launch_bounds__(NW * 32)
attn_split_mma_kernel(const __grid_constant__ CUtensorMap tmC, const bf16* __restrict__ q, int ldq, const bf16* __restrict__ cache,
                      const int* __restrict__ block_table, int max_blocks, const int* __restrict__ row_seg,
                      const int* __restrict__ positions, float* __restrict__ part_acc, float* __restrict__ part_ml,
                      int n_chunks, float scale, int window, int page_size, int H, int G) {
    kp_pdl_begin_early_if(gridDim.z > 1);
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem_raw = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    bf16* Ks = reinterpret_cast<bf16*>(smem_raw);                 // [NW][64][HD]
    bf16* Vs = Ks + NW * AM_TILE * HD;                            // [NW][64][HD]
    float* wO = reinterpret_cast<float*>(Vs + NW * AM_TILE * HD); // [NW][AM_RMAX][HD]
    float* wm = wO + NW * AM_RMAX * HD;                           // [NW][AM_RMAX]
    float* wl = wm + NW * AM_RMAX;                                // [NW][AM_RMAX]
    uint64_t* bar = reinterpret_cast<uint64_t*>(wl + NW * AM_RMAX);
    constexpr int CHUNK = NW * AM_TILE;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int chunk = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
    const int R = H / G;
    const int pos = positions[row];
    const int k_lo = window > 0 ? max(0, pos - window + 1) : 0, k_hi = pos;
    const int c0 = chunk * CHUNK;
    if (c0 > k_hi || c0 + CHUNK - 1 < k_lo) return;
    const int* bt = block_table + (size_t)row_seg[row] * max_blocks;
    const size_t page_stride = (size_t)2 * G * page_size * HD;
    const size_t k_off = (size_t)kvh * page_size * HD, v_off = ((size_t)G + kvh) * page_size * HD;

    if (TMA) {
        if (tid == 0) {
            kp_mbar_init(bar, 1);
            kp_mbar_init_fence();
            const int box = min(page_size, AM_TILE);               // keys a box
            uint32_t bytes = 0;
            for (int key0 = c0; key0 < c0 + CHUNK; key0 += box)
                if (key0 <= k_hi && key0 + box - 1 >= k_lo) bytes += 2 * box * HD * 2;
            kp_mbar_expect_tx(bar, bytes);
            for (int key0 = c0; key0 < c0 + CHUNK; key0 += box) {
                if (!(key0 <= k_hi && key0 + box - 1 >= k_lo)) continue;
                const int page = bt[key0 / page_size];
                const int row_k = ((page * 2) * G + kvh) * page_size + key0 % page_size;   // row of the 2-D view
                const int row_v = row_k + G * page_size;
                const int in_chunk = key0 - c0;
                bf16* kd = Ks + (size_t)(in_chunk / AM_TILE) * AM_TILE * HD + (size_t)(in_chunk % AM_TILE) * 64;
                bf16* vd = Vs + (size_t)(in_chunk / AM_TILE) * AM_TILE * HD + (size_t)(in_chunk % AM_TILE) * 64;
#pragma unroll
                for (int half = 0; half < HD / 64; half++) {
                    kp_tma_load_2d(kd + half * (AM_TILE * 64), &tmC, half * 64, row_k, bar);
                    kp_tma_load_2d(vd + half * (AM_TILE * 64), &tmC, half * 64, row_v, bar);
                }
            }
        }
    } else {
#pragma unroll
        for (int w = 0; w < NW; w++)
            load_kv_tile<HD>(Ks + w * AM_TILE * HD, Vs + w * AM_TILE * HD, cache, bt, page_stride, k_off, v_off, page_size,
                             c0 + w * AM_TILE, k_lo, k_hi, tid, NW * 32);
        cp_async_commit();
    }

    // Q of the R heads of this kv head as rows 0..R-1 of the m16 tile (rows 8..15 do not exist: R <= 8)
    uint32_t qf[HD / 16][4];
    {
        const bf16* qr = q + (size_t)row * ldq + (size_t)(kvh * R + min(g, R - 1)) * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            uint32_t lo = *reinterpret_cast<const uint32_t*>(qr + ks * 16 + 2 * t);
            uint32_t hi = *reinterpret_cast<const uint32_t*>(qr + ks * 16 + 8 + 2 * t);
            if (g >= R) lo = hi = 0;
            qf[ks][0] = lo; qf[ks][1] = 0; qf[ks][2] = hi; qf[ks][3] = 0;
        }
    }
    bf16* Kt = Ks + warp * AM_TILE * HD;
    bf16* Vt = Vs + warp * AM_TILE * HD;
    const int t0 = c0 + warp * AM_TILE;                           // first key of this warp's tile
    if (TMA) {
        __syncthreads();                                          // the barrier is initialised
        if (!kp_mbar_wait_bounded(bar, 0)) {
            if (lane == 0) atomicExch(&g_attn_status, 1);
            return;                                                // (every thread sees the same barrier)
        }
        // V rows of keys that this row does not read hold whatever was there: zero them (P is 0 there, but
        // 0 * NaN is not); K rows need nothing, their scores are masked
        if (t0 < k_lo || t0 + AM_TILE - 1 > k_hi) {
            for (int idx = lane; idx < AM_TILE * (HD / 8); idx += 32) {
                const int r = idx / (HD / 8), c = idx % (HD / 8);
                if (t0 + r < k_lo || t0 + r > k_hi) *reinterpret_cast<uint4*>(tile_chunk<HD>(Vt, r, c)) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }
    } else {
        cp_async_wait<0>();
        __syncthreads();
    }
    float s[8][4];
    qk_tile<HD>(s, qf, Kt, lane);
    // row g of the tile: columns 2t, 2t+1 of each n-tile are keys t0 + nt*8 + 2t (+1)
    float m = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int key = t0 + nt * 8 + 2 * t + i;
            const float v = (key >= k_lo && key <= k_hi) ? s[nt][i] * scale : -INFINITY;
            s[nt][i] = v;
            m = fmaxf(m, v);
        }
    }
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    float l = 0.f;
    uint32_t pf[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
        const float p0 = m == -INFINITY ? 0.f : expf(s[nt][0] - m), p1 = m == -INFINITY ? 0.f : expf(s[nt][1] - m);
        // the sum runs over the values as they enter the product (rounded to bfloat16)
        const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
        l += __low2float(pb) + __high2float(pb);
        pf[nt >> 1][(nt & 1) * 2] = *reinterpret_cast<const uint32_t*>(&pb);
        pf[nt >> 1][(nt & 1) * 2 + 1] = 0;
    }
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    float o[HD / 8][4];
#pragma unroll
    for (int dn = 0; dn < HD / 8; dn++)
#pragma unroll
        for (int i = 0; i < 4; i++) o[dn][i] = 0.f;
    pv_tile<HD>(o, pf, Vt, lane);

    if (g < R) {
#pragma unroll
        for (int dn = 0; dn < HD / 8; dn++) {
            wO[((size_t)warp * AM_RMAX + g) * HD + dn * 8 + 2 * t] = o[dn][0];
            wO[((size_t)warp * AM_RMAX + g) * HD + dn * 8 + 2 * t + 1] = o[dn][1];
        }
        if (t == 0) { wm[warp * AM_RMAX + g] = m; wl[warp * AM_RMAX + g] = l; }
    }
    __syncthreads();
    // the warps' partial results, combined in warp order
    for (int e = tid; e < R * HD; e += NW * 32) {
        const int r = e / HD, d = e % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; w++) M = fmaxf(M, wm[w * AM_RMAX + r]);
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) {
            const float mw = wm[w * AM_RMAX + r];
            if (mw != -INFINITY) acc = fmaf(wO[((size_t)w * AM_RMAX + r) * HD + d], expf(mw - M), acc);
        }
        part_acc[(((size_t)row * H + kvh * R + r) * n_chunks + chunk) * HD + d] = acc;
    }
    if (tid < R) {
        float M = -INFINITY, L = 0.f;
        for (int w = 0; w < NW; w++) M = fmaxf(M, wm[w * AM_RMAX + tid]);
        for (int w = 0; w < NW; w++) {
            const float mw = wm[w * AM_RMAX + tid];
            if (mw != -INFINITY) L = fmaf(wl[w * AM_RMAX + tid], expf(mw - M), L);
        }
        float* ml = part_ml + (((size_t)row * H + kvh * R + tid) * n_chunks + chunk) * 2;
        ml[0] = M;
        ml[1] = L;
    }
}

// ------------------------------------------------------------------ decode, persistent (head size 64, chunks of 256 keys)
// The same chunk pass as attn_split_mma_kernel<64, 4, true>, built so that the cache streams without a break:
// one persistent CTA an SM; a producer warp walks the CTA's share of the (row, kv head, chunk) items, looks up
// the pages and issues the TMA loads of an item's K and V tiles (and a bulk copy of its Q rows) into a ring of
// AR_STAGES stages; as many groups of four consumer warps take the items in turn (item k: stage and group
// k % AR_STAGES), each warp one 64-key tile as above, and write the chunk's partial result in the same format.
// (One CTA an item spends most of its life on the chain position -> block table -> first byte, and only three
// fit an SM: 2.9 TB/s at 8 rows, 4.2 at 64.)  Every wait is bounded; a wait that gives up sets the status word.
#define AR_GROUPS 3                          // groups of consumer warps = stages of the ring: group g reads stage g
#define AR_STAGES AR_GROUPS
#define AR_NW 4
#define AR_THREADS ((AR_GROUPS * AR_NW + 1) * 32)
#define AR_CHUNK (AR_NW * AM_TILE)

struct ArMeta { int row, kvh, chunk, k_lo, k_hi, pad0, pad1, pad2; };

template <int HD>
__host__ __device__ constexpr size_t ar_stage_bytes() { return (size_t)2 * AR_NW * AM_TILE * HD * 2 + 1024; }
template <int HD>
static size_t ar_smem_bytes() {
    return 1024 + AR_STAGES * ar_stage_bytes<HD>() + AR_STAGES * sizeof(ArMeta) + 2 * AR_STAGES * 8 +
           AR_GROUPS * sizeof(float) * (AR_NW * AM_RMAX * HD + 2 * AR_NW * AM_RMAX) + 32;
}

template <int HD>
__global__ void __launch_bounds__(AR_THREADS)
attn_split_ring_kernel(const __grid_constant__ CUtensorMap tmC, const bf16* __restrict__ q, int ldq,
                       const int* __restrict__ block_table, int max_blocks, const int* __restrict__ row_seg,
                       const int* __restrict__ positions, float* __restrict__ part_acc, float* __restrict__ part_ml,
                       int n_chunks, float scale, int window, int page_size, int H, int G, int n_rows) {
    kp_pdl_begin_early_if(n_rows > 1);
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    constexpr size_t STAGE = ar_stage_bytes<HD>();
    constexpr size_t KV = (size_t)AR_NW * AM_TILE * HD * 2;                // bytes of a stage's K tiles (and of its V tiles)
    ArMeta* metas = reinterpret_cast<ArMeta*>(base + AR_STAGES * STAGE);
    uint64_t* full = reinterpret_cast<uint64_t*>(metas + AR_STAGES);
    uint64_t* empty = full + AR_STAGES;
    volatile int* gave_up = reinterpret_cast<volatile int*>(empty + AR_STAGES);   // [group, padded to 4]: a warp's wait ran out
    float* scratch = reinterpret_cast<float*>(empty + AR_STAGES) + 4;   // [group]: wO [NW][RMAX][HD], wm, wl [NW][RMAX]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int R = H / G;

    if (tid == 0) {
        for (int s = 0; s < AR_STAGES; s++) { kp_mbar_init(&full[s], 1); kp_mbar_init(&empty[s], AR_NW); }
        for (int g2 = 0; g2 < 4; g2++) gave_up[g2] = 0;
        kp_mbar_init_fence();
    }
    __syncthreads();

    if (warp == AR_GROUPS * AR_NW) {
        // ---- producer
        const int n_items = n_rows * G * n_chunks;
        const int box = min(page_size, AM_TILE), n_boxes = AR_CHUNK / box;   // keys a box; at most 32 boxes (pages of 8 keys)
        int k = 0;
        bool alive = true;
        for (int it0 = blockIdx.x; it0 < n_items && alive; it0 += 32 * gridDim.x) {
            // 32 candidates at a time, one a lane: which of them have keys to read
            const int it = it0 + lane * gridDim.x;
            int c_row = 0, c_kvh = 0, c_chunk = 0, c_lo = 0, c_hi = -1, c_seg = 0;
            bool valid = false;
            if (it < n_items) {
                // chunk by chunk, so that the chunks that exist (the first ones, or a window's band) spread evenly
                // over the CTAs whatever the numbers of chunks and CTAs
                c_chunk = it / (n_rows * G);
                const int rest = it - c_chunk * (n_rows * G);
                c_kvh = rest % G;
                c_row = rest / G;
                const int pos = positions[c_row];
                c_lo = window > 0 ? max(0, pos - window + 1) : 0;
                c_hi = pos;
                const int c0 = c_chunk * AR_CHUNK;
                valid = !(c0 > c_hi || c0 + AR_CHUNK - 1 < c_lo);
                if (valid) c_seg = row_seg[c_row];
            }
            unsigned todo = __ballot_sync(0xffffffffu, valid);
            while (todo && alive) {
                const int src = __ffs(todo) - 1;
                todo &= todo - 1;
                const int row = __shfl_sync(0xffffffffu, c_row, src), kvh = __shfl_sync(0xffffffffu, c_kvh, src);
                const int chunk = __shfl_sync(0xffffffffu, c_chunk, src), seg = __shfl_sync(0xffffffffu, c_seg, src);
                const int k_lo = __shfl_sync(0xffffffffu, c_lo, src), k_hi = __shfl_sync(0xffffffffu, c_hi, src);
                const int c0 = chunk * AR_CHUNK;
                // lane b: box b of the chunk
                const int key0 = c0 + lane * box;
                const bool need = lane < n_boxes && key0 <= k_hi && key0 + box - 1 >= k_lo;
                const int page = need ? block_table[(size_t)seg * max_blocks + key0 / page_size] : 0;
                const unsigned boxes = __ballot_sync(0xffffffffu, need);
                const int s = k % AR_STAGES;
                uint64_t* fbar = &full[s];
                unsigned char* st = base + (size_t)s * STAGE;
                int ok = 1;
                if (lane == 0) {
                    ok = kp_mbar_wait_bounded(&empty[s], ((k / AR_STAGES) & 1) ^ 1) ? 1 : 0;
                    if (ok) {
                        ArMeta m;
                        m.row = row; m.kvh = kvh; m.chunk = chunk; m.k_lo = k_lo; m.k_hi = k_hi; m.pad0 = m.pad1 = m.pad2 = 0;
                        metas[s] = m;
                        const uint32_t q_bytes = (uint32_t)R * HD * 2;
                        kp_mbar_expect_tx(fbar, (uint32_t)__popc(boxes) * 2 * box * HD * 2 + q_bytes);
                        kp_bulk_g2s(st + 2 * KV, q + (size_t)row * ldq + (size_t)kvh * R * HD, q_bytes, fbar);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { alive = false; break; }
                if (need) {
                    const int row_k = ((page * 2) * G + kvh) * page_size + key0 % page_size;       // row of the 2-D view
                    const int row_v = row_k + G * page_size;
                    const int in_chunk = key0 - c0;
                    const size_t off = ((size_t)(in_chunk / AM_TILE) * AM_TILE * HD + (size_t)(in_chunk % AM_TILE) * 64) * 2;
                    kp_tma_load_2d(st + off, &tmC, 0, row_k, fbar);
                    kp_tma_load_2d(st + KV + off, &tmC, 0, row_v, fbar);
                }
                k++;
            }
        }
        // no more items: a mark for each group
        for (int e = 0; e < AR_GROUPS && alive; e++, k++) {
            const int s = k % AR_STAGES;
            if (lane == 0) {
                if (kp_mbar_wait_bounded(&empty[s], ((k / AR_STAGES) & 1) ^ 1)) {
                    metas[s].row = -1;
                    kp_mbar_arrive(&full[s]);
                } else {
                    alive = false;
                }
            }
            alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
        }
        if (!alive && lane == 0) atomicExch(&g_attn_status, 1);
        return;
    }

    // ---- consumers: group grp, warp wg of it
    const int grp = warp / AR_NW, wg = warp % AR_NW, g = lane >> 2, t = lane & 3;
    float* wO = scratch + (size_t)grp * (AR_NW * AM_RMAX * HD + 2 * AR_NW * AM_RMAX);
    float* wm = wO + AR_NW * AM_RMAX * HD;
    float* wl = wm + AR_NW * AM_RMAX;
    const int gtid = tid - grp * AR_NW * 32;                          // thread of the group
    auto group_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "n"(AR_NW * 32) : "memory"); };
    for (int k = grp;; k += AR_GROUPS) {
        const int s = k % AR_STAGES;
        // The four warps of the group leave the loop together or not at all (the group's barriers below count all
        // of them): a warp whose wait ran out says so, and all of them look after a barrier.
        if (!kp_mbar_wait_bounded(&full[s], (k / AR_STAGES) & 1)) {
            if (lane == 0) { atomicExch(&g_attn_status, 1); gave_up[grp] = 1; }
        }
        group_sync();
        if (gave_up[grp]) break;
        const ArMeta me = metas[s];
        if (me.row < 0) break;
        unsigned char* st = base + (size_t)s * STAGE;
        bf16* Kt = reinterpret_cast<bf16*>(st) + (size_t)wg * AM_TILE * HD;
        bf16* Vt = reinterpret_cast<bf16*>(st + KV) + (size_t)wg * AM_TILE * HD;
        const bf16* Qs = reinterpret_cast<const bf16*>(st + 2 * KV);
        const int k_lo = me.k_lo, k_hi = me.k_hi;
        const int t0 = me.chunk * AR_CHUNK + wg * AM_TILE;            // first key of this warp's tile
        uint32_t qf[HD / 16][4];
        {
            const bf16* qr = Qs + (size_t)min(g, R - 1) * HD;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ks++) {
                uint32_t lo = *reinterpret_cast<const uint32_t*>(qr + ks * 16 + 2 * t);
                uint32_t hi = *reinterpret_cast<const uint32_t*>(qr + ks * 16 + 8 + 2 * t);
                if (g >= R) lo = hi = 0;
                qf[ks][0] = lo; qf[ks][1] = 0; qf[ks][2] = hi; qf[ks][3] = 0;
            }
        }
        // V rows of keys that this row does not read hold whatever was there: zero them (P is 0 there, but
        // 0 * NaN is not); K rows need nothing, their scores are masked
        if (t0 < k_lo || t0 + AM_TILE - 1 > k_hi) {
            for (int idx = lane; idx < AM_TILE * (HD / 8); idx += 32) {
                const int r = idx / (HD / 8), c = idx % (HD / 8);
                if (t0 + r < k_lo || t0 + r > k_hi) *reinterpret_cast<uint4*>(tile_chunk<HD>(Vt, r, c)) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }
        float sc[8][4];
        qk_tile<HD>(sc, qf, Kt, lane);
        float m = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const int key = t0 + nt * 8 + 2 * t + i;
                const float v = (key >= k_lo && key <= k_hi) ? sc[nt][i] * scale : -INFINITY;
                sc[nt][i] = v;
                m = fmaxf(m, v);
            }
        }
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        float l = 0.f;
        uint32_t pf[4][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            const float p0 = m == -INFINITY ? 0.f : expf(sc[nt][0] - m), p1 = m == -INFINITY ? 0.f : expf(sc[nt][1] - m);
            // the sum runs over the values as they enter the product (rounded to bfloat16)
            const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
            l += __low2float(pb) + __high2float(pb);
            pf[nt >> 1][(nt & 1) * 2] = *reinterpret_cast<const uint32_t*>(&pb);
            pf[nt >> 1][(nt & 1) * 2 + 1] = 0;
        }
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        float o[HD / 8][4];
#pragma unroll
        for (int dn = 0; dn < HD / 8; dn++)
#pragma unroll
            for (int i = 0; i < 4; i++) o[dn][i] = 0.f;
        pv_tile<HD>(o, pf, Vt, lane);
        __syncwarp();
        if (lane == 0) kp_mbar_arrive(&empty[s]);                     // this warp has read its tiles (and Q, and the item)

        if (g < R) {
#pragma unroll
            for (int dn = 0; dn < HD / 8; dn++) {
                wO[((size_t)wg * AM_RMAX + g) * HD + dn * 8 + 2 * t] = o[dn][0];
                wO[((size_t)wg * AM_RMAX + g) * HD + dn * 8 + 2 * t + 1] = o[dn][1];
            }
            if (t == 0) { wm[wg * AM_RMAX + g] = m; wl[wg * AM_RMAX + g] = l; }
        }
        group_sync();
        // the warps' partial results, combined in warp order
        for (int e = gtid; e < R * HD; e += AR_NW * 32) {
            const int r = e / HD, d = e % HD;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < AR_NW; w++) M = fmaxf(M, wm[w * AM_RMAX + r]);
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < AR_NW; w++) {
                const float mw = wm[w * AM_RMAX + r];
                if (mw != -INFINITY) acc = fmaf(wO[((size_t)w * AM_RMAX + r) * HD + d], expf(mw - M), acc);
            }
            part_acc[(((size_t)me.row * H + me.kvh * R + r) * n_chunks + me.chunk) * HD + d] = acc;
        }
        if (gtid < R) {
            float M = -INFINITY, L = 0.f;
            for (int w = 0; w < AR_NW; w++) M = fmaxf(M, wm[w * AM_RMAX + gtid]);
            for (int w = 0; w < AR_NW; w++) {
                const float mw = wm[w * AM_RMAX + gtid];
                if (mw != -INFINITY) L = fmaf(wl[w * AM_RMAX + gtid], expf(mw - M), L);
            }
            float* ml = part_ml + (((size_t)me.row * H + me.kvh * R + gtid) * n_chunks + me.chunk) * 2;
            ml[0] = M;
            ml[1] = L;
        }
        group_sync();                                                 // the group's scratch is free for its next item
    }
}

// ------------------------------------------------------------------ prefill (segments of many rows)
// One CTA: 64 consecutive rows (tile `qt` of segment `seg`) of one head.  tile_seg / tile_q0 list the tiles.
template <int HD>
__global__ void __launch_bounds__(128)
attn_prefill_mma_kernel(const bf16* __restrict__ q, int ldq, const bf16* __restrict__ cache,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_rows,
                        const int* __restrict__ seg_pos, const int* __restrict__ tile_seg,
                        const int* __restrict__ tile_row0, bf16* __restrict__ out, int ldo, float scale, int window,
                        int page_size, int H, int G) {
    kp_pdl_begin();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* Ks = reinterpret_cast<bf16*>(smem_raw);                 // [2][64][HD]
    bf16* Vs = Ks + 2 * AM_TILE * HD;                             // [2][64][HD]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int h = blockIdx.y, kvh = h / (H / G);
    const int seg = tile_seg[blockIdx.x];
    const int row0 = tile_row0[blockIdx.x];                        // first row of this tile (global row index)
    const int seg_end = cu_rows[seg + 1];
    const int n_rows = min(64, seg_end - row0);
    const int pos0 = seg_pos[seg] + (row0 - cu_rows[seg]);         // position of the tile's first row
    const int* bt = block_table + (size_t)seg * max_blocks;
    const size_t page_stride = (size_t)2 * G * page_size * HD;
    const size_t k_off = (size_t)kvh * page_size * HD, v_off = ((size_t)G + kvh) * page_size * HD;

    // keys any row of the tile may read
    const int k_hi_all = pos0 + n_rows - 1;
    const int k_lo_all = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int tile_lo = k_lo_all / AM_TILE, tile_hi = k_hi_all / AM_TILE;

    // this warp's 16 rows: rows r0 = warp*16 + g and r0 + 8
    const int ra = warp * 16 + g, rb = ra + 8;
    const int pos_a = pos0 + ra, pos_b = pos0 + rb;
    const bool has_a = ra < n_rows, has_b = rb < n_rows;
    uint32_t qf[HD / 16][4];
    {
        const bf16* qa = q + (size_t)(row0 + min(ra, n_rows - 1)) * ldq + (size_t)h * HD;
        const bf16* qb = q + (size_t)(row0 + min(rb, n_rows - 1)) * ldq + (size_t)h * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            qf[ks][0] = *reinterpret_cast<const uint32_t*>(qa + ks * 16 + 2 * t);
            qf[ks][1] = *reinterpret_cast<const uint32_t*>(qb + ks * 16 + 2 * t);
            qf[ks][2] = *reinterpret_cast<const uint32_t*>(qa + ks * 16 + 8 + 2 * t);
            qf[ks][3] = *reinterpret_cast<const uint32_t*>(qb + ks * 16 + 8 + 2 * t);
        }
    }
    const int lo_a = window > 0 ? max(0, pos_a - window + 1) : 0, lo_b = window > 0 ? max(0, pos_b - window + 1) : 0;

    float o[HD / 8][4];
#pragma unroll
    for (int dn = 0; dn < HD / 8; dn++)
#pragma unroll
        for (int i = 0; i < 4; i++) o[dn][i] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    load_kv_tile<HD>(Ks, Vs, cache, bt, page_stride, k_off, v_off, page_size, tile_lo * AM_TILE, k_lo_all, k_hi_all,
                     tid, 128);
    cp_async_commit();
    for (int kt = tile_lo; kt <= tile_hi; kt++) {
        const int buf = (kt - tile_lo) & 1;
        if (kt + 1 <= tile_hi) {
            load_kv_tile<HD>(Ks + (buf ^ 1) * AM_TILE * HD, Vs + (buf ^ 1) * AM_TILE * HD, cache, bt, page_stride, k_off,
                             v_off, page_size, (kt + 1) * AM_TILE, k_lo_all, k_hi_all, tid, 128);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int t0 = kt * AM_TILE;
        // a warp whose rows all lie before this tile (causal) or after its window has nothing to do in it
        const int w_pos_hi = pos0 + min(warp * 16 + 15, n_rows - 1);
        const int w_lo = window > 0 ? max(0, pos0 + warp * 16 - window + 1) : 0;
        if (warp * 16 < n_rows && t0 <= w_pos_hi && t0 + AM_TILE - 1 >= w_lo) {
            float s[8][4];
            qk_tile<HD>(s, qf, Ks + buf * AM_TILE * HD, lane);
            float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const int key = t0 + nt * 8 + 2 * t + i;
                    const float va = (has_a && key <= pos_a && key >= lo_a) ? s[nt][i] * scale : -INFINITY;
                    const float vb = (has_b && key <= pos_b && key >= lo_b) ? s[nt][2 + i] * scale : -INFINITY;
                    s[nt][i] = va; s[nt][2 + i] = vb;
                    mx_a = fmaxf(mx_a, va); mx_b = fmaxf(mx_b, vb);
                }
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
            const float ca = (m_a == -INFINITY) ? 0.f : expf(m_a - mn_a), cb = (m_b == -INFINITY) ? 0.f : expf(m_b - mn_b);
            float sa = 0.f, sb = 0.f;
            uint32_t pf[4][4];
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                const float pa0 = mn_a == -INFINITY ? 0.f : expf(s[nt][0] - mn_a), pa1 = mn_a == -INFINITY ? 0.f : expf(s[nt][1] - mn_a);
                const float pb0 = mn_b == -INFINITY ? 0.f : expf(s[nt][2] - mn_b), pb1 = mn_b == -INFINITY ? 0.f : expf(s[nt][3] - mn_b);
                const __nv_bfloat162 xa = __floats2bfloat162_rn(pa0, pa1), xb = __floats2bfloat162_rn(pb0, pb1);
                sa += __low2float(xa) + __high2float(xa);
                sb += __low2float(xb) + __high2float(xb);
                pf[nt >> 1][(nt & 1) * 2] = *reinterpret_cast<const uint32_t*>(&xa);
                pf[nt >> 1][(nt & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&xb);
            }
            sa += __shfl_xor_sync(0xffffffffu, sa, 1); sa += __shfl_xor_sync(0xffffffffu, sa, 2);
            sb += __shfl_xor_sync(0xffffffffu, sb, 1); sb += __shfl_xor_sync(0xffffffffu, sb, 2);
            l_a = l_a * ca + sa; l_b = l_b * cb + sb;
            m_a = mn_a; m_b = mn_b;
#pragma unroll
            for (int dn = 0; dn < HD / 8; dn++) { o[dn][0] *= ca; o[dn][1] *= ca; o[dn][2] *= cb; o[dn][3] *= cb; }
            pv_tile<HD>(o, pf, Vs + buf * AM_TILE * HD, lane);
        }
        __syncthreads();                                          // the buffer is free for the load after next
    }
    const float ia = l_a > 0.f ? 1.0f / l_a : 0.f, ib = l_b > 0.f ? 1.0f / l_b : 0.f;
    if (has_a) {
        bf16* oa = out + (size_t)(row0 + ra) * ldo + (size_t)h * HD;
#pragma unroll
        for (int dn = 0; dn < HD / 8; dn++)
            *reinterpret_cast<uint32_t*>(oa + dn * 8 + 2 * t) = pack_bf16(o[dn][0] * ia, o[dn][1] * ia);
    }
    if (has_b) {
        bf16* ob = out + (size_t)(row0 + rb) * ldo + (size_t)h * HD;
#pragma unroll
        for (int dn = 0; dn < HD / 8; dn++)
            *reinterpret_cast<uint32_t*>(ob + dn * 8 + 2 * t) = pack_bf16(o[dn][2] * ib, o[dn][3] * ib);
    }
}

#ifndef USE_RING
#define USE_RING 1
#endif
static int am_n_sm() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int HD, int NW>
static int launch_split(const void* q, int ldq, const void* cache, long long n_pages, const int* block_table,
                        int max_blocks, const int* row_seg, const int* positions, float* part_acc, float* part_ml,
                        int n_chunks, float scale, int window, int page_size, int n, int H, int G, cudaStream_t s) {
    const size_t smem = 1024 + (size_t)2 * NW * AM_TILE * HD * 2 + sizeof(float) * (NW * AM_RMAX * HD + 2 * NW * AM_RMAX) + 16;
    alignas(64) CUtensorMap tm = {};
    // tiles by TMA where the pages allow it (and the cache is known by its size), else by cp.async
    const bool tma = n_pages > 0 && n_pages * 2 * G * page_size < 2147483647LL && (page_size % 8 == 0) && (page_size % AM_TILE == 0 || AM_TILE % page_size == 0) &&
                     !((uintptr_t)cache & 15) &&
                     kp_make_map_bf16_2d(&tm, cache, (unsigned long long)n_pages * 2 * G * page_size, HD, HD, 64,
                                         page_size < AM_TILE ? page_size : AM_TILE) == 0;
    if constexpr (HD == 64 && NW == AR_NW) {
        // the persistent form where its Q copy can run: 16-byte aligned rows of Q, whole 16 bytes of Q a kv head
        if (USE_RING && tma && !((uintptr_t)q & 15) && (ldq % 8) == 0 && ((H / G) * HD * 2) % 16 == 0) {
            const size_t rs = ar_smem_bytes<HD>();
            static bool ready = false;
            if (!ready) {
                cudaError_t e = cudaFuncSetAttribute(attn_split_ring_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rs);
                if (e != cudaSuccess) return (int)e;
                ready = true;
            }
            const long long items = (long long)n * G * n_chunks;
            const int sms = am_n_sm();
            kp_launch_pdl(attn_split_ring_kernel<HD>, dim3((unsigned)(items < sms ? items : sms)), dim3(AR_THREADS), rs, s, tm,
                          (const bf16*)q, ldq, block_table, max_blocks, row_seg, positions, part_acc, part_ml, n_chunks, scale,
                          window, page_size, H, G, n);
            return kp_launch_status();
        }
    }
    auto kern = tma ? attn_split_mma_kernel<HD, NW, true> : attn_split_mma_kernel<HD, NW, false>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    kp_launch_pdl(kern, dim3(dim3(n_chunks, G, n)), dim3(NW * 32), smem, s, tm,
        (const bf16*)q, ldq, (const bf16*)cache, block_table, max_blocks, row_seg, positions, part_acc, part_ml,
        n_chunks, scale, window, page_size, H, G);
    return kp_launch_status();
}

template <int HD>
static int launch_prefill(const void* q, int ldq, const void* cache, const int* block_table, int max_blocks,
                          const int* cu_rows, const int* seg_pos, const int* tile_seg, const int* tile_row0, int n_tiles,
                          void* out, int ldo, float scale, int window, int page_size, int H, int G, cudaStream_t s) {
    const size_t smem = (size_t)4 * AM_TILE * HD * 2;
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    kp_launch_pdl(attn_prefill_mma_kernel<HD>, dim3(dim3(n_tiles, H)), dim3(128), smem, s, 
        (const bf16*)q, ldq, (const bf16*)cache, block_table, max_blocks, cu_rows, seg_pos, tile_seg, tile_row0,
        (bf16*)out, ldo, scale, window, page_size, H, G);
    return kp_launch_status();
}

extern "C" {

// The chunk partials of the split pass (bfloat16, head size 64 or 128, H/G <= 8); chunks of `chunk_keys` keys
// (64, 128 or 256), n_chunks of them, into `scratch` (n * H * n_chunks * (hd + 2) floats).  The caller runs the
// merge of attention_decode.cu afterwards (kp_attention_merge, same chunk size) on the same scratch.
int kp_attention_split_mma(const void* q, int ldq, const void* cache, long long n_pages, const int* block_table, int max_blocks,
                           const int* row_seg, const int* positions, float* scratch, int n_chunks, int chunk_keys,
                           float scale, int window, int page_size, int n, int H, int G, int hd, void* stream) {
    if (n <= 0) return 0;
    if ((hd != 64 && hd != 128) || G < 1 || H % G || H / G > AM_RMAX || page_size < 1 || n_chunks < 1 || n > 65535 ||
        G > 65535 || (ldq & 1) || (chunk_keys != 64 && chunk_keys != 128 && chunk_keys != 256))
        return KP_ERR_UNSUPPORTED;
    float* part_acc = scratch;
    float* part_ml = scratch + (size_t)n * H * n_chunks * hd;
    cudaStream_t s = (cudaStream_t)stream;
#define AM_SPLIT(HD, NW)                                                                                          \
    return launch_split<HD, NW>(q, ldq, cache, n_pages, block_table, max_blocks, row_seg, positions, part_acc, part_ml, \
                                n_chunks, scale, window, page_size, n, H, G, s)
    if (hd == 64) {
        if (chunk_keys == 64) AM_SPLIT(64, 1);
        if (chunk_keys == 128) AM_SPLIT(64, 2);
        AM_SPLIT(64, 4);
    }
    if (chunk_keys == 64) AM_SPLIT(128, 1);
    if (chunk_keys == 128) AM_SPLIT(128, 2);
    AM_SPLIT(128, 4);
#undef AM_SPLIT
}

// tile_seg / tile_row0: for each tile of 64 rows its segment and its first row (device arrays, n_tiles long)
int kp_attention_prefill_mma(const void* q, int ldq, const void* cache, const int* block_table, int max_blocks,
                             const int* cu_rows, const int* seg_pos, const int* tile_seg, const int* tile_row0,
                             int n_tiles, void* out, int ldo, float scale, int window, int page_size, int H, int G,
                             int hd, void* stream) {
    if (n_tiles <= 0) return 0;
    if ((hd != 64 && hd != 128) || G < 1 || H % G || page_size < 1 || H > 65535 || (ldq & 1) || (ldo & 1))
        return KP_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (hd == 64) return launch_prefill<64>(q, ldq, cache, block_table, max_blocks, cu_rows, seg_pos, tile_seg, tile_row0,
                                            n_tiles, out, ldo, scale, window, page_size, H, G, s);
    return launch_prefill<128>(q, ldq, cache, block_table, max_blocks, cu_rows, seg_pos, tile_seg, tile_row0, n_tiles,
                               out, ldo, scale, window, page_size, H, G, s);
}


}  // extern "C"
