// Causal attention of prompt portions over the paged cache on the 5th-generation tensor cores
// (bfloat16, head size 64).
//
// One CTA: 128 consecutive rows of a segment x one head, looping over tiles of 128 keys up to the causal
// limit.  Per tile (formulas as in attention.cu; src/backend/cpu/scalar/core.c:383-433):
//   S  = Q K^T        tcgen05.mma, 128 x 128 x 64, Q and the K tile K-major in shared memory (TMA, 128-byte
//                     swizzle), S in tensor memory (128 columns);
//   P  = exp(S*scale - m), row statistics in float32 by 128 threads (one a row) that read S from tensor
//        memory, mask keys outside [pos - window + 1, pos], and write P as bfloat16 into shared memory in the
//        K-major swizzled layout of an MMA operand;
//   PV = P V          tcgen05.mma, 128 x 64 x 128, V tile as it lies in the cache (keys x head size: the
//                     MN-major B operand), into 64 more columns of tensor memory, not accumulated there:
//   O  = O*corr + PV  in registers of the row's thread, so a change of the row maximum needs no pass over
//                     tensor memory.
// Roles by warp: 0 TMA producer (Q once; K double-buffered, V single: the next K tile is requested as soon as
// S has been computed from the buffer, the next V tile as soon as PV has), 1 tensor-memory owner and MMA
// issuer, 2-5 the rows.  The MMA warp issues the next tile's S right behind PV, so it overlaps the rows'
// update of O.  Two CTAs fit an SM (96 KB of shared memory, 256 columns of tensor memory each) and fill each
// other's waits.
//
// K/V tiles come from the cache seen as one 2-D tensor (rows = page, K|V, kv head, key of the page), one box
// of min(page size, 128) keys each; boxes wholly outside the CTA's keys are not loaded (V starts zeroed, so
// what an unloaded part holds is finite and meets P = 0).  Tiles start at multiples of 128 of the absolute
// key index.  The caller lists the 128-row tiles from the one that reads the most keys to the one that reads
// the fewest; a CTA takes the i-th and the i-th last, so every CTA has about the same work.
// Every mbarrier wait is bounded; a wait that gives up sets the status word, and the CTA frees its tensor
// memory and returns.
#include <type_traits>

#include "tcgen05.cuh"

#define AT_BM 128
#define AT_BN 128
#define AT_HD 64
#define AT_THREADS 192
#define AT_TILE_BYTES (128 * 64 * 2)         // a 128 x 64 bf16 tile: 16 KB

KP_STATUS_WORD(g_attn_tc_status, attention_tc)          // 0 ok; 1: a bounded wait gave up

__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// the largest of three (one instruction on this architecture)
__device__ __forceinline__ float at_max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

struct AtArgs {
    const int* block_table; int max_blocks;
    const int* cu_rows; const int* seg_pos; const int* tile_seg; const int* tile_row0;
    bf16* out; int ldo;
    float scale; int window; int page_size; int H, G; int n_tiles;
};

// One piece of work: 128 rows (or the segment's last few) of one segment
struct AtItem {
    int row0, n_rows, pos0, k_hi_all, k_lo_all, kt_lo, kt_hi;
    const int* bt;
};
__device__ __forceinline__ AtItem at_item(const AtArgs& p, int tile) {
    AtItem it;
    const int seg = p.tile_seg[tile];
    it.row0 = p.tile_row0[tile];
    const int seg_begin = p.cu_rows[seg], seg_end = p.cu_rows[seg + 1];
    it.n_rows = min(AT_BM, seg_end - it.row0);
    it.pos0 = p.seg_pos[seg] + (it.row0 - seg_begin);            // position of the first row
    it.k_hi_all = it.pos0 + it.n_rows - 1;
    it.k_lo_all = p.window > 0 ? max(0, it.pos0 - p.window + 1) : 0;
    it.kt_lo = it.k_lo_all / AT_BN;
    it.kt_hi = it.k_hi_all / AT_BN;
    it.bt = p.block_table + (size_t)seg * p.max_blocks;
    return it;
}

__global__ void __launch_bounds__(AT_THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmC, const AtArgs p) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* sm = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    unsigned char* Qs = sm;                                     // 16 KB
    unsigned char* Ks = Qs + AT_TILE_BYTES;                     // 2 x 16 KB
    unsigned char* Vs = Ks + 2 * AT_TILE_BYTES;                 // 16 KB
    unsigned char* Ps = Vs + AT_TILE_BYTES;                     // 2 x 16 KB: keys 0..63 | keys 64..127
    uint64_t* bars = reinterpret_cast<uint64_t*>(Ps + 2 * AT_TILE_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;                                // [2]
    uint64_t* k_empty = bars + 3;                               // [2]
    uint64_t* v_full = bars + 5;
    uint64_t* v_empty = bars + 6;
    uint64_t* s_full = bars + 7;
    uint64_t* p_full = bars + 8;
    uint64_t* pv_full = bars + 9;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y, kvh = h / (p.H / p.G);
    // The tiles are listed from the one that reads the most keys to the one that reads the fewest; this CTA
    // takes the blockIdx.x-th and the blockIdx.x-th last, so every CTA has about the same work.
    const int n_items = ((int)blockIdx.x < p.n_tiles - 1 - (int)blockIdx.x) ? 2 : 1;
    auto item_tile = [&](int idx) { return idx == 0 ? (int)blockIdx.x : p.n_tiles - 1 - (int)blockIdx.x; };

    if (threadIdx.x == 0) {
        kp_mbar_init(q_full, 1);
        for (int i = 0; i < 2; i++) { kp_mbar_init(&k_full[i], 1); kp_mbar_init(&k_empty[i], 1); }
        kp_mbar_init(v_full, 1); kp_mbar_init(v_empty, 1);
        kp_mbar_init(s_full, 1); kp_mbar_init(p_full, 128); kp_mbar_init(pv_full, 1);
        *abort_flag = 0;
        kp_mbar_init_fence();
    }
    // V starts zeroed: a part of a tile that is never loaded then holds something finite
    for (int i = threadIdx.x; i < AT_TILE_BYTES / 16; i += AT_THREADS) reinterpret_cast<uint4*>(Vs)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1) kp_tmem_alloc(tmem_slot, 256);
    kp_tc_fence_before();
    __syncthreads();
    kp_tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_pv = tmem_base + 128;
    kp_pdl_begin();

    // The three roles walk the same items and key tiles; `i` counts the key tiles over both items, and the
    // mbarrier parities follow from it (buffer uses: K buffer i & 1 for the (i >> 1)-th time, V, S, P, PV for
    // the i-th time).
    if (warp == 0) {
        if (lane == 0) {
            const int box = min(p.page_size, AT_BN);
            int i = 0;
            bool ok = true;
            for (int idx = 0; idx < n_items && ok; idx++) {
                const AtItem it = at_item(p, item_tile(idx));
                if (idx > 0) {
                    // Q is read by the S products; the last of the item before has freed its K buffer when done
                    const int last = i - 1;
                    if (!kp_mbar_wait_bounded(&k_empty[last & 1], (last >> 1) & 1)) { *abort_flag = 1; break; }
                }
                kp_mbar_expect_tx(q_full, AT_TILE_BYTES);
                kp_tma_load_2d(Qs, &tmQ, h * AT_HD, it.row0, q_full);
                // the boxes of a tile that hold keys of this item; `dst` a K or V buffer, kv 0 or 1
                auto load_tile = [&](unsigned char* dst, int kt, int kv, uint64_t* bar) {
                    uint32_t bytes = 0;
                    for (int key0 = kt * AT_BN; key0 < (kt + 1) * AT_BN; key0 += box)
                        if (key0 <= it.k_hi_all && key0 + box - 1 >= it.k_lo_all) bytes += box * AT_HD * 2;
                    kp_mbar_expect_tx(bar, bytes);
                    for (int key0 = kt * AT_BN; key0 < (kt + 1) * AT_BN; key0 += box) {
                        if (!(key0 <= it.k_hi_all && key0 + box - 1 >= it.k_lo_all)) continue;
                        const int page = it.bt[key0 / p.page_size];
                        const int row = ((page * 2 + kv) * p.G + kvh) * p.page_size + key0 % p.page_size;
                        kp_tma_load_2d(dst + (size_t)(key0 - kt * AT_BN) * 128, &tmC, 0, row, bar);
                    }
                };
                for (int kt = it.kt_lo; kt <= it.kt_hi; kt++, i++) {
                    const int kb = i & 1;
                    if (*abort_flag || !kp_mbar_wait_bounded(&k_empty[kb], ((i >> 1) & 1) ^ 1)) { *abort_flag = 1; ok = false; break; }
                    load_tile(Ks + kb * AT_TILE_BYTES, kt, 0, &k_full[kb]);
                    if (!kp_mbar_wait_bounded(v_empty, (i & 1) ^ 1)) { *abort_flag = 1; ok = false; break; }
                    load_tile(Vs, kt, 1, v_full);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = kp_umma_idesc(AT_BM, AT_BN, false);
            constexpr uint32_t idesc_pv = kp_umma_idesc(AT_BM, AT_HD, true);
            const uint64_t qdesc = kp_umma_desc(kp_smem_u32(Qs));
            bool ok = true;
            int base = 0;                                                // key tiles of the items before
            for (int idx = 0; idx < n_items && ok; idx++) {
                const AtItem it = at_item(p, item_tile(idx));
                const int n_kt = it.kt_hi - it.kt_lo + 1;
                ok = kp_mbar_wait_bounded(q_full, idx & 1);
                auto issue_s = [&](int i) {                               // S of key tile i (counted over the items)
                    const int kb = i & 1;
                    if (!kp_mbar_wait_bounded(&k_full[kb], (i >> 1) & 1)) return false;
                    // S is free once the rows have read the tile before (they say so with p_full)
                    if (i > 0 && !kp_mbar_wait_bounded(p_full, (i - 1) & 1)) return false;
                    kp_tc_fence_after();
                    const uint64_t kdesc = kp_umma_desc(kp_smem_u32(Ks + kb * AT_TILE_BYTES));
#pragma unroll
                    for (int k = 0; k < AT_HD / 16; k++) kp_umma_bf16(tmem_s, qdesc + 2 * k, kdesc + 2 * k, idesc_s, k ? 1u : 0u);
                    kp_umma_commit(s_full);
                    kp_umma_commit(&k_empty[kb]);
                    return true;
                };
                if (ok) ok = issue_s(base);
                for (int j = 0; j < n_kt && ok; j++) {
                    const int i = base + j;
                    // PV of tile i: P is in shared memory (p_full), V has come
                    if (!kp_mbar_wait_bounded(p_full, i & 1) || !kp_mbar_wait_bounded(v_full, i & 1)) { ok = false; break; }
                    kp_tc_fence_after();
                    const uint32_t pa = kp_smem_u32(Ps), va = kp_smem_u32(Vs);
#pragma unroll
                    for (int kk = 0; kk < AT_BN / 16; kk++)
                        kp_umma_bf16(tmem_pv, kp_umma_desc(pa + (kk >> 2) * AT_TILE_BYTES) + 2 * (kk & 3), kp_umma_desc(va + kk * 2048),
                                idesc_pv, kk ? 1u : 0u);
                    kp_umma_commit(pv_full);
                    kp_umma_commit(v_empty);
                    if (j + 1 < n_kt) ok = issue_s(i + 1);
                }
                base += n_kt;
            }
            if (!ok) { *abort_flag = 1; atomicExch(&g_attn_tc_status, 1); }
        }
    } else {
        // ---- the rows: thread r of the four warps owns row r (lane r of tensor memory)
        const int q4 = warp & 3;
        const int r = q4 * 32 + lane;
        const uint32_t lane_off = (uint32_t)(q4 * 32) << 16;
        const float sl2 = p.scale * 1.4426950408889634f;              // scale * log2(e)
        bool ok = true;
        int i = 0;
        for (int idx = 0; idx < n_items && ok; idx++) {
            const AtItem it = at_item(p, item_tile(idx));
            const int pos = it.pos0 + r;                                  // this row's position (rows >= n_rows: masked)
            const bool live = r < it.n_rows;
            const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
            const int lo_max = p.window > 0 ? max(0, it.k_hi_all - p.window + 1) : 0;    // the last row's first key
            float o[AT_HD];
#pragma unroll
            for (int d = 0; d < AT_HD; d++) o[d] = 0.f;
            float m = -INFINITY, l = 0.f;
            for (int kt = it.kt_lo; kt <= it.kt_hi && ok; kt++, i++) {
                if (!kp_mbar_wait_bounded(s_full, i & 1) || *abort_flag) { ok = false; break; }
                kp_tc_fence_after();
                // Most tiles lie wholly inside every row's keys; only the tile on the diagonal, a window's edge
                // and rows past the end of the segment need the mask.  Scores are taken in base 2:
                // exp(x) = 2^(x log2 e).
                const bool masked = !(kt * AT_BN + AT_BN - 1 <= it.pos0 && kt * AT_BN >= lo_max && it.n_rows == AT_BM);
                // pass 1: the row maximum of this tile
                float tmax = -INFINITY;
#pragma unroll 1
                for (int c = 0; c < AT_BN; c += 32) {
                    uint32_t s[32];
                    kp_tmem_ld32(tmem_s + lane_off + c, s);
                    if (masked) {
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const int key = kt * AT_BN + c + j;
                            if (live && key >= lo && key <= pos) tmax = fmaxf(tmax, __uint_as_float(s[j]));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) tmax = at_max3(tmax, __uint_as_float(s[j]), __uint_as_float(s[j + 1]));
                    }
                }
                const float m_new = fmaxf(m, tmax * sl2);                       // in units of log2
                const float corr = (m_new == -INFINITY) ? 0.f : exp2f(m - m_new);       // m = -inf: 2^(-inf) = 0
                const float m_sub = (m_new == -INFINITY) ? 0.f : m_new;
                // pass 2: P = 2^(S*scale*log2e - m_new), rounded to bfloat16 as it enters the product; its row sum
                float lsum = 0.f;
                // (the masked form is a separate instance: in the common, unmasked one no instruction looks at
                // keys.  With one body and the test inside it the compiler predicated the mask's compares and
                // selects instead of branching around them, and the ALU pipe, not the exponentials, set the pace.)
                auto pass2 = [&](auto masked_c) {
                    constexpr bool MASKED = decltype(masked_c)::value;
#pragma unroll 1
                    for (int c = 0; c < AT_BN; c += 32) {
                        uint32_t s[32];
                        kp_tmem_ld32(tmem_s + lane_off + c, s);
                        unsigned char* prow = Ps + (c >> 6) * AT_TILE_BYTES + r * 128;
#pragma unroll
                        for (int j8 = 0; j8 < 4; j8++) {
                            uint32_t w[4];
#pragma unroll
                            for (int j2 = 0; j2 < 4; j2++) {
                                float pv[2];
#pragma unroll
                                for (int e = 0; e < 2; e++) {
                                    const int j = j8 * 8 + j2 * 2 + e;
                                    float pe = at_exp2(fmaf(__uint_as_float(s[j]), sl2, -m_sub));
                                    if (MASKED) {
                                        const int key = kt * AT_BN + c + j;
                                        if (!(live && key >= lo && key <= pos)) pe = 0.f;
                                    }
                                    pv[e] = pe;
                                }
                                lsum += pv[0] + pv[1];
                                const __nv_bfloat162 pb = __floats2bfloat162_rn(pv[0], pv[1]);
                                w[j2] = *reinterpret_cast<const uint32_t*>(&pb);
                            }
                            const int chunk = ((c & 63) >> 3) + j8;           // 16-byte piece of the 128-byte row
                            *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                };
                if (masked) pass2(std::true_type{}); else pass2(std::false_type{});
                l = l * corr + lsum;
                m = m_new;
                kp_tc_fence_before();                                           // the reads of S are done
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor core
                kp_mbar_arrive(p_full);
                // O = O * corr + P V
                if (!kp_mbar_wait_bounded(pv_full, i & 1)) { ok = false; break; }
                kp_tc_fence_after();
#pragma unroll
                for (int c = 0; c < AT_HD; c += 32) {
                    uint32_t v[32];
                    kp_tmem_ld32(tmem_pv + lane_off + c, v);
#pragma unroll
                    for (int j = 0; j < 32; j++) o[c + j] = o[c + j] * corr + __uint_as_float(v[j]);
                }
                kp_tc_fence_before();
            }
            if (ok && live) {
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                bf16* dst = p.out + (size_t)(it.row0 + r) * p.ldo + (size_t)h * AT_HD;
#pragma unroll
                for (int d = 0; d < AT_HD; d += 8) {
                    uint4 w;
                    __nv_bfloat162* w2 = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
                    for (int e = 0; e < 4; e++) w2[e] = __floats2bfloat162_rn(o[d + 2 * e] * inv, o[d + 2 * e + 1] * inv);
                    *reinterpret_cast<uint4*>(dst + d) = w;
                }
            }
        }
        if (!ok && lane == 0) atomicExch(&g_attn_tc_status, 1);
    }
    kp_tc_fence_before();
    __syncthreads();
    if (warp == 1) kp_tmem_dealloc(tmem_base, 256);
}

// ------------------------------------------------------------------ two heads a CTA
// The same tiles and formulas with the work laid out so that the tensor core and the softmax overlap: a CTA
// takes TWO query heads that share a kv head (the same rows, the same key tiles, so K and V are loaded once
// for both) and has one group of four row warps for each.  Every row thread holds its whole row of S in
// registers (one pass: maximum, exponentials, P), which frees the S columns of tensor memory at once: the
// MMA warp computes the next tile's S for a head while that head's rows are still at their softmax.  O is
// accumulated by the MMAs in tensor memory; the rows rescale it there (load, multiply, store) only when a
// row maximum of their warp has grown, which after the first tiles of a row is rare.  One CTA an SM: 160 KB
// of shared memory (Q 2 x 16, K 2 x 16, V 2 x 16, P 2 x 32), all 512 columns of tensor memory (S 2 x 128,
// O 2 x 64), 320 threads.  Needs an even number of query heads a kv head.
#define A2_THREADS 320

__global__ void __launch_bounds__(A2_THREADS, 1)
attn_prefill_tc_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmC, const AtArgs p) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* sm = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    unsigned char* Qs = sm;                                     // 2 x 16 KB: the two heads
    unsigned char* Ks = Qs + 2 * AT_TILE_BYTES;                 // 2 stages
    unsigned char* Vs = Ks + 2 * AT_TILE_BYTES;                 // 2 stages
    unsigned char* Ps = Vs + 2 * AT_TILE_BYTES;                 // 2 heads x (keys 0..63 | keys 64..127)
    uint64_t* bars = reinterpret_cast<uint64_t*>(Ps + 4 * AT_TILE_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;  uint64_t* k_empty = bars + 3;     // [2] each
    uint64_t* v_full = bars + 5;  uint64_t* v_empty = bars + 7;
    uint64_t* s_full = bars + 9;  uint64_t* s_free = bars + 11;     // [2]: one a head
    uint64_t* p_full = bars + 13; uint64_t* o_done = bars + 15;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h0 = 2 * blockIdx.y, kvh = h0 / (p.H / p.G);
    const int n_items = ((int)blockIdx.x < p.n_tiles - 1 - (int)blockIdx.x) ? 2 : 1;
    auto item_tile = [&](int idx) { return idx == 0 ? (int)blockIdx.x : p.n_tiles - 1 - (int)blockIdx.x; };

    if (threadIdx.x == 0) {
        kp_mbar_init(q_full, 1);
        for (int i = 0; i < 2; i++) {
            kp_mbar_init(&k_full[i], 1); kp_mbar_init(&k_empty[i], 1);
            kp_mbar_init(&v_full[i], 1); kp_mbar_init(&v_empty[i], 1);
            kp_mbar_init(&s_full[i], 1); kp_mbar_init(&s_free[i], 128);
            kp_mbar_init(&p_full[i], 128); kp_mbar_init(&o_done[i], 1);
        }
        *abort_flag = 0;
        kp_mbar_init_fence();
    }
    // V starts zeroed: a part of a tile that is never loaded then holds something finite
    for (int i = threadIdx.x; i < 2 * AT_TILE_BYTES / 16; i += A2_THREADS) reinterpret_cast<uint4*>(Vs)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1) kp_tmem_alloc(tmem_slot, 512);
    kp_tc_fence_before();
    __syncthreads();
    kp_tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    kp_pdl_begin();

    // registers: the first four warps need few, the row warps many (a row of S: 128)

    // `i` counts the key tiles over both items; stage i & 1 of K and V is used for the (i >> 1)-th time, the
    // per-head barriers for the i-th time.
    if (warp == 0) {
        if (lane == 0) {
            const int box = min(p.page_size, AT_BN);
            int i = 0;
            bool ok = true;
            for (int idx = 0; idx < n_items && ok; idx++) {
                const AtItem it = at_item(p, item_tile(idx));
                if (idx > 0) {
                    // Q is read by the S products; the last ones of the item before free their K stage when done
                    const int last = i - 1;
                    if (!kp_mbar_wait_bounded(&k_empty[last & 1], (last >> 1) & 1)) { *abort_flag = 1; break; }
                }
                kp_mbar_expect_tx(q_full, 2 * AT_TILE_BYTES);
                kp_tma_load_2d(Qs, &tmQ, h0 * AT_HD, it.row0, q_full);
                kp_tma_load_2d(Qs + AT_TILE_BYTES, &tmQ, (h0 + 1) * AT_HD, it.row0, q_full);
                auto load_tile = [&](unsigned char* dst, int kt, int kv, uint64_t* bar) {
                    uint32_t bytes = 0;
                    for (int key0 = kt * AT_BN; key0 < (kt + 1) * AT_BN; key0 += box)
                        if (key0 <= it.k_hi_all && key0 + box - 1 >= it.k_lo_all) bytes += box * AT_HD * 2;
                    kp_mbar_expect_tx(bar, bytes);
                    for (int key0 = kt * AT_BN; key0 < (kt + 1) * AT_BN; key0 += box) {
                        if (!(key0 <= it.k_hi_all && key0 + box - 1 >= it.k_lo_all)) continue;
                        const int page = it.bt[key0 / p.page_size];
                        const int row = ((page * 2 + kv) * p.G + kvh) * p.page_size + key0 % p.page_size;
                        kp_tma_load_2d(dst + (size_t)(key0 - kt * AT_BN) * 128, &tmC, 0, row, bar);
                    }
                };
                for (int kt = it.kt_lo; kt <= it.kt_hi; kt++, i++) {
                    const int st = i & 1, par = ((i >> 1) & 1) ^ 1;
                    if (*abort_flag || !kp_mbar_wait_bounded(&k_empty[st], par)) { *abort_flag = 1; ok = false; break; }
                    load_tile(Ks + st * AT_TILE_BYTES, kt, 0, &k_full[st]);
                    if (!kp_mbar_wait_bounded(&v_empty[st], par)) { *abort_flag = 1; ok = false; break; }
                    load_tile(Vs + st * AT_TILE_BYTES, kt, 1, &v_full[st]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = kp_umma_idesc(AT_BM, AT_BN, false);
            constexpr uint32_t idesc_pv = kp_umma_idesc(AT_BM, AT_HD, true);
            bool ok = true;
            // S of key tile i for head g: its columns are free once the head's rows hold tile i - 1 in registers
            auto issue_s = [&](int i, int g) {
                if (i > 0 && !kp_mbar_wait_bounded(&s_free[g], (i - 1) & 1)) return false;
                kp_tc_fence_after();
                const uint64_t qdesc = kp_umma_desc(kp_smem_u32(Qs + g * AT_TILE_BYTES));
                const uint64_t kdesc = kp_umma_desc(kp_smem_u32(Ks + (i & 1) * AT_TILE_BYTES));
#pragma unroll
                for (int k = 0; k < AT_HD / 16; k++)
                    kp_umma_bf16(tmem_base + 128 * g, qdesc + 2 * k, kdesc + 2 * k, idesc_s, k ? 1u : 0u);
                kp_umma_commit(&s_full[g]);
                return true;
            };
            auto issue_s_both = [&](int i) {
                if (!kp_mbar_wait_bounded(&k_full[i & 1], (i >> 1) & 1)) return false;
                if (!issue_s(i, 0) || !issue_s(i, 1)) return false;
                kp_umma_commit(&k_empty[i & 1]);
                return true;
            };
            int base = 0;
            for (int idx = 0; idx < n_items && ok; idx++) {
                const AtItem it = at_item(p, item_tile(idx));
                const int n_kt = it.kt_hi - it.kt_lo + 1;
                ok = kp_mbar_wait_bounded(q_full, idx & 1);
                if (ok) ok = issue_s_both(base);
                for (int j = 0; j < n_kt && ok; j++) {
                    const int i = base + j;
                    if (j + 1 < n_kt && !issue_s_both(i + 1)) { ok = false; break; }
                    if (!kp_mbar_wait_bounded(&v_full[i & 1], (i >> 1) & 1)) { ok = false; break; }
                    const uint32_t va = kp_smem_u32(Vs + (i & 1) * AT_TILE_BYTES);
                    for (int g = 0; g < 2 && ok; g++) {
                        // P of the head is in shared memory, and its rows have rescaled O if they had to
                        if (!kp_mbar_wait_bounded(&p_full[g], i & 1)) { ok = false; break; }
                        kp_tc_fence_after();
                        const uint32_t pa = kp_smem_u32(Ps + g * 2 * AT_TILE_BYTES);
#pragma unroll
                        for (int kk = 0; kk < AT_BN / 16; kk++)
                            kp_umma_bf16(tmem_base + 256 + 64 * g, kp_umma_desc(pa + (kk >> 2) * AT_TILE_BYTES) + 2 * (kk & 3),
                                         kp_umma_desc(va + kk * 2048), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                        kp_umma_commit(&o_done[g]);
                    }
                    if (ok) kp_umma_commit(&v_empty[i & 1]);
                }
                base += n_kt;
            }
            if (!ok) { *abort_flag = 1; atomicExch(&g_attn_tc_status, 1); }
        }
    } else {
        // ---- the rows: warps 2-5 head 0, warps 6-9 head 1; thread r of a group owns row r
        const int g = (warp - 2) >> 2;
        const int q4 = warp & 3;
        const int r = q4 * 32 + lane;
        const uint32_t lane_off = (uint32_t)(q4 * 32) << 16;
        const uint32_t tmem_s = tmem_base + 128 * g + lane_off, tmem_o = tmem_base + 256 + 64 * g + lane_off;
        unsigned char* Pg = Ps + g * 2 * AT_TILE_BYTES;
        const int h = h0 + g;
        const float sl2 = p.scale * 1.4426950408889634f;              // scale * log2(e)
        // A wait that gives up ends all waiting (ok = false) but not the walk: the arrivals that others count on
        // are still made.
        bool ok = true;
        int i = 0;
        for (int idx = 0; idx < n_items; idx++) {
            const AtItem it = at_item(p, item_tile(idx));
            const int pos = it.pos0 + r;
            const bool live = r < it.n_rows;
            const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
            const int lo_max = p.window > 0 ? max(0, it.k_hi_all - p.window + 1) : 0;
            float m = -INFINITY, l = 0.f;
            for (int kt = it.kt_lo; kt <= it.kt_hi; kt++, i++) {
                if (ok && (*abort_flag || !kp_mbar_wait_bounded(&s_full[g], i & 1))) ok = false;
                kp_tc_fence_after();
                uint32_t s0[32], s1[32], s2[32], s3[32];
                kp_tmem_ld32_issue(tmem_s, s0);
                kp_tmem_ld32_issue(tmem_s + 32, s1);
                kp_tmem_ld32_issue(tmem_s + 64, s2);
                kp_tmem_ld32_issue(tmem_s + 96, s3);
                kp_tmem_ld_wait();
                kp_tc_fence_before();
                kp_mbar_arrive(&s_free[g]);                                     // the next tile's S may be computed
                const bool masked = !(kt * AT_BN + AT_BN - 1 <= it.pos0 && kt * AT_BN >= lo_max && it.n_rows == AT_BM);
                float tmax = -INFINITY;
                auto max32 = [&](const uint32_t (&s)[32], int c) {
                    if (masked) {
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const int key = kt * AT_BN + c + j;
                            if (live && key >= lo && key <= pos) tmax = fmaxf(tmax, __uint_as_float(s[j]));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) tmax = at_max3(tmax, __uint_as_float(s[j]), __uint_as_float(s[j + 1]));
                    }
                };
                max32(s0, 0); max32(s1, 32); max32(s2, 64); max32(s3, 96);
                const float m_new = fmaxf(m, tmax * sl2);                       // in units of log2
                const float corr = (m_new == -INFINITY) ? 0.f : exp2f(m - m_new);       // m = -inf: 2^(-inf) = 0
                const float m_sub = (m_new == -INFINITY) ? 0.f : m_new;
                if (kt > it.kt_lo) {
                    // the product of the tile before has read P and added to O
                    if (ok && !kp_mbar_wait_bounded(&o_done[g], (i - 1) & 1)) ok = false;
                    if (__any_sync(0xffffffffu, corr != 1.0f)) {
                        kp_tc_fence_after();
#pragma unroll 1
                        for (int c = 0; c < AT_HD; c += 32) {
                            uint32_t v[32];
                            kp_tmem_ld32(tmem_o + c, v);
#pragma unroll
                            for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
                            kp_tmem_st32(tmem_o + c, v);
                        }
                        kp_tmem_st_wait();
                    }
                }
                float lsum = 0.f;
                auto p32 = [&](const uint32_t (&s)[32], int c, auto masked_c) {
                    constexpr bool MASKED = decltype(masked_c)::value;
                    unsigned char* prow = Pg + (c >> 6) * AT_TILE_BYTES + r * 128;
#pragma unroll
                    for (int j8 = 0; j8 < 4; j8++) {
                        uint32_t w[4];
#pragma unroll
                        for (int j2 = 0; j2 < 4; j2++) {
                            float pv[2];
#pragma unroll
                            for (int e = 0; e < 2; e++) {
                                const int j = j8 * 8 + j2 * 2 + e;
                                float pe = at_exp2(fmaf(__uint_as_float(s[j]), sl2, -m_sub));
                                if (MASKED) {
                                    const int key = kt * AT_BN + c + j;
                                    if (!(live && key >= lo && key <= pos)) pe = 0.f;
                                }
                                pv[e] = pe;
                            }
                            lsum += pv[0] + pv[1];
                            const __nv_bfloat162 pb = __floats2bfloat162_rn(pv[0], pv[1]);
                            w[j2] = *reinterpret_cast<const uint32_t*>(&pb);
                        }
                        const int chunk = ((c & 63) >> 3) + j8;               // 16-byte piece of the 128-byte row
                        *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                };
                if (masked) {
                    p32(s0, 0, std::true_type{}); p32(s1, 32, std::true_type{}); p32(s2, 64, std::true_type{}); p32(s3, 96, std::true_type{});
                } else {
                    p32(s0, 0, std::false_type{}); p32(s1, 32, std::false_type{}); p32(s2, 64, std::false_type{}); p32(s3, 96, std::false_type{});
                }
                l = l * corr + lsum;
                m = m_new;
                kp_tc_fence_before();                                           // O (if rescaled) is written
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor core
                kp_mbar_arrive(&p_full[g]);
            }
            // the row is complete when the last product is
            if (ok && !kp_mbar_wait_bounded(&o_done[g], (i - 1) & 1)) ok = false;
            kp_tc_fence_after();
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* dst = p.out + (size_t)(it.row0 + r) * p.ldo + (size_t)h * AT_HD;
#pragma unroll 1
            for (int c = 0; c < AT_HD; c += 32) {
                uint32_t v[32];
                kp_tmem_ld32(tmem_o + c, v);
                if (ok && live) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint4 w;
                        __nv_bfloat162* w2 = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            w2[e] = __floats2bfloat162_rn(__uint_as_float(v[d + 2 * e]) * inv, __uint_as_float(v[d + 2 * e + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c + d) = w;
                    }
                }
            }
            kp_tc_fence_before();
        }
        if (!ok && lane == 0) atomicExch(&g_attn_tc_status, 1);
    }
    kp_tc_fence_before();
    __syncthreads();
    if (warp == 1) kp_tmem_dealloc(tmem_base, 512);
}

static int g_at_pair = 1;                     // 1: two heads a CTA where the head counts allow it; 0: never

extern "C" {

// tile_seg / tile_row0: the 128-row tiles of the step, most keys first (device arrays, n_tiles long);
// n_rows_total: rows of q.
int kp_attention_prefill_tc(const void* q, int ldq, int n_rows_total, const void* cache, long long n_pages,
                            const int* block_table, int max_blocks, const int* cu_rows, const int* seg_pos,
                            const int* tile_seg, const int* tile_row0, int n_tiles, void* out, int ldo, float scale,
                            int window, int page_size, int H, int G, int hd, void* stream) {
    if (n_tiles <= 0) return 0;
    if (hd != AT_HD || G < 1 || H % G || H > 65535 || (ldq & 7) || (ldo & 7) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) ||
        ((uintptr_t)cache & 15) || page_size < 8 || (page_size % 8) || !(page_size % AT_BN == 0 || AT_BN % page_size == 0) ||
        n_pages <= 0 || n_pages * 2 * G * page_size >= 2147483647LL)
        return KP_ERR_UNSUPPORTED;
    alignas(64) CUtensorMap tq, tc;
    int st = kp_make_map_bf16_2d(&tq, q, (unsigned long long)n_rows_total, H * hd, ldq, AT_HD, AT_BM);
    if (st) return st;
    st = kp_make_map_bf16_2d(&tc, cache, (unsigned long long)n_pages * 2 * G * page_size, hd, hd, AT_HD,
                             page_size < AT_BN ? page_size : AT_BN);
    if (st) return st;
    AtArgs a = {};
    a.block_table = block_table; a.max_blocks = max_blocks; a.cu_rows = cu_rows; a.seg_pos = seg_pos;
    a.tile_seg = tile_seg; a.tile_row0 = tile_row0; a.out = (bf16*)out; a.ldo = ldo; a.scale = scale; a.window = window;
    a.page_size = page_size; a.H = H; a.G = G; a.n_tiles = n_tiles;
    if (g_at_pair && (H / G) % 2 == 0) {
        const size_t smem2 = 1024 + 10 * AT_TILE_BYTES + 17 * 8 + 16;
        static bool attr2_set = false;
        if (!attr2_set) {
            cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
            if (e != cudaSuccess) return (int)e;
            attr2_set = true;
        }
        kp_launch_pdl(attn_prefill_tc_pair_kernel, dim3((n_tiles + 1) / 2, H / 2), dim3(A2_THREADS), smem2, (cudaStream_t)stream, tq, tc, a);
        return kp_launch_status();
    }
    const size_t smem = 1024 + 6 * AT_TILE_BYTES + 10 * 8 + 16;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    kp_launch_pdl(attn_prefill_tc_kernel, dim3((n_tiles + 1) / 2, H), dim3(AT_THREADS), smem, (cudaStream_t)stream, tq, tc, a);
    return kp_launch_status();
}

// 1 (default): two heads a CTA where the head counts allow it; 0: one head a CTA always.  For measurements and tests.
void kp_attention_tc_set_pair(int on) { g_at_pair = on ? 1 : 0; }


}  // extern "C"
