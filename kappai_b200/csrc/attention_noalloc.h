/* Split-KV decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference (System64fumo/kappai);
 * it exists for users of this library.
 *
 * Who needs it: code that runs where cudaMalloc is off limits -- inside a CUDA
 * graph capture, inside a host callback or a real-time loop that must not take
 * the allocator's locks, or in a process whose device memory was handed out in
 * full at start-up and has no allocator to ask.  The ordinary entry point,
 * kp_attention_split, needs a scratch buffer from its caller (the per-chunk
 * partial results that the merge pass reads); such callers have nowhere to get
 * one.  Here the scratch is a fixed array that lives inside the library.
 *
 * What it costs: every GPU on which this library is loaded holds the array
 * (KP_NOALLOC_SCRATCH_FLOATS floats, 4 MiB) from load until the process ends,
 * whether or not the entry point is ever called.  That is why it is a library
 * of its own and not part of the one the engine loads.
 *
 * Limits and rules
 *  - n_rows * H * n_chunks * (head_dim + 2) must not exceed
 *    KP_NOALLOC_SCRATCH_FLOATS; a larger call is refused with
 *    KP_NOALLOC_TOO_LARGE and nothing is launched.
 *  - n_chunks (chunks of 256 keys) must reach the largest position of the
 *    batch: positions[r] < n_chunks * 256 for every row, and the block table
 *    must cover that position.  A row beyond it is merged from the chunks
 *    that exist (its result is then wrong, but nothing is read out of range).
 *  - The first call on a device looks up the array's device address (one
 *    cudaGetSymbolAddress, with that device current) and keeps it.  Make that
 *    first call outside any stream capture.
 *  - All calls share the one array and it keeps what the last call left.  The
 *    kernels write every partial result before they read it, so nothing has to
 *    be cleared between calls; but two calls that overlap on the GPU (different
 *    streams, no ordering between them) race on it.  Order them.
 *  - It calls no cudaMalloc, cudaFree or other allocating routine.
 *
 * Arguments are those of kp_attention_split without the scratch pointer; the
 * result is the same.
 */
#ifndef KAPPAI_B200_ATTENTION_NOALLOC_H
#define KAPPAI_B200_ATTENTION_NOALLOC_H

#ifdef __cplusplus
extern "C" {
#endif

#define KP_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define KP_NOALLOC_TOO_LARGE (-27)

/* 0, a cudaError_t, KP_NOALLOC_TOO_LARGE, or the argument errors of kp_attention_split (-22, -95). */
int kp_attention_split_noalloc(const void* q, int ldq, const void* cache, const int* block_table, int max_blocks,
                               const int* row_seg, const int* positions, void* out, int ldo, int n_chunks,
                               float scale, int window, int page_size, int n_rows, int H, int G, int head_dim,
                               int dtype, void* stream);

/* Floats of scratch a call with these sizes needs (compare with KP_NOALLOC_SCRATCH_FLOATS). */
long long kp_attention_split_noalloc_need(int n_rows, int H, int head_dim, int n_chunks);

/* A sentence for a return code of kp_attention_split_noalloc. */
const char* kp_attention_split_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif
