// The allocation-free variant of the split-KV decode attention: see attention_noalloc.h for who it is
// for and what it costs.  It runs the kernels of attention_decode.cu (included below, unchanged) with
// their scratch in a fixed array inside this library.
#include "attention_noalloc.h"

#include "attention_decode.cu"

// The scratch of every call: chunk partials (unnormalised sums, then maxima and sums of exponentials).
// In host code this name is only a handle for the runtime -- it is not a device address, and a kernel
// handed it would read and write the wrong memory -- so the address is asked for once per device below.
static __device__ __align__(256) float g_noalloc_scratch[KP_NOALLOC_SCRATCH_FLOATS];

#define KP_NOALLOC_MAX_DEVICES 64
static float* s_scratch_of_device[KP_NOALLOC_MAX_DEVICES];      // device address of the array, per device

// The array's address on the current device; looked up at the first call on that device.
static int scratch_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= KP_NOALLOC_MAX_DEVICES) return KP_ERR_UNSUPPORTED;
    if (s_scratch_of_device[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        s_scratch_of_device[dev] = static_cast<float*>(p);
    }
    *out = s_scratch_of_device[dev];
    return 0;
}

extern "C" {

long long kp_attention_split_noalloc_need(int n_rows, int H, int head_dim, int n_chunks) {
    return kp_attention_split_scratch(n_rows, H, head_dim, n_chunks);
}

const char* kp_attention_split_noalloc_strerror(int code) {
    switch (code) {
        case 0: return "ok";
        case KP_NOALLOC_TOO_LARGE:
            return "the call needs more scratch than the library's fixed array holds "
                   "(n_rows * H * n_chunks * (head_dim + 2) floats against 1048576); split the batch";
        case KP_ERR_BAD_ARG: return "bad argument";
        case KP_ERR_UNSUPPORTED: return "sizes not supported by the kernel";
        default: return "CUDA error (the code is a cudaError_t)";
    }
}

int kp_attention_split_noalloc(const void* q, int ldq, const void* cache, const int* block_table, int max_blocks,
                               const int* row_seg, const int* positions, void* out, int ldo, int n_chunks,
                               float scale, int window, int page_size, int n_rows, int H, int G, int head_dim,
                               int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (H < 1 || head_dim < 1 || n_chunks < 1) return KP_ERR_BAD_ARG;
    if (kp_attention_split_scratch(n_rows, H, head_dim, n_chunks) > (long long)KP_NOALLOC_SCRATCH_FLOATS)
        return KP_NOALLOC_TOO_LARGE;
    float* scratch = nullptr;
    const int st = scratch_address(&scratch);
    if (st) return st;
    // the chunk pass writes each (row, head, chunk) partial that the merge pass reads, so the array's old
    // contents never matter and nothing is cleared here
    return kp_attention_split(q, ldq, cache, block_table, max_blocks, row_seg, positions, out, ldo, scratch,
                              n_chunks, scale, window, page_size, n_rows, H, G, head_dim, dtype, stream);
}

}  // extern "C"
