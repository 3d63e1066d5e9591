// C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) on the CUDA cores, float32 FMA.
//
// This is the matrix product of the true 32-bit path (no tensor-core mode of
// reduced precision is involved) and the general fallback of the bfloat16 path
// for shapes the tensor-core kernels refuse.  W is row-major [out][in] as in
// the reference (src/backend/cpu/scalar/quants.c:1367-1414); each output
// element sums k = 0..K-1 in order, so a row's result does not depend on M.
#include "common.cuh"

#define EPI_STORE 0      // C (type T) = acc
#define EPI_STORE_F32 1  // C (float)  = acc
#define EPI_ACCUM_F32 2  // C (float) += acc        (residual sum in 32-bit)

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
gemm_nt_simt_kernel(const T* __restrict__ A, const T* __restrict__ W, const float* __restrict__ bias,
                    void* __restrict__ Cv, int M, int N, int K, int lda, int ldw, int ldc) {
    kp_pdl_begin();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;          // 16 x 16 threads, 4x4 outputs each
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64x16 elements per operand, 256 threads: 4 each
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int e = tid + i * 256;
            const int r = e / BK, c = e % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
            Ws[c][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; i++) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; j++) b[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[gn];
            const size_t o = (size_t)gm * ldc + gn;
            if (EPI == EPI_STORE) ((T*)Cv)[o] = from_f32<T>(v);
            else if (EPI == EPI_STORE_F32) ((float*)Cv)[o] = v;
            else ((float*)Cv)[o] += v;
        }
    }
}

template <typename T>
static int launch(const void* A, const void* W, const float* bias, void* C, int M, int N, int K, int lda, int ldw,
                  int ldc, int epi, cudaStream_t s) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (epi == EPI_STORE)
        kp_launch_pdl(gemm_nt_simt_kernel<T, EPI_STORE>, dim3(grid), dim3(256), 0, s, (const T*)A, (const T*)W, bias, C, M, N, K, lda, ldw, ldc);
    else if (epi == EPI_STORE_F32)
        kp_launch_pdl(gemm_nt_simt_kernel<T, EPI_STORE_F32>, dim3(grid), dim3(256), 0, s, (const T*)A, (const T*)W, bias, C, M, N, K, lda, ldw, ldc);
    else if (epi == EPI_ACCUM_F32)
        kp_launch_pdl(gemm_nt_simt_kernel<T, EPI_ACCUM_F32>, dim3(grid), dim3(256), 0, s, (const T*)A, (const T*)W, bias, C, M, N, K, lda, ldw, ldc);
    else
        return KP_ERR_BAD_ARG;
    return kp_launch_status();
}

extern "C" int kp_gemm_nt_simt(const void* A, const void* W, const float* bias, void* C, int M, int N, int K, int lda,
                               int ldw, int ldc, int epi, int dtype, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return KP_ERR_BAD_ARG;
    if ((long long)((M + BM - 1) / BM) > 65535) return KP_ERR_UNSUPPORTED;
    KP_DISPATCH_DTYPE(dtype, T, return launch<T>(A, W, bias, C, M, N, K, lda, ldw, ldc, epi, (cudaStream_t)stream));
    return 0;
}
