// True float32 matrix product for the 32-bit path:  C = A @ W^T (+ bias),
// A [M, K] row-major, W [N, K] row-major (the [out, in] layout of the model
// file, andre-fu/prism engine/weight_pool.py:46-70; F.linear at
// engine/executor.py:109,122,125,127,130).  CUDA-core FFMA only: no tensor
// cores, no TF32, no split-K.  Every output element is accumulated over k in
// ascending order inside one thread, so its value does not depend on M, on
// the row's place in the batch, or on the grid.
#include "common.cuh"

namespace prism {

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
sgemm_nt_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                const void* __restrict__ bias, int bias_bf16, float* __restrict__ C, int ldc,
                int M, int N, int K) {
    pdl_trigger();
    pdl_wait();
    constexpr int THREADS = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int idx = tid; idx < BM * BK; idx += THREADS) {
            const int r = idx / BK, c = idx % BK;
            As[c][r] = (m0 + r < M && k0 + c < K) ? A[(size_t)(m0 + r) * lda + k0 + c] : 0.f;
        }
        for (int idx = tid; idx < BN * BK; idx += THREADS) {
            const int r = idx / BK, c = idx % BK;
            Ws[c][r] = (n0 + r < N && k0 + c < K) ? W[(size_t)(n0 + r) * ldw + k0 + c] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias != nullptr) v += load_param(bias, bias_bf16, n);
            C[(size_t)m * ldc + n] = v;
        }
    }
}

}  // namespace prism

PRISM_EXPORT int prism_sgemm_nt(const float* A, int lda, const float* W, int ldw, const void* bias,
                                int bias_dtype, float* C, int ldc, int M, int N, int K,
                                cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    const int bb = bias_dtype == PRISM_DTYPE_BF16;
    if (M <= 16) {
        dim3 grid((N + 63) / 64, (M + 15) / 16);
        prism::sgemm_nt_kernel<16, 64, 32, 1, 4><<<grid, 256, 0, stream>>>(A, lda, W, ldw, bias, bb, C, ldc, M, N, K);
    } else {
        dim3 grid((N + 63) / 64, (M + 63) / 64);
        prism::sgemm_nt_kernel<64, 64, 16, 4, 4><<<grid, 256, 0, stream>>>(A, lda, W, ldw, bias, bb, C, ldc, M, N, K);
    }
    return (int)cudaPeekAtLastError();
}
