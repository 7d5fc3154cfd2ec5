// True float32 matrix product for the 32-bit path: C[M,N] = A[M,K] * W[N,K]^T.
//
// Plain FMA on the CUDA cores, no tensor-core mode of reduced precision. Every
// output element is one chain of fused multiply-adds over k = 0..K-1 in order,
// so a row's result does not depend on M, on the row's place in the batch or on
// the tiling: the 32-bit path is bitwise the same however the tokens are cut.
// Weights are stored [out, in] row-major as in the checkpoint
// (python/stride_worker/model.py:258-260).
#include "common.cuh"

namespace stride {

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256) gemm_nt_f32_kernel(const float* __restrict__ A, const float* __restrict__ W,
                                                          float* __restrict__ C, int M, int N, int K, int lda, int ldw,
                                                          int ldc) {
    pdl_trigger();
    pdl_wait();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4] = {};
    // each thread loads 4 elements of each tile: row = tid / 4 (+0), k = (tid % 4) * 4 .. +3
    const int lrow = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + j][lrow] = (am < M && k < K) ? A[static_cast<size_t>(am) * lda + k] : 0.f;
            Ws[lk + j][lrow] = (wn < N && k < K) ? W[static_cast<size_t>(wn) * ldw + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[static_cast<size_t>(m) * ldc + n] = acc[i][j];
        }
    }
}

}  // namespace stride

extern "C" int stride_gemm_nt_f32(const float* A, const float* W, float* C, int M, int N, int K, int lda, int ldw, int ldc,
                                  cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0 || lda < K || ldw < K || ldc < N) return STRIDE_BAD_ARGUMENT;
    if (M == 0) return 0;
    dim3 grid((N + stride::BN - 1) / stride::BN, (M + stride::BM - 1) / stride::BM);
    if (grid.y > 65535) return STRIDE_UNSUPPORTED;
    stride::launch(stride::gemm_nt_f32_kernel, dim3(grid), dim3(256), 0, stream, A, W, C, M, N, K, lda, ldw, ldc);
    return STRIDE_LAUNCH_STATUS();
}
