// True float32 matrix product for the 32-bit path: C[M,N] = A[M,K] * W[N,K]^T.
//
// FFMA on the CUDA cores only: no tensor-core instruction, so no TF32 anywhere.  Every output
// element is accumulated over k = 0 .. K-1 in ascending order by one thread, so its value
// does not depend on M, on the row's place in the batch, or on the launch shape.
#include "common.cuh"

#define GF_BM 64
#define GF_BN 64
#define GF_BK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K, int lda, int ldw, int ldc) {
    __shared__ float As[GF_BK][GF_BM + 4];
    __shared__ float Ws[GF_BK][GF_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;          // tx: 4 columns, ty: 4 rows
    const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GF_BK) {
        // 64 x 16 elements per operand, 256 threads: 4 each, k fastest for coalescing
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int e = tid + r * 256;
            const int row = e >> 4, kk = e & 15;
            const int k = k0 + kk;
            const int m = m0 + row, n = n0 + row;
            As[kk][row] = (m < M && k < K) ? A[(size_t)m * lda + k] : 0.f;
            Ws[kk][row] = (n < N && k < K) ? W[(size_t)n * ldw + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GF_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
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
            if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
        }
    }
}

RB_EXPORT int rb_gemm_f32(const float* A, const float* W, float* C, int M, int N, int K,
                          int lda, int ldw, int ldc, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
    gemm_f32_kernel<<<grid, 256, 0, st>>>(A, W, C, M, N, K, lda, ldw, ldc);
    return rb_launch_status();
}
