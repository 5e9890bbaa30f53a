// True 32-bit matrix product for the float32 path: C[n, m] = sum_k A[n, k] * W[m, k], no tensor cores, no TF32.
// Every output element is one float accumulator fed by fmaf in ascending k, so its value depends on neither the
// number of rows in the call nor on the tile it falls into: the 32-bit path gives the same logits however the tokens
// are cut into steps.
#include "common.cuh"

#define TILE 64
#define BK 16

__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W,
                                                        float* __restrict__ C, int N, int M, int K) {
    __shared__ float As[BK][TILE + 4];
    __shared__ float Ws[BK][TILE + 4];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;       // tx: 4 output columns (m), ty: 4 output rows (n)
    const int n0 = blockIdx.y * TILE, m0 = blockIdx.x * TILE;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 x 16 values of each operand, 4 per thread: thread t loads row t / 4, k columns (t % 4) * 4 .. + 3
        const int lr = threadIdx.x / 4, lk = (threadIdx.x % 4) * 4;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k = k0 + lk + j;
            const int an = n0 + lr, wm = m0 + lr;
            As[lk + j][lr] = (an < N && k < K) ? A[(size_t)an * K + k] : 0.0f;
            Ws[lk + j][lr] = (wm < M && k < K) ? W[(size_t)wm * K + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int n = n0 + ty * 4 + i;
        if (n >= N) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int m = m0 + tx * 4 + j;
            if (m < M) C[(size_t)n * M + m] = acc[i][j];
        }
    }
}

MB_API int mb_gemm_f32(const float* A, const float* W, float* C, int N, int M, int K, cudaStream_t st) {
    if (N == 0 || M == 0) return 0;
    dim3 grid((M + TILE - 1) / TILE, (N + TILE - 1) / TILE);
    if (grid.y > 65535) return -2;
    gemm_f32_kernel<<<grid, 256, 0, st>>>(A, W, C, N, M, K);
    MB_LAUNCH_CHECK();
    return 0;
}
