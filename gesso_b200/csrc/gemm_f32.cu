// True 32-bit matrix product on CUDA cores: C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]).
//
// This is the matrix product of the float32 path.  No tensor-core mode is involved (TF32
// would round the inputs to 10 mantissa bits), every product is an FP32 FMA, and the sum over
// k runs in the same order for every output element whatever M and N are, so a row's result
// does not depend on how many other rows share the batch.  W is stored (out, in) as the
// reference stores projection weights (src/Operators/cpu.jl:629-630).
//
// Tile 64x64x16, 256 threads, 4x4 outputs per thread; edges are bounds-checked (any M, N, K).
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const float* __restrict__ bias,
                float* __restrict__ C, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = threadIdx.x + e * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * K + gk]) : 0.f;
            Ws[kk][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
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
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)gm * N + gn] = acc[i][j] + (bias ? bias[gn] : 0.f);
        }
    }
}

GESSO_API int gesso_gemm_f32(const void* A, int a_dtype, const void* W, int w_dtype, const float* bias, float* C,
                             int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return GESSO_ERR_BAD_SIZE;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return GESSO_ERR_BAD_SIZE;
    if (a_dtype == GESSO_F32 && w_dtype == GESSO_F32)
        gemm_f32_kernel<float, float><<<grid, 256, 0, stream>>>((const float*)A, (const float*)W, bias, C, M, N, K);
    else if (a_dtype == GESSO_F32 && w_dtype == GESSO_BF16)
        gemm_f32_kernel<float, bf16><<<grid, 256, 0, stream>>>((const float*)A, (const bf16*)W, bias, C, M, N, K);
    else if (a_dtype == GESSO_BF16 && w_dtype == GESSO_F32)
        gemm_f32_kernel<bf16, float><<<grid, 256, 0, stream>>>((const bf16*)A, (const float*)W, bias, C, M, N, K);
    else if (a_dtype == GESSO_BF16 && w_dtype == GESSO_BF16)
        gemm_f32_kernel<bf16, bf16><<<grid, 256, 0, stream>>>((const bf16*)A, (const bf16*)W, bias, C, M, N, K);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}
