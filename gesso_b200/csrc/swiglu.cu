// SwiGLU activation on the fused gate/up projection.
//
// Input [N, 2F]: columns [0,F) are the gate projection g, [F,2F) the up projection u.
// out = (g / (1 + exp(-g))) * u  (src/Operators/cpu.jl:482-488), evaluated in float32.
#include <math.h>

#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, long long n_rows, int F) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * F) return;
    const long long r = i / F;
    const int f = (int)(i % F);
    const float g = to_f32(gu[r * 2 * F + f]);
    const float u = to_f32(gu[r * 2 * F + F + f]);
    out[i] = from_f32<T>((g / (1.f + expf(-g))) * u);
}

GESSO_API int gesso_swiglu(const void* gu, void* out, int dtype, int n_rows, int F, cudaStream_t stream) {
    if (n_rows <= 0 || F <= 0) return 0;
    const long long total = (long long)n_rows * F;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    if (dtype == GESSO_F32)
        swiglu_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>((const float*)gu, (float*)out, n_rows, F);
    else if (dtype == GESSO_BF16)
        swiglu_kernel<bf16><<<(unsigned)blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, n_rows, F);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}
