// SwiGLU activation on the fused gate/up projection.
//
// Input [N, 2F].  Plain layout: columns [0,F) are the gate projection g, [F,2F) the up projection
// u.  Packed layout: every group of 16 columns holds 8 gate columns and then the matching 8 up
// columns (the row order in which the skinny matrix product wants the fused weight).
// out = (g / (1 + exp(-g))) * u  (src/Operators/cpu.jl:482-488), evaluated in float32.
#include <math.h>

#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, long long n_rows, int F, int packed) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * F) return;
    const long long r = i / F;
    const int f = (int)(i % F);
    const T* row = gu + r * 2 * F;
    const int gi = packed ? 16 * (f >> 3) + (f & 7) : f;
    const int ui = packed ? gi + 8 : F + f;
    const float g = to_f32(row[gi]);
    const float u = to_f32(row[ui]);
    out[i] = from_f32<T>((g / (1.f + expf(-g))) * u);
}

GESSO_API int gesso_swiglu(const void* gu, void* out, int dtype, int n_rows, int F, int packed, cudaStream_t stream) {
    if (n_rows <= 0 || F <= 0) return 0;
    if (packed && F % 8 != 0) return GESSO_ERR_BAD_SIZE;
    const long long total = (long long)n_rows * F;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    if (dtype == GESSO_F32)
        swiglu_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>((const float*)gu, (float*)out, n_rows, F, packed);
    else if (dtype == GESSO_BF16)
        swiglu_kernel<bf16><<<(unsigned)blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, n_rows, F, packed);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}
