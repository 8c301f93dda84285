// What an architecture may do to its logits after the head: a scale and a soft cap.
//
// logits = cap * tanh(scale * logits / cap)   (without a cap: scale * logits), in place, float32.
// LFM2 does neither (no soft cap, no bias on its head, src/Inference/Inference.jl:2747-2800), so its steps
// never launch this; the model spec carries both values for architectures that do.
#include <math.h>

#include "common.cuh"

__global__ void logit_transform_kernel(float* __restrict__ logits, long long n, float scale, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float x = logits[i] * scale;
    if (cap > 0.f) x = cap * tanhf(x / cap);
    logits[i] = x;
}

// logits: float32 [n]; cap <= 0: no soft cap.
GESSO_API int gesso_logit_transform(float* logits, long long n, float scale, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    const long long blocks = (n + threads - 1) / threads;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    launch_pdl(logit_transform_kernel, dim3((unsigned)blocks), dim3(threads), 0, stream, logits, n, scale, cap);
    return launch_status();
}
