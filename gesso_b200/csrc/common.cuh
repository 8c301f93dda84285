// Shared helpers of the sm_100a kernel library.
//
// Every launcher is `extern "C"`, takes raw device pointers, sizes and the stream to launch
// on, and returns 0 or a negative refusal code / positive cudaError_t.  A launcher never
// allocates and never synchronises.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define GESSO_API extern "C" __attribute__((visibility("default")))

// refusal codes (sizes a kernel does not take); positive values are cudaError_t
#define GESSO_ERR_BAD_DTYPE (-2)
#define GESSO_ERR_BAD_SIZE (-3)
#define GESSO_ERR_UNSUPPORTED (-4)

enum GessoDtype { GESSO_F32 = 0, GESSO_BF16 = 1 };

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the total.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();   // `red` may still be read from an earlier call
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

static inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return (int)e;
}

// ---- programmatic dependent launch ------------------------------------------------------------------
// Kernels of a decoding step are launched with the "programmatic stream serialization" attribute: a
// kernel may be scheduled while its predecessor still runs, does what does not depend on earlier
// kernels (its weight prefetch), and executes pdl_wait() before it touches anything an earlier
// kernel produced; pdl_launch_dependents() lets its own successor in.  Without the attribute both
// calls do nothing, so every kernel also runs correctly when launched the plain way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

extern int gesso_pdl_enabled;   // runtime.cu; set through gesso_set_pdl()
extern "C" int gesso_sm_count();  // runtime.cu; streaming multiprocessors of the current device

template <typename... KArgs, typename... Args>
static inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gesso_pdl_enabled ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
