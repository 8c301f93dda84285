// Greedy token selection with library-owned scratch memory; see argmax_static.h for the contract.
//
// Same two steps as the regular wide-row argmax: 32 blocks per row each scan a slice and leave
// (value, index, nonfinite) in scratch, a second kernel picks the winner.  The scratch is the
// file-scope device array below instead of caller memory.
#include <math.h>

#include "argmax_static.h"

// One record per (row, slice): value, index, nonfinite flag.
struct __align__(4) SliceBest { float value; int index; int nonfinite; };

// In host code this name is only a handle for cudaGetSymbolAddress, not a device address: the
// launcher below asks the runtime for the address once per device and passes that to the kernels.
static __device__ __align__(256) SliceBest g_scratch[GESSO_ARGMAX_STATIC_MAX_ROWS * GESSO_ARGMAX_STATIC_SPLIT];
static_assert(sizeof(g_scratch) == GESSO_ARGMAX_STATIC_SCRATCH_BYTES, "scratch size differs from the header");

__global__ void __launch_bounds__(256)
argmax_static_partial(const float* __restrict__ logits, int V, SliceBest* __restrict__ scratch) {
    __shared__ float s_val[8];
    __shared__ int s_idx[8], s_bad[8];
    const int row = blockIdx.y, part = blockIdx.x;
    const int per = (V + GESSO_ARGMAX_STATIC_SPLIT - 1) / GESSO_ARGMAX_STATIC_SPLIT;
    const int lo = part * per, hi = min(V, lo + per);
    const float* r = logits + (size_t)row * V;
    float best = -INFINITY;
    int bi = 0x7fffffff, bad = 0;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = r[i];
        if (!isfinite(v)) bad = 1;
        if (v > best) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        bad |= __shfl_xor_sync(0xffffffffu, bad, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) { s_val[wid] = best; s_idx[wid] = bi; s_bad[wid] = bad; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
            if (s_val[w] > best || (s_val[w] == best && s_idx[w] < bi)) { best = s_val[w]; bi = s_idx[w]; }
            bad |= s_bad[w];
        }
        SliceBest out;
        out.value = best;
        out.index = bi;
        out.nonfinite = bad;
        scratch[row * GESSO_ARGMAX_STATIC_SPLIT + part] = out;   // every slot that is read is written first
    }
}

__global__ void argmax_static_final(const SliceBest* __restrict__ scratch, int* __restrict__ ids,
                                    int* __restrict__ nonfinite) {
    const int row = blockIdx.x, lane = threadIdx.x;     // 32 threads, one per slice
    const SliceBest mine = scratch[row * GESSO_ARGMAX_STATIC_SPLIT + lane];
    float best = mine.value;
    int bi = mine.index, bad = mine.nonfinite;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        bad |= __shfl_xor_sync(0xffffffffu, bad, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { ids[row] = bi == 0x7fffffff ? 0 : bi; nonfinite[row] = bad; }
}

#define MAX_DEVICES 64
static SliceBest* g_scratch_addr[MAX_DEVICES];   // device address of g_scratch, per device, once looked up

extern "C" int gesso_argmax_rows_static(const float* logits, int n_rows, int vocab, int* ids, int* nonfinite,
                                        cudaStream_t stream) {
    if (n_rows == 0) return 0;
    if (n_rows < 0 || vocab < 1 || !logits || !ids || !nonfinite) return GESSO_ARGMAX_STATIC_BAD_ARGUMENT;
    if (n_rows > GESSO_ARGMAX_STATIC_MAX_ROWS) return GESSO_ARGMAX_STATIC_TOO_MANY_ROWS;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return GESSO_ARGMAX_STATIC_BAD_ARGUMENT;
    if (!g_scratch_addr[dev]) {
        // Set-up, once per device, with that device current: the array's address on THIS device.
        // (Passing `g_scratch` itself to a kernel from host code would hand it a host-side stand-in.)
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_scratch);
        if (e != cudaSuccess) return (int)e;
        g_scratch_addr[dev] = static_cast<SliceBest*>(p);
    }
    SliceBest* scratch = g_scratch_addr[dev];
    argmax_static_partial<<<dim3(GESSO_ARGMAX_STATIC_SPLIT, n_rows), 256, 0, stream>>>(logits, vocab, scratch);
    argmax_static_final<<<n_rows, 32, 0, stream>>>(scratch, ids, nonfinite);
    return (int)cudaGetLastError();
}
