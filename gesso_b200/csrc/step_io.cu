// Small copies between steps, done by a kernel instead of by the copy engines.
//
// Between two decoding steps the stream carries a handful of tiny transfers: the next step's metadata
// from pinned host memory (a few KB), the sampled ids from the selection's output into that metadata,
// the status words and the ids back to pinned host memory.  As memcpy operations each of them costs
// 3 us of its own plus 2 to 7 us for the change between the compute and the copy engines, in a chain
// where the next step can only start when the last one has finished.  A kernel reads and writes pinned
// host memory directly (it is mapped into the device's address space), several segments per launch,
// and the chain stays on one engine.  What a kernel wrote to host memory is seen by the host once it has
// waited for an event recorded behind the kernel.
#include "common.cuh"

#define COPY_SEGS 6

struct CopySegs {
    int* dst[COPY_SEGS];
    const int* src[COPY_SEGS];
    long long n[COPY_SEGS];      // 32-bit words
};

// Segments of one launch must not overlap one another (blocks work on all of them at once).
__global__ void __launch_bounds__(256) copy_words_kernel(const CopySegs s, int n_segs) {
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
    for (int k = 0; k < n_segs; ++k) {
        int* __restrict__ d = s.dst[k];
        const int* __restrict__ a = s.src[k];
        const long long n = s.n[k];
        if ((((size_t)d | (size_t)a) & 15) == 0) {
            const long long n4 = n / 4;
            for (long long i = tid; i < n4; i += stride) reinterpret_cast<int4*>(d)[i] = reinterpret_cast<const int4*>(a)[i];
            for (long long i = 4 * n4 + tid; i < n; i += stride) d[i] = a[i];
        } else {
            for (long long i = tid; i < n; i += stride) d[i] = a[i];
        }
    }
}

// dst / src: device memory or pinned (mapped) host memory; n: words of 32 bits; at most COPY_SEGS segments.
GESSO_API int gesso_copy_words(int n_segs, void* const* dst, const void* const* src, const long long* n,
                               cudaStream_t stream) {
    if (n_segs <= 0) return 0;
    if (n_segs > COPY_SEGS) return GESSO_ERR_BAD_SIZE;
    CopySegs s = {};
    long long most = 0;
    for (int k = 0; k < n_segs; ++k) {
        if (n[k] < 0 || (n[k] > 0 && (!dst[k] || !src[k]))) return GESSO_ERR_BAD_SIZE;
        s.dst[k] = (int*)dst[k];
        s.src[k] = (const int*)src[k];
        s.n[k] = n[k];
        if (n[k] > most) most = n[k];
    }
    if (most == 0) return 0;
    long long blocks = (most / 4 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 4LL * gesso_sm_count()) blocks = 4LL * gesso_sm_count();
    copy_words_kernel<<<(unsigned)blocks, 256, 0, stream>>>(s, n_segs);
    return launch_status();
}
