// Paged causal attention for any head size, in float32 arithmetic (CUDA cores).
//
// This is the kernel of the true 32-bit path, and the bfloat16 path uses it for head sizes its
// tensor-core kernels do not take.  One warp per (token, query head).  A query at absolute
// position p reads keys lo..p of its own request, lo = max(0, p - window + 1) with a window,
// else 0 (src/Inference/Inference.jl:1206-1207).  Query head h reads kv head h / (nh/nkv)
// (src/Inference/Inference.jl:1398).  Score = (q . k) / sqrt(hd); softmax and the weighted sum
// of values are float32 with a running maximum per lane (lanes stride over keys) that is
// merged across the warp at the end, so the result does not depend on which pages hold the keys
// or on what else is in the batch.
#include <math.h>

#include "common.cuh"

template <typename T, int HD_PAD>
__global__ void __launch_bounds__(128)
paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                               const T* __restrict__ v_pages, const int* __restrict__ block_table,
                               int max_pages, int page_size, const int* __restrict__ positions,
                               const int* __restrict__ seg_of_token, T* __restrict__ out, int n_tokens,
                               int nh, int nkv, int hd, int window, float scale) {
    __shared__ float q_s[4][HD_PAD];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const long long wi = (long long)blockIdx.x * 4 + wid;
    if (wi >= (long long)n_tokens * nh) return;   // whole warps leave together; no block barrier below
    const int t = (int)(wi / nh), h = (int)(wi % nh);
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    const int* bt = block_table + (size_t)seg_of_token[t] * max_pages;
    const T* qrow = q + ((size_t)t * nh + h) * hd;
    for (int j = lane; j < HD_PAD; j += 32) q_s[wid][j] = j < hd ? to_f32(qrow[j]) : 0.f;
    __syncwarp();

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    float m = -INFINITY, l = 0.f;
    float acc[HD_PAD];
#pragma unroll
    for (int j = 0; j < HD_PAD; ++j) acc[j] = 0.f;

    for (int u = lo + lane; u <= pos; u += 32) {
        const int page = bt[u / page_size];
        if (page < 0) continue;
        const T* kr = k_pages + (((size_t)page * nkv + kvh) * page_size + (u % page_size)) * hd;
        // V is stored [feature][slot] inside a page
        const T* vr = v_pages + ((size_t)page * nkv + kvh) * hd * page_size + (u % page_size);
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < HD_PAD; ++j)
            if (j < hd) dot += q_s[wid][j] * to_f32(kr[j]);
        const float sc = dot * scale;
        if (sc > m) {
            const float corr = expf(m - sc);   // exp(-inf) = 0 on the first key
            l *= corr;
#pragma unroll
            for (int j = 0; j < HD_PAD; ++j) acc[j] *= corr;
            m = sc;
        }
        const float p = expf(sc - m);
        l += p;
#pragma unroll
        for (int j = 0; j < HD_PAD; ++j)
            if (j < hd) acc[j] += p * to_f32(vr[(size_t)j * page_size]);
    }
    const float M = warp_max(m);
    const float f = (m == -INFINITY) ? 0.f : expf(m - M);
    const float L = warp_sum(l * f);
    T* orow = out + ((size_t)t * nh + h) * hd;
#pragma unroll
    for (int j = 0; j < HD_PAD; ++j) {
        const float a = warp_sum(acc[j] * f);
        if (j < hd && (j & 31) == lane) orow[j] = from_f32<T>(a / L);
    }
}

template <typename T>
static int launch_generic(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                          int max_pages, int page_size, const int* positions, const int* seg_of_token,
                          void* out, int n_tokens, int nh, int nkv, int hd, int window, float scale,
                          cudaStream_t stream) {
    const long long total = (long long)n_tokens * nh;
    const long long blocks = (total + 3) / 4;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
#define GO(PAD)                                                                                          \
    paged_attention_generic_kernel<T, PAD><<<(unsigned)blocks, 128, 0, stream>>>(                        \
        (const T*)q, (const T*)k_pages, (const T*)v_pages, block_table, max_pages, page_size, positions, \
        seg_of_token, (T*)out, n_tokens, nh, nkv, hd, window, scale)
    if (hd <= 32) GO(32);
    else if (hd <= 64) GO(64);
    else if (hd <= 128) GO(128);
    else if (hd <= 256) GO(256);
    else return GESSO_ERR_BAD_SIZE;
#undef GO
    return launch_status();
}

GESSO_API int gesso_paged_attention_generic(const void* q, const void* k_pages, const void* v_pages, int dtype,
                                            const int* block_table, int max_pages, int page_size,
                                            const int* positions, const int* seg_of_token, void* out,
                                            int n_tokens, int nh, int nkv, int hd, int window, float scale,
                                            cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || page_size <= 0) return GESSO_ERR_BAD_SIZE;
    if (dtype == GESSO_F32)
        return launch_generic<float>(q, k_pages, v_pages, block_table, max_pages, page_size, positions,
                                     seg_of_token, out, n_tokens, nh, nkv, hd, window, scale, stream);
    if (dtype == GESSO_BF16)
        return launch_generic<bf16>(q, k_pages, v_pages, block_table, max_pages, page_size, positions,
                                    seg_of_token, out, n_tokens, nh, nkv, hd, window, scale, stream);
    return GESSO_ERR_BAD_DTYPE;
}
