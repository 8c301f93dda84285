// Per-head q/k RMSNorm, rotary position encoding and the write of K and V into cache pages.
//
// Input is the fused projection [N, (nh + 2*nkv) * hd] with features head-major
// (f = head*hd + j, src/Inference/Inference.jl:1573-1583): q heads, then k heads, then v heads.
// q and k heads are normed over hd (weight [hd] shared by all heads, same eps as every other
// norm) BEFORE the rotation (src/Inference/Inference.jl:2401-2416); v is copied.  The rotation
// pairs element i with i + hd/2 (half-split layout, src/Operators/cpu.jl:357-371):
//   x_i' = x_i cos - x_{i+hd/2} sin,   x_{i+hd/2}' = x_i sin + x_{i+hd/2} cos.
// cos/sin come from a float32 table [max_positions, hd/2] that the host fills from float64
// angles, so the angle itself never loses precision at large positions.  The cache holds the
// normed, rotated K and the raw V (src/Inference/Inference.jl:2417-2421).  Page layouts:
// K [page][kv head][slot][feature], V [page][kv head][feature][slot].
//
// One warp per (token, head).  Everything is float32 inside; stores round to the run type.
#include "common.cuh"

template <typename T>
__global__ void qk_norm_rope_store_kernel(
    const T* __restrict__ qkv, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int* __restrict__ positions,
    const int* __restrict__ seg_of_token, const int* __restrict__ block_table, int max_pages, int page_size,
    T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages, int n_tokens, int nh, int nkv,
    int hd, int write_kv, int* __restrict__ status) {
    // let the successor in first (it only prefetches what no running kernel writes until its own wait)
    pdl_launch_dependents();
    pdl_wait();
    const int heads = write_kv ? nh + 2 * nkv : nh;   // without a cache write the input holds q heads only
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const long long wi = (long long)blockIdx.x * warps + (threadIdx.x >> 5);
    if (wi >= (long long)n_tokens * heads) return;
    const int t = (int)(wi / heads), head = (int)(wi % heads);
    const int half = hd >> 1;
    const T* src = qkv + (size_t)t * heads * hd + (size_t)head * hd;
    const int pos = positions[t];

    const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * nh + head) * hd;
    } else {
        const int kvh = is_k ? head - nh : head - nh - nkv;
        const int s = seg_of_token[t];
        const int page = block_table[(size_t)s * max_pages + pos / page_size];
        if (page < 0) {   // a position without a page: record it and write nothing
            if (lane == 0) atomicExch(status, 1);
            return;
        }
        if (!is_k) {
            // v is stored transposed inside its page, [head size][page size], so that the attention
            // kernels read the values of consecutive keys of one feature as one contiguous piece
            T* vt = v_pages + ((size_t)page * nkv + kvh) * hd * page_size + (pos % page_size);
            for (int j = lane; j < hd; j += 32) vt[(size_t)j * page_size] = src[j];
            return;
        }
        dst = k_pages + (((size_t)page * nkv + kvh) * page_size + (pos % page_size)) * hd;
    }
    const float* w = is_q ? q_w : k_w;
    float ss = 0.f;
    for (int i = lane; i < half; i += 32) {
        const float a = to_f32(src[i]), b = to_f32(src[i + half]);
        ss += a * a + b * b;
    }
    ss = warp_sum(ss);
    const float denom = w ? sqrtf(ss / (float)hd + eps) : 1.f;
    const bool rotate = cos_t != nullptr;   // no table: the mixer has no position encoding
    const float* cs = rotate ? cos_t + (size_t)pos * half : nullptr;
    const float* sn = rotate ? sin_t + (size_t)pos * half : nullptr;
    for (int i = lane; i < half; i += 32) {
        float a = to_f32(src[i]), b = to_f32(src[i + half]);
        if (w) { a = (a / denom) * w[i]; b = (b / denom) * w[i + half]; }
        const float c = rotate ? cs[i] : 1.f, s = rotate ? sn[i] : 0.f;
        dst[i] = from_f32<T>(a * c - b * s);
        dst[i + half] = from_f32<T>(a * s + b * c);
    }
}

GESSO_API int gesso_qk_norm_rope_store(const void* qkv, int dtype, const float* q_w, const float* k_w, float eps,
                                       const float* cos_t, const float* sin_t, const int* positions,
                                       const int* seg_of_token, const int* block_table, int max_pages,
                                       int page_size, void* q_out, void* k_pages, void* v_pages, int n_tokens,
                                       int nh, int nkv, int hd, int write_kv, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd <= 0 || (hd & 1) || nh <= 0 || nkv <= 0 || page_size <= 0) return GESSO_ERR_BAD_SIZE;
    const int warps = 4;
    const long long total = (long long)n_tokens * (write_kv ? nh + 2 * nkv : nh);
    const long long blocks = (total + warps - 1) / warps;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    if (dtype == GESSO_F32)
        launch_pdl(qk_norm_rope_store_kernel<float>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
            (const float*)qkv, q_w, k_w, eps, cos_t, sin_t, positions, seg_of_token, block_table, max_pages,
            page_size, (float*)q_out, (float*)k_pages, (float*)v_pages, n_tokens, nh, nkv, hd, write_kv, status);
    else if (dtype == GESSO_BF16)
        launch_pdl(qk_norm_rope_store_kernel<bf16>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
            (const bf16*)qkv, q_w, k_w, eps, cos_t, sin_t, positions, seg_of_token, block_table, max_pages,
            page_size, (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages, n_tokens, nh, nkv, hd, write_kv, status);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}
