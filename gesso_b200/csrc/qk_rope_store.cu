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
// Pages are handed from request to request as they are, so the slots behind a request's last
// position hold whatever the page's last owner left, a NaN or an infinity included.  The tensor-core
// attention kernels multiply masked probabilities (exact zeros) with the V slots of the whole 16-key
// block that holds the last position, and 0 x NaN is NaN.  So the writer keeps this invariant: the
// V slots between a request's last written position and the end of that position's 16-slot block
// are zero.  The token that ends a request's portion in a step writes those zeros along with its own
// values (the same 32-byte sectors); no other token of the step touches them.
//
// The position part may rotate only the first `rot_dim` features of a head (the rest are normed and
// passed on as they are) and may pair neighbours (2i, 2i+1) instead of the halves (i, i + rot_dim/2);
// the tables are [max_positions, rot_dim/2] then.  The kernel that works by 64-token tiles takes the
// full half-split layout only; everything else goes through the one below.
//
// One warp per (token, head).  Everything is float32 inside; stores round to the run type.
#include "common.cuh"

template <typename T>
__global__ void qk_norm_rope_store_kernel(
    const T* __restrict__ qkv, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int* __restrict__ positions,
    const int* __restrict__ seg_of_token, const int* __restrict__ block_table, int max_pages, int page_size,
    T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages, int n_tokens, int nh, int nkv,
    int hd, int write_kv, int rot_dim, int interleaved, int* __restrict__ status) {
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
            const int slot = pos % page_size;
            T* vt = v_pages + ((size_t)page * nkv + kvh) * hd * page_size + slot;
            // the last token of its request in this step clears the rest of its 16-slot block
            const bool last = t == n_tokens - 1 || seg_of_token[t + 1] != s;
            const int clear = last ? min(page_size, ((slot >> 4) + 1) << 4) - slot : 1;
            for (int j = lane; j < hd; j += 32) {
                vt[(size_t)j * page_size] = src[j];
                for (int z = 1; z < clear; ++z) vt[(size_t)j * page_size + z] = from_f32<T>(0.f);
            }
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
    const int rot_half = rotate ? rot_dim >> 1 : 0;
    const float* cs = rotate ? cos_t + (size_t)pos * rot_half : nullptr;
    const float* sn = rotate ? sin_t + (size_t)pos * rot_half : nullptr;
    for (int i = lane; i < rot_half; i += 32) {            // the rotated pairs
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + rot_half;
        float a = to_f32(src[ia]), b = to_f32(src[ib]);
        if (w) { a = (a / denom) * w[ia]; b = (b / denom) * w[ib]; }
        const float c = cs[i], s = sn[i];
        dst[ia] = from_f32<T>(a * c - b * s);
        dst[ib] = from_f32<T>(a * s + b * c);
    }
    for (int i = 2 * rot_half + lane; i < hd; i += 32) {   // features the position part leaves alone
        float a = to_f32(src[i]);
        if (w) a = (a / denom) * w[i];
        dst[i] = from_f32<T>(a);
    }
}

// The same for steps with prompt portions in bfloat16: a block takes one 64-token tile of a portion
// (tile_seg / tile_q0, the tiles the prefill attention walks) and one q or k head.  HD / 8 lanes share a
// (token, head): each holds 4 + 4 elements of the two rotation halves (8-byte loads and stores).  A block
// of a k head also moves the matching v head: the tile goes through shared memory and is written along
// the slot axis of its transposed page, 8 consecutive positions (16 bytes) per store, instead of one
// 2-byte store per element.
template <int HD>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_tile_kernel(
    const bf16* __restrict__ qkv, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int* __restrict__ seg_start,
    const int* __restrict__ seg_pos0, const int* __restrict__ tile_seg, const int* __restrict__ tile_q0,
    const int* __restrict__ block_table, int max_pages, int page_size, bf16* __restrict__ q_out,
    bf16* __restrict__ k_pages, bf16* __restrict__ v_pages, int nh, int nkv, int* __restrict__ status) {
    constexpr int LPH = HD / 8, HALF = HD / 2;
    __shared__ __align__(16) bf16 vt[64][HD + 8];
    // launched programmatically: let the successor be set up, then wait for what earlier kernels wrote (every
    // block waits, also one with nothing to do, so that the chain of dependences stays whole)
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.x, hs = blockIdx.y;            // hs < nh: a q head; else k head hs - nh (and its v head)
    const int seg = tile_seg[tile], q0 = tile_q0[tile];
    const int t0 = seg_start[seg], n = seg_start[seg + 1] - t0;
    const int rows = min(64, n - q0);
    if (rows <= 0) return;
    const int pos0 = seg_pos0[seg] + q0;
    const int heads = nh + 2 * nkv;
    const bool is_q = hs < nh;
    const int kvh = hs - nh;
    const int* bt = block_table + (size_t)seg * max_pages;
    const float* w = is_q ? q_w : k_w;
    const bool rotate = cos_t != nullptr;
    const int l = threadIdx.x % LPH;
    for (int r0 = threadIdx.x / LPH; r0 < 64; r0 += 256 / LPH) {      // the same trip count for every lane
        const bool valid = r0 < rows;
        const int r = valid ? r0 : rows - 1;
        const int t = t0 + q0 + r, pos = pos0 + r;
        const bf16* src = qkv + ((size_t)t * heads + hs) * HD;
        const uint2 ua = *reinterpret_cast<const uint2*>(src + 4 * l);
        const uint2 ub = *reinterpret_cast<const uint2*>(src + HALF + 4 * l);
        float a[4], b[4];
        {
            const __nv_bfloat162 a0 = *reinterpret_cast<const __nv_bfloat162*>(&ua.x), a1 = *reinterpret_cast<const __nv_bfloat162*>(&ua.y);
            const __nv_bfloat162 b0 = *reinterpret_cast<const __nv_bfloat162*>(&ub.x), b1 = *reinterpret_cast<const __nv_bfloat162*>(&ub.y);
            a[0] = __low2float(a0); a[1] = __high2float(a0); a[2] = __low2float(a1); a[3] = __high2float(a1);
            b[0] = __low2float(b0); b[1] = __high2float(b0); b[2] = __low2float(b1); b[3] = __high2float(b1);
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) ss += a[i] * a[i] + b[i] * b[i];
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (w) {
            const float denom = sqrtf(ss / (float)HD + eps);
            const float4 wa = *reinterpret_cast<const float4*>(w + 4 * l);
            const float4 wb = *reinterpret_cast<const float4*>(w + HALF + 4 * l);
            a[0] = (a[0] / denom) * wa.x; a[1] = (a[1] / denom) * wa.y; a[2] = (a[2] / denom) * wa.z; a[3] = (a[3] / denom) * wa.w;
            b[0] = (b[0] / denom) * wb.x; b[1] = (b[1] / denom) * wb.y; b[2] = (b[2] / denom) * wb.z; b[3] = (b[3] / denom) * wb.w;
        }
        float c[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
        if (rotate) {
            const float4 cc = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * HALF + 4 * l);
            const float4 sv = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * HALF + 4 * l);
            c[0] = cc.x; c[1] = cc.y; c[2] = cc.z; c[3] = cc.w;
            sn[0] = sv.x; sn[1] = sv.y; sn[2] = sv.z; sn[3] = sv.w;
        }
        if (!valid) continue;
        bf16* dst;
        if (is_q) {
            dst = q_out + ((size_t)t * nh + hs) * HD;
        } else {
            const int page = bt[pos / page_size];
            if (page < 0) {       // a position without a page: record it and write nothing
                if (l == 0) atomicExch(status, 1);
                continue;
            }
            dst = k_pages + (((size_t)page * nkv + kvh) * page_size + (pos % page_size)) * HD;
        }
        uint2 oa, ob;
        {
            __nv_bfloat162 v0 = __floats2bfloat162_rn(a[0] * c[0] - b[0] * sn[0], a[1] * c[1] - b[1] * sn[1]);
            __nv_bfloat162 v1 = __floats2bfloat162_rn(a[2] * c[2] - b[2] * sn[2], a[3] * c[3] - b[3] * sn[3]);
            __nv_bfloat162 v2 = __floats2bfloat162_rn(a[0] * sn[0] + b[0] * c[0], a[1] * sn[1] + b[1] * c[1]);
            __nv_bfloat162 v3 = __floats2bfloat162_rn(a[2] * sn[2] + b[2] * c[2], a[3] * sn[3] + b[3] * c[3]);
            oa.x = *reinterpret_cast<unsigned*>(&v0); oa.y = *reinterpret_cast<unsigned*>(&v1);
            ob.x = *reinterpret_cast<unsigned*>(&v2); ob.y = *reinterpret_cast<unsigned*>(&v3);
        }
        *reinterpret_cast<uint2*>(dst + 4 * l) = oa;
        *reinterpret_cast<uint2*>(dst + HALF + 4 * l) = ob;
    }
    if (is_q) return;
    // ---- the v head of this kv head: tile -> shared memory -> transposed pages ----
    for (int idx = threadIdx.x; idx < 64 * (HD / 8); idx += 256) {
        const int r = idx / (HD / 8), cpiece = idx % (HD / 8);
        if (r < rows)
            *reinterpret_cast<uint4*>(&vt[r][8 * cpiece]) = *reinterpret_cast<const uint4*>(
                qkv + ((size_t)(t0 + q0 + r) * heads + nh + nkv + kvh) * HD + 8 * cpiece);
    }
    __syncthreads();
    const int g0 = pos0 >> 3, ng = ((pos0 + rows - 1) >> 3) - g0 + 1;      // groups of 8 positions
    for (int idx = threadIdx.x; idx < ng * HD; idx += 256) {
        const int j = idx / ng, gi = idx % ng;
        const int p_lo = (g0 + gi) << 3;
        const int page = bt[p_lo / page_size];
        if (page < 0) {
            if (gi == 0 && j == 0) atomicExch(status, 1);
            continue;
        }
        bf16* dst = v_pages + (((size_t)page * nkv + kvh) * HD + j) * page_size + (p_lo % page_size);
        const int lo = max(p_lo, pos0), hi = min(p_lo + 8, pos0 + rows);
        if (hi - lo == 8) {
            unsigned u[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 v2 = __halves2bfloat162(vt[p_lo - pos0 + 2 * i][j], vt[p_lo - pos0 + 2 * i + 1][j]);
                u[i] = *reinterpret_cast<const unsigned*>(&v2);
            }
            *reinterpret_cast<uint4*>(dst) = make_uint4(u[0], u[1], u[2], u[3]);
        } else {
            for (int p = lo; p < hi; ++p) dst[p - p_lo] = vt[p - pos0][j];
        }
    }
    // the tile that ends the portion clears the rest of the last position's 16-slot block
    if (q0 + rows == n) {
        const int last = pos0 + rows - 1, slot = last % page_size;
        const int clear = min(page_size, ((slot >> 4) + 1) << 4) - slot - 1;
        const int page = bt[last / page_size];
        if (clear > 0 && page >= 0) {
            bf16* dst = v_pages + ((size_t)page * nkv + kvh) * HD * page_size + slot + 1;
            for (int idx = threadIdx.x; idx < HD * clear; idx += 256)
                dst[(size_t)(idx / clear) * page_size + idx % clear] = __float2bfloat16_rn(0.f);
        }
    }
}

GESSO_API int gesso_qk_rope_store_tiles_takes(int hd, int page_size, int nh, int nkv) {
    return (hd == 32 || hd == 64 || hd == 128) && page_size > 0 && page_size % 8 == 0 && nh > 0 && nkv > 0 &&
           nh + nkv <= 65535;
}

// bfloat16, prompt portions: qkv [N, (nh + 2 nkv) hd]; the step's tiles as for the prefill attention.
GESSO_API int gesso_qk_norm_rope_store_tiles(const void* qkv, const float* q_w, const float* k_w, float eps,
                                             const float* cos_t, const float* sin_t, const int* seg_start,
                                             const int* seg_pos0, const int* tile_seg, const int* tile_q0,
                                             int n_tiles, const int* block_table, int max_pages, int page_size,
                                             void* q_out, void* k_pages, void* v_pages, int nh, int nkv, int hd,
                                             int* status, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (!gesso_qk_rope_store_tiles_takes(hd, page_size, nh, nkv)) return GESSO_ERR_BAD_SIZE;
    const dim3 grid(n_tiles, nh + nkv);
#define GO(HD)                                                                                                  \
    launch_pdl(qk_norm_rope_store_tile_kernel<HD>, grid, dim3(256), 0, stream,                                  \
        (const bf16*)qkv, q_w, k_w, eps, cos_t, sin_t, seg_start, seg_pos0, tile_seg, tile_q0, block_table,     \
        max_pages, page_size, (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages, nh, nkv, status)
    if (hd == 32) GO(32);
    else if (hd == 64) GO(64);
    else GO(128);
#undef GO
    return launch_status();
}

GESSO_API int gesso_qk_norm_rope_store(const void* qkv, int dtype, const float* q_w, const float* k_w, float eps,
                                       const float* cos_t, const float* sin_t, const int* positions,
                                       const int* seg_of_token, const int* block_table, int max_pages,
                                       int page_size, void* q_out, void* k_pages, void* v_pages, int n_tokens,
                                       int nh, int nkv, int hd, int write_kv, int rot_dim, int interleaved,
                                       int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd <= 0 || (hd & 1) || nh <= 0 || nkv <= 0 || page_size <= 0) return GESSO_ERR_BAD_SIZE;
    if (cos_t != nullptr && (rot_dim < 2 || (rot_dim & 1) || rot_dim > hd)) return GESSO_ERR_BAD_SIZE;
    const int warps = 4;
    const long long total = (long long)n_tokens * (write_kv ? nh + 2 * nkv : nh);
    const long long blocks = (total + warps - 1) / warps;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    if (dtype == GESSO_F32)
        launch_pdl(qk_norm_rope_store_kernel<float>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
            (const float*)qkv, q_w, k_w, eps, cos_t, sin_t, positions, seg_of_token, block_table, max_pages,
            page_size, (float*)q_out, (float*)k_pages, (float*)v_pages, n_tokens, nh, nkv, hd, write_kv, rot_dim,
            interleaved, status);
    else if (dtype == GESSO_BF16)
        launch_pdl(qk_norm_rope_store_kernel<bf16>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
            (const bf16*)qkv, q_w, k_w, eps, cos_t, sin_t, positions, seg_of_token, block_table, max_pages,
            page_size, (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages, n_tokens, nh, nkv, hd, write_kv, rot_dim,
            interleaved, status);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}
