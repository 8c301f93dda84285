// The double-gated short convolution between in_proj and out_proj, on the flat token axis.
//
// bcx holds B, C and X side by side ([N, 3H]: columns [0,H)=B, [H,2H)=C, [2H,3H)=X).  For token
// t and channel c: bx = B*X;  y = sum_{p<L-1} hist[p]*w[c,p] + bx*w[c,L-1];  out = C*y; the
// history then shifts by one and takes bx (src/Inference/lfm2.jl:253-271).  Taps run oldest to
// newest, the newest multiplies the current token (:256).  A FIR has no recurrence, so all
// tokens of a portion run in parallel: the L-1 earlier values of a token come from earlier
// tokens of the same portion (recomputed from bcx) or, before the portion's start, from the
// request's state slot, which holds the last L-1 values of bx in float32.
//
// Two launches keep the slot free of read/write races: `mix` only reads the slot, `state_update`
// (one thread per (portion, channel), which owns that slot column) rewrites it afterwards.
// When every portion is short (decoding), `mix_update_small` does both in one launch with the
// same ownership.
//
// `packed` rows of bcx hold the three parts in groups of 24 columns (B, C, X of 8 channels), the order in
// which the packed input projection (whose decoding form has this convolution in its epilogue) gives them.
#include "common.cuh"

// column of part p (0 = B, 1 = C, 2 = X) of channel c in a row of bcx
__device__ __forceinline__ int bcx_col(int part, int c, int H, int packed) {
    return packed ? 24 * (c >> 3) + 8 * part + (c & 7) : part * H + c;
}

template <typename T>
__device__ __forceinline__ float bx_at(const T* __restrict__ bcx, const float* __restrict__ in_bias,
                                       int tok, int c, int H, int packed) {
    const T* row = bcx + (size_t)tok * 3 * H;
    float b = to_f32(row[bcx_col(0, c, H, packed)]), x = to_f32(row[bcx_col(2, c, H, packed)]);
    if (in_bias) { b += in_bias[c]; x += in_bias[2 * H + c]; }
    return b * x;
}

// state layout for one layer: state[slot * slot_stride + q * H + c], q = 0 (oldest) .. L-2 (newest)
template <typename T>
__global__ void conv_mix_kernel(const T* __restrict__ bcx, const float* __restrict__ in_bias,
                                const float* __restrict__ taps, const float* __restrict__ conv_bias,
                                const float* __restrict__ state, long long slot_stride,
                                const int* __restrict__ seg_of_token, const int* __restrict__ seg_start,
                                const int* __restrict__ seg_pos0, const int* __restrict__ slots,
                                T* __restrict__ out, int n_tokens, int H, int L, int packed) {
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t = blockIdx.x;
    if (c >= H || t >= n_tokens) return;
    const int s = seg_of_token[t];
    const int off = t - seg_start[s];          // index of this token inside its portion
    const int pos = seg_pos0[s] + off;         // absolute position
    const float* st = state + (size_t)slots[s] * slot_stride;
    const float* w = taps + (size_t)c * L;
    float y = 0.f;
    for (int p = 0; p < L - 1; ++p) {
        const int back = (L - 1) - p;          // how many tokens before t
        float v;
        if (back > pos) v = 0.f;               // before the start of the sequence
        else if (back <= off) v = bx_at(bcx, in_bias, t - back, c, H, packed);
        else v = st[(size_t)((L - 1) - (back - off)) * H + c];
        y += v * w[p];
    }
    y += bx_at(bcx, in_bias, t, c, H, packed) * w[L - 1];
    if (conv_bias) y += conv_bias[c];
    const T* row = bcx + (size_t)t * 3 * H;
    float cg = to_f32(row[bcx_col(1, c, H, packed)]);
    if (in_bias) cg += in_bias[H + c];
    out[(size_t)t * H + c] = from_f32<T>(cg * y);
}

// The same for VEC consecutive channels per thread (16-byte loads): the form long portions take.
template <typename T> struct ConvVec;
template <> struct ConvVec<float> { static constexpr int N = 4; };
template <> struct ConvVec<bf16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float (&v)[ConvVec<T>::N]);
template <>
__device__ __forceinline__ void load_vec<float>(const float* p, float (&v)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <>
__device__ __forceinline__ void load_vec<bf16>(const bf16* p, float (&v)[8]) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const unsigned u[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h2 = *reinterpret_cast<const __nv_bfloat162*>(&u[i]);
        v[2 * i] = __low2float(h2);
        v[2 * i + 1] = __high2float(h2);
    }
}
__device__ __forceinline__ void store_vec(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store_vec(bf16* p, const float (&v)[8]) {
    unsigned u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        u[i] = *reinterpret_cast<unsigned*>(&h2);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(u[0], u[1], u[2], u[3]);
}

template <typename T>
__global__ void conv_mix_vec_kernel(const T* __restrict__ bcx, const float* __restrict__ in_bias,
                                    const float* __restrict__ taps, const float* __restrict__ conv_bias,
                                    const float* __restrict__ state, long long slot_stride,
                                    const int* __restrict__ seg_of_token, const int* __restrict__ seg_start,
                                    const int* __restrict__ seg_pos0, const int* __restrict__ slots,
                                    T* __restrict__ out, int n_tokens, int H, int L, int packed) {
    constexpr int V = ConvVec<T>::N;
    const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    const int t = blockIdx.x;
    if (c0 >= H || t >= n_tokens) return;
    const int s = seg_of_token[t];
    const int off = t - seg_start[s];
    const int pos = seg_pos0[s] + off;
    const float* st = state + (size_t)slots[s] * slot_stride;
    float y[V];
#pragma unroll
    for (int v = 0; v < V; ++v) y[v] = 0.f;
    for (int p = 0; p < L; ++p) {
        const int back = (L - 1) - p;          // how many tokens before t (0: the token itself)
        float val[V];
        if (back > pos) {
#pragma unroll
            for (int v = 0; v < V; ++v) val[v] = 0.f;
        } else if (back <= off) {
            const T* row = bcx + (size_t)(t - back) * 3 * H;
            float b[V], x[V];
            load_vec<T>(row + bcx_col(0, c0, H, packed), b);
            load_vec<T>(row + bcx_col(2, c0, H, packed), x);
#pragma unroll
            for (int v = 0; v < V; ++v) {
                if (in_bias) { b[v] += in_bias[c0 + v]; x[v] += in_bias[2 * H + c0 + v]; }
                val[v] = b[v] * x[v];
            }
        } else {
            const float* sp = st + (size_t)((L - 1) - (back - off)) * H + c0;
#pragma unroll
            for (int v = 0; v < V; ++v) val[v] = sp[v];
        }
#pragma unroll
        for (int v = 0; v < V; ++v) y[v] += val[v] * taps[(size_t)(c0 + v) * L + p];
    }
    float cg[V];
    load_vec<T>(bcx + (size_t)t * 3 * H + bcx_col(1, c0, H, packed), cg);
#pragma unroll
    for (int v = 0; v < V; ++v) {
        if (conv_bias) y[v] += conv_bias[c0 + v];
        if (in_bias) cg[v] += in_bias[H + c0 + v];
        y[v] *= cg[v];
    }
    store_vec(out + (size_t)t * H + c0, y);
}

// The same for runs of TB consecutive tokens per thread (long portions, at most 4 taps): the products
// B*X of the last L-1 tokens stay in registers from one token to the next, so a token costs one read of
// its own B, C and X instead of L reads of B and X; the history is fetched afresh only at the start of a
// run and where a new portion begins inside it.
template <typename T, int TB, int L>
__global__ void conv_mix_run_kernel(const T* __restrict__ bcx, const float* __restrict__ in_bias,
                                    const float* __restrict__ taps, const float* __restrict__ conv_bias,
                                    const float* __restrict__ state, long long slot_stride,
                                    const int* __restrict__ seg_of_token, const int* __restrict__ seg_start,
                                    const int* __restrict__ seg_pos0, const int* __restrict__ slots,
                                    T* __restrict__ out, int n_tokens, int H, int packed) {
    // launched programmatically: let the successor be set up, then wait for what earlier kernels wrote (every
    // block waits, also one with nothing to do, so that the chain of dependences stays whole)
    pdl_launch_dependents();
    pdl_wait();
    constexpr int V = ConvVec<T>::N;
    const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    const int tbeg = blockIdx.x * TB, tend = min(n_tokens, tbeg + TB);
    if (c0 >= H || tbeg >= n_tokens) return;
    float w[L][V], hist[L - 1][V];
#pragma unroll
    for (int p = 0; p < L; ++p)
#pragma unroll
        for (int v = 0; v < V; ++v) w[p][v] = taps[(size_t)(c0 + v) * L + p];
    for (int t = tbeg; t < tend; ++t) {
        const int s = seg_of_token[t];
        const int off = t - seg_start[s];
        const int pos = seg_pos0[s] + off;
        const T* row = bcx + (size_t)t * 3 * H;
        if (t == tbeg || off == 0) {
            // hist[q] = bx of the token (L-1-q) places before t, for the taps q = 0 .. L-2 (oldest first)
            const float* st = state + (size_t)slots[s] * slot_stride;
#pragma unroll
            for (int q = 0; q < L - 1; ++q) {
                const int back = (L - 1) - q;
                if (back > pos) {
#pragma unroll
                    for (int v = 0; v < V; ++v) hist[q][v] = 0.f;
                } else if (back <= off) {
                    const T* prow = row - (size_t)back * 3 * H;
                    float b[V], x[V];
                    load_vec<T>(prow + bcx_col(0, c0, H, packed), b);
                    load_vec<T>(prow + bcx_col(2, c0, H, packed), x);
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        if (in_bias) { b[v] += in_bias[c0 + v]; x[v] += in_bias[2 * H + c0 + v]; }
                        hist[q][v] = b[v] * x[v];
                    }
                } else {
                    const float* sp = st + (size_t)((L - 1) - (back - off)) * H + c0;
#pragma unroll
                    for (int v = 0; v < V; ++v) hist[q][v] = sp[v];
                }
            }
        }
        float b[V], x[V], cg[V], y[V];
        load_vec<T>(row + bcx_col(0, c0, H, packed), b);
        load_vec<T>(row + bcx_col(2, c0, H, packed), x);
        load_vec<T>(row + bcx_col(1, c0, H, packed), cg);
#pragma unroll
        for (int v = 0; v < V; ++v) {
            if (in_bias) { b[v] += in_bias[c0 + v]; x[v] += in_bias[2 * H + c0 + v]; cg[v] += in_bias[H + c0 + v]; }
            const float cur = b[v] * x[v];
            // taps oldest to newest, in the order of the other kernels
            float acc = 0.f;
#pragma unroll
            for (int q = 0; q < L - 1; ++q) acc += hist[q][v] * w[q][v];
            acc += cur * w[L - 1][v];
            if (conv_bias) acc += conv_bias[c0 + v];
            y[v] = acc * cg[v];
            // the history moves up by one place and takes this token's product at its newest place
#pragma unroll
            for (int q = 0; q < L - 2; ++q) hist[q][v] = hist[q + 1][v];
            hist[L - 2][v] = cur;
        }
        store_vec(out + (size_t)t * H + c0, y);
    }
}

template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ bcx, const float* __restrict__ in_bias,
                                         float* __restrict__ state, long long slot_stride,
                                         const int* __restrict__ seg_start, const int* __restrict__ seg_pos0,
                                         const int* __restrict__ slots, int n_segs, int H, int L, int packed) {
    // launched programmatically: let the successor be set up, then wait for what earlier kernels wrote (every
    // block waits, also one with nothing to do, so that the chain of dependences stays whole)
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int s = blockIdx.x;
    if (c >= H || s >= n_segs) return;
    const int t0 = seg_start[s], n = seg_start[s + 1] - t0;
    const int pos_end = seg_pos0[s] + n;       // sequence length after this step
    float* st = state + (size_t)slots[s] * slot_stride;
    // new entry q holds bx of the token (L-1-q) places before the end; ascending q never
    // overwrites an old entry that is still to be read (it reads index q+n > q).
    for (int q = 0; q < L - 1; ++q) {
        const int back = (L - 1) - q;          // 1 = last token of the portion
        float v;
        if (back > pos_end) v = 0.f;
        else if (back <= n) v = bx_at(bcx, in_bias, t0 + n - back, c, H, packed);
        else v = st[(size_t)(q + n) * H + c];
        st[(size_t)q * H + c] = v;
    }
}

// Both steps for short portions (n <= 8): one thread per (portion, channel) walks its tokens in
// order with the history in registers, as the reference's per-channel loop does.
template <typename T, int LMAX>
__global__ void conv_mix_update_small_kernel(const T* __restrict__ bcx, const float* __restrict__ in_bias,
                                             const float* __restrict__ taps, const float* __restrict__ conv_bias,
                                             float* __restrict__ state, long long slot_stride,
                                             const int* __restrict__ seg_start, const int* __restrict__ seg_pos0,
                                             const int* __restrict__ slots, T* __restrict__ out, int n_segs,
                                             int H, int L, int packed) {
    // let the successor in first (it only prefetches what no running kernel writes until its own wait)
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int s = blockIdx.x;
    if (c >= H || s >= n_segs) return;
    const int t0 = seg_start[s], n = seg_start[s + 1] - t0;
    float* st = state + (size_t)slots[s] * slot_stride;
    float hist[LMAX], w[LMAX];
    const bool fresh = seg_pos0[s] == 0;
#pragma unroll
    for (int q = 0; q < LMAX; ++q) {
        hist[q] = (q < L - 1 && !fresh) ? st[(size_t)q * H + c] : 0.f;
        w[q] = q < L ? taps[(size_t)c * L + q] : 0.f;
    }
    for (int i = 0; i < n; ++i) {
        const int t = t0 + i;
        const float bx = bx_at(bcx, in_bias, t, c, H, packed);
        float y = 0.f;
#pragma unroll
        for (int p = 0; p < LMAX; ++p)
            if (p < L - 1) y += hist[p] * w[p];
        float wl = 0.f;
#pragma unroll
        for (int p = 0; p < LMAX; ++p)
            if (p == L - 1) wl = w[p];
        y += bx * wl;
        if (conv_bias) y += conv_bias[c];
        const T* row = bcx + (size_t)t * 3 * H;
        float cg = to_f32(row[bcx_col(1, c, H, packed)]);
        if (in_bias) cg += in_bias[H + c];
        out[(size_t)t * H + c] = from_f32<T>(cg * y);
#pragma unroll
        for (int p = 0; p < LMAX - 1; ++p)
            if (p < L - 2) hist[p] = hist[p + 1];
#pragma unroll
        for (int p = 0; p < LMAX; ++p)
            if (p == L - 2) hist[p] = bx;
    }
#pragma unroll
    for (int q = 0; q < LMAX; ++q)
        if (q < L - 1) st[(size_t)q * H + c] = hist[q];
}

GESSO_API int gesso_short_conv(const void* bcx, int dtype, const float* in_bias, const float* taps,
                               const float* conv_bias, float* state, long long slot_stride,
                               const int* seg_of_token, const int* seg_start, const int* seg_pos0,
                               const int* slots, void* out, int n_tokens, int n_segs, int max_seg_len,
                               int H, int L, int packed, cudaStream_t stream) {
    if (n_tokens <= 0 || n_segs <= 0) return 0;
    if (L < 2 || H <= 0 || (packed && H % 8 != 0)) return GESSO_ERR_BAD_SIZE;
    if (dtype != GESSO_F32 && dtype != GESSO_BF16) return GESSO_ERR_BAD_DTYPE;
    const int threads = 128;
    const int cblocks = (H + threads - 1) / threads;
    if (max_seg_len <= 8 && L <= 8) {
        dim3 grid(n_segs, cblocks);
        if (dtype == GESSO_F32)
            launch_pdl(conv_mix_update_small_kernel<float, 8>, grid, dim3(threads), 0, stream,
                (const float*)bcx, in_bias, taps, conv_bias, state, slot_stride, seg_start, seg_pos0, slots,
                (float*)out, n_segs, H, L, packed);
        else
            launch_pdl(conv_mix_update_small_kernel<bf16, 8>, grid, dim3(threads), 0, stream,
                (const bf16*)bcx, in_bias, taps, conv_bias, state, slot_stride, seg_start, seg_pos0, slots,
                (bf16*)out, n_segs, H, L, packed);
        return launch_status();
    }
    dim3 grid(n_tokens, cblocks), sgrid(n_segs, cblocks);
    const int vec = dtype == GESSO_F32 ? 4 : 8;
    if (H % vec == 0) {
        // 16 bytes of channels per thread
        const int vthreads = 128;
        dim3 vgrid(n_tokens, (H / vec + vthreads - 1) / vthreads);
        if (L <= 4 && n_tokens >= 256) {
            // long portions: runs of 8 tokens per thread with the history in registers
            constexpr int TB = 8;
            dim3 rgrid((n_tokens + TB - 1) / TB, (H / vec + vthreads - 1) / vthreads);
#define RUN(T, LL)                                                                                              \
    launch_pdl(conv_mix_run_kernel<T, TB, LL>, rgrid, dim3(vthreads), 0, stream,                                \
        (const T*)bcx, in_bias, taps, conv_bias, (const float*)state, slot_stride, seg_of_token, seg_start,     \
        seg_pos0, slots, (T*)out, n_tokens, H, packed)
            if (dtype == GESSO_F32) {
                if (L == 2) RUN(float, 2); else if (L == 3) RUN(float, 3); else RUN(float, 4);
                launch_pdl(conv_state_update_kernel<float>, sgrid, dim3(threads), 0, stream,
                    (const float*)bcx, in_bias, state, slot_stride, seg_start, seg_pos0, slots, n_segs, H, L, packed);
            } else {
                if (L == 2) RUN(bf16, 2); else if (L == 3) RUN(bf16, 3); else RUN(bf16, 4);
                launch_pdl(conv_state_update_kernel<bf16>, sgrid, dim3(threads), 0, stream,
                    (const bf16*)bcx, in_bias, state, slot_stride, seg_start, seg_pos0, slots, n_segs, H, L, packed);
            }
#undef RUN
            return launch_status();
        }
        if (dtype == GESSO_F32) {
            conv_mix_vec_kernel<float><<<vgrid, vthreads, 0, stream>>>(
                (const float*)bcx, in_bias, taps, conv_bias, state, slot_stride, seg_of_token, seg_start, seg_pos0, slots,
                (float*)out, n_tokens, H, L, packed);
            conv_state_update_kernel<float><<<sgrid, threads, 0, stream>>>((const float*)bcx, in_bias, state, slot_stride,
                                                                           seg_start, seg_pos0, slots, n_segs, H, L, packed);
        } else {
            conv_mix_vec_kernel<bf16><<<vgrid, vthreads, 0, stream>>>(
                (const bf16*)bcx, in_bias, taps, conv_bias, state, slot_stride, seg_of_token, seg_start, seg_pos0, slots,
                (bf16*)out, n_tokens, H, L, packed);
            conv_state_update_kernel<bf16><<<sgrid, threads, 0, stream>>>((const bf16*)bcx, in_bias, state, slot_stride,
                                                                          seg_start, seg_pos0, slots, n_segs, H, L, packed);
        }
        return launch_status();
    }
    if (dtype == GESSO_F32) {
        conv_mix_kernel<float><<<grid, threads, 0, stream>>>((const float*)bcx, in_bias, taps, conv_bias, state,
                                                             slot_stride, seg_of_token, seg_start, seg_pos0, slots,
                                                             (float*)out, n_tokens, H, L, packed);
        conv_state_update_kernel<float><<<sgrid, threads, 0, stream>>>((const float*)bcx, in_bias, state, slot_stride,
                                                                       seg_start, seg_pos0, slots, n_segs, H, L, packed);
    } else {
        conv_mix_kernel<bf16><<<grid, threads, 0, stream>>>((const bf16*)bcx, in_bias, taps, conv_bias, state,
                                                            slot_stride, seg_of_token, seg_start, seg_pos0, slots,
                                                            (bf16*)out, n_tokens, H, L, packed);
        conv_state_update_kernel<bf16><<<sgrid, threads, 0, stream>>>((const bf16*)bcx, in_bias, state, slot_stride,
                                                                      seg_start, seg_pos0, slots, n_segs, H, L, packed);
    }
    return launch_status();
}
