// Embedding gather and the fused residual-add + RMSNorm.
//
// The residual stream `h` is float32 in both run types; the sum `h + delta (+ bias)` and the
// norm statistics are computed in float32.  RMSNorm divides first and scales second,
// y = (x / sqrt(mean(x^2) + eps)) * w, as the reference's row kernel does
// (src/Operators/cpu.jl:293-311).  The reference fuses the residual add with the norm that
// follows it on its decode path (src/Inference/Inference.jl:3239-3247); here that fusion is
// the only form.
#include "common.cuh"

// ---- embedding ------------------------------------------------------------------------------
template <typename T>
__global__ void embed_gather_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                    float* __restrict__ h, int H, int V, float scale) {
    // let the successor in first (it only prefetches what no running kernel writes until its own wait)
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = tokens[t];
    if (id < 0 || id >= V) id = 0;   // ids are validated on the host; never read outside the table
    const T* row = table + (size_t)id * H;
    float* out = h + (size_t)t * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) out[c] = to_f32(row[c]) * scale;
}

GESSO_API int gesso_embed_gather(const int* tokens, const void* table, int table_dtype, float* h,
                                 int n_tokens, int H, int V, float scale, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == GESSO_F32)
        launch_pdl(embed_gather_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const float*)table, h, H, V, scale);
    else if (table_dtype == GESSO_BF16)
        launch_pdl(embed_gather_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const bf16*)table, h, H, V, scale);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}

// ---- h += delta (+ bias); out = rmsnorm(h) * w ------------------------------------------------
// One block per output row.  `rows` (optional) selects which rows of h are normed: then h is
// not written back (the selected rows are the last use of the stream).  The row is staged in
// dynamic shared memory (H floats) so it is read from global memory once.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                   const float* __restrict__ delta_bias, const float* __restrict__ w,
                                   float eps, TO* __restrict__ out, const int* __restrict__ rows, int H) {
    extern __shared__ float srow[];
    __shared__ float red[33];
    // launched programmatically: let the successor be set up, then wait for what earlier kernels wrote (every
    // block waits, also one with nothing to do, so that the chain of dependences stays whole)
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* hrow = h + (size_t)src * H;
    const TD* drow = delta ? delta + (size_t)src * H : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float x = hrow[c];
        if (drow) {
            float d = to_f32(drow[c]);
            if (delta_bias) d += delta_bias[c];
            x += d;
            if (!rows) hrow[c] = x;
        }
        srow[c] = x;
        ss += x * x;
    }
    ss = block_sum(ss, red);
    const float denom = sqrtf(ss / (float)H + eps);
    TO* orow = out + (size_t)r * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) orow[c] = from_f32<TO>((srow[c] / denom) * (w ? w[c] : 1.f));
}

// The same, four elements at a time, the row kept in registers (H a multiple of 4, at most 8192):
// the form steps with many tokens take, where the kernel is bound by its memory traffic.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x), b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&a);
    u.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

#define NORM_VEC_THREADS 512
#define NORM_VEC_MAX 4

template <typename TD, typename TO>
__global__ void __launch_bounds__(NORM_VEC_THREADS)
add_rmsnorm_vec_kernel(float* __restrict__ h, const TD* __restrict__ delta, const float* __restrict__ delta_bias,
                       const float* __restrict__ w, float eps, TO* __restrict__ out, const int* __restrict__ rows,
                       int H) {
    __shared__ float red[33];
    // launched programmatically: let the successor be set up, then wait for what earlier kernels wrote (every
    // block waits, also one with nothing to do, so that the chain of dependences stays whole)
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* hrow = h + (size_t)src * H;
    const TD* drow = delta ? delta + (size_t)src * H : nullptr;
    const int nv = H >> 2;
    float4 x[NORM_VEC_MAX];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < NORM_VEC_MAX; ++v) {
        const int i = (threadIdx.x + v * NORM_VEC_THREADS) * 4;
        if (i < nv * 4) {
            float4 a = load4(hrow + i);
            if (drow) {
                float4 d = load4(drow + i);
                if (delta_bias) {
                    const float4 b = load4(delta_bias + i);
                    d.x += b.x; d.y += b.y; d.z += b.z; d.w += b.w;
                }
                a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
                if (!rows) store4(hrow + i, a);
            }
            x[v] = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
    }
    ss = block_sum(ss, red);
    const float denom = sqrtf(ss / (float)H + eps);
    TO* orow = out + (size_t)r * H;
#pragma unroll
    for (int v = 0; v < NORM_VEC_MAX; ++v) {
        const int i = (threadIdx.x + v * NORM_VEC_THREADS) * 4;
        if (i < nv * 4) {
            const float4 ww = w ? load4(w + i) : make_float4(1.f, 1.f, 1.f, 1.f);
            store4(orow + i, make_float4((x[v].x / denom) * ww.x, (x[v].y / denom) * ww.y, (x[v].z / denom) * ww.z,
                                         (x[v].w / denom) * ww.w));
        }
    }
}

// The same for steps of many rows: a warp per row, the whole row in registers (VPL float4 per lane), no
// block-wide barrier between the sum of squares and the scaling; four rows per block.
#define NORM_WARP_ROWS 4
template <typename TD, typename TO, int VPL>
__global__ void __launch_bounds__(NORM_WARP_ROWS * 32)
add_rmsnorm_warp_kernel(float* __restrict__ h, const TD* __restrict__ delta, const float* __restrict__ delta_bias,
                        const float* __restrict__ w, float eps, TO* __restrict__ out, const int* __restrict__ rows,
                        int n_rows) {
    constexpr int H = VPL * 128;
    // launched programmatically: let the successor be set up, then wait for what earlier kernels wrote (every
    // block waits, also one with nothing to do, so that the chain of dependences stays whole)
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * NORM_WARP_ROWS + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const int src = rows ? rows[r] : r;
    float* hrow = h + (size_t)src * H;
    const TD* drow = delta ? delta + (size_t)src * H : nullptr;
    float4 x[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) x[v] = load4(hrow + (v * 32 + lane) * 4);
    if (drow) {
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            const int i = (v * 32 + lane) * 4;
            float4 d = load4(drow + i);
            if (delta_bias) {
                const float4 b = load4(delta_bias + i);
                d.x += b.x; d.y += b.y; d.z += b.z; d.w += b.w;
            }
            x[v].x += d.x; x[v].y += d.y; x[v].z += d.z; x[v].w += d.w;
            if (!rows) store4(hrow + i, x[v]);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v) ss += x[v].x * x[v].x + x[v].y * x[v].y + x[v].z * x[v].z + x[v].w * x[v].w;
    ss = warp_sum(ss);
    const float denom = sqrtf(ss / (float)H + eps);
    TO* orow = out + (size_t)r * H;
    if constexpr (sizeof(TO) == 2) {
        // bfloat16 output: one reciprocal and a multiplication per element (the last bit of the float32
        // quotient is far below the output's rounding); the float32 output keeps the division
        const float inv = 1.f / denom;
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            const int i = (v * 32 + lane) * 4;
            const float4 ww = w ? load4(w + i) : make_float4(1.f, 1.f, 1.f, 1.f);
            store4(orow + i, make_float4((x[v].x * inv) * ww.x, (x[v].y * inv) * ww.y, (x[v].z * inv) * ww.z,
                                         (x[v].w * inv) * ww.w));
        }
    } else {
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            const int i = (v * 32 + lane) * 4;
            const float4 ww = w ? load4(w + i) : make_float4(1.f, 1.f, 1.f, 1.f);
            store4(orow + i, make_float4((x[v].x / denom) * ww.x, (x[v].y / denom) * ww.y, (x[v].z / denom) * ww.z,
                                         (x[v].w / denom) * ww.w));
        }
    }
}

template <typename TD, typename TO>
static bool launch_norm_warp(float* h, const void* delta, const float* delta_bias, const float* w, float eps, void* out,
                             const int* rows, int n_rows, int H, cudaStream_t stream) {
    const int grid = (n_rows + NORM_WARP_ROWS - 1) / NORM_WARP_ROWS;
#define WLAUNCH(VPL)                                                                                         \
    launch_pdl(add_rmsnorm_warp_kernel<TD, TO, VPL>, dim3(grid), dim3(NORM_WARP_ROWS * 32), 0, stream, h, (const TD*)delta, delta_bias, w, \
                                                                                   eps, (TO*)out, rows, n_rows)
    switch (H) {
        case 512: WLAUNCH(4); return true;
        case 1024: WLAUNCH(8); return true;
        case 1536: WLAUNCH(12); return true;
        case 2048: WLAUNCH(16); return true;
        case 2560: WLAUNCH(20); return true;
        default: return false;
    }
#undef WLAUNCH
}

GESSO_API int gesso_add_rmsnorm(float* h, const void* delta, int delta_dtype, const float* delta_bias,
                                const float* w, float eps, void* out, int out_dtype, const int* rows,
                                int n_rows, int H, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || (size_t)H * sizeof(float) > 200 * 1024) return GESSO_ERR_BAD_SIZE;
    if (n_rows >= 256) {      // many rows: a warp per row, for the widths it is compiled for
        bool done = false;
        if (delta_dtype == GESSO_F32 && out_dtype == GESSO_F32)
            done = launch_norm_warp<float, float>(h, delta, delta_bias, w, eps, out, rows, n_rows, H, stream);
        else if (delta_dtype == GESSO_BF16 && out_dtype == GESSO_BF16)
            done = launch_norm_warp<bf16, bf16>(h, delta, delta_bias, w, eps, out, rows, n_rows, H, stream);
        else if (delta_dtype == GESSO_F32 && out_dtype == GESSO_BF16)
            done = launch_norm_warp<float, bf16>(h, delta, delta_bias, w, eps, out, rows, n_rows, H, stream);
        else if (delta_dtype == GESSO_BF16 && out_dtype == GESSO_F32)
            done = launch_norm_warp<bf16, float>(h, delta, delta_bias, w, eps, out, rows, n_rows, H, stream);
        if (done) return launch_status();
    }
    if (H % 4 == 0 && H <= 4 * NORM_VEC_THREADS * NORM_VEC_MAX) {
#define VLAUNCH(TD, TO)                                                                             \
    launch_pdl(add_rmsnorm_vec_kernel<TD, TO>, dim3(n_rows), dim3(NORM_VEC_THREADS), 0, stream, h, (const TD*)delta, delta_bias, w, eps, \
                                                                             (TO*)out, rows, H)
        if (delta_dtype == GESSO_F32 && out_dtype == GESSO_F32) VLAUNCH(float, float);
        else if (delta_dtype == GESSO_BF16 && out_dtype == GESSO_BF16) VLAUNCH(bf16, bf16);
        else if (delta_dtype == GESSO_F32 && out_dtype == GESSO_BF16) VLAUNCH(float, bf16);
        else if (delta_dtype == GESSO_BF16 && out_dtype == GESSO_F32) VLAUNCH(bf16, float);
        else return GESSO_ERR_BAD_DTYPE;
#undef VLAUNCH
        return launch_status();
    }
    int threads = 128;
    while (threads < 1024 && threads * 4 < H) threads <<= 1;
    const size_t smem = (size_t)H * sizeof(float);
#define LAUNCH(TD, TO)                                                                              \
    do {                                                                                            \
        if (smem > 48 * 1024)                                                                       \
            cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                        \
        launch_pdl(add_rmsnorm_kernel<TD, TO>, dim3(n_rows), dim3(threads), smem, stream,           \
            h, (const TD*)delta, delta_bias, w, eps, (TO*)out, rows, H);                            \
    } while (0)
    if (delta_dtype == GESSO_F32 && out_dtype == GESSO_F32) LAUNCH(float, float);
    else if (delta_dtype == GESSO_BF16 && out_dtype == GESSO_BF16) LAUNCH(bf16, bf16);
    else if (delta_dtype == GESSO_F32 && out_dtype == GESSO_BF16) LAUNCH(float, bf16);
    else if (delta_dtype == GESSO_BF16 && out_dtype == GESSO_F32) LAUNCH(bf16, float);
    else return GESSO_ERR_BAD_DTYPE;
#undef LAUNCH
    return launch_status();
}

// ---- plain RMSNorm over the last axis of a [rows, D] tensor (per-head norms, tests) ----------------
template <typename T>
__global__ void rmsnorm_rows_kernel(const T* __restrict__ x, const float* __restrict__ w, float eps,
                                    T* __restrict__ out, int n_rows, int D) {
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * warps + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const T* xr = x + (size_t)r * D;
    float ss = 0.f;
    for (int c = lane; c < D; c += 32) { float v = to_f32(xr[c]); ss += v * v; }
    ss = warp_sum(ss);
    const float denom = sqrtf(ss / (float)D + eps);
    T* o = out + (size_t)r * D;
    for (int c = lane; c < D; c += 32) o[c] = from_f32<T>((to_f32(xr[c]) / denom) * w[c]);
}

GESSO_API int gesso_rmsnorm_rows(const void* x, const float* w, float eps, void* out, int dtype,
                                 int n_rows, int D, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const int warps = 4;
    const int blocks = (n_rows + warps - 1) / warps;
    if (dtype == GESSO_F32)
        rmsnorm_rows_kernel<float><<<blocks, warps * 32, 0, stream>>>((const float*)x, w, eps, (float*)out, n_rows, D);
    else if (dtype == GESSO_BF16)
        rmsnorm_rows_kernel<bf16><<<blocks, warps * 32, 0, stream>>>((const bf16*)x, w, eps, (bf16*)out, n_rows, D);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}
