// Entry points of the skinny matrix product (gemm_skinny.cuh has the kernel).  The kernel's
// instantiations are compiled in gemm_skinny_t{1,2}{,_norm}.cu, one file per (token tiles, fused
// norm) pair; this file only checks the arguments and picks one.
#include "gemm_skinny.cuh"

#define SKINNY_DECLARE(NT, NORM)                                                                        \
    extern template int skinny_launch<NT, NORM>(const void*, const float*, const float*, float, const void*, void*, \
                                                const float*, int, int, int, int, void*, long long,   \
                                                const ConvEpi&, cudaStream_t)
SKINNY_DECLARE(1, false);
SKINNY_DECLARE(1, true);
SKINNY_DECLARE(2, false);
SKINNY_DECLARE(2, true);

static int launch_skinny(const void* x, const float* h_in, const float* norm_w, float eps, const void* W, void* out,
                         const float* bias, int M, int N, int K, int epi, void* ws, long long ws_bytes,
                         const ConvEpi& cv, cudaStream_t stream) {
#define GO(NT, NM) return skinny_launch<NT, NM>(x, h_in, norm_w, eps, W, out, bias, M, N, K, epi, ws, ws_bytes, cv, stream)
    if (M <= 8) {
        if (h_in) GO(1, true);
        GO(1, false);
    }
    if (h_in) GO(2, true);
    GO(2, false);
#undef GO
}

GESSO_API int gesso_skinny_gemm_takes(int M, int N, int K) {
    return M >= 1 && M <= 16 && N >= 16 && N % 16 == 0 && K >= 32 && K % 32 == 0;
}

// x: bf16 [M,K] (or null with h_in/norm_w: the norm is fused); W: bf16 [N,K]; out by `epi`.
// ws: optional workspace for products split along K (zeroed once by the caller, at least 16 KB of
// tickets plus the partial tiles; products it is too small for are not split); one per stream.
GESSO_API int gesso_skinny_gemm(const void* x, const float* h_in, const float* norm_w, float eps, const void* W,
                                void* out, const float* bias, int M, int N, int K, int epi, void* ws,
                                long long ws_bytes, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (!gesso_skinny_gemm_takes(M, N, K)) return GESSO_ERR_BAD_SIZE;
    if ((x == nullptr) == (h_in == nullptr)) return GESSO_ERR_UNSUPPORTED;
    if (h_in && M > 16) return GESSO_ERR_BAD_SIZE;      // the fused norm is for a handful of rows
    if (epi == EPI_CONV) return GESSO_ERR_UNSUPPORTED;   // has an entry point of its own
    if (ws_bytes < (long long)SK_TICKETS * 4) ws = nullptr;
    const ConvEpi none = {};
    return launch_skinny(x, h_in, norm_w, eps, W, out, bias, M, N, K, epi, ws, ws_bytes, none, stream);
}

GESSO_API int gesso_skinny_conv_takes(int M, int H, int K, int L) {
    return M >= 1 && M <= 16 && H >= 8 && H % 8 == 0 && K >= 32 && K % 32 == 0 && L >= 2 && L <= 8;
}

// The input projection of the short convolution with the convolution in its epilogue, for a step of
// single tokens (token i belongs to request i).  W: bf16 [3H, K] packed in groups of 24 rows (B, C, X
// of 8 channels); x or h_in/norm_w as above; y: bf16 [M, H]; state: this layer's [slot][L-1][H] float32.
GESSO_API int gesso_skinny_gemm_conv(const void* x, const float* h_in, const float* norm_w, float eps, const void* W,
                                     void* y, int M, int H, int K, const float* taps, const float* conv_bias,
                                     const float* in_bias, float* state, long long slot_stride, const int* slots,
                                     const int* seg_pos0, int L, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (!gesso_skinny_conv_takes(M, H, K, L)) return GESSO_ERR_BAD_SIZE;
    if ((x == nullptr) == (h_in == nullptr)) return GESSO_ERR_UNSUPPORTED;
    const ConvEpi cv = {taps, conv_bias, in_bias, state, slot_stride, slots, seg_pos0, L, H};
    return launch_skinny(x, h_in, norm_w, eps, W, y, nullptr, M, 3 * H, K, EPI_CONV, nullptr, 0, cv, stream);
}
