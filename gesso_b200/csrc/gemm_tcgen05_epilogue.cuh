// What an epilogue thread of the tcgen05 matrix products does with 32 consecutive accumulator columns of
// its row: store them as bfloat16 or float32, add them into the float32 residual stream, or apply SwiGLU
// to packed gate/up columns (8 gate columns then their 8 up columns: 32 columns give 16 outputs).
#pragma once
#include <math.h>

#include "common.cuh"

enum { TC_EPI_BF16 = 0, TC_EPI_F32 = 1, TC_EPI_RESID = 2, TC_EPI_SWIGLU = 3 };

// r: the 32 float32 values (as bits); row < M and col < N are the caller's checks; N is the row pitch of C.
template <int EPI>
__device__ __forceinline__ void tc_store_32(const unsigned (&r)[32], void* __restrict__ out,
                            const float* __restrict__ bias, int row, int col, int N) {
    if (EPI == TC_EPI_SWIGLU) {
        // packed columns: 8 gate then their 8 up; 32 columns give 16 outputs
        bf16* o = reinterpret_cast<bf16*>(out) + (size_t)row * (N / 2) + col / 2;
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
            if (col + grp * 16 >= N) break;
            unsigned pk[4];
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                const float g0 = __uint_as_float(r[grp * 16 + i]), g1 = __uint_as_float(r[grp * 16 + i + 1]);
                const float u0 = __uint_as_float(r[grp * 16 + 8 + i]), u1 = __uint_as_float(r[grp * 16 + 9 + i]);
                __nv_bfloat162 v = __floats2bfloat162_rn((g0 / (1.f + expf(-g0))) * u0,
                                                         (g1 / (1.f + expf(-g1))) * u1);
                pk[i / 2] = *reinterpret_cast<unsigned*>(&v);
            }
            *reinterpret_cast<uint4*>(o + grp * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
    } else if (EPI == TC_EPI_BF16) {
        bf16* o = reinterpret_cast<bf16*>(out) + (size_t)row * N + col;
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
            if (col + i >= N) break;
            unsigned pk[4];
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[i + j]), __uint_as_float(r[i + j + 1]));
                pk[j / 2] = *reinterpret_cast<unsigned*>(&v);
            }
            *reinterpret_cast<uint4*>(o + i) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
    } else {
        float* o = reinterpret_cast<float*>(out) + (size_t)row * N + col;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            if (col + i >= N) break;
            float4 v = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                                   __uint_as_float(r[i + 3]));
            if (EPI == TC_EPI_RESID) {
                const float4 old = *reinterpret_cast<const float4*>(o + i);
                v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                if (bias) {
                    v.x += bias[col + i]; v.y += bias[col + i + 1]; v.z += bias[col + i + 2]; v.w += bias[col + i + 3];
                }
            }
            *reinterpret_cast<float4*>(o + i) = v;
        }
    }
}
