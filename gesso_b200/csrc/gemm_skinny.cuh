// Skinny matrix products for steps of few tokens (decoding): Y[M,N] = X[M,K] * W[N,K]^T, M <= 16.
//
// With so few rows the product is bound by the one pass over W, so the kernel is built around that
// stream: a block owns 16 rows of W and its 8 warps walk K in interleaved 32-element chunks (the
// block reads 512 contiguous bytes of each row per round).  Every thread streams 16 bytes of two W
// rows per chunk through a private ring in shared memory (asynchronous copies, ten chunks in
// flight) into the A fragment of mma.m16n8k16 (the sum over k is order-free, so the k index of a
// fragment slot is whatever the load delivers; the X fragment uses the same assignment), and
// accumulates in float32.  The weights sit on
// the M side of the MMA and the tokens on its N side (8 per tile), so no tensor work is wasted on
// padding.  The 8 partial sums of a block are added in shared memory in a fixed order: a row's
// result does not depend on the grid or on how many other tokens share the step.
//
// Fused into the kernel, to save launches and passes over activations:
//   prologue NORM:   X = rmsnorm(h) * w computed from the float32 residual stream (each block
//                    recomputes the row statistics: M*K floats from L2);
//   epilogue BF16:   Y stored as bfloat16;       F32: Y stored as float32 (logits);
//            RESID:  h[M,N] += Y (+ bias), the residual add of the sublayer, in float32;
//            SWIGLU: rows g and g+8 of a block are gate_i and up_i (the caller packs the fused
//                    gate/up matrix in groups of 8), out[M, N/2] = silu(gate) * up;
//            CONV:   24 rows of a block are B, C and X of 8 channels (the caller packs the input
//                    projection of the short convolution so); for a step of single tokens the
//                    epilogue forms bx = B X, runs the FIR over the request's state and bx, gates
//                    with C, stores y[M, H] and shifts bx into the state: no kernel of its own.
// A long inner size with a narrow output (the feed-forward's down projection) is split along K over
// S blocks per tile, so that a block's share of K is short enough for its token-side fragments to
// stay in registers and there are enough blocks to fill the device.  The S blocks of a tile are a
// thread-block cluster (S = 2, 4, 8): each leaves its partial tile in its own shared memory, the
// cluster meets at its barrier, and every block adds the S parts of its share of the tile's elements
// through distributed shared memory, in the order 0..S-1, and runs the epilogue on them: one barrier
// per tile, no trip through global memory.  Where no cluster can be had (S = 16) the partial tiles go
// to a workspace and the block that arrives last (a ticket per tile) adds them in the same order.
// Formulas: src/Operators/cpu.jl:293-311 (norm), 482-488 (SwiGLU), 629-630 (x W^T).
#pragma once
#include <math.h>

#include "common.cuh"

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_RESID = 2, EPI_SWIGLU = 3, EPI_CONV = 4 };

// What the short-convolution epilogue needs beside the product (see short_conv.cu for the layer).
struct ConvEpi {
    const float* taps;        // [H][L], oldest to newest
    const float* conv_bias;   // [H] or null
    const float* in_bias;     // [3H] (B, C, X) or null
    float* state;             // this layer's state: [slot][L-1][H] float32
    long long slot_stride;
    const int* slots;         // per token (a step of single tokens: token i is request i)
    const int* seg_pos0;      // per token: its position (0: the request starts, the history is zero)
    int L, H;
};

__device__ __forceinline__ void mma16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;   // weights are read once: do not keep them in L1
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// a load that stays where it is written (the compiler may not move it down to its use)
__device__ __forceinline__ float ld_f32_now(const float* p) {
    float v;
    asm volatile("ld.global.f32 %0, [%1];\n" : "=f"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned pack2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<unsigned*>(&v);
}

#define SK_WARPS 8

// the address of this block's shared-memory object `addr` in block `rank` of the cluster, and a read from there
__device__ __forceinline__ unsigned sk_cluster_map(unsigned addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float sk_ld_cluster(unsigned addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
// all threads of all blocks of the cluster; what a block wrote to its shared memory before is visible after
__device__ __forceinline__ void sk_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
#ifndef SK_RING_UNITS
#define SK_RING_UNITS 160                    // ring size in units of 512 bytes per block (160: 80 KB)
#endif
#ifndef SK_MIN_BLOCKS
#define SK_MIN_BLOCKS 1                      // blocks per SM the register allocation leaves room for
#endif
#ifndef SK_BLOCKS_PER_SM
#define SK_BLOCKS_PER_SM 2                               // persistent blocks per SM (two fit by shared memory and registers)
#endif
#define SK_STAGES_FOR(ROWS) (SK_RING_UNITS / (ROWS))   // chunks in flight per thread: 10 of 32 bytes or 20 of 16 bytes

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// W is streamed through a ring of SK_STAGES private slots per thread (asynchronous copies global ->
// shared, read back by the same thread), so the bytes in flight do not cost registers and no
// block-wide barrier sits in the inner loop.  Blocks are persistent: a block walks the tiles
// blockIdx.x, blockIdx.x + gridDim.x, ... and its stream runs on across tile borders, so the fixed
// costs (norm statistics, pipeline fill) are paid once per block.  ROWS = 16 or 8 rows of W per tile
// (8 when there are too few 16-row tiles to fill the device; rows 8..15 of the MMA are then zero).
// XC: chunks per warp and tile whose token-side fragments are kept in registers across tiles (0: reload).
// Two blocks have to fit an SM (the grid is sized for that): with two token tiles the register allocation
// would otherwise go a few registers past half of the file and leave every second block waiting.
template <int NT, int EPI, bool NORM, int ROWS, int XC, bool CL = false>
__global__ void __launch_bounds__(SK_WARPS * 32, NT >= 2 ? SK_BLOCKS_PER_SM : SK_MIN_BLOCKS)
skinny_gemm_kernel(const bf16* __restrict__ x, const float* __restrict__ h_in, const float* __restrict__ norm_w,
                   float eps, const bf16* __restrict__ W, void* __restrict__ out, const float* __restrict__ bias,
                   int M, int N, int K, int ldk, int S, float* __restrict__ ws, int* __restrict__ tickets,
                   const ConvEpi cv) {
    // K: this block's share of the inner size; ldk: the row pitch of W and x (K * S)
    constexpr int RSLOTS = ROWS / 8;                      // 16-byte pieces per thread and chunk
    constexpr int STAGES = SK_STAGES_FOR(ROWS);           // ring depth: 80 KB of W in flight per block
    extern __shared__ uint4 ring[];                       // [stage][RSLOTS][256 threads]
    __shared__ float part[2][SK_WARPS][ROWS][NT * 8 + 1];
    __shared__ float rinv[NT * 8];
    __shared__ float ssw[SK_WARPS][NT * 8];
    __shared__ int s_last;
    __shared__ float cl_part[CL ? 2 : 1][CL ? ROWS * NT * 8 : 1];    // this block's partial tile, for its cluster
    const int ks = S > 1 ? (int)(blockIdx.x % (unsigned)S) : 0;      // which share of K
    const int bid = S > 1 ? (int)(blockIdx.x / (unsigned)S) : (int)blockIdx.x;
    const int gdim = S > 1 ? (int)(gridDim.x / (unsigned)S) : (int)gridDim.x;
    // NORM with norm_w == nullptr: the norm's weight was folded into W's columns by the caller.  Then
    // X = bf16(h) goes into the MMA as it is, sum(h^2) is gathered from the very fragments the warps
    // load anyway, and 1/sqrt(mean(h^2) + eps) scales the result in the epilogue: no extra pass over h.
    const bool folded = NORM && norm_w == nullptr;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int n_chunks = K / 32;
    const int CH = (n_chunks + SK_WARPS - 1) / SK_WARPS;  // loop steps per tile (chunk w + 8 i, if it exists)
    const int n_tiles = N / ROWS;
    const int my_tiles = bid < n_tiles ? (n_tiles - bid + gdim - 1) / gdim : 0;
    const int total = my_tiles * CH;
    // Blocks start at different places along K (step i of a tile covers chunk w + 8 ((i + rot) mod CH)):
    // otherwise every block reads the same offset of its rows at the same time, and with a row pitch
    // that is a large power of two those addresses crowd onto few memory channels.
    const int rot = (int)(((unsigned)bid * 7u) % (unsigned)CH);
    auto chunk_of = [&](int i) -> int {
        if (i >= CH) return n_chunks;                     // padding step of the register queue
        int r = i + rot;
        if (r >= CH) r -= CH;
        return w + r * SK_WARPS;
    };

    uint4* slot = ring + threadIdx.x;
    constexpr int stage_stride = RSLOTS * SK_WARPS * 32;
    const bf16* wbase = W + (size_t)g * ldk + (size_t)ks * K + 8 * t;   // + tile row offset + chunk offset

    // producer cursor: item (tile, step) -> asynchronous copies into the ring
    int p_tile = bid, p_i = 0, p_stage = 0, p_item = 0;
    auto issue = [&]() {
        if (p_item < total) {
            const int c = chunk_of(p_i);
            if (c < n_chunks) {
                const bf16* src = wbase + (size_t)p_tile * ROWS * ldk + (size_t)c * 32;
#pragma unroll
                for (int rs = 0; rs < RSLOTS; ++rs)
                    cp_async16(slot + p_stage * stage_stride + rs * SK_WARPS * 32, src + (size_t)(8 * rs) * ldk);
            }
            ++p_item;
            if (++p_i == CH) { p_i = 0; p_tile += gdim; }
            if (++p_stage == STAGES) p_stage = 0;
        }
        cp_async_commit();                                // an empty group keeps the count in step
    };
#pragma unroll
    for (int sidx = 0; sidx < STAGES; ++sidx) issue();   // start the stream before anything else
    // The weights do not depend on earlier kernels; everything below does.  Let the next kernel in
    // (it starts its own weight stream) and wait for the producers of the activations.
    pdl_launch_dependents();
    pdl_wait();

    if (NORM && !folded) {
        // 1 / sqrt(mean(h^2) + eps) of every token row; warp w takes rows w, w+8, ...
        for (int m = w; m < M; m += SK_WARPS) {
            const float4* row = reinterpret_cast<const float4*>(h_in + (size_t)m * K);
            float ss = 0.f;
#pragma unroll 8
            for (int i = lane; i < K / 4; i += 32) {      // independent loads: keep several in flight
                const float4 v = row[i];
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
            ss = warp_sum(ss);
            if (lane == 0) rinv[m] = 1.f / sqrtf(ss / (float)K + eps);
        }
        __syncthreads();
    }

    // the token side of the product for chunk c and token tile j
    float ssq[NT];                                        // folded norm: this thread's share of sum(h^2)
#pragma unroll
    for (int j = 0; j < NT; ++j) ssq[j] = 0.f;
    auto load_x = [&](int c, int j, bool count) -> uint4 {
        const int m = j * 8 + g;
        const int k = c * 32 + 8 * t;
        uint4 xb = make_uint4(0, 0, 0, 0);
        if (m < M && c < n_chunks) {
            if (NORM && folded) {
                const float4 h0 = *reinterpret_cast<const float4*>(h_in + (size_t)m * K + k);
                const float4 h1 = *reinterpret_cast<const float4*>(h_in + (size_t)m * K + k + 4);
                if (count)
                    ssq[j] += h0.x * h0.x + h0.y * h0.y + h0.z * h0.z + h0.w * h0.w + h1.x * h1.x + h1.y * h1.y +
                              h1.z * h1.z + h1.w * h1.w;
                xb.x = pack2(h0.x, h0.y);
                xb.y = pack2(h0.z, h0.w);
                xb.z = pack2(h1.x, h1.y);
                xb.w = pack2(h1.z, h1.w);
            } else if (NORM) {
                const float4 h0 = *reinterpret_cast<const float4*>(h_in + (size_t)m * K + k);
                const float4 h1 = *reinterpret_cast<const float4*>(h_in + (size_t)m * K + k + 4);
                const float4 w0 = *reinterpret_cast<const float4*>(norm_w + k);
                const float4 w1 = *reinterpret_cast<const float4*>(norm_w + k + 4);
                const float r = rinv[m];
                xb.x = pack2((h0.x * r) * w0.x, (h0.y * r) * w0.y);
                xb.y = pack2((h0.z * r) * w0.z, (h0.w * r) * w0.w);
                xb.z = pack2((h1.x * r) * w1.x, (h1.y * r) * w1.y);
                xb.w = pack2((h1.z * r) * w1.z, (h1.w * r) * w1.w);
            } else {
                xb = *reinterpret_cast<const uint4*>(x + (size_t)m * ldk + (size_t)ks * K + k);
            }
        }
        return xb;
    };
    // Token-side fragments live in a small register queue: slot ii serves the items i = ii, ii + XD,
    // ... of every tile.  With XC > 0 a tile has at most XC items per warp and the queue is filled
    // once; otherwise a slot is refilled right after it is used, XD items ahead, so that the L2
    // latency of the activations never sits between the arrival of W and the MMA.
    constexpr int XD = XC > 0 ? XC : 4;
    uint4 xq[XD][NT];
#pragma unroll
    for (int i = 0; i < XD; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) xq[i][j] = load_x(chunk_of(i), j, true);

    float acc[NT][4];
    float acc2[NT][4];                                    // rows 16..23 of a 24-row tile (upper half unused)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
        acc2[j][0] = acc2[j][1] = acc2[j][2] = acc2[j][3] = 0.f;
    }

    int c_stage = 0, buf = 0;
    for (int tk = 0; tk < my_tiles; ++tk) {
        const int tile = bid + tk * gdim;
        // residual epilogue: the element of the stream this thread will add to is asked for now, so that its trip
        // from the cache runs beside the tile's products instead of behind them (one element per thread: a tile
        // has at most 256)
        float h_old = 0.f;
        if (EPI == EPI_RESID && (CL || S == 1)) {
            const int idx = CL ? ks + S * (int)threadIdx.x : (int)threadIdx.x;
            const int r = idx % ROWS, m = idx / ROWS;
            if (idx < ROWS * NT * 8 && m < M) h_old = ld_f32_now(reinterpret_cast<const float*>(out) + (size_t)m * N + tile * ROWS + r);
        }
#pragma unroll 1
        for (int i0 = 0; i0 < CH; i0 += XD) {
#pragma unroll
            for (int ii = 0; ii < XD; ++ii) {
                const int i = i0 + ii;
                if (i >= CH) break;
                const int c = chunk_of(i);
                uint4 xb[NT];
#pragma unroll
                for (int j = 0; j < NT; ++j) xb[j] = xq[ii][j];
                if (XC == 0) {
                    // slot ii serves the items ii, ii + XD, ... of a tile, then item ii of the next tile
                    int ni = i + XD;
                    const bool wrapped = ni >= CH;
                    if (wrapped) ni = ii;
#pragma unroll
                    for (int j = 0; j < NT; ++j) xq[ii][j] = load_x(chunk_of(ni), j, tk == 0 && !wrapped);
                }
                cp_async_wait<STAGES - 1>();              // the oldest group (this item) has landed
                const uint4 fa = slot[c_stage * stage_stride];
                const uint4 fb = RSLOTS >= 2 ? slot[c_stage * stage_stride + SK_WARPS * 32] : make_uint4(0, 0, 0, 0);
                const uint4 fc = RSLOTS == 3 ? slot[c_stage * stage_stride + 2 * SK_WARPS * 32] : make_uint4(0, 0, 0, 0);
                if (++c_stage == STAGES) c_stage = 0;
                issue();                                  // refill the slot with the item SK_STAGES ahead
                if (c < n_chunks) {
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        mma16816(acc[j], fa.x, fb.x, fa.y, fb.y, xb[j].x, xb[j].y);
                        mma16816(acc[j], fa.z, fb.z, fa.w, fb.w, xb[j].z, xb[j].w);
                        if (RSLOTS == 3) {
                            mma16816(acc2[j], fc.x, 0u, fc.y, 0u, xb[j].x, xb[j].y);
                            mma16816(acc2[j], fc.z, 0u, fc.w, 0u, xb[j].z, xb[j].w);
                        }
                    }
                }
            }
        }
        // ---- add the 8 partial sums of the block in a fixed order ----
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            part[buf][w][g][j * 8 + 2 * t] = acc[j][0];
            part[buf][w][g][j * 8 + 2 * t + 1] = acc[j][1];
            if (ROWS >= 16) {
                part[buf][w][(g + 8) % ROWS][j * 8 + 2 * t] = acc[j][2];
                part[buf][w][(g + 8) % ROWS][j * 8 + 2 * t + 1] = acc[j][3];
            }
            if (ROWS == 24) {
                part[buf][w][(g + 16) % ROWS][j * 8 + 2 * t] = acc2[j][0];
                part[buf][w][(g + 16) % ROWS][j * 8 + 2 * t + 1] = acc2[j][1];
                acc2[j][0] = acc2[j][1] = 0.f;
            }
            acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
        }
        if (NORM && folded && tk == 0) {
            // every chunk of h has passed through some warp during the first tile: finish sum(h^2)
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                float v = ssq[j];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                if (t == 0) ssw[w][j * 8 + g] = v;
            }
        }
        __syncthreads();      // one barrier per tile: `part` is double buffered
        if (NORM && folded && tk == 0) {
            if (threadIdx.x < NT * 8) {
                float v = 0.f;
#pragma unroll
                for (int ww = 0; ww < SK_WARPS; ++ww) v += ssw[ww][threadIdx.x];
                rinv[threadIdx.x] = 1.f / sqrtf(v / (float)K + eps);
            }
            __syncthreads();
        }
        const int n0 = tile * ROWS;
        if (CL) {
            // the S blocks of this tile are one cluster (rank ks): partial tiles through distributed shared memory
            constexpr int TILE = ROWS * NT * 8;
            for (int idx = threadIdx.x; idx < TILE; idx += blockDim.x) {
                const int r = idx % ROWS, m = idx / ROWS;
                float v = 0.f;
#pragma unroll
                for (int ww = 0; ww < SK_WARPS; ++ww) v += part[buf][ww][r][m];
                cl_part[buf][idx] = v;
            }
            // One barrier per tile is enough: cl_part is double buffered, and a block writes a buffer again only
            // after the barrier of the tile in between, which every block reaches after its reads of this one.
            sk_cluster_sync();
            const unsigned mine = (unsigned)__cvta_generic_to_shared(&cl_part[buf][0]);
            for (int idx = ks + S * (int)threadIdx.x; idx < TILE; idx += S * (int)blockDim.x) {
                const int r = idx % ROWS, m = idx / ROWS;
                if (m >= M) continue;
                float v = 0.f;
                for (int sp = 0; sp < S; ++sp) v += sk_ld_cluster(sk_cluster_map(mine + 4u * (unsigned)idx, (unsigned)sp));
                const size_t o = (size_t)m * N + n0 + r;
                if (EPI == EPI_BF16) reinterpret_cast<bf16*>(out)[o] = __float2bfloat16_rn(v);
                else if (EPI == EPI_F32) reinterpret_cast<float*>(out)[o] = v;
                else reinterpret_cast<float*>(out)[o] = h_old + (v + (bias ? bias[n0 + r] : 0.f));
            }
        } else if (EPI != EPI_SWIGLU && EPI != EPI_CONV && !NORM && S > 1) {
            // this block's partial tile -> workspace; the last of the S blocks adds them up
            constexpr int TILE = ROWS * NT * 8;
            float* wsp = ws + (size_t)tile * S * TILE;
            for (int idx = threadIdx.x; idx < TILE; idx += blockDim.x) {
                const int r = idx % ROWS, m = idx / ROWS;
                float v = 0.f;
#pragma unroll
                for (int ww = 0; ww < SK_WARPS; ++ww) v += part[buf][ww][r][m];
                __stcg(wsp + ks * TILE + idx, v);
            }
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) {
                const int old = atomicAdd(tickets + tile, 1);
                s_last = old == S - 1;
                if (old == S - 1) tickets[tile] = 0;      // all S have arrived: ready for the next launch
            }
            __syncthreads();
            if (s_last) {
                __threadfence();
                for (int idx = threadIdx.x; idx < TILE; idx += blockDim.x) {
                    const int r = idx % ROWS, m = idx / ROWS;
                    if (m >= M) continue;
                    float v = 0.f;
                    for (int sp = 0; sp < S; ++sp) v += __ldcg(wsp + sp * TILE + idx);
                    const size_t o = (size_t)m * N + n0 + r;
                    if (EPI == EPI_BF16) reinterpret_cast<bf16*>(out)[o] = __float2bfloat16_rn(v);
                    else if (EPI == EPI_F32) reinterpret_cast<float*>(out)[o] = v;
                    else reinterpret_cast<float*>(out)[o] += v + (bias ? bias[n0 + r] : 0.f);
                }
            }
        } else if (EPI == EPI_CONV) {
            // 8 channels per token: rows r, r + 8, r + 16 are B, C, X of channel tile * 8 + r (ROWS == 24)
            for (int idx = threadIdx.x; idx < 8 * NT * 8; idx += blockDim.x) {
                const int r = idx & 7, m = idx >> 3;
                if (m >= M) continue;
                float b = 0.f, cg = 0.f, xv = 0.f;
#pragma unroll
                for (int ww = 0; ww < SK_WARPS; ++ww) {
                    b += part[buf][ww][r][m];
                    cg += part[buf][ww][(r + 8) % ROWS][m];
                    xv += part[buf][ww][(r + 16) % ROWS][m];
                }
                if (NORM && folded) { b *= rinv[m]; cg *= rinv[m]; xv *= rinv[m]; }
                // the projection's output is a bfloat16 tensor wherever it is stored: round as a store would
                b = __bfloat162float(__float2bfloat16_rn(b));
                cg = __bfloat162float(__float2bfloat16_rn(cg));
                xv = __bfloat162float(__float2bfloat16_rn(xv));
                const int ch = tile * 8 + r, H = cv.H, L = cv.L;
                if (cv.in_bias) { b += cv.in_bias[ch]; cg += cv.in_bias[H + ch]; xv += cv.in_bias[2 * H + ch]; }
                const float bx = b * xv;
                float* st = cv.state + (size_t)cv.slots[m] * cv.slot_stride + ch;
                const bool fresh = cv.seg_pos0[m] == 0;
                const float* tp = cv.taps + (size_t)ch * L;
                float y = 0.f;
                for (int q = 0; q < L - 1; ++q) {
                    const float hq = fresh ? 0.f : st[(size_t)q * H];
                    y += hq * tp[q];
                    if (q > 0) st[(size_t)(q - 1) * H] = hq;      // the history moves up by one place
                }
                st[(size_t)(L - 2) * H] = bx;
                y += bx * tp[L - 1];
                if (cv.conv_bias) y += cv.conv_bias[ch];
                reinterpret_cast<bf16*>(out)[(size_t)m * H + ch] = __float2bfloat16_rn(cg * y);
            }
        } else if (EPI == EPI_SWIGLU) {
            // 8 outputs per token: row r is gate, row r + 8 is up (ROWS == 16)
            for (int idx = threadIdx.x; idx < 8 * NT * 8; idx += blockDim.x) {
                const int r = idx & 7, m = idx >> 3;
                if (m >= M) continue;
                float gt = 0.f, up = 0.f;
#pragma unroll
                for (int ww = 0; ww < SK_WARPS; ++ww) { gt += part[buf][ww][r][m]; up += part[buf][ww][(r + 8) % ROWS][m]; }
                if (NORM && folded) { gt *= rinv[m]; up *= rinv[m]; }
                reinterpret_cast<bf16*>(out)[(size_t)m * (N / 2) + tile * 8 + r] =
                    __float2bfloat16_rn((gt / (1.f + expf(-gt))) * up);
            }
        } else {
            for (int idx = threadIdx.x; idx < ROWS * NT * 8; idx += blockDim.x) {
                const int r = idx % ROWS, m = idx / ROWS;
                if (m >= M) continue;
                float v = 0.f;
#pragma unroll
                for (int ww = 0; ww < SK_WARPS; ++ww) v += part[buf][ww][r][m];
                if (NORM && folded) v *= rinv[m];
                const size_t o = (size_t)m * N + n0 + r;
                if (EPI == EPI_BF16) reinterpret_cast<bf16*>(out)[o] = __float2bfloat16_rn(v);
                else if (EPI == EPI_F32) reinterpret_cast<float*>(out)[o] = v;
                else reinterpret_cast<float*>(out)[o] = h_old + (v + (bias ? bias[n0 + r] : 0.f));
            }
        }
        buf ^= 1;
    }
    cp_async_wait<0>();
    if (CL) sk_cluster_sync();     // nobody leaves while a block of its cluster may still read its partial tile
}

#define SK_RING_BYTES(ROWS) (SK_STAGES_FOR(ROWS) * ((ROWS) / 8) * SK_WARPS * 32 * 16)
#define SK_MAX_BLOCKS (SK_BLOCKS_PER_SM * gesso_sm_count())

#define SK_TICKETS 4096                                  // tiles a split product may have (ints at the head of the workspace)

template <int NT, int EPI, bool NORM, int ROWS, int XC>
static int launch_one(const void* x, const float* h_in, const float* norm_w, float eps, const void* W, void* out,
                      const float* bias, int M, int N, int K, int S, void* ws, const ConvEpi& cv, cudaStream_t stream) {
    static bool configured = false;   // once per instantiation, outside any stream capture
    if (!configured) {
        cudaFuncSetAttribute(skinny_gemm_kernel<NT, EPI, NORM, ROWS, XC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SK_RING_BYTES(ROWS));
        configured = true;
    }
    const int n_tiles = N / ROWS;
    const int per_share = n_tiles < SK_MAX_BLOCKS / S ? n_tiles : SK_MAX_BLOCKS / S;
    const int blocks = per_share * S;
    launch_pdl(skinny_gemm_kernel<NT, EPI, NORM, ROWS, XC>, dim3(blocks), dim3(SK_WARPS * 32), SK_RING_BYTES(ROWS), stream,
               (const bf16*)x, h_in, norm_w, eps, (const bf16*)W, out, bias, M, N, K / S, K, S,
               (float*)((int*)ws + SK_TICKETS), (int*)ws, cv);
    return launch_status();
}

// The same for a product split along K whose S blocks per tile form a cluster (S = 2, 4, 8): no workspace.
template <int NT, int EPI, int ROWS, int XC>
static int launch_cluster(const void* x, const void* W, void* out, const float* bias, int M, int N, int K, int S,
                          cudaStream_t stream) {
    auto kernel = skinny_gemm_kernel<NT, EPI, false, ROWS, XC, true>;
    static bool configured = false;   // once per instantiation, outside any stream capture
    if (!configured) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_RING_BYTES(ROWS));
        configured = true;
    }
    const int n_tiles = N / ROWS;
    const int per_share = n_tiles < SK_MAX_BLOCKS / S ? n_tiles : SK_MAX_BLOCKS / S;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(per_share * S);
    cfg.blockDim = dim3(SK_WARPS * 32);
    cfg.dynamicSmemBytes = SK_RING_BYTES(ROWS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gesso_pdl_enabled ? 2 : 1;
    const ConvEpi none = {};
    cudaLaunchKernelEx(&cfg, kernel, (const bf16*)x, (const float*)nullptr, (const float*)nullptr, 0.f, (const bf16*)W, out,
                       bias, M, N, K / S, K, S, (float*)nullptr, (int*)nullptr, none);
    return launch_status();
}

template <int NT, int EPI, bool NORM>
static int launch_shape(const void* x, const float* h_in, const float* norm_w, float eps, const void* W, void* out,
                        const float* bias, int M, int N, int K, void* ws, long long ws_bytes, const ConvEpi& cv,
                        cudaStream_t stream) {
    // token-side fragments stay in registers when a warp has at most 8 chunks per tile (K <= 2048); the queue
    // has 2, 4 or 8 places, of which a tile uses the first ceil(chunks / warps)
    auto per_warp = [](int k) { return (k / 32 + SK_WARPS - 1) / SK_WARPS; };
    auto cacheable = [&](int k) { return k % 32 == 0 && per_warp(k) <= 8 && NT * per_warp(k) <= 16; };
    int S = 1;
    if (!cacheable(K) && !NORM && EPI != EPI_SWIGLU && EPI != EPI_CONV) {
        // split K over S blocks per tile, the smallest S whose share is cacheable: a cluster up to 8 blocks
        // (no workspace); 16 blocks through the workspace if it is there and large enough
        for (int s = 2; s <= 16; s *= 2) {
            // sized for 16 token rows whatever M is: the choice of S must not depend on the batch
            const long long need = (long long)SK_TICKETS * 4 + (long long)N * s * 16 * 4;
            const bool room = s <= 8 || (ws != nullptr && N / 8 <= SK_TICKETS && need <= ws_bytes);
            if (K % (32 * s) == 0 && cacheable(K / s)) {
                if (room) S = s;
                break;
            }
        }
    }
    const int Ks = K / S;
    const bool cache_x = cacheable(Ks);
    const bool small_rows = EPI != EPI_SWIGLU && (N / 16) * S < SK_MAX_BLOCKS && N % 8 == 0;
    const int xc = !cache_x ? 0 : per_warp(Ks) <= 2 ? 2 : per_warp(Ks) <= 4 ? 4 : 8;
#define GO(ROWS, XC) return launch_one<NT, EPI, NORM, ROWS, XC>(x, h_in, norm_w, eps, W, out, bias, M, N, K, S, ws, cv, stream)
    if constexpr (!NORM && EPI != EPI_SWIGLU && EPI != EPI_CONV) {
        if (S > 1 && S <= 8) {       // a split product whose share is cacheable: xc is 2, 4 or 8
#define GC(ROWS, XC) return launch_cluster<NT, EPI, ROWS, XC>(x, W, out, bias, M, N, K, S, stream)
            if (small_rows) {
                if (xc == 8) GC(8, 8);
                if (xc == 4) GC(8, 4);
                if (xc == 2) GC(8, 2);
            } else {
                if (xc == 8) GC(16, 8);
                if (xc == 4) GC(16, 4);
                if (xc == 2) GC(16, 2);
            }
#undef GC
            S = 1;                   // no cached shape for it: unsplit (never the case for the sizes that split)
        }
    }
    if constexpr (EPI == EPI_CONV) {
        if (xc == 8) GO(24, 8);
        if (xc == 4) GO(24, 4);
        GO(24, 0);
    } else {
    if (EPI != EPI_SWIGLU && small_rows) {
        if (xc == 8) GO(8, 8);
        if (xc == 4) GO(8, 4);
        if (xc == 2) GO(8, 2);
        GO(8, 0);
    }
    if (xc == 8) GO(16, 8);
    if (xc == 4) GO(16, 4);
    if (xc == 2) GO(16, 2);
    GO(16, 0);
    }
#undef GO
}

// Every epilogue for one (token tiles, fused norm) pair: each pair is compiled in a file of its
// own (gemm_skinny_*.cu), since the instantiations are what takes the time to compile.
template <int NT, bool NORM>
int skinny_launch(const void* x, const float* h_in, const float* norm_w, float eps, const void* W, void* out,
                  const float* bias, int M, int N, int K, int epi, void* ws, long long ws_bytes,
                  const ConvEpi& cv, cudaStream_t stream) {
#define GO(E) return launch_shape<NT, E, NORM>(x, h_in, norm_w, eps, W, out, bias, M, N, K, ws, ws_bytes, cv, stream)
    if (epi == EPI_BF16) GO(EPI_BF16);
    if (epi == EPI_F32) GO(EPI_F32);
    if (epi == EPI_SWIGLU) GO(EPI_SWIGLU);
    if (epi == EPI_CONV) GO(EPI_CONV);
    if constexpr (!NORM) {
        if (epi == EPI_RESID) GO(EPI_RESID);
    }
    return GESSO_ERR_UNSUPPORTED;
#undef GO
}
