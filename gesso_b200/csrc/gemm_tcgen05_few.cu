// Dense bfloat16 matrix product for a few dozen rows (17 .. 128 tokens: a decoding step of many
// requests, a small mixed step) on the 5th-generation tensor cores:
//   C[M,N] = A[M,K] * W[N,K]^T, float32 accumulation in tensor memory.
//
// Such a product is bound by reading W once, so the operands are swapped: 128 rows of W are the
// MMA's M side and the tokens (rounded up to MT, a multiple of 16) its N side.  A tile is 128 rows
// of W times all tokens.  Where W has fewer tiles than the device has SMs, a cluster of S = 2 .. 8
// blocks shares a tile: block r of the cluster multiplies the r-th part of K, and the partial tiles
// are added through distributed shared memory, in the order of the ranks.
//   warp 0   one elected thread issues TMA loads (128-byte swizzle) of a 128 x 64 tile of W and the
//            MT x 64 tile of A per stage into a ring of up to ten stages; the first ring of W tiles is
//            requested before the wait on the preceding kernel (W does not depend on it);
//   warp 1   allocates tensor memory (two accumulators of MT columns); one elected thread issues
//            tcgen05.mma (M = 128, N = MT, K = 16; four per stage) and commits stages and accumulators;
//   warps 2..17  the epilogue: warp e works on tensor-memory lanes 32 (e % 4) .. + 31 (rows of the tile,
//            output columns of C) and on every fourth group of 8 tokens (e / 4, + 4, ...), read with
//            tcgen05.ld; sixteen warps, because one warp's chain of dependent instructions per value
//            would otherwise be what a single-tile block waits for at its end.
// Without a cluster a block walks whole tiles (blockIdx.x, + gridDim.x, ...) and stores them directly.
// In a cluster every block has one part of one tile.  When all have finished their products (first
// cluster barrier: the rings are free), each sends the values of token slice j (MT / S tokens, rounded up) to the
// ring of block j (st.shared::cluster); after the second barrier block j adds the S parts of its slice
// from its own shared memory in the order 0 .. S-1 and stores them.  Epilogues: bfloat16 / float32
// store, add into the float32 residual stream (with bias), SwiGLU of packed gate/up rows (8 gate rows
// then their 8 up rows: the partner value comes from the lane 8 further on).
// Formulas: src/Operators/cpu.jl:629-630 (x W^T), 482-488 (SwiGLU).
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT failed polls the thread records a code in
// the status word and leaves its loop; every thread still arrives at both cluster barriers, so the
// kernel always ends and frees its tensor memory.  Rows beyond M / N and columns beyond K are zero
// filled by TMA and predicated on the way out.
#include <math.h>

#include "tcgen05.cuh"
#include "gemm_tcgen05_epilogue.cuh"
#include "tensor_map.cuh"

#define FW_BN 128            // rows of W per tile
#define FW_BK 64
#define FW_EPI_WARPS 16       // four per quarter of the tensor-memory lanes, each with every fourth group of 8 tokens
#define FW_THREADS (64 + 32 * FW_EPI_WARPS)
#define FW_SMS gesso_sm_count()
#define FW_MAX_ROWS 128      // tokens
#define FW_MAX_STAGES 10
#define FW_RING_BYTES (192 * 1024)
#define FW_W_BYTES (FW_BN * FW_BK * 2)

struct FewShared {
    unsigned long long full[FW_MAX_STAGES], empty[FW_MAX_STAGES], acc_full[2], acc_empty[2];
    unsigned tmem_base;
};

// the address of this block's shared-memory object `addr` in block `rank` of the cluster
__device__ __forceinline__ unsigned cluster_map(unsigned addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(unsigned addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}

// every warp arrives as one (its threads have converged before)
__device__ __forceinline__ void cluster_sync_warps() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

template <int EPI>
__device__ __forceinline__ void few_store(float v, void* __restrict__ out, const float* __restrict__ bias, int tok,
                                          int n, int N, int lane) {
    if (EPI == TC_EPI_SWIGLU) {
        const float up = __shfl_xor_sync(0xffffffffu, v, 8);
        if ((lane & 8) == 0 && n < N)
            reinterpret_cast<bf16*>(out)[(size_t)tok * (N / 2) + (n >> 4) * 8 + (n & 7)] =
                __float2bfloat16(__fdividef(v, 1.f + __expf(-v)) * up);
    } else if (n < N) {
        if (EPI == TC_EPI_BF16) reinterpret_cast<bf16*>(out)[(size_t)tok * N + n] = __float2bfloat16(v);
        else if (EPI == TC_EPI_F32) reinterpret_cast<float*>(out)[(size_t)tok * N + n] = v;
        else {
            float* o = reinterpret_cast<float*>(out) + (size_t)tok * N + n;
            *o = *o + v + (bias ? bias[n] : 0.f);
        }
    }
}

// S: blocks per cluster (1: launched without clusters).  With S > 1 the grid has exactly S blocks per tile.
template <int EPI>
__global__ void __launch_bounds__(FW_THREADS, 1)
gemm_tcgen05_few_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                        void* __restrict__ out, const float* __restrict__ bias, int M, int N, int K, int MT, int stages,
                        int S, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ FewShared s;
    unsigned char* ring = reinterpret_cast<unsigned char*>(((size_t)smem_raw + 1023) & ~(size_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned stage_bytes = FW_W_BYTES + (unsigned)MT * FW_BK * 2;
    const int KB = (K + FW_BK - 1) / FW_BK, n_tiles = (N + FW_BN - 1) / FW_BN;
    const int rank = S > 1 ? (int)cluster_ctarank() : 0;
    const int tile0 = (int)blockIdx.x / S, tile_step = (int)gridDim.x / S;
    const int kb_lo = (int)((long long)rank * KB / S), n_kb = (int)((long long)(rank + 1) * KB / S) - kb_lo;
    const int my_tiles = tile0 < n_tiles ? (n_tiles - tile0 + tile_step - 1) / tile_step : 0;
    const int mine = my_tiles * n_kb;       // stages this block loads

    const int early = mine < stages ? mine : stages;
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_a) : "memory");
        for (int i = 0; i < stages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s.acc_full[i], 1);
            mbar_init(&s.acc_empty[i], FW_EPI_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        // The first ring of W tiles depends neither on the preceding kernel nor on the rest of the
        // set-up: it is requested at once.
        for (int i = 0; i < early; ++i) {
            mbar_expect_tx(&s.full[i], stage_bytes);
            tma_load_2d(ring + (size_t)i * stage_bytes, &map_w, (kb_lo + i % n_kb) * FW_BK,
                        (tile0 + (i / n_kb) * tile_step) * FW_BN, &s.full[i]);
        }
    }
    if (warp == 1) {
        tmem_alloc(&s.tmem_base, 2 * FW_MAX_ROWS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = s.tmem_base;
    pdl_launch_dependents();
    bool have_tile = false;     // epilogue warps of a cluster: the partial tile is in tensor memory

    if (warp == 0) {
        // ---- producer ----
        if (elect_one()) {
            pdl_wait();      // the tokens come from the preceding kernel
            for (int i = 0; i < early; ++i)
                tma_load_2d(ring + (size_t)i * stage_bytes + FW_W_BYTES, &map_a, (kb_lo + i % n_kb) * FW_BK, 0, &s.full[i]);
            for (int i = early; i < mine; ++i) {
                const int st = i % stages;
                const unsigned phase = (unsigned)(i / stages) & 1;
                if (!mbar_wait_idle(&s.empty[st], phase ^ 1)) { atomicExch(status, 32); break; }
                const int k0 = (kb_lo + i % n_kb) * FW_BK;
                mbar_expect_tx(&s.full[st], stage_bytes);
                tma_load_2d(ring + (size_t)st * stage_bytes, &map_w, k0, (tile0 + (i / n_kb) * tile_step) * FW_BN, &s.full[st]);
                tma_load_2d(ring + (size_t)st * stage_bytes + FW_W_BYTES, &map_a, k0, 0, &s.full[st]);
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core issue ----
        if (elect_one()) {
            const unsigned idesc = make_idesc(FW_BN, MT);
            int i = 0;
            bool ok = true;
            for (int t = 0; t < my_tiles && ok; ++t) {
                const unsigned buf = t & 1;
                if (!mbar_wait(&s.acc_empty[buf], ((t >> 1) & 1) ^ 1)) { atomicExch(status, 35); break; }
                tc_fence_after();
                const unsigned acc = tmem + buf * FW_MAX_ROWS;
                for (int kb = 0; kb < n_kb; ++kb, ++i) {
                    const int st = i % stages;
                    const unsigned phase = (unsigned)(i / stages) & 1;
                    if (!mbar_wait(&s.full[st], phase)) { atomicExch(status, 33); ok = false; break; }
                    tc_fence_after();
                    const unsigned base = smem_u32(ring + (size_t)st * stage_bytes);
                    const unsigned long long dw = make_desc(base), da = make_desc(base + FW_W_BYTES);
#pragma unroll
                    for (int k = 0; k < FW_BK / 16; ++k)
                        umma_f16(acc, dw + 2 * k, da + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&s.empty[st]);
                }
                umma_commit(&s.acc_full[buf]);     // arrives even after a failure, so the epilogue ends
            }
        }
    } else {
        // ---- epilogue: warp e may touch tensor-memory lanes 32 (e % 4) .. + 31 ----
        const int e = warp - 2, q = warp & 3, part = e >> 2;
        const int nl = q * 32 + lane;      // row of the tile
        pdl_wait();                        // this role reads and writes what earlier kernels used
        if (S > 1) {
            if (my_tiles > 0) {
                have_tile = mbar_wait(&s.acc_full[0], 0);
                if (!have_tile && lane == 0) atomicExch(status, 34);
                tc_fence_after();
            }
        } else {
            for (int t = 0; t < my_tiles; ++t) {
                const unsigned buf = t & 1;
                if (!mbar_wait(&s.acc_full[buf], (t >> 1) & 1)) {
                    if (lane == 0) atomicExch(status, 34);
                    break;
                }
                tc_fence_after();
                const unsigned acc = tmem + buf * FW_MAX_ROWS + ((unsigned)(q * 32) << 16);
                const int n = (tile0 + t * tile_step) * FW_BN + nl;
#pragma unroll 1
                for (int c = part * 8; c < MT; c += 32) {
                    unsigned v[8];
                    tmem_ld8(acc + (unsigned)c, v);
                    tmem_ld_wait();
                    if (EPI == TC_EPI_RESID) {
                        // all reads of the residual stream first: they do not wait for one another
                        float* o = reinterpret_cast<float*>(out) + (size_t)c * N + n;
                        const float b = (bias && n < N) ? bias[n] : 0.f;
                        float old[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) old[j] = (c + j < M && n < N) ? o[(size_t)j * N] : 0.f;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (c + j < M && n < N) o[(size_t)j * N] = old[j] + __uint_as_float(v[j]) + b;
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (c + j < M) few_store<EPI>(__uint_as_float(v[j]), out, bias, c + j, n, N, lane);
                    }
                }
                // this warp has read its lanes of the buffer: hand it back to the MMA thread
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.acc_empty[buf]);
            }
        }
    }
    if (S > 1) {
        // Every thread of every block arrives at both barriers, whatever happened above.
        const int slice = (MT + S - 1) / S;            // tokens whose sum each block owns
        const unsigned recv = smem_u32(ring);          // [S parts][slice tokens][128 rows] float32, over the ring
        cluster_sync_warps();                          // all products done: every ring is free
        if (warp >= 2 && have_tile) {
            const int q = warp & 3, part = (warp - 2) >> 2, nl = q * 32 + lane;
            const unsigned acc = tmem + ((unsigned)(q * 32) << 16);
#pragma unroll 1
            for (int c = part * 8; c < MT; c += 32) {
                unsigned v[8];
                tmem_ld8(acc + (unsigned)c, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int tok = c + j, dst = tok / slice, t = tok - dst * slice;
                    st_cluster_f32(cluster_map(recv + (unsigned)(((rank * slice + t) * FW_BN + nl) * 4), (unsigned)dst),
                                   __uint_as_float(v[j]));
                }
            }
        }
        cluster_sync_warps();                          // all parts have arrived
        if (warp >= 2 && my_tiles > 0) {
            // warp (q, part) adds up and stores every fourth token of this block's slice
            const int q = warp & 3, part = (warp - 2) >> 2, nl = q * 32 + lane;
            const int n = tile0 * FW_BN + nl;
            const float* mine_parts = reinterpret_cast<const float*>(ring);
            const int tok0 = rank * slice;
            const int count = M - tok0 < slice ? M - tok0 : slice;      // may be negative: nothing to store
            for (int t = part; t < count; t += 4) {
                float old = 0.f;
                if (EPI == TC_EPI_RESID && n < N) old = reinterpret_cast<const float*>(out)[(size_t)(tok0 + t) * N + n];
                float sum = 0.f;
                for (int src = 0; src < S; ++src) sum += mine_parts[(src * slice + t) * FW_BN + nl];
                if (EPI == TC_EPI_RESID) {
                    if (n < N)
                        reinterpret_cast<float*>(out)[(size_t)(tok0 + t) * N + n] = old + sum + (bias ? bias[n] : 0.f);
                } else {
                    few_store<EPI>(sum, out, bias, tok0 + t, n, N, lane);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 2 * FW_MAX_ROWS);
    }
}

// ---- host side ------------------------------------------------------------------------------------------
static int few_mt(int M) { return M <= 16 ? 16 : (M + 15) / 16 * 16; }

GESSO_API int gesso_gemm_tcgen05_few_takes(int M, int N, int K) {
    // TMA: 16-byte aligned rows (K % 8)
    return M >= 1 && M <= FW_MAX_ROWS && N >= 8 && K >= 8 && K % 8 == 0;
}

template <int EPI>
static void few_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int grid, int S, size_t smem,
                       cudaStream_t stream) {
    *cfg = cudaLaunchConfig_t{};
    cfg->gridDim = dim3(grid);
    cfg->blockDim = dim3(FW_THREADS);
    cfg->dynamicSmemBytes = smem;
    cfg->stream = stream;
    int n = 0;
    if (S > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = S;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (gesso_pdl_enabled) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg->attrs = attr;
    cfg->numAttrs = n;
}

template <int EPI>
static int launch_few(const CUtensorMap& mw, const CUtensorMap& ma, void* out, const float* bias, int M, int N, int K,
                      int want_S, int* status, cudaStream_t stream) {
    const int MT = few_mt(M);
    const unsigned stage_bytes = FW_W_BYTES + MT * FW_BK * 2;
    int stages = FW_RING_BYTES / stage_bytes;
    if (stages > FW_MAX_STAGES) stages = FW_MAX_STAGES;
    const size_t smem = (size_t)stages * stage_bytes + 1024;
    static bool configured = false;
    static int max_clusters[9];      // clusters of S blocks the device runs at the same time
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tcgen05_few_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 FW_RING_BYTES + 1024) != cudaSuccess)
            return (int)cudaGetLastError();
        for (int S = 2; S <= 8; ++S) {
            few_config<EPI>(&cfg, attr, S, S, FW_RING_BYTES + 1024, stream);
            cfg.numAttrs = 1;       // the cluster size alone
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_few_kernel<EPI>, &cfg) != cudaSuccess) {
                cudaGetLastError();
                n = 0;
            }
            max_clusters[S] = n;
        }
        configured = true;
    }
    const int n_tiles = (N + FW_BN - 1) / FW_BN, KB = (K + FW_BK - 1) / FW_BK;
    // the largest cluster whose blocks all run at once, with at least two steps along K for each block
    int S = 1;
    for (int c = 8; c >= 2; --c)
        if ((want_S == 0 || want_S == c) && n_tiles * c <= FW_SMS && n_tiles <= max_clusters[c] && KB >= 2 * c) {
            S = c;
            break;
        }
    const int grid = S > 1 ? n_tiles * S : (n_tiles < FW_SMS ? n_tiles : FW_SMS);
    few_config<EPI>(&cfg, attr, grid, S, smem, stream);
    cudaLaunchKernelEx(&cfg, gemm_tcgen05_few_kernel<EPI>, mw, ma, out, bias, M, N, K, MT, stages, S, status);
    return launch_status();
}

// A: bfloat16 [M,K], M <= 128; W: bfloat16 [N,K]; out by `epi` (bf16 [M,N], f32 [M,N], f32 residual [M,N]
// +=, bf16 [M,N/2] SwiGLU of packed gate/up rows of W); cluster: 0 lets the kernel choose the blocks per
// tile, 1 .. 8 asks for that many where it fits; status: one int, 0 unless a wait ran out.
GESSO_API int gesso_gemm_tcgen05_few(const void* A, const void* W, void* out, const float* bias, int M, int N, int K,
                                     int epi, int cluster, int* status, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (!gesso_gemm_tcgen05_few_takes(M, N, K)) return GESSO_ERR_BAD_SIZE;
    if (epi == TC_EPI_SWIGLU && N % 16 != 0) return GESSO_ERR_BAD_SIZE;
    if (((size_t)A & 15) || ((size_t)W & 15)) return GESSO_ERR_BAD_SIZE;
    CUtensorMap mw, ma;
    int r = make_matrix_map(&mw, W, N, K, FW_BN);
    if (r) return r;
    r = make_matrix_map(&ma, A, M, K, few_mt(M));
    if (r) return r;
    switch (epi) {
        case TC_EPI_BF16: return launch_few<TC_EPI_BF16>(mw, ma, out, bias, M, N, K, cluster, status, stream);
        case TC_EPI_F32: return launch_few<TC_EPI_F32>(mw, ma, out, bias, M, N, K, cluster, status, stream);
        case TC_EPI_RESID: return launch_few<TC_EPI_RESID>(mw, ma, out, bias, M, N, K, cluster, status, stream);
        case TC_EPI_SWIGLU: return launch_few<TC_EPI_SWIGLU>(mw, ma, out, bias, M, N, K, cluster, status, stream);
        default: return GESSO_ERR_UNSUPPORTED;
    }
}
