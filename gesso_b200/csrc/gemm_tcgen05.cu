// Dense bfloat16 matrix product on the 5th-generation tensor cores:
//   C[M,N] = A[M,K] * W[N,K]^T, float32 accumulation in tensor memory.
//
// A block computes 128 x BN tiles of C (BN = 256 or 128), one after the other.  Three roles:
//   warp 0  one elected thread issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of a
//           128 x 64 tile of A and a BN x 64 tile of W per stage into a ring of shared-memory
//           stages, each guarded by a "full" mbarrier (transaction bytes) and an "empty" mbarrier;
//   warp 1  allocates 2 x BN tensor-memory columns; one elected thread issues tcgen05.mma
//           (cta_group::1, kind::f16, M = 128, N = BN, K = 16; four per stage) on shared-memory
//           descriptors, frees a stage with tcgen05.commit -> its "empty" barrier and signals the
//           finished accumulator through a last commit;
//   warps 2..5  the epilogue: tcgen05.ld (32 lanes x 32 columns per warp and step) brings the
//           accumulator rows to registers; each thread owns one row of C and stores 32 consecutive
//           columns per step as bfloat16 / float32, or adds them into the float32 residual stream, or
//           applies SwiGLU to packed gate/up columns.
// Both operands are K-major (A row-major, W stored (out, in) as the reference stores projection
// weights, src/Operators/cpu.jl:629-630), which is the canonical layout of the shared-memory
// descriptor: 8-row groups 1024 bytes apart, 128-byte rows, 16-byte chunks XOR-swizzled by the row.
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT failed polls the thread records a code in
// the status word, and every role then leaves its loop, so the kernel always ends, frees its
// tensor memory and the host reads the status.  Rows beyond M and columns beyond N / K are zero
// filled by TMA on the way in and predicated on the way out.
#include <math.h>

#include "tcgen05.cuh"
#include "gemm_tcgen05_epilogue.cuh"
#include "tensor_map.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_SMS gesso_sm_count()

template <int BN, int STAGES>
struct __align__(1024) TcSmem {
    bf16 a[STAGES][TC_BM * TC_BK];     // 16 KB per stage
    bf16 b[STAGES][BN * TC_BK];        // 32 or 16 KB per stage
    unsigned long long full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    unsigned tmem_base;
};

// Blocks are persistent: block b computes tiles b, b + gridDim.x, ... (tile = n_block * m_blocks +
// m_block, so blocks that run together share W tiles in L2).  The accumulator is double buffered in
// tensor memory (2 x BN columns): while the epilogue warps drain one buffer, the MMA thread already
// fills the other, and the TMA ring runs on across tile borders.
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    void* __restrict__ out, const float* __restrict__ bias, int M, int N, int K,
                    int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    // the swizzled stages must start on a 1024-byte boundary
    TcSmem<BN, STAGES>& s =
        *reinterpret_cast<TcSmem<BN, STAGES>*>(((size_t)smem_raw + 1023) & ~(size_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    const int m_blocks = (M + TC_BM - 1) / TC_BM, n_blocks = (N + BN - 1) / BN;
    const int n_tiles = m_blocks * n_blocks;
    constexpr unsigned STAGE_BYTES = (TC_BM + BN) * TC_BK * sizeof(bf16);

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s.acc_full[i], 1);
            mbar_init(&s.acc_empty[i], 4);      // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {               // this warp owns the tensor memory: two accumulators of BN columns
        tmem_alloc(&s.tmem_base, 2 * BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = s.tmem_base;
    // Launched programmatically: the set-up above ran while the kernel before still worked; nothing below
    // reads or writes global memory before that kernel is complete.
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        // ---- producer ----
        if (elect_one()) {
            unsigned it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % m_blocks) * TC_BM, n0 = (tile / m_blocks) * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int st = it % STAGES;
                    const unsigned phase = (it / STAGES) & 1;
                    if (!mbar_wait(&s.empty[st], phase ^ 1)) { atomicExch(status, 2); ok = false; break; }
                    mbar_expect_tx(&s.full[st], STAGE_BYTES);
                    tma_load_2d(s.a[st], &map_a, kb * TC_BK, m0, &s.full[st]);
                    tma_load_2d(s.b[st], &map_w, kb * TC_BK, n0, &s.full[st]);
                }
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core issue ----
        if (elect_one()) {
            constexpr unsigned idesc = make_idesc(TC_BM, BN);
            unsigned it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++local) {
                const unsigned buf = local & 1;
                // the epilogue must have drained this buffer (two tiles ago)
                if (!mbar_wait(&s.acc_empty[buf], ((local >> 1) & 1) ^ 1)) { atomicExch(status, 5); ok = false; break; }
                tc_fence_after();
                const unsigned acc = tmem + buf * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int st = it % STAGES;
                    const unsigned phase = (it / STAGES) & 1;
                    if (!mbar_wait(&s.full[st], phase)) { atomicExch(status, 3); ok = false; break; }
                    tc_fence_after();
                    const unsigned long long da = make_desc(smem_u32(s.a[st]));
                    const unsigned long long db = make_desc(smem_u32(s.b[st]));
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)     // 16 elements = 32 bytes = 2 descriptor units
                        umma_f16(acc, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&s.empty[st]);               // the stage is free once these MMAs have read it
                }
                umma_commit(&s.acc_full[buf]);                // arrives even after a failure, so the epilogue ends
            }
        }
    } else {
        // ---- epilogue: warp q may touch tensor-memory lanes 32q .. 32q+31 ----
        const int q = warp & 3;
        unsigned local = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
            const int m0 = (tile % m_blocks) * TC_BM, n0 = (tile / m_blocks) * BN;
            const unsigned buf = local & 1;
            const bool ready = mbar_wait(&s.acc_full[buf], (local >> 1) & 1);
            if (!ready) {
                if (lane == 0) atomicExch(status, 4);
                break;
            }
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const unsigned acc = tmem + buf * BN + ((unsigned)(q * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                unsigned r[32];
                tmem_ld32(acc + (unsigned)c, r);
                tmem_ld_wait();
                const int col = n0 + c;
                if (row >= M || col >= N) continue;
                tc_store_32<EPI>(r, out, bias, row, col, N);
            }
            // this warp has read its lanes of the buffer: hand it back to the MMA thread
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 2 * BN);
    }
}

// ---- host side ------------------------------------------------------------------------------------------
GESSO_API int gesso_gemm_tcgen05_takes(int M, int N, int K) {
    // TMA: 16-byte aligned rows (K % 8); vector stores: N % 8 (bfloat16) / N % 4 (float32)
    return M >= 1 && N >= 8 && N % 8 == 0 && K >= 8 && K % 8 == 0;
}

template <int BN, int STAGES, int EPI>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mw, void* out, const float* bias, int M, int N, int K,
                     int* status, cudaStream_t stream) {
    const size_t smem = sizeof(TcSmem<BN, STAGES>) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    const int tiles = ((N + BN - 1) / BN) * ((M + TC_BM - 1) / TC_BM);
    const dim3 grid(tiles < TC_SMS ? tiles : TC_SMS);
    launch_pdl(gemm_tcgen05_kernel<BN, STAGES, EPI>, grid, dim3(TC_THREADS), smem, stream, ma, mw, out, bias, M, N, K,
               status);
    return launch_status();
}

// A: bfloat16 [M,K]; W: bfloat16 [N,K]; out by `epi` (bf16 [M,N], f32 [M,N], f32 residual [M,N] +=,
// bf16 [M,N/2] SwiGLU of packed gate/up columns); status: one int, 0 unless a wait ran out.
GESSO_API int gesso_gemm_tcgen05(const void* A, const void* W, void* out, const float* bias, int M, int N, int K,
                                 int epi, int* status, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (!gesso_gemm_tcgen05_takes(M, N, K)) return GESSO_ERR_BAD_SIZE;
    if (epi == TC_EPI_SWIGLU && N % 16 != 0) return GESSO_ERR_BAD_SIZE;
    if (((size_t)A & 15) || ((size_t)W & 15) || ((size_t)out & 15)) return GESSO_ERR_BAD_SIZE;
    const bool wide = N % 256 == 0 || N >= 1024;
    CUtensorMap ma, mw;
    int r = make_matrix_map(&ma, A, M, K, TC_BM);
    if (r) return r;
    r = make_matrix_map(&mw, W, N, K, wide ? 256 : 128);
    if (r) return r;
#define GO(BN, ST)                                                                                              \
    switch (epi) {                                                                                              \
        case TC_EPI_BF16: return launch_tc<BN, ST, TC_EPI_BF16>(ma, mw, out, bias, M, N, K, status, stream);    \
        case TC_EPI_F32: return launch_tc<BN, ST, TC_EPI_F32>(ma, mw, out, bias, M, N, K, status, stream);      \
        case TC_EPI_RESID: return launch_tc<BN, ST, TC_EPI_RESID>(ma, mw, out, bias, M, N, K, status, stream);  \
        case TC_EPI_SWIGLU: return launch_tc<BN, ST, TC_EPI_SWIGLU>(ma, mw, out, bias, M, N, K, status, stream); \
        default: return GESSO_ERR_UNSUPPORTED;                                                                  \
    }
    if (wide) { GO(256, 4) } else { GO(128, 4) }
#undef GO
}
