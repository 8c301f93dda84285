// Dense bfloat16 matrix product on the 5th-generation tensor cores with two blocks per tile:
//   C[M,N] = A[M,K] * W[N,K]^T, float32 accumulation in tensor memory.
//
// The blocks of a cluster of two compute a 256 x 256 tile of C together (tcgen05.mma.cta_group::2): each
// block stages its own 128 rows of A and HALF of the tile's rows of W (128 x 64 each per stage), the tensor
// cores of both SMs read both halves, and each block's tensor memory receives its 128 rows of the
// accumulator.  Per SM and k step that is 32 KB of operands from L2 instead of the 48 KB a block working
// alone on 128 x 256 needs: the single-block kernel (gemm_tcgen05.cu) is bound by exactly that traffic.
// The smaller stages also allow a ring six deep.
//
// Roles in each block: warp 0 issues the TMA loads (their bytes are counted on the LEADER block's "full"
// barrier; the leader alone arms it); warp 1 allocates the tensor memory, and in the leader block one
// thread issues the MMAs for both blocks, frees a stage in both blocks with one multicast commit and
// signals a finished accumulator to both blocks' epilogues the same way; warps 2..5 are the epilogue of
// the block's own 128 rows (as in the single-block kernel) and hand the accumulator back by an arrival on
// the leader's barrier.  All waits are bounded and report through the status word; the blocks meet at a
// cluster barrier before the tensor memory is given back.
#include <math.h>

#include "tcgen05.cuh"
#include "gemm_tcgen05_epilogue.cuh"
#include "tensor_map.cuh"

#define TP_BM 128            // rows of C per block (256 per pair)
#define TP_BN 256            // columns of C per pair; each block stages 128 rows of W
#define TP_BK 64
#define TP_STAGES 6
#define TP_THREADS 192

struct __align__(1024) TpSmem {
    bf16 a[TP_STAGES][TP_BM * TP_BK];          // 16 KB per stage
    bf16 b[TP_STAGES][(TP_BN / 2) * TP_BK];    // 16 KB per stage
    unsigned long long full[TP_STAGES], empty[TP_STAGES], acc_full[2], acc_empty[2];
    unsigned tmem_base;
};

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TP_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         void* __restrict__ out, const float* __restrict__ bias, int M, int N, int K,
                         int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    TpSmem& s = *reinterpret_cast<TpSmem*>(((size_t)smem_raw + 1023) & ~(size_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_ctarank();          // 0: the leader of the pair
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int k_blocks = (K + TP_BK - 1) / TP_BK;
    const int m_blocks = (M + 2 * TP_BM - 1) / (2 * TP_BM), n_blocks = (N + TP_BN - 1) / TP_BN;
    const int n_tiles = m_blocks * n_blocks;
    constexpr unsigned STAGE_BYTES = (TP_BM + TP_BN / 2) * TP_BK * sizeof(bf16);     // per block

    if (threadIdx.x == 0) {
        for (int i = 0; i < TP_STAGES; ++i) {
            mbar_init(&s.full[i], 1);           // used in the leader: its own arming arrival + both blocks' bytes
            mbar_init(&s.empty[i], 1);          // in each block: the leader's multicast commit
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s.acc_full[i], 1);       // in each block: the leader's multicast commit
            mbar_init(&s.acc_empty[i], 8);      // used in the leader: the epilogue warps of both blocks
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {               // the same warp in both blocks: two accumulators of 256 columns
        tmem_alloc_pair(&s.tmem_base, 2 * TP_BN);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    cluster_sync_all();            // both blocks' barriers are initialised before anybody signals across
    tc_fence_after();
    const unsigned tmem = s.tmem_base;
    // Launched programmatically: what stands above (barriers, tensor memory) ran while the kernel before
    // still worked; nothing below reads or writes global memory before that kernel is complete.
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        // ---- producer (both blocks) ----
        if (elect_one()) {
            unsigned it = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
                const int m0 = (tile % m_blocks) * 2 * TP_BM + (int)rank * TP_BM;
                const int n0 = (tile / m_blocks) * TP_BN + (int)rank * (TP_BN / 2);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int st = it % TP_STAGES;
                    const unsigned phase = (it / TP_STAGES) & 1;
                    if (!mbar_wait(&s.empty[st], phase ^ 1)) { atomicExch(status, 22); ok = false; break; }
                    if (rank == 0) mbar_expect_tx(&s.full[st], 2 * STAGE_BYTES);
                    tma_load_2d_pair(s.a[st], &map_a, kb * TP_BK, m0, &s.full[st]);
                    tma_load_2d_pair(s.b[st], &map_w, kb * TP_BK, n0, &s.full[st]);
                }
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core issue (the leader block, for both) ----
        if (rank == 0 && elect_one()) {
            constexpr unsigned idesc = make_idesc(2 * TP_BM, TP_BN);
            unsigned it = 0, local = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++local) {
                const unsigned buf = local & 1;
                // the epilogues of both blocks must have drained this buffer (two tiles ago)
                if (!mbar_wait(&s.acc_empty[buf], ((local >> 1) & 1) ^ 1)) { atomicExch(status, 25); ok = false; break; }
                tc_fence_after();
                const unsigned acc = tmem + buf * TP_BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int st = it % TP_STAGES;
                    const unsigned phase = (it / TP_STAGES) & 1;
                    if (!mbar_wait(&s.full[st], phase)) { atomicExch(status, 23); ok = false; break; }
                    tc_fence_after();
                    const unsigned long long da = make_desc(smem_u32(s.a[st]));
                    const unsigned long long db = make_desc(smem_u32(s.b[st]));
#pragma unroll
                    for (int k = 0; k < TP_BK / 16; ++k)
                        umma_f16_pair(acc, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&s.empty[st]);           // the stage is free in both blocks
                }
                umma_commit_pair(&s.acc_full[buf]);            // arrives even after a failure, so the epilogues end
            }
        }
    } else {
        // ---- epilogue of this block's 128 rows: warp q may touch tensor-memory lanes 32q .. 32q+31 ----
        const int q = warp & 3;
        unsigned local = 0;
        for (int tile = pair; tile < n_tiles; tile += n_pairs, ++local) {
            const int m0 = (tile % m_blocks) * 2 * TP_BM + (int)rank * TP_BM, n0 = (tile / m_blocks) * TP_BN;
            const unsigned buf = local & 1;
            const bool ready = mbar_wait(&s.acc_full[buf], (local >> 1) & 1);
            if (!__all_sync(0xffffffffu, ready)) {
                if (lane == 0) atomicExch(status, 24);
                break;
            }
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const unsigned acc = tmem + buf * TP_BN + ((unsigned)(q * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < TP_BN; c += 32) {
                unsigned r[32];
                tmem_ld32(acc + (unsigned)c, r);
                tmem_ld_wait();
                const int col = n0 + c;
                if (row >= M || col >= N) continue;
                tc_store_32<EPI>(r, out, bias, row, col, N);
            }
            // this warp has read its lanes of the buffer: hand it back to the MMA thread in the leader
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&s.acc_empty[buf]);
        }
    }
    tc_fence_before();
    cluster_sync_all();            // nobody gives tensor memory back while the other block still reads or writes
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem, 2 * TP_BN);
    }
}

// ---- host side ------------------------------------------------------------------------------------------
// The pair kernel takes what the single-block kernel takes, and pays from 256 rows and 256 columns on.
GESSO_API int gesso_gemm_tcgen05_pair_takes(int M, int N, int K) {
    return M >= 256 && N >= 256 && N % 8 == 0 && K >= 8 && K % 8 == 0;
}

template <int EPI>
static int tp_launch(const CUtensorMap& ma, const CUtensorMap& mw, void* out, const float* bias, int M, int N, int K,
                     int* status, cudaStream_t stream) {
    const size_t smem = sizeof(TpSmem) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    const int tiles = ((N + TP_BN - 1) / TP_BN) * ((M + 2 * TP_BM - 1) / (2 * TP_BM));
    const int max_pairs = gesso_sm_count() / 2;            // one pair of blocks per two SMs
    const int pairs = tiles < max_pairs ? tiles : max_pairs;
    launch_pdl(gemm_tcgen05_pair_kernel<EPI>, dim3(2 * pairs), dim3(TP_THREADS), smem, stream, ma, mw, out, bias, M, N, K,
               status);
    return launch_status();
}

// A: bfloat16 [M,K]; W: bfloat16 [N,K]; out by `epi` as for gesso_gemm_tcgen05; status: one int, 0 unless a
// wait ran out.
GESSO_API int gesso_gemm_tcgen05_pair(const void* A, const void* W, void* out, const float* bias, int M, int N, int K,
                                      int epi, int* status, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (!gesso_gemm_tcgen05_pair_takes(M, N, K)) return GESSO_ERR_BAD_SIZE;
    if (epi == TC_EPI_SWIGLU && N % 16 != 0) return GESSO_ERR_BAD_SIZE;
    if (((size_t)A & 15) || ((size_t)W & 15) || ((size_t)out & 15)) return GESSO_ERR_BAD_SIZE;
    CUtensorMap ma, mw;
    int r = make_matrix_map(&ma, A, M, K, 128);
    if (r) return r;
    r = make_matrix_map(&mw, W, N, K, 128);
    if (r) return r;
    switch (epi) {
        case TC_EPI_BF16: return tp_launch<TC_EPI_BF16>(ma, mw, out, bias, M, N, K, status, stream);
        case TC_EPI_F32: return tp_launch<TC_EPI_F32>(ma, mw, out, bias, M, N, K, status, stream);
        case TC_EPI_RESID: return tp_launch<TC_EPI_RESID>(ma, mw, out, bias, M, N, K, status, stream);
        case TC_EPI_SWIGLU: return tp_launch<TC_EPI_SWIGLU>(ma, mw, out, bias, M, N, K, status, stream);
        default: return GESSO_ERR_UNSUPPORTED;
    }
}
