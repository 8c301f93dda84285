// Flash prefill attention on the 5th-generation tensor cores (bfloat16, head size 64, paged cache).
//
// A block owns up to 128 query rows: floor(128/G) consecutive tokens of one request times the G query
// heads of one kv group (G = 2 .. 16; where G does not divide 128 the last 128 - G floor(128/G) rows
// are zero and idle), so a single copy of K and V serves every head of the group (the GQA map
// h -> h / (nh/nkv) of src/Inference/Inference.jl:1398).  It walks the keys in blocks of 128:
//
//   TMA warps     one brings Q once (3-D tensor map [token][head][feature], 128-byte swizzle) and per key block
//                 the 8 K pages ([slot][feature] rows of 128 bytes, 128-byte swizzle), another the 8 V pages
//                 ([feature][slot] rows of 32 bytes, 32-byte swizzle), each into a two-stage ring with barriers
//                 of its own: a K stage is free again when its block's scores are computed, a V stage after
//                 O += P V, so the keys of block j + 2 are under way during the softmax of block j;
//   MMA thread    S[128 x 128] = Q K^T   (tcgen05.mma, M 128, N 128, K 4 x 16) into tensor memory, issued
//                 for block j+1 as soon as the softmax warps hold S of block j in registers;
//                 O[128 x 64] += P V     (A operand P read from tensor memory, B = one V page per K = 16
//                 step), accumulated in tensor memory over all blocks; the thread watches the barriers of
//                 both and issues whichever product is ready;
//   4 softmax warps  one thread per query row, all 128 scores of a block in registers (four tcgen05.ld, no
//                 second pass, no exchange between threads): mask, maximum, base-2 exponentials with
//                 log2(e)/sqrt(d) folded into one multiply-add, sum, P as packed bfloat16 back to tensor memory
//                 (tcgen05.st).  These warps hold 208 registers a thread: the four other warps of the block
//                 (two of them idle) give theirs up (setmaxnreg), so that two blocks still fit an SM.
// The running maximum is only raised when a block exceeds it by more than 8 (a factor 256, far inside
// the range of bfloat16 and float32): then the row of O in tensor memory and the running sum are scaled
// down, which after the first blocks is rare; the result O / l is the same function either way.
// Formulas: scores q.k/sqrt(d), query at position p reads keys max(0, p-window+1)..p, softmax, weighted
// sum of values (src/Inference/Inference.jl:1201-1207, 1414-1457).  All waits are bounded mbarrier
// waits that report through the status word (no block-wide barrier between the roles).  Two blocks fit
// an SM (80 KB of shared memory, 256 tensor-memory columns each), so one block's softmax overlaps the
// other's tensor work.
#include <math.h>

#include "tcgen05.cuh"
#include "tensor_map.cuh"

#define FA_HD 64
#define FA_BK 128
#define FA_STAGES 2
#define FA_THREADS 256                 // warps 0..3: softmax (one thread per query row), warp 4: TMA, warp 5: MMA, 6 and 7 idle
#define FA_REGS_SOFTMAX 208             // registers per softmax thread: the other warp group gives most of its own away
#define FA_REGS_OTHER 40
#define FA_LOG2E 1.4426950408889634f
#define FA_RAISE 8.f                   // the reference maximum follows the true one at this distance

struct __align__(1024) FaSmem {
    bf16 q[128 * FA_HD];                       // 16 KB
    bf16 k[FA_STAGES][FA_BK * FA_HD];          // 16 KB per stage: 8 pages x [16][64]
    bf16 v[FA_STAGES][FA_BK * FA_HD];          // 16 KB per stage: 8 pages x [64][16]
    unsigned long long q_full, k_full[FA_STAGES], k_empty[FA_STAGES], v_full[FA_STAGES], v_empty[FA_STAGES], s_full, s_free,
        p_ready, o_full;
    unsigned tmem_base;
};

__global__ void __launch_bounds__(FA_THREADS, 2)
prefill_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                                 int max_pages, int page_size, const int* __restrict__ seg_start,
                                 const int* __restrict__ seg_pos0, const int* __restrict__ tile_seg,
                                 const int* __restrict__ tile_q0, bf16* __restrict__ out, int nh, int nkv, int G,
                                 int window, float scale_log2, int num_pages, int* __restrict__ status) {
    extern __shared__ unsigned char fa_raw[];
    FaSmem& s = *reinterpret_cast<FaSmem*>(((size_t)fa_raw + 1023) & ~(size_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // launched programmatically: let the successor be set up, then wait for what earlier kernels wrote (every
    // block waits, also one with nothing to do, so that the chain of dependences stays whole)
    pdl_launch_dependents();
    pdl_wait();
    const int TOK = 128 / G;                      // tokens per block
    const int sub = (64 + TOK - 1) / TOK;         // blocks per 64-token tile of the step's tile list
    // Long tiles first: the queries at the end of a prompt have the most keys to read (up to 17 key blocks
    // at 2,048 tokens where the first tiles have one).  Blocks are handed out in the order of blockIdx.x, so
    // the kv heads of one tile are neighbours there and the tiles go from the longest to the shortest:
    // a greedy schedule by decreasing work, which ends nearly level on every SM.
    const int kvh = (int)(blockIdx.x % (unsigned)nkv);
    const int bx = (int)(gridDim.x / (unsigned)nkv) - 1 - (int)(blockIdx.x / (unsigned)nkv);
    const int tile = bx / sub;
    const int seg = tile_seg[tile];
    const int t0 = seg_start[seg], n = seg_start[seg + 1] - t0;
    const int q_in_tile = (bx % sub) * TOK;
    const int q0 = tile_q0[tile] + q_in_tile;
    if (q0 >= n) return;                          // nothing of this block lies inside the portion
    const int p0 = seg_pos0[seg];
    const int rows_tok = min(min(TOK, 64 - q_in_tile), n - q0);       // valid tokens of this block
    const int pos_first = p0 + q0, pos_last = p0 + q0 + rows_tok - 1;
    const int first_key = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int kb0 = first_key / FA_BK, kb1 = pos_last / FA_BK;         // key blocks kb0..kb1
    const int n_blocks = kb1 - kb0 + 1;
    const int* bt = block_table + (size_t)seg * max_pages;

    if (threadIdx.x == 0) {
        mbar_init(&s.q_full, 1);
        for (int i = 0; i < FA_STAGES; ++i) {
            mbar_init(&s.k_full[i], 1); mbar_init(&s.k_empty[i], 1);
            mbar_init(&s.v_full[i], 1); mbar_init(&s.v_empty[i], 1);
        }
        mbar_init(&s.s_full, 1);
        mbar_init(&s.s_free, 128);
        mbar_init(&s.p_ready, 128);
        mbar_init(&s.o_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 5) {       // S: columns 0..127, P: 128..191 (bfloat16 pairs), O: 192..255
        tmem_alloc(&s.tmem_base, 256);
        tmem_relinquish();
    }
    if (TOK * G < 128) {
        // the rows behind the last whole token are not written by the load of Q: zero them for the tensor cores
        // (rows are independent, so what they hold could not reach another row, but NaN patterns would wander
        // through these rows' softmax for nothing)
        for (int i = TOK * G * FA_HD + (int)threadIdx.x; i < 128 * FA_HD; i += FA_THREADS) s.q[i] = __float2bfloat16(0.f);
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = s.tmem_base;
    const unsigned tm_s = tmem, tm_p = tmem + 128, tm_o = tmem + 192;

    if (warp >= 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(FA_REGS_OTHER));
    }
    if (warp == 4 || warp == 6) {
        // ---- TMA producers: warp 4 brings Q and the K pages, warp 6 the V pages ----
        // The two rings have barriers of their own: a K stage is free again when the scores of its block are
        // computed, long before the block's V stage (free after O += P V), so the keys of block j + 2 are on
        // their way while block j is still in its softmax.
        // Lanes 0..7 each own one 16-key page of a block: they look their page up (one coalesced read of
        // the block table, one block ahead) and issue its TMA load themselves, so the eight lookups and
        // loads of a block go out side by side instead of one after the other.
        const bool keys = warp == 4;
        if (keys && lane == 0) {
            mbar_expect_tx(&s.q_full, TOK * G * FA_HD * sizeof(bf16));
            tma_load_3d(s.q, &map_q, 0, kvh * G, t0 + q0, &s.q_full);
        }
        // A page beyond the sequence or given back behind a window is wholly masked.  Its probabilities
        // are exact zeros, but 0 x NaN is NaN and such a page may hold anything, so nothing of it is
        // read: its loads start past the last row of the tensor map, where TMA fills in zeros.
        auto lookup = [&](int j) -> int {
            const int key0 = (kb0 + j) * FA_BK + lane * 16;
            return (lane < FA_BK / 16 && j < n_blocks && key0 <= pos_last) ? bt[key0 / page_size] : -1;
        };
        unsigned long long* full = keys ? s.k_full : s.v_full;
        unsigned long long* empty = keys ? s.k_empty : s.v_empty;
        int page = lookup(0);
        bool ok = true;
        for (int j = 0; j < n_blocks && ok; ++j) {
            const int st = j % FA_STAGES;
            const int next_page = lookup(j + 1);
            if (lane == 0) {
                if (!mbar_wait_idle(&empty[st], ((j / FA_STAGES) & 1) ^ 1)) { atomicExch(status, keys ? 12 : 11); ok = false; }
                else mbar_expect_tx(&full[st], FA_BK * FA_HD * sizeof(bf16));
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (ok && lane < FA_BK / 16) {
                const int sl = ((kb0 + j) * FA_BK + lane * 16) % page_size;
                const int pg = page < 0 ? num_pages : page;          // num_pages: the first row past the end
                if (keys) tma_load_2d(s.k[st] + lane * 16 * FA_HD, &map_k, 0, (pg * nkv + kvh) * page_size + sl, &full[st]);
                else tma_load_2d(s.v[st] + lane * 16 * FA_HD, &map_v, sl, (pg * nkv + kvh) * FA_HD, &full[st]);
            }
            page = next_page;
        }
    } else if (warp == 5) {
        // ---- tensor-core issue ----
        // One thread issues both kinds of product and takes whichever is ready: the scores of the next block
        // (its keys have landed, the softmax warps hold the scores before it in registers) or O += P V of the
        // oldest block whose probabilities are written and whose values have landed.  Neither waits for the other.
        if (elect_one()) {
            constexpr unsigned idesc_s = make_idesc(128, FA_BK);
            constexpr unsigned idesc_o = make_idesc(128, FA_HD);
            bool ok = mbar_wait_idle(&s.q_full, 0);
            if (!ok) atomicExch(status, 13);
            const unsigned long long dq = make_desc(smem_u32(s.q));
            unsigned long long dk[FA_STAGES], dv[FA_STAGES];
#pragma unroll
            for (int i = 0; i < FA_STAGES; ++i) {
                dk[i] = make_desc(smem_u32(s.k[i]));
                dv[i] = make_desc_sw32(smem_u32(s.v[i]));
            }
            int s_next = 0, pv_next = 0;             // the next block whose scores / whose P V is to be issued
            unsigned idle = 0;
            while (pv_next < n_blocks && ok) {
                bool progressed = false;
                if (s_next < n_blocks && mbar_test(&s.k_full[s_next % FA_STAGES], (s_next / FA_STAGES) & 1) &&
                    (s_next == 0 || mbar_test(&s.s_free, (s_next - 1) & 1))) {
                    tc_fence_after();
                    const unsigned long long d = dk[s_next % FA_STAGES];
#pragma unroll
                    for (int k = 0; k < FA_HD / 16; ++k) umma_f16(tm_s, dq + 2 * k, d + 2 * k, idesc_s, k > 0 ? 1u : 0u);
                    umma_commit(&s.s_full);
                    umma_commit(&s.k_empty[s_next % FA_STAGES]);      // the keys are free when the scores are done
                    ++s_next;
                    progressed = true;
                }
                if (pv_next < s_next && mbar_test(&s.p_ready, pv_next & 1) &&
                    mbar_test(&s.v_full[pv_next % FA_STAGES], (pv_next / FA_STAGES) & 1)) {
                    tc_fence_after();
                    const unsigned long long d = dv[pv_next % FA_STAGES];
#pragma unroll
                    for (int kk = 0; kk < FA_BK / 16; ++kk)          // one V page (16 keys x 64 features, 2 KB) per step
                        umma_f16_ts(tm_o, tm_p + 8 * kk, d + kk * (16 * FA_HD * (int)sizeof(bf16) / 16), idesc_o,
                                    (pv_next > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(&s.o_full);
                    umma_commit(&s.v_empty[pv_next % FA_STAGES]);
                    ++pv_next;
                    progressed = true;
                }
                if (progressed) idle = 0;
                else if (++idle > WAIT_LIMIT) { atomicExch(status, 14); ok = false; }
            }
        }
    } else if (warp < 4) {
        // ---- softmax: one thread per query row (warps 0..3: the four quarters of the tensor-memory lanes) ----
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(FA_REGS_SOFTMAX));
        const int r = warp * 32 + lane;                   // row = token * G + head
        const int tok = r / G, hg = r % G;
        const bool valid = tok < rows_tok;
        const int pos = p0 + q0 + min(tok, rows_tok - 1);
        const int lo = window > 0 ? max(0, pos - window + 1) : 0;
        const unsigned lane_base = (unsigned)(warp * 32) << 16;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        // a wait that ran out ends the whole warp: the tensor-memory loads and stores below are warp-wide
        auto wait_all = [&](void* bar, unsigned parity, int code) -> bool {
            const bool got = mbar_wait(bar, parity);
            if (__all_sync(0xffffffffu, got)) return true;
            if (lane == 0) atomicExch(status, code);
            return false;
        };
        for (int j = 0; j < n_blocks && ok; ++j) {
            const int key0 = (kb0 + j) * FA_BK;
            if (!wait_all(&s.s_full, j & 1, 16)) { ok = false; break; }
            tc_fence_after();
            unsigned v[FA_BK];
#pragma unroll
            for (int c = 0; c < FA_BK; c += 32) tmem_ld32(tm_s + lane_base + c, reinterpret_cast<unsigned(&)[32]>(v[c]));
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(&s.s_free);                       // S may be overwritten by the next block's scores
            // masking is a pass of its own behind a warp-wide branch: most blocks lie wholly inside the
            // visible range, and their inner loops then carry no compare at all
            if (__any_sync(0xffffffffu, key0 + FA_BK - 1 > pos || key0 < lo)) {
#pragma unroll
                for (int i = 0; i < FA_BK; ++i) {
                    const int key = key0 + i;
                    if (key > pos || key < lo) v[i] = 0xff800000u;      // -inf
                }
            }
            // four independent chains of three-input maxima: 64 instructions for 128 scores
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < FA_BK; i += 8) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    mx4[u] = max3(mx4[u], __uint_as_float(v[i + 2 * u]), __uint_as_float(v[i + 2 * u + 1]));
            }
            // rounded up to a whole number: every rescaling is then by an exact power of two, and the
            // rounding of a probability to bfloat16 does not depend on which reference it was taken against
            // (nor, therefore, on how a row's keys were cut into blocks and steps)
            const float m_blk = ceilf(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2);
            // O += P V of the block before has finished: P may be rewritten, O may be rescaled
            if (j > 0) {
                if (!wait_all(&s.o_full, (j - 1) & 1, 17)) { ok = false; break; }
                tc_fence_after();
            }
            // raise the reference maximum?  (the warp acts as one, rows that stay are scaled by 1)
            const bool raise = m_blk > m_ref + FA_RAISE;
            const float alpha = (raise && m_ref != -INFINITY) ? ex2_approx(m_ref - m_blk) : 1.f;
            if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
                for (int c = 0; c < FA_HD; c += 16) {     // seldom taken: keep its registers few
                    unsigned o[16];
                    tmem_ld16(tm_o + lane_base + c, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st16(tm_o + lane_base + c, o);
                }
            }
            l *= alpha;
            if (raise) m_ref = m_blk;
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            // score * scale - maximum and the running sums as packed pairs (one instruction for two values);
            // the exponentials one by one (the special-function unit has no packed form in float32); the
            // probabilities go back to tensor memory 32 at a time as packed bfloat16
            const unsigned long long scale2 = pack_f32x2(scale_log2, scale_log2), neg_m2 = pack_f32x2(-m_use, -m_use);
            unsigned long long l2[4] = {0ull, 0ull, 0ull, 0ull};      // four chains of pairs of partial sums
#pragma unroll
            for (int c = 0; c < FA_BK; c += 32) {
                unsigned pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float x0, x1;
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(v[c + i]), __uint_as_float(v[c + i + 1])), scale2, neg_m2),
                                 x0, x1);
                    const float e0 = ex2_approx(x0), e1 = ex2_approx(x1);
                    l2[(i >> 1) & 3] = add_f32x2(l2[(i >> 1) & 3], pack_f32x2(e0, e1));
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(e0, e1);
                    pk[i / 2] = *reinterpret_cast<unsigned*>(&b2);
                }
                tmem_st16(tm_p + lane_base + c / 2, pk);
            }
            {
                float a0, a1;
                unpack_f32x2(add_f32x2(add_f32x2(l2[0], l2[1]), add_f32x2(l2[2], l2[3])), a0, a1);
                l += a0 + a1;
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&s.p_ready);
        }
        if (ok) {
            // the last O += P V, and out = O / l
            if (!wait_all(&s.o_full, (n_blocks - 1) & 1, 17)) ok = false;
        }
        if (ok) {
            tc_fence_after();
            const float inv = 1.f / l;
            bf16* dst = out + ((size_t)(t0 + q0 + tok) * nh + (size_t)kvh * G + hg) * FA_HD;
#pragma unroll
            for (int c = 0; c < FA_HD; c += 32) {
                unsigned o[32];
                tmem_ld32(tm_o + lane_base + c, o);
                tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        unsigned w4[4];
#pragma unroll
                        for (int i = 0; i < 8; i += 2) {
                            __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(o[d + i]) * inv,
                                                                      __uint_as_float(o[d + i + 1]) * inv);
                            w4[i / 2] = *reinterpret_cast<unsigned*>(&b2);
                        }
                        *reinterpret_cast<uint4*>(dst + c + d) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, 256);
    }
}

// ---- host side ------------------------------------------------------------------------------------------
GESSO_API int gesso_attention_tcgen05_takes(int hd, int page_size, int nh, int nkv) {
    if (hd != FA_HD || page_size < 16 || page_size % 16 != 0 || nkv <= 0 || nh % nkv != 0) return 0;
    const int G = nh / nkv;
    return G >= 2 && G <= 16;
}

// q: bf16 [n_tokens, nh, 64]; k_pages bf16 [pages, nkv, page_size, 64]; v_pages bf16 [pages, nkv, 64, page_size];
// tile_seg / tile_q0: the step's 64-token tiles; out bf16 [n_tokens, nh*64].
GESSO_API int gesso_prefill_attention_tcgen05(const void* q, const void* k_pages, const void* v_pages, int num_pages,
                                              const int* block_table, int max_pages, int page_size,
                                              const int* seg_start, const int* seg_pos0, const int* tile_seg,
                                              const int* tile_q0, int n_tiles, int n_tokens, void* out, int nh, int nkv,
                                              int window, float scale, int* status, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (!gesso_attention_tcgen05_takes(FA_HD, page_size, nh, nkv)) return GESSO_ERR_BAD_SIZE;
    TensorMapEncodeFn fn = tensor_map_encoder();
    if (!fn) return GESSO_ERR_UNSUPPORTED;
    const int G = nh / nkv, TOK = 128 / G;
    CUtensorMap mq, mk, mv;
    {
        const cuuint64_t dims[3] = {FA_HD, (cuuint64_t)nh, (cuuint64_t)n_tokens};
        const cuuint64_t strides[2] = {FA_HD * sizeof(bf16), (cuuint64_t)nh * FA_HD * sizeof(bf16)};
        const cuuint32_t box[3] = {FA_HD, (cuuint32_t)G, (cuuint32_t)TOK};
        const cuuint32_t elem[3] = {1, 1, 1};
        if (fn(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return GESSO_ERR_UNSUPPORTED;
    }
    {
        const cuuint64_t dims[2] = {FA_HD, (cuuint64_t)num_pages * nkv * page_size};
        const cuuint64_t strides[1] = {FA_HD * sizeof(bf16)};
        const cuuint32_t box[2] = {FA_HD, 16};
        const cuuint32_t elem[2] = {1, 1};
        if (fn(&mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(k_pages), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return GESSO_ERR_UNSUPPORTED;
    }
    {
        const cuuint64_t dims[2] = {(cuuint64_t)page_size, (cuuint64_t)num_pages * nkv * FA_HD};
        const cuuint64_t strides[1] = {(cuuint64_t)page_size * sizeof(bf16)};
        const cuuint32_t box[2] = {16, FA_HD};
        const cuuint32_t elem[2] = {1, 1};
        if (fn(&mv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(v_pages), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return GESSO_ERR_UNSUPPORTED;
    }
    const size_t smem = sizeof(FaSmem) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(prefill_attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    const int sub = (64 + TOK - 1) / TOK;
    if ((long long)n_tiles * sub * nkv > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    const dim3 grid((unsigned)(n_tiles * sub * nkv));
    launch_pdl(prefill_attention_tcgen05_kernel, grid, dim3(FA_THREADS), smem, stream,
        mq, mk, mv, block_table, max_pages, page_size, seg_start, seg_pos0, tile_seg, tile_q0, (bf16*)out, nh, nkv, G,
        window, scale * FA_LOG2E, num_pages, status);
    return launch_status();
}
