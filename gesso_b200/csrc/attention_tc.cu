// Tensor-core paged attention for bfloat16: a split-KV kernel for steps of single tokens and a
// flash kernel for steps with prompt portions.  Head sizes 32, 64, 96, 128; page sizes that are
// multiples of 16.  Other sizes are refused (the caller then takes the FP32-arithmetic kernel).
//
// Both kernels take K and V fragments from the cache pages as they lie, with no transposition (the
// decode kernel through a per-thread ring of asynchronous copies, the prefill kernel straight into
// registers):
//   * scores S = Q K^T use mma.m16n8k16 with K as the B operand: b(k = feature, n = key) is two
//     consecutive features of one K row, so a thread reads 16 contiguous bytes of a K row and
//     uses them for two k16 steps.  The sum over features is order-free, so features are assigned
//     to fragment slots as the loads deliver them (thread t of a quad holds features 8t..8t+7 of
//     each 32-feature chunk), and Q's A fragment uses the same assignment.
//   * outputs O = P V use V as the B operand: b(k = key, n = feature) is two consecutive keys of
//     one feature, contiguous because V pages are stored [feature][slot].  The 16 keys of a block
//     are assigned to the two 8-key score tiles so that a thread's four probabilities are keys
//     4t..4t+3, which is one 8-byte read of a V^T row.
// Softmax statistics and the output accumulate in float32 with a running maximum (base-2
// exponentials with the 1/sqrt(d) scale folded in; the maximum is rounded up to a whole number, see
// attend_block).  Reference design inputs: the split-K decode
// kernels of ext/cuda_attention.jl:421-550 (block = kv head x key chunk, all query heads of the
// group from one read, LSE combine); formulas as src/Inference/Inference.jl:1201-1207, 1398,
// 1414-1457.
#include <math.h>

#include "common.cuh"

#define LOG2E 1.4426950408889634f

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// K and V fragments of one 16-key block for one kv head.
template <int HD>
struct KVFrag {
    uint4 k[2][HD / 32];     // [score tile][32-feature chunk]
    uint2 v[HD / 8];         // [8-feature tile]
};

template <int HD>
__device__ __forceinline__ void load_block(KVFrag<HD>& f, const bf16* __restrict__ k_pages,
                                           const bf16* __restrict__ v_pages, const int* __restrict__ bt,
                                           int block, int page_size, int nkv, int kvh, int g, int t) {
    const int key0 = block * 16;
    const int page = bt[key0 / page_size];
    const int sub = key0 % page_size;
    if (page < 0) {   // a page that was given back (behind a window): masked anyway, read nothing
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) f.k[0][c] = f.k[1][c] = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) f.v[j] = make_uint2(0, 0);
        return;
    }
    const size_t pk = ((size_t)page * nkv + kvh);
    // score tile 0 column g is key 4(g/2) + g%2, tile 1 column g is key 4(g/2) + 2 + g%2
    const int key_a = 4 * (g >> 1) + (g & 1);
    const bf16* ka = k_pages + (pk * page_size + sub + key_a) * HD + 8 * t;
    const bf16* kb = ka + 2 * HD;
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) {
        f.k[0][c] = *reinterpret_cast<const uint4*>(ka + 32 * c);
        f.k[1][c] = *reinterpret_cast<const uint4*>(kb + 32 * c);
    }
    const bf16* vt = v_pages + (pk * HD + g) * page_size + sub + 4 * t;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) f.v[j] = *reinterpret_cast<const uint2*>(vt + (size_t)(8 * j) * page_size);
}

// One 16-key block against one m16 tile of queries: scores, running softmax, outputs.
// qf[c] / qg[c]: Q rows g and g+8, features 32c+8t..+8.  pos_a / pos_b: last visible key of rows g
// and g+8; lo_a / lo_b: first visible key.  key0: first key of the block.
// UPPER = false: rows 8..15 of the tile carry no query (a decoding step with at most 8 query heads per kv
// head): their scores are not looked at, their probabilities are zero and their outputs are never read.
template <int HD, bool UPPER = true>
__device__ __forceinline__ void attend_block(const KVFrag<HD>& f, const uint4 (&qf)[HD / 32],
                                             const uint4 (&qg)[HD / 32], float (&o)[HD / 8][4], float (&m)[2],
                                             float (&l)[2], int key0, int t, int pos_a, int pos_b, int lo_a,
                                             int lo_b, float scale_log2, bool need_mask) {
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) {
        mma_bf16(s0, qf[c].x, qg[c].x, qf[c].y, qg[c].y, f.k[0][c].x, f.k[0][c].y);
        mma_bf16(s0, qf[c].z, qg[c].z, qf[c].w, qg[c].w, f.k[0][c].z, f.k[0][c].w);
        mma_bf16(s1, qf[c].x, qg[c].x, qf[c].y, qg[c].y, f.k[1][c].x, f.k[1][c].y);
        mma_bf16(s1, qf[c].z, qg[c].z, qf[c].w, qg[c].w, f.k[1][c].z, f.k[1][c].w);
    }
    // this thread's keys: key0 + 4t + {0,1} (tile 0) and + {2,3} (tile 1); rows g (idx 0,1) and g+8 (2,3)
    float sa[4] = {s0[0], s0[1], s1[0], s1[1]};
    float sb[4] = {s0[2], s0[3], s1[2], s1[3]};
    const int kbase = key0 + 4 * t;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        sa[i] *= scale_log2;
        if (UPPER) sb[i] *= scale_log2;
        if (need_mask) {
            const int key = kbase + i;
            if (key > pos_a || key < lo_a) sa[i] = -INFINITY;
            if (UPPER && (key > pos_b || key < lo_b)) sb[i] = -INFINITY;
        }
    }
    // The running maximum is kept as a whole number (scores are in the base-2 domain): rescaling by
    // 2^(old - new) is then exact, and a probability rounded to bfloat16 against one whole number is the
    // probability rounded against another times an exact power of two.  So what a row's keys add up to does
    // not depend on the order of the blocks, on the warps and splits that share them, or on how the
    // maximum grew on the way: only on the row's final maximum.
    const float ma = ceilf(quad_max(fmaxf(fmaxf(sa[0], sa[1]), fmaxf(sa[2], sa[3]))));
    const float na = fmaxf(m[0], ma);
    const float ua = na == -INFINITY ? 0.f : na;                                      // all masked so far
    const float alpha_a = exp2f(m[0] - ua);
    m[0] = na;
    float pa[4], pb[4] = {0.f, 0.f, 0.f, 0.f};
    float la = 0.f, lb = 0.f, alpha_b = 1.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        pa[i] = exp2f(sa[i] - ua);
        la += pa[i];
    }
    l[0] = l[0] * alpha_a + la;
    if (UPPER) {
        const float mb = ceilf(quad_max(fmaxf(fmaxf(sb[0], sb[1]), fmaxf(sb[2], sb[3]))));
        const float nb = fmaxf(m[1], mb);
        const float ub = nb == -INFINITY ? 0.f : nb;
        alpha_b = exp2f(m[1] - ub);
        m[1] = nb;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            pb[i] = exp2f(sb[i] - ub);
            lb += pb[i];
        }
        l[1] = l[1] * alpha_b + lb;
    }
    const unsigned a0 = pack_bf16(pa[0], pa[1]), a1 = UPPER ? pack_bf16(pb[0], pb[1]) : 0u;
    const unsigned a2 = pack_bf16(pa[2], pa[3]), a3 = UPPER ? pack_bf16(pb[2], pb[3]) : 0u;
    // the running maximum seldom moves after the first blocks: rescale only when some row's did
    const bool rescale = __any_sync(0xffffffffu, alpha_a != 1.f || alpha_b != 1.f);
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) {
        if (rescale) {
            o[j][0] *= alpha_a;
            o[j][1] *= alpha_a;
            if (UPPER) {
                o[j][2] *= alpha_b;
                o[j][3] *= alpha_b;
            }
        }
        mma_bf16(o[j], a0, a1, a2, a3, f.v[j].x, f.v[j].y);
    }
}

// ================================ decode: split-KV ==============================================
// grid (nkv, segments, splits), 128 threads; a step of single tokens (token i is segment i).  The
// m16 rows are the query heads of the kv group (up to 16).  Every warp walks its share of the
// split's 16-key blocks; the warps are merged in shared memory; with more than one split the
// partial (m, l, O) goes to the workspace and the last split to arrive merges them (a ticket per
// (segment, kv head), reset for the next launch).
//
// How many of the grid's splits a request uses is decided per step from two numbers the host packs
// beside the positions (the longest sequence and the average one): few requests are cut so that one
// wave of blocks fills the device, as many pieces each as that takes; and where the lengths are
// uneven (the longest more than 1.5 times the average) no piece is longer than the average request,
// so that a long request among short ones does not run alone at the end.  Pieces are never shorter
// than DA_MIN_PER key blocks.  The splits a request does not use leave at once; they are the last
// in launch order.  Without the two numbers every request uses every split.
//
// The kernel is bound by the stream of K and V, so that stream is kept deep and started early:
// every thread copies the fragments it will need (64 bytes of K rows, 64 bytes of V^T rows per block
// at head size 64) asynchronously into a private ring in shared memory, DA_STAGES blocks ahead; the
// page ids of a warp's blocks are fetched by its lanes in one go, so no lookup sits in the chain;
// and everything but the block that holds the step's own token is requested before the wait for
// the preceding kernels (which write that token's K and V and the queries), so the first keys are
// on their way while those still run.
#define DA_STAGES_DEEP 6          // few blocks (small batches): a deep ring per warp, two blocks per SM
#define DA_STAGES_WIDE 3          // many blocks: four blocks per SM hide each other's latencies instead
#define DA_MIN_PER 16             // key blocks (256 keys): finer pieces cost more in set-up and merge than they win

__device__ __forceinline__ void cp_async_zfill16(void* smem_dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(valid ? 16 : 0));
}
__device__ __forceinline__ void cp_async_zfill8(void* smem_dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(d), "l"(src), "r"(valid ? 8 : 0));
}

template <int HD, int DA_STAGES, bool UPPER>
__global__ void __launch_bounds__(128)
decode_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages,
                        const bf16* __restrict__ v_pages, const int* __restrict__ block_table, int max_pages,
                        int page_size, int page_shift, const int* __restrict__ positions,
                        bf16* __restrict__ out, int nh, int nkv, int window, float scale_log2, int n_splits,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ tickets,
                        const int* __restrict__ kv_span, int slots) {
    // ring: [stage][piece][128 threads]: HD/16 pieces of 16 bytes for K, then HD/8 pieces of 8 bytes for V;
    // afterwards the same memory serves the merge of the warps ([4 warps][16 rows][HD + 2] floats)
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* smem = reinterpret_cast<float*>(smem_raw);
    __shared__ int s_last;
    constexpr int KP = HD / 16, VP = HD / 8;
    constexpr int STAGE_BYTES = (KP * 16 + VP * 8) * 128;
    const int kvh = blockIdx.x, seg = blockIdx.y, split = blockIdx.z;
    const int G = nh / nkv;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int tok = seg;                     // a step of single tokens
    const int pos = positions[tok];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* bt = block_table + (size_t)seg * max_pages;

    const int first_block = lo / 16, last_block = pos / 16;
    const int n_blocks = last_block - first_block + 1;
    int used = n_splits;                     // pieces this request is cut into
    if (n_splits > 1 && kv_span != nullptr) {
        const int n_segs = (int)gridDim.y;
        int longest = kv_span[0], average = kv_span[1];
        if (window > 0) {
            longest = min(longest, window);
            average = min(average, window);
        }
        const int long_b = (longest + 15) / 16;
        const int avg_b = max(1, average / 16);
        const int base = n_segs * nkv;
        int chunk = 0x7fffffff;
        if (5 * base <= 4 * slots) {         // the requests' own blocks leave room in one wave: fill it
            const long long work = (long long)(avg_b + 1) * n_segs * nkv;
            chunk = max(DA_MIN_PER, (int)((work + slots - base - 1) / (slots - base)));
        }
        if (2 * long_b > 3 * avg_b) chunk = min(chunk, max(DA_MIN_PER, avg_b));
        used = chunk == 0x7fffffff ? 1 : min(n_splits, max(1, (n_blocks + chunk - 1) / chunk));
    }
    if (split >= used) {                     // a piece this request does not need
        pdl_launch_dependents();
        return;
    }
    const int per = (n_blocks + used - 1) / used;
    const int b0 = first_block + split * per;
    const int b1 = min(last_block + 1, b0 + per);
    const int mine_n = b0 + w < b1 ? (b1 - b0 - w + 3) / 4 : 0;      // blocks b0 + w + 4 i of this warp

    // page ids of this warp's blocks, 32 at a time: lane i holds the page of block i of the batch
    // (page_shift >= 0: the page size is that power of two, and no division is needed)
    int pages = 0;
    auto fetch_pages = [&](int first_i) {
        const int i = first_i + lane;
        const int key = (b0 + w + 4 * i) * 16;
        pages = i < mine_n ? bt[page_shift >= 0 ? key >> page_shift : key / page_size] : -1;
    };
    fetch_pages(0);

    unsigned char* ring = smem_raw;
    const int key_a = 4 * (g >> 1) + (g & 1);
    // what does not change from block to block is added up once: this thread's place inside a page of its kv
    // head, for K ([slot][feature]) and for V ([feature][slot]); a page is page_elems elements of either
    const size_t page_elems = (size_t)nkv * page_size * HD;
    const bf16* k_mine = k_pages + ((size_t)kvh * page_size + key_a) * HD + 8 * t;
    const bf16* v_mine = v_pages + ((size_t)kvh * HD + g) * page_size + 4 * t;
    unsigned char* ring_mine_k = ring + (size_t)threadIdx.x * 16;
    unsigned char* ring_mine_v = ring + (size_t)KP * 16 * 128 + (size_t)threadIdx.x * 8;
    int issued = 0, issue_stage = 0;
    auto issue = [&]() {                     // request block `issued` of this warp into its ring stage
        if (issued < mine_n) {
            const int key0 = (b0 + w + 4 * issued) * 16;
            const int page = __shfl_sync(0xffffffffu, pages, issued & 31);
            const bool valid = page >= 0;    // a page given back behind a window: masked, zero-filled
            const int sub = page_shift >= 0 ? key0 & (page_size - 1) : key0 % page_size;
            const size_t at = (size_t)(valid ? page : 0) * page_elems;
            const int stage_off = issue_stage * STAGE_BYTES;
            const bf16* ka = k_mine + at + sub * HD;
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                cp_async_zfill16(ring_mine_k + stage_off + (2 * c) * 128 * 16, ka + 32 * c, valid);
                cp_async_zfill16(ring_mine_k + stage_off + (2 * c + 1) * 128 * 16, ka + 2 * HD + 32 * c, valid);
            }
            const bf16* vt = v_mine + at + sub;
#pragma unroll
            for (int j = 0; j < VP; ++j)
                cp_async_zfill8(ring_mine_v + stage_off + j * 128 * 8, vt + (size_t)(8 * j) * page_size, valid);
            ++issued;
            if (++issue_stage == DA_STAGES) issue_stage = 0;
            if ((issued & 31) == 0) fetch_pages(issued);
        }
        asm volatile("cp.async.commit_group;\n" ::);      // an empty group keeps the count in step
    };
    // before the wait: everything but the block of the step's own token
    int early = 0;
#pragma unroll 1
    for (; early < DA_STAGES; ++early) {
        if (issued < mine_n && b0 + w + 4 * issued == last_block) break;
        issue();
    }
    // let the successor in first (it only prefetches what no running kernel writes until its own wait)
    pdl_launch_dependents();
    pdl_wait();
#pragma unroll 1
    for (; early < DA_STAGES; ++early) issue();

    // Q fragments: row g is head kvh*G + g (zero rows beyond the group)
    uint4 qf[HD / 32], qg[HD / 32];
    {
        const bf16* qa = q + ((size_t)tok * nh + (size_t)kvh * G + g) * HD + 8 * t;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
            qf[c] = g < G ? *reinterpret_cast<const uint4*>(qa + 32 * c) : make_uint4(0, 0, 0, 0);
            qg[c] = (UPPER && g + 8 < G) ? *reinterpret_cast<const uint4*>(qa + 8 * HD + 32 * c) : make_uint4(0, 0, 0, 0);
        }
    }

    float o[HD / 8][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

    int read_stage = 0;
#pragma unroll 1
    for (int i = 0; i < mine_n; ++i) {
        const int b = b0 + w + 4 * i;
        asm volatile("cp.async.wait_group %0;\n" ::"n"(DA_STAGES - 1));
        const int stage_off = read_stage * STAGE_BYTES;
        if (++read_stage == DA_STAGES) read_stage = 0;
        KVFrag<HD> cur;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
            cur.k[0][c] = *reinterpret_cast<const uint4*>(ring_mine_k + stage_off + (2 * c) * 128 * 16);
            cur.k[1][c] = *reinterpret_cast<const uint4*>(ring_mine_k + stage_off + (2 * c + 1) * 128 * 16);
        }
#pragma unroll
        for (int j = 0; j < VP; ++j) cur.v[j] = *reinterpret_cast<const uint2*>(ring_mine_v + stage_off + j * 128 * 8);
        issue();                                          // refill the stage just read
        const bool need_mask = (b * 16 + 15 > pos) || (b * 16 < lo);
        attend_block<HD, UPPER>(cur, qf, qg, o, m, l, b * 16, t, pos, pos, lo, lo, scale_log2, need_mask);
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();                                      // the ring is free: it becomes the merge buffer
    l[0] = quad_sum(l[0]);
    l[1] = quad_sum(l[1]);

    // ---- merge the four warps ----
    float* mine = smem + (size_t)w * 16 * (HD + 2);
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) {
        mine[g * (HD + 2) + 8 * j + 2 * t] = o[j][0];
        mine[g * (HD + 2) + 8 * j + 2 * t + 1] = o[j][1];
        mine[(g + 8) * (HD + 2) + 8 * j + 2 * t] = o[j][2];
        mine[(g + 8) * (HD + 2) + 8 * j + 2 * t + 1] = o[j][3];
    }
    if (t == 0) {
        mine[g * (HD + 2) + HD] = m[0];
        mine[g * (HD + 2) + HD + 1] = l[0];
        mine[(g + 8) * (HD + 2) + HD] = m[1];
        mine[(g + 8) * (HD + 2) + HD + 1] = l[1];
    }
    __syncthreads();
    // thread -> (head row r, feature d): G*HD outputs
    for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
        const int r = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int ww = 0; ww < 4; ++ww) M = fmaxf(M, smem[((size_t)ww * 16 + r) * (HD + 2) + HD]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int ww = 0; ww < 4; ++ww) {
            const float* row = smem + ((size_t)ww * 16 + r) * (HD + 2);
            const float f = row[HD] == -INFINITY ? 0.f : exp2f(row[HD] - M);
            L += row[HD + 1] * f;
            acc += row[d] * f;
        }
        const int head = kvh * G + r;
        if (used == 1) {
            out[((size_t)tok * nh + head) * HD + d] = __float2bfloat16_rn(acc / L);
        } else {
            const size_t pi = ((size_t)seg * nh + head) * n_splits + split;
            part_o[pi * HD + d] = acc;
            if (d == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
        }
    }
    if (used == 1) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int ticket = atomicAdd(&tickets[seg * nkv + kvh], 1);
        s_last = ticket == used - 1;
        if (s_last) tickets[seg * nkv + kvh] = 0;     // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
        const int r = idx / HD, d = idx % HD;
        const int head = kvh * G + r;
        const size_t p0 = ((size_t)seg * nh + head) * n_splits;
        float M = -INFINITY;
#pragma unroll 8
        for (int s = 0; s < used; ++s) M = fmaxf(M, __ldcg(part_ml + (p0 + s) * 2));
        float L = 0.f, acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < used; ++s) {
            const float ms = __ldcg(part_ml + (p0 + s) * 2);
            const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
            L += __ldcg(part_ml + (p0 + s) * 2 + 1) * f;
            acc += __ldcg(part_o + (p0 + s) * HD + d) * f;
        }
        out[((size_t)tok * nh + head) * HD + d] = __float2bfloat16_rn(acc / L);
    }
}

// ================================ prefill: flash ================================================
// grid (64-token tiles, nkv, G / HPW), 128 threads.  A warp owns 16 consecutive tokens of one
// request and HPW query heads of one kv group; it walks the 16-key blocks up to its last row's
// position.  tile_seg / tile_q0 list the tiles (a tile never crosses a request).
template <int HD, int HPW>
__global__ void __launch_bounds__(128)
prefill_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages,
                         const bf16* __restrict__ v_pages, const int* __restrict__ block_table, int max_pages,
                         int page_size, const int* __restrict__ seg_start, const int* __restrict__ seg_pos0,
                         const int* __restrict__ tile_seg, const int* __restrict__ tile_q0,
                         bf16* __restrict__ out, int nh, int nkv, int window, float scale_log2) {
    // Long tiles first: the queries at the end of a prompt have the most keys to read.  Blocks are handed
    // out in the order of blockIdx.x: the (kv head, head pair) blocks of one tile are neighbours there and
    // the tiles go from the longest to the shortest, a greedy schedule by decreasing work.
    const int G = nh / nkv;
    const unsigned per_tile = (unsigned)nkv * (unsigned)(G / HPW);
    const int tile = (int)(gridDim.x / per_tile) - 1 - (int)(blockIdx.x / per_tile);
    const int kvh = (int)((blockIdx.x % per_tile) / (unsigned)(G / HPW));
    const int hpair = (int)(blockIdx.x % (unsigned)(G / HPW));
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int seg = tile_seg[tile];
    const int t0 = seg_start[seg], n = seg_start[seg + 1] - t0;
    const int q0 = tile_q0[tile] + 16 * w;          // first row of this warp inside the request's portion
    if (q0 >= n) return;
    const int rows = min(16, n - q0);
    const int p0 = seg_pos0[seg];
    // rows beyond the portion repeat its last row (computed, never stored)
    const int ra = min(g, rows - 1), rb = min(g + 8, rows - 1);
    const int pos_a = p0 + q0 + ra, pos_b = p0 + q0 + rb;
    const int lo_a = window > 0 ? max(0, pos_a - window + 1) : 0;
    const int lo_b = window > 0 ? max(0, pos_b - window + 1) : 0;
    const int pos_first = p0 + q0, pos_last = p0 + q0 + rows - 1;
    const int first_block = (window > 0 ? max(0, pos_first - window + 1) : 0) / 16;
    const int last_block = pos_last / 16;
    const int* bt = block_table + (size_t)seg * max_pages;
    const int head0 = kvh * G + hpair * HPW;

    uint4 qf[HPW][HD / 32], qg[HPW][HD / 32];
    float o[HPW][HD / 8][4], m[HPW][2], l[HPW][2];
#pragma unroll
    for (int h = 0; h < HPW; ++h) {
        const bf16* qa = q + ((size_t)(t0 + q0 + ra) * nh + head0 + h) * HD + 8 * t;
        const bf16* qb = q + ((size_t)(t0 + q0 + rb) * nh + head0 + h) * HD + 8 * t;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
            qf[h][c] = *reinterpret_cast<const uint4*>(qa + 32 * c);
            qg[h][c] = *reinterpret_cast<const uint4*>(qb + 32 * c);
        }
        m[h][0] = m[h][1] = -INFINITY;
        l[h][0] = l[h][1] = 0.f;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) o[h][j][0] = o[h][j][1] = o[h][j][2] = o[h][j][3] = 0.f;
    }
    KVFrag<HD> cur, nxt;
    load_block<HD>(cur, k_pages, v_pages, bt, first_block, page_size, nkv, kvh, g, t);
    for (int b = first_block; b <= last_block; ++b) {
        const bool more = b < last_block;
        if (more) load_block<HD>(nxt, k_pages, v_pages, bt, b + 1, page_size, nkv, kvh, g, t);
        // a block needs masking if some row cannot see its last key, or a window cuts into it
        const bool need_mask = (b * 16 + 15 > pos_first) || (window > 0 && b * 16 < max(lo_a, lo_b));
#pragma unroll
        for (int h = 0; h < HPW; ++h)
            attend_block<HD>(cur, qf[h], qg[h], o[h], m[h], l[h], b * 16, t, pos_a, pos_b, lo_a, lo_b, scale_log2,
                             need_mask);
        if (more) cur = nxt;
    }
#pragma unroll
    for (int h = 0; h < HPW; ++h) {
        const float la = quad_sum(l[h][0]), lb = quad_sum(l[h][1]);
        const float ia = 1.f / la, ib = 1.f / lb;
        bf16* oa = out + ((size_t)(t0 + q0 + g) * nh + head0 + h) * HD + 2 * t;
        bf16* ob = out + ((size_t)(t0 + q0 + g + 8) * nh + head0 + h) * HD + 2 * t;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) {
            if (g < rows)
                *reinterpret_cast<__nv_bfloat162*>(oa + 8 * j) = __floats2bfloat162_rn(o[h][j][0] * ia, o[h][j][1] * ia);
            if (g + 8 < rows)
                *reinterpret_cast<__nv_bfloat162*>(ob + 8 * j) = __floats2bfloat162_rn(o[h][j][2] * ib, o[h][j][3] * ib);
        }
    }
}

// ---- launchers -------------------------------------------------------------------------------------
GESSO_API int gesso_attention_tc_takes(int hd, int page_size, int nh, int nkv) {
    if (!(hd == 32 || hd == 64 || hd == 96 || hd == 128)) return 0;
    if (page_size <= 0 || page_size % 16 != 0) return 0;
    if (nkv <= 0 || nh % nkv != 0) return 0;
    return 1;
}

// Workspace sizes (in elements) of the split-KV kernel for `segs` single-token requests.
GESSO_API long long gesso_decode_attention_workspace(int segs, int nh, int nkv, int hd, int n_splits,
                                                     long long* part_ml_floats, long long* ticket_ints) {
    *part_ml_floats = (long long)segs * nh * n_splits * 2;
    *ticket_ints = (long long)segs * nkv;
    return (long long)segs * nh * n_splits * hd;
}

GESSO_API int gesso_decode_attention(const void* q, const void* k_pages, const void* v_pages,
                                     const int* block_table, int max_pages, int page_size, const int* positions,
                                     void* out, int n_segs, int nh, int nkv, int hd,
                                     int window, float scale, int n_splits, float* part_o, float* part_ml,
                                     int* tickets, const int* kv_span, cudaStream_t stream) {
    if (n_segs <= 0) return 0;
    if (!gesso_attention_tc_takes(hd, page_size, nh, nkv)) return GESSO_ERR_BAD_SIZE;
    const int G = nh / nkv;
    if (G > 16 || n_splits < 1 || n_splits > 65535 || n_segs > 65535 || nkv > 65535) return GESSO_ERR_BAD_SIZE;
    if (n_splits > 1 && (!part_o || !part_ml || !tickets)) return GESSO_ERR_BAD_SIZE;
    dim3 grid(nkv, n_segs, n_splits);
    int page_shift = -1;
    if ((page_size & (page_size - 1)) == 0)
        for (page_shift = 0; (1 << page_shift) < page_size; ++page_shift) {}
    // Few blocks: two per SM with a deep ring each (a block must cover the memory latency by itself).  Many
    // blocks (large batches): four per SM with a shallow ring each; the same bytes are in flight, and twice
    // the warps keep the issue slots busy where one warp's chain of dependent instructions would not.
    // (counted by the pieces that a step of even lengths uses: at most what two blocks per SM hold at once)
    const long long base = (long long)nkv * n_segs;
    const long long even = kv_span ? (2LL * gesso_sm_count() / base < 1 ? 1 : 2LL * gesso_sm_count() / base) : n_splits;
    const long long blocks = base * (even < n_splits ? even : n_splits);
    const bool wide = blocks >= 3LL * gesso_sm_count();
    const int slots = (wide ? 4 : 2) * gesso_sm_count();
    const int stages = wide ? DA_STAGES_WIDE : DA_STAGES_DEEP;
    const size_t merge = (size_t)4 * 16 * (hd + 2) * sizeof(float);
    const size_t ring = (size_t)stages * (hd / 16 * 16 + hd / 8 * 8) * 128;
    const size_t smem = ring > merge ? ring : merge;
    const float scale_log2 = scale * LOG2E;
#define GO3(HD, ST, UP)                                                                                     \
    do {                                                                                                    \
        static bool configured = false;   /* once per instantiation, outside any stream capture */          \
        if (!configured) {                                                                                  \
            cudaFuncSetAttribute(decode_attention_kernel<HD, ST, UP>,                                       \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                   \
            configured = true;                                                                              \
        }                                                                                                   \
        launch_pdl(decode_attention_kernel<HD, ST, UP>, grid, dim3(128), smem, stream,                      \
            (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, block_table, max_pages, page_size,  \
            page_shift, positions, (bf16*)out, nh, nkv, window, scale_log2, n_splits, part_o, part_ml,      \
            tickets, kv_span, slots);                                                                       \
    } while (0)
#define GO(HD)                                                                                              \
    do {                                                                                                    \
        if (wide) { if (G > 8) GO3(HD, DA_STAGES_WIDE, true); else GO3(HD, DA_STAGES_WIDE, false); }        \
        else { if (G > 8) GO3(HD, DA_STAGES_DEEP, true); else GO3(HD, DA_STAGES_DEEP, false); }             \
    } while (0)
    if (hd == 32) GO(32);
    else if (hd == 64) GO(64);
    else if (hd == 96) GO(96);
    else GO(128);
#undef GO
#undef GO3
    return launch_status();
}

GESSO_API int gesso_prefill_attention(const void* q, const void* k_pages, const void* v_pages,
                                      const int* block_table, int max_pages, int page_size, const int* seg_start,
                                      const int* seg_pos0, const int* tile_seg, const int* tile_q0, int n_tiles,
                                      void* out, int nh, int nkv, int hd, int window, float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (!gesso_attention_tc_takes(hd, page_size, nh, nkv)) return GESSO_ERR_BAD_SIZE;
    const int G = nh / nkv;
    if ((long long)n_tiles * nh > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    const float scale_log2 = scale * LOG2E;
#define GO(HD, HPW)                                                                                          \
    prefill_attention_kernel<HD, HPW><<<dim3((unsigned)(n_tiles * nkv * (G / HPW))), 128, 0, stream>>>(      \
        (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, block_table, max_pages, page_size,       \
        seg_start, seg_pos0, tile_seg, tile_q0, (bf16*)out, nh, nkv, window, scale_log2)
    if (hd <= 64 && G % 2 == 0) {
        if (hd == 32) GO(32, 2); else GO(64, 2);
    } else {
        if (hd == 32) GO(32, 1); else if (hd == 64) GO(64, 1); else if (hd == 96) GO(96, 1); else GO(128, 1);
    }
#undef GO
    return launch_status();
}
