// Token selection on the device: greedy argmax and temperature / nucleus sampling.
//
// Greedy: argmax with ties going to the lowest id; a non-finite logit anywhere in the row is
// reported through `nonfinite[row]` and no token may be emitted for it
// (src/Inference/session.jl:447-458).
//
// Sampling follows the reference's sampler (src/Inference/sampling.jl:43-74): weights
// w_i = exp((logit_i - max) / T) in float64; with top_p = 1 the draw walks the ids in order and
// returns the first id whose running sum exceeds r = u * total; with top_p < 1 the smallest set of
// most likely ids (ties: lower id first) whose mass reaches top_p * total is kept, and the walk
// runs over that set in descending order of weight.  The uniform u (one per row per call) comes
// from the host's splitmix64 stream of the request, so a request's tokens do not depend on the
// batch it is in.  No sort is needed: the kept set and the drawn id are both "first position in
// descending order at which the running mass crosses a target", which is found by narrowing the
// 64-bit pattern of the weight eight bits at a time (positive doubles order like their bits).  The
// weights are computed once into a scratch row (float64, read back from L2 by the later passes).  A
// cluster of eight blocks works on a row, each on an eighth of the ids; what the blocks must agree on
// (the total, a byte pass's histogram) they read from one another's shared memory.
#include <math.h>

#include "common.cuh"

#define SAMPLE_THREADS 1024

// ---- greedy ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_rows_kernel(const float* __restrict__ logits, int V, int* __restrict__ ids, int* __restrict__ nonfinite,
                   int* __restrict__ host_out) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ int s_bad;
    const float* row = logits + (size_t)blockIdx.x * V;
    if (threadIdx.x == 0) s_bad = 0;
    __syncthreads();
    float best = -INFINITY;
    int bi = 0x7fffffff;
    int bad = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (!isfinite(v)) bad = 1;
        if (v > best) { best = v; bi = i; }      // ascending i per thread: first maximum kept
    }
    if (bad) s_bad = 1;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { s_val[wid] = best; s_idx[wid] = bi; }
    __syncthreads();
    if (wid == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? s_val[lane] : -INFINITY;
        bi = lane < nw ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) {
            ids[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
            nonfinite[blockIdx.x] = s_bad;
            // pinned host memory [2][rows]: the result goes there without a copy of its own (the host sees it once
            // it has waited for an event behind this kernel)
            if (host_out) {
                host_out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
                host_out[gridDim.x + blockIdx.x] = s_bad;
            }
        }
    }
}

// Wide rows: ARGMAX_SPLIT blocks per row scan a slice each and leave (value, id, nonfinite) in the
// caller's scratch; a second small kernel picks the winner (ties still go to the lowest id).
#define ARGMAX_SPLIT 32

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, int V, float* __restrict__ pval, int* __restrict__ pidx) {
    __shared__ float s_val[8];
    __shared__ int s_idx[8], s_bad[8];
    const int row = blockIdx.y, part = blockIdx.x;
    const int per = (V + ARGMAX_SPLIT - 1) / ARGMAX_SPLIT;
    const int lo = part * per, hi = min(V, lo + per);
    const float* r = logits + (size_t)row * V;
    float best = -INFINITY;
    int bi = 0x7fffffff, bad = 0;
    pdl_launch_dependents();
    pdl_wait();                 // the logits come from the kernel before
    if (((V | per) & 3) == 0 && (((size_t)logits) & 15) == 0) {
        // 16-byte reads; a thread meets its elements in ascending order, so ">" keeps the lowest id of a tie
        for (int i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(r + i);
            if (!isfinite(v.x) || !isfinite(v.y) || !isfinite(v.z) || !isfinite(v.w)) bad = 1;
            if (v.x > best) { best = v.x; bi = i; }
            if (v.y > best) { best = v.y; bi = i + 1; }
            if (v.z > best) { best = v.z; bi = i + 2; }
            if (v.w > best) { best = v.w; bi = i + 3; }
        }
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            const float v = r[i];
            if (!isfinite(v)) bad = 1;
            if (v > best) { best = v; bi = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        bad |= __shfl_xor_sync(0xffffffffu, bad, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) { s_val[wid] = best; s_idx[wid] = bi; s_bad[wid] = bad; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
            if (s_val[w] > best || (s_val[w] == best && s_idx[w] < bi)) { best = s_val[w]; bi = s_idx[w]; }
            bad |= s_bad[w];
        }
        pval[row * ARGMAX_SPLIT + part] = best;
        pidx[(row * ARGMAX_SPLIT + part) * 2] = bi;
        pidx[(row * ARGMAX_SPLIT + part) * 2 + 1] = bad;
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ pval, const int* __restrict__ pidx,
                                    int* __restrict__ ids, int* __restrict__ nonfinite, int* __restrict__ host_out) {
    const int row = blockIdx.x, lane = threadIdx.x;     // 32 threads, one per slice
    pdl_launch_dependents();
    pdl_wait();
    float best = pval[row * ARGMAX_SPLIT + lane];
    int bi = pidx[(row * ARGMAX_SPLIT + lane) * 2], bad = pidx[(row * ARGMAX_SPLIT + lane) * 2 + 1];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        bad |= __shfl_xor_sync(0xffffffffu, bad, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
        ids[row] = bi == 0x7fffffff ? 0 : bi;
        nonfinite[row] = bad;
        if (host_out) {          // pinned host memory [2][rows]: the result goes there without a copy of its own
            host_out[row] = bi == 0x7fffffff ? 0 : bi;
            host_out[gridDim.x + row] = bad;
        }
    }
}

// scratch: n_rows * ARGMAX_SPLIT floats and 2 * n_rows * ARGMAX_SPLIT ints (may be null for narrow rows)
// host_out: null, or pinned host memory of 2 * n_rows ints that takes the ids and the flags as well
GESSO_API int gesso_argmax_rows(const float* logits, int n_rows, int V, int* ids, int* nonfinite,
                                float* scratch_val, int* scratch_idx, int* host_out, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (V <= 0) return GESSO_ERR_BAD_SIZE;
    if (V < 8192 || !scratch_val || !scratch_idx || n_rows > 65535) {
        argmax_rows_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, V, ids, nonfinite, host_out);
        return launch_status();
    }
    launch_pdl(argmax_partial_kernel, dim3(ARGMAX_SPLIT, n_rows), dim3(256), 0, stream, logits, V, scratch_val,
               scratch_idx);
    launch_pdl(argmax_final_kernel, dim3(n_rows), dim3(32), 0, stream, (const float*)scratch_val,
               (const int*)scratch_idx, ids, nonfinite, host_out);
    return launch_status();
}

// ---- temperature / nucleus ----------------------------------------------------------------------
__device__ __forceinline__ double block_sum_d(double v, double* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        double t = lane < (blockDim.x >> 5) ? red[lane] : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ double weight_of(float logit, float hi, double inv_t) {
    return exp(((double)logit - (double)hi) * inv_t);
}

// The weight of element i: from the row's cache of weights (written by the first pass) if there is one.
struct Weights {
    const float* row;
    const double* cache;
    float hi;
    double inv_t;
    __device__ __forceinline__ double operator()(int i) const {
        return cache ? __ldcg(cache + i) : weight_of(row[i], hi, inv_t);
    }
};

// ---- a cluster of SAMPLE_CLUSTER blocks per row: block r works on the r-th slice of the ids ----------
#define SAMPLE_CLUSTER 8      // at most; fewer blocks per row when there are many rows (see the launch)
#define SAMPLE_WARPS (SAMPLE_THREADS / 32)

__device__ __forceinline__ unsigned sample_blocks() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(r));
    return r;
}

__device__ __forceinline__ unsigned sample_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// every warp arrives as one: its threads have converged before
__device__ __forceinline__ void sample_cluster_sync() {
    __syncthreads();
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// reads of another block's shared memory (the address of the same object in block `rank`)
__device__ __forceinline__ unsigned peer_addr(const void* p, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"((unsigned)__cvta_generic_to_shared(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ double peer_f64(const void* p, unsigned rank) {
    double v;
    asm volatile("ld.shared::cluster.f64 %0, [%1];\n" : "=d"(v) : "r"(peer_addr(p, rank)) : "memory");
    return v;
}
__device__ __forceinline__ int peer_i32(const void* p, unsigned rank) {
    int v;
    asm volatile("ld.shared::cluster.s32 %0, [%1];\n" : "=r"(v) : "r"(peer_addr(p, rank)) : "memory");
    return v;
}

// One byte pass's histogram: mass, elements and highest id per byte value.
struct ByteHist {
    double mass[256];
    int count[256];
    int last[256];
};

struct CrossShared {
    ByteHist mine[2];          // this block's slice (two copies: peers may still read the pass before)
    ByteHist all;              // the whole row: the blocks' histograms added in rank order
    ByteHist top[2];           // the whole row's histograms of the two top bytes, as the first walk over the row
    unsigned long long top_prefix[2];     // built them, and the prefix each was built under: a later walk that
    int top_valid[2];                     // comes by with the same prefix takes them as they are
    double red[33];
    double exchange[2];        // a value each block shows its peers (two copies, as above)
    unsigned long long prefix;
    double above, mass;
    int id, done;
    int cnt[SAMPLE_THREADS];
};

// Finds, in descending order of weight (ties: ascending id), the first element at which the
// running mass exceeds `target` (strict: running > target) or reaches it (running >= target).
// Returns the element's id and the running mass up to and including it.  Every thread of every
// block of the cluster must call it; all blocks return the same result.
//
// The weight's bit pattern is narrowed from the top byte down.  `prefix` holds the bytes fixed so
// far; `above` is the mass of all weights whose pattern is larger than any with this prefix.  Each
// warp keeps a histogram of its own over its part of the block's slice: in a step of 32 elements
// the lanes with the same byte value form a group (match.any), the group's first lane adds the
// group's weights up in lane order and adds the sum to the warp's histogram (steps with at most six
// values, the usual case in the top bytes, take one butterfly per value instead, the other lanes
// adding zero).  The warps' histograms are added in warp order, the blocks' in rank order (read from
// the peers' shared memory), and the walk down the 256 values is a warp's scan in lane order, so the
// sums do not depend on timing.  As soon as the chosen value holds a single element, that element is
// the answer and the remaining bytes are skipped.  The histograms of the two top bytes are kept with
// the prefix they were built under: the draw's walk follows the nucleus cut's path there nearly
// always and then scans the row for neither.
struct CrossResult { int id; double mass; };

__device__ CrossResult descending_cross(const Weights& W, int V, int lo, int hi_id, double target, bool strict,
                                        CrossShared& sh, ByteHist* wh_all, unsigned& round) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned C = sample_blocks();
    ByteHist& wh = wh_all[warp];
    if (threadIdx.x == 0) { sh.prefix = 0ull; sh.above = 0.0; sh.done = 0; }
    __syncthreads();
    for (int byte = 7; byte >= 0; --byte) {
        const unsigned long long prefix = sh.prefix;
        const int shift = byte * 8;
        // a histogram depends on the prefix, not on the target: where the second walk over a row follows the first
        // one's path through the two top bytes (nearly all of the mass lies there) it takes the first one's histograms
        const int lvl = 7 - byte;
        const bool keep = lvl < 2;
        if (keep && sh.top_valid[lvl] && sh.top_prefix[lvl] == prefix) {
            const ByteHist& top = sh.top[lvl];
            for (int b = threadIdx.x; b < 256; b += blockDim.x) {
                sh.all.mass[b] = top.mass[b]; sh.all.count[b] = top.count[b]; sh.all.last[b] = top.last[b];
            }
        } else {
        for (int b = lane; b < 256; b += 32) { wh.mass[b] = 0.0; wh.count[b] = 0; wh.last[b] = -1; }
        __syncwarp();
        for (int base = lo + warp * 32; base < hi_id; base += SAMPLE_THREADS) {
            const int i = base + lane;
            const bool valid = i < hi_id;
            const double w = valid ? W(i) : 0.0;
            const unsigned long long bits = (unsigned long long)__double_as_longlong(w);
            const bool match = valid && (byte == 7 || ((bits >> (shift + 8)) == (prefix >> (shift + 8))));
            const int b = match ? (int)((bits >> shift) & 0xff) : -1;
            const int b0 = __shfl_sync(0xffffffffu, b, 0);
            if (__all_sync(0xffffffffu, b == b0)) {
                if (b0 < 0) continue;                        // nobody matches
                double sum = w;                              // fixed butterfly: the same sum every time
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                if (lane == 0) { wh.mass[b0] += sum; wh.count[b0] += 32; wh.last[b0] = base + 31; }
            } else {
                const unsigned grp = __match_any_sync(0xffffffffu, b);
                const bool leader = match && lane == __ffs(grp) - 1;
                unsigned leaders = __ballot_sync(0xffffffffu, leader);
                double sum = 0.0;
                if (__popc(leaders) <= 6) {
                    // few values, large groups (the top bytes): one butterfly per value, the others adding zero
                    while (leaders) {
                        const int src = __ffs(leaders) - 1;
                        leaders &= leaders - 1;
                        const int bv = __shfl_sync(0xffffffffu, b, src);
                        double t = (match && b == bv) ? w : 0.0;
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
                        if (lane == src) sum = t;
                    }
                } else {
                    // many values, small groups: every lane walks the members of its group in lane order
                    unsigned m = match ? grp : 0u;
                    while (__any_sync(0xffffffffu, m != 0u)) {
                        const int src = m ? __ffs(m) - 1 : lane;
                        const double v = __shfl_sync(0xffffffffu, w, src);
                        if (m) { sum += v; m &= m - 1; }
                    }
                }
                if (leader) {
                    wh.mass[b] += sum;
                    wh.count[b] += __popc(grp);
                    wh.last[b] = base + (31 - __clz(grp));     // bases ascend: the last write is the highest id
                }
            }
            __syncwarp();
        }
        __syncthreads();
        ByteHist& mine = sh.mine[round & 1];
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            double mass = 0.0;
            int count = 0, last = -1;
            for (int k = 0; k < SAMPLE_WARPS; ++k) {
                mass += wh_all[k].mass[b];
                count += wh_all[k].count[b];
                last = max(last, wh_all[k].last[b]);
            }
            mine.mass[b] = mass; mine.count[b] = count; mine.last[b] = last;
        }
        sample_cluster_sync();                     // every block's histogram of this pass is written
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            double mass = 0.0;
            int count = 0, last = -1;
            for (unsigned r = 0; r < C; ++r) {
                mass += peer_f64(&mine.mass[b], r);
                count += peer_i32(&mine.count[b], r);
                last = max(last, peer_i32(&mine.last[b], r));
            }
            sh.all.mass[b] = mass; sh.all.count[b] = count; sh.all.last[b] = last;
            if (keep && !sh.top_valid[lvl]) { sh.top[lvl].mass[b] = mass; sh.top[lvl].count[b] = count; sh.top[lvl].last[b] = last; }
        }
        ++round;
        }
        __syncthreads();
        if (warp == 0) {
            // The walk down the 256 values, by one warp: lane l owns the values 255 - 8 l .. 248 - 8 l, adds its
            // occupied ones up, the lanes' sums are scanned in lane order (a fixed order: the same sums every
            // time), and every lane then walks its eight values from the mass above them; the first lane with a
            // crossing holds the answer.
            double m[8];
            int c[8];
            double local = 0.0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int b = 255 - 8 * lane - k;
                c[k] = sh.all.count[b];
                m[k] = c[k] > 0 ? sh.all.mass[b] : 0.0;
                local += m[k];
            }
            double incl = local;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            double run = __shfl_up_sync(0xffffffffu, incl, 1);
            run = sh.above + (lane == 0 ? 0.0 : run);
            int pick = -1, low = -1;                 // low: this lane's smallest occupied value
            double run_pick = 0.0, run_low = 0.0;    // the mass above them
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (c[k] <= 0) continue;
                const double next = run + m[k];
                const bool crossed = strict ? (next > target) : (next >= target);
                if (crossed && pick < 0) { pick = 255 - 8 * lane - k; run_pick = run; }
                low = 255 - 8 * lane - k;
                run_low = run;
                run = next;
            }
            const unsigned crossed_in = __ballot_sync(0xffffffffu, pick >= 0);
            const unsigned occupied_in = __ballot_sync(0xffffffffu, low >= 0);
            int src;
            if (crossed_in) {
                src = __ffs(crossed_in) - 1;
            } else {
                // nothing crossed (rounding): the walk ends in the smallest occupied value
                src = occupied_in ? 31 - __clz(occupied_in) : 0;
                pick = low;
                run_pick = run_low;
            }
            pick = __shfl_sync(0xffffffffu, pick, src);
            run_pick = __shfl_sync(0xffffffffu, run_pick, src);
            if (pick < 0) { pick = 0; run_pick = sh.above; }         // an empty histogram: nothing matched
            if (lane == 0) {
                if (keep && !sh.top_valid[lvl]) { sh.top_valid[lvl] = 1; sh.top_prefix[lvl] = prefix; }
                sh.above = run_pick;
                sh.prefix = prefix | ((unsigned long long)pick << shift);
                if (sh.all.count[pick] == 1) {        // one element left: it is the answer
                    sh.id = sh.all.last[pick];
                    sh.mass = run_pick + sh.all.mass[pick];
                    sh.done = 1;
                }
            }
        }
        __syncthreads();
        if (sh.done) {
            CrossResult r;
            r.id = sh.id;
            r.mass = sh.mass;
            __syncthreads();
            return r;
        }
    }
    // All weights equal to the found pattern tie; they are taken in ascending id order.  Every block
    // does this part over the whole row by itself (it is rare, and all arrive at the same answer).
    const unsigned long long pat = sh.prefix;
    const double wv = __longlong_as_double((long long)pat);
    const double above = sh.above;
    // how many of the tied elements are needed for the running mass to cross
    long long need;
    if (wv > 0.0) {
        double k = floor((target - above) / wv);
        need = (long long)k + 1;                 // strict: above + need*wv > target
        if (!strict && above + (double)(need - 1) * wv >= target && need > 1) need -= 1;
        if (need < 1) need = 1;
    } else {
        need = 1;
    }
    // the need-th tied id in ascending order: count ties per thread chunk, then scan
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int i0 = threadIdx.x * chunk, i1 = min(V, i0 + chunk);
    int cnt = 0;
    for (int i = i0; i < i1; ++i)
        if ((unsigned long long)__double_as_longlong(W(i)) == pat) ++cnt;
    sh.cnt[threadIdx.x] = cnt;
    __syncthreads();
    if (threadIdx.x == 0) {
        long long run = 0, total = 0;
        for (int t = 0; t < (int)blockDim.x; ++t) total += sh.cnt[t];
        if (need > total) need = total;          // rounding: take the last tie
        int owner = 0;
        long long before = 0;
        for (int t = 0; t < (int)blockDim.x; ++t) {
            if (run + sh.cnt[t] >= need) { owner = t; before = run; break; }
            run += sh.cnt[t];
        }
        sh.id = owner;
        sh.mass = above + (double)need * wv;
        sh.red[0] = (double)(need - before);     // rank inside the owner's chunk
    }
    __syncthreads();
    const int owner = sh.id;
    const long long rank = (long long)sh.red[0];
    __syncthreads();
    if ((int)threadIdx.x == owner) {
        long long seen = 0;
        int found = i1 - 1;
        for (int i = i0; i < i1; ++i)
            if ((unsigned long long)__double_as_longlong(W(i)) == pat) {
                if (++seen == rank) { found = i; break; }
            }
        sh.id = found;
    }
    __syncthreads();
    CrossResult r;
    r.id = sh.id;
    r.mass = sh.mass;
    __syncthreads();
    return r;
}

// Every block shows `v` to its peers; returns the values of all blocks (the same in every block).
__device__ void cluster_gather(double v, double (&out)[SAMPLE_CLUSTER], CrossShared& sh, unsigned& round) {
    double* slot = &sh.exchange[round & 1];
    if (threadIdx.x == 0) *slot = v;
    sample_cluster_sync();
    const unsigned C = sample_blocks();
    for (unsigned r = 0; r < SAMPLE_CLUSTER; ++r) out[r] = r < C ? peer_f64(slot, r) : 0.0;
    ++round;
    sample_cluster_sync();      // all have read: a block may leave after this without a peer still reading it
}

// A cluster of 1, 2, 4 or 8 blocks per row (the launch's cluster size).  u[row] in [0,1).  top_p[row] in (0,1]; temperature[row] > 0.
// wcache: [rows, V] float64 scratch for the weights (computed once, read by the later passes), or null
// (every pass then computes them again).
__global__ void __launch_bounds__(SAMPLE_THREADS, 1)
sample_rows_kernel(const float* __restrict__ logits, int V, const double* __restrict__ temperature,
                   const double* __restrict__ top_p, const double* __restrict__ u, int* __restrict__ ids,
                   int* __restrict__ nonfinite, double* __restrict__ wcache) {
    extern __shared__ unsigned char sample_smem[];
    ByteHist* wh_all = reinterpret_cast<ByteHist*>(sample_smem);      // one histogram per warp
    __shared__ CrossShared sh;
    __shared__ float s_max[33];
    __shared__ double s_part[SAMPLE_THREADS];
    __shared__ int s_bad;
    const int C = (int)sample_blocks();
    const int rowi = blockIdx.x / C;
    const unsigned rank = sample_rank();
    unsigned round = 0;                          // exchanges with the peers so far (picks the copy to write)
    const float* row = logits + (size_t)rowi * V;
    // this block's slice of the ids, in whole steps of 32
    const int per = ((V + C - 1) / C + 31) / 32 * 32;
    const int lo = min(V, (int)rank * per), hi_id = min(V, lo + per);
    if (threadIdx.x == 0) { s_bad = 0; sh.top_valid[0] = sh.top_valid[1] = 0; }
    __syncthreads();
    // the maximum and the check for non-finite values: every block over its slice, the cluster puts them together
    // (a slice with a non-finite value shows its peers a NaN)
    float hi = -INFINITY;
    int bad = 0;
#pragma unroll 8
    for (int i = lo + threadIdx.x; i < hi_id; i += blockDim.x) {
        const float v = row[i];
        if (!isfinite(v)) bad = 1;
        hi = fmaxf(hi, v);
    }
    if (bad) s_bad = 1;
    hi = warp_max(hi);
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = hi;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? s_max[threadIdx.x] : -INFINITY;
        v = warp_max(v);
        if (threadIdx.x == 0) s_max[32] = v;
    }
    __syncthreads();
    {
        double maxima[SAMPLE_CLUSTER];
        cluster_gather(s_bad ? (double)NAN : (double)s_max[32], maxima, sh, round);
        bad = 0;
        hi = -INFINITY;
        for (int r = 0; r < C; ++r) {
            if (maxima[r] != maxima[r]) bad = 1;
            else hi = fmaxf(hi, (float)maxima[r]);
        }
    }
    if (bad) {                                   // the same in every block: nobody waits at a barrier below
        if (threadIdx.x == 0 && rank == 0) { nonfinite[rowi] = 1; ids[rowi] = 0; }
        return;
    }
    const double inv_t = 1.0 / temperature[rowi];
    double* row_cache = wcache ? wcache + (size_t)rowi * V : nullptr;
    double part = 0.0;
    for (int i = lo + threadIdx.x; i < hi_id; i += blockDim.x) {
        const double w = weight_of(row[i], hi, inv_t);
        if (row_cache) __stcg(row_cache + i, w);
        part += w;
    }
    const double slice_total = block_sum_d(part, sh.red);
    double totals[SAMPLE_CLUSTER];
    cluster_gather(slice_total, totals, sh, round);       // its barrier also publishes the cached weights
    double total = 0.0;
    for (int r = 0; r < SAMPLE_CLUSTER; ++r) total += totals[r];
    const Weights W = {row, row_cache, hi, inv_t};
    const double p = top_p[rowi];
    const double r01 = u[rowi];

    if (p >= 1.0) {
        // walk in id order: the slice that holds the draw, then its thread chunks, then its elements
        const double r = r01 * total;
        double run = 0.0;
        int slice = -1;
        for (int k = 0; k < SAMPLE_CLUSTER; ++k) {
            if (r < run + totals[k]) { slice = k; break; }
            run += totals[k];
        }
        if (slice < 0) {                         // rounding: the last id
            if (threadIdx.x == 0 && rank == 0) { ids[rowi] = V - 1; nonfinite[rowi] = 0; }
            return;
        }
        if ((int)rank != slice) return;
        const int n = hi_id - lo;
        const int chunk = (n + (int)blockDim.x - 1) / (int)blockDim.x;
        const int i0 = min(hi_id, lo + (int)threadIdx.x * chunk), i1 = min(hi_id, i0 + chunk);
        double mine = 0.0;
        for (int i = i0; i < i1; ++i) mine += W(i);
        s_part[threadIdx.x] = mine;
        __syncthreads();
        if (threadIdx.x < 32) {
            // the thread whose chunk holds the draw: lane l adds up the chunks of threads 32 l .. 32 l + 31, the
            // lanes' sums are scanned in lane order, and each lane then walks its 32 chunks from the mass before them
            const int lane = threadIdx.x, per_lane = (int)blockDim.x / 32;
            double local = 0.0;
            for (int t = 0; t < per_lane; ++t) local += s_part[lane * per_lane + t];
            double incl = local;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            double before = __shfl_up_sync(0xffffffffu, incl, 1);
            before = run + (lane == 0 ? 0.0 : before);
            int owner = -1;
            double at = 0.0;
            for (int t = 0; t < per_lane; ++t) {
                const double next = before + s_part[lane * per_lane + t];
                if (r < next) { owner = lane * per_lane + t; at = before; break; }
                before = next;
            }
            const unsigned found = __ballot_sync(0xffffffffu, owner >= 0);
            const int src = found ? __ffs(found) - 1 : 0;
            owner = __shfl_sync(0xffffffffu, owner, src);
            at = __shfl_sync(0xffffffffu, at, src);
            if (lane == 0) { sh.id = found ? owner : -1; sh.above = at; }
        }
        __syncthreads();
        const int owner = sh.id;
        if (owner < 0) {                         // rounding: the slice's last id
            if (threadIdx.x == 0) { ids[rowi] = hi_id - 1; nonfinite[rowi] = 0; }
            return;
        }
        if ((int)threadIdx.x == owner) {
            double acc = sh.above;
            int found = i1 - 1;
            for (int i = i0; i < i1; ++i) {
                acc += W(i);
                if (r < acc) { found = i; break; }
            }
            ids[rowi] = found;
            nonfinite[rowi] = 0;
        }
        return;
    }
    // nucleus: kept mass = running mass at the first position where it reaches top_p * total
    const CrossResult cut = descending_cross(W, V, lo, hi_id, p * total, false, sh, wh_all, round);
    const double r = r01 * cut.mass;
    const CrossResult pick = descending_cross(W, V, lo, hi_id, r, true, sh, wh_all, round);
    if (threadIdx.x == 0 && rank == 0) { ids[rowi] = pick.id; nonfinite[rowi] = 0; }
    sample_cluster_sync();                       // no block leaves while a peer may still read its shared memory
}

// wcache: n_rows * V doubles of scratch, or null.
GESSO_API int gesso_sample_rows(const float* logits, int n_rows, int V, const double* temperature,
                                const double* top_p, const double* u, int* ids, int* nonfinite, double* wcache,
                                cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (V <= 0) return GESSO_ERR_BAD_SIZE;
    const size_t smem = sizeof(ByteHist) * SAMPLE_WARPS;
    static bool configured = false;
    static int max_clusters[SAMPLE_CLUSTER + 1];     // clusters of that many blocks the device runs at once
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(SAMPLE_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (!configured) {
        if (cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        for (int c = 2; c <= SAMPLE_CLUSTER; c *= 2) {
            attr[0].val.clusterDim.x = c;
            cfg.gridDim = dim3(c);
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, sample_rows_kernel, &cfg) != cudaSuccess) {
                cudaGetLastError();
                n = 0;
            }
            max_clusters[c] = n;
        }
        configured = true;
    }
    // the most blocks per row with which all rows still run at the same time
    int C = 1;
    for (int c = SAMPLE_CLUSTER; c >= 2; c /= 2)
        if (n_rows <= max_clusters[c]) { C = c; break; }
    attr[0].val.clusterDim.x = C;
    cfg.gridDim = dim3(n_rows * C);
    cudaLaunchKernelEx(&cfg, sample_rows_kernel, logits, V, temperature, top_p, u, ids, nonfinite, wcache);
    return launch_status();
}
