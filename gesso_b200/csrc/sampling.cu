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
// 64-bit pattern of the weight eight bits at a time (positive doubles order like their bits).
#include <math.h>

#include "common.cuh"

#define SAMPLE_THREADS 1024

// ---- greedy ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_rows_kernel(const float* __restrict__ logits, int V, int* __restrict__ ids, int* __restrict__ nonfinite) {
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
                                    int* __restrict__ ids, int* __restrict__ nonfinite) {
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
    if (lane == 0) { ids[row] = bi == 0x7fffffff ? 0 : bi; nonfinite[row] = bad; }
}

// scratch: n_rows * ARGMAX_SPLIT floats and 2 * n_rows * ARGMAX_SPLIT ints (may be null for narrow rows)
GESSO_API int gesso_argmax_rows(const float* logits, int n_rows, int V, int* ids, int* nonfinite,
                                float* scratch_val, int* scratch_idx, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (V <= 0) return GESSO_ERR_BAD_SIZE;
    if (V < 8192 || !scratch_val || !scratch_idx || n_rows > 65535) {
        argmax_rows_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, V, ids, nonfinite);
        return launch_status();
    }
    launch_pdl(argmax_partial_kernel, dim3(ARGMAX_SPLIT, n_rows), dim3(256), 0, stream, logits, V, scratch_val,
               scratch_idx);
    launch_pdl(argmax_final_kernel, dim3(n_rows), dim3(32), 0, stream, (const float*)scratch_val,
               (const int*)scratch_idx, ids, nonfinite);
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

// Finds, in descending order of weight (ties: ascending id), the first element at which the
// running mass exceeds `target` (strict: running > target) or reaches it (running >= target).
// Returns through shared memory: the element's id and the running mass up to and including it.
// Every thread of the block must call it.  hist[256] doubles, red[33] doubles of shared memory.
struct CrossResult { int id; double mass; };

__device__ CrossResult descending_cross(const float* __restrict__ row, int V, float hi, double inv_t,
                                        double target, bool strict, double* hist, double* red,
                                        unsigned long long* s_prefix, double* s_above, int* s_id,
                                        double* s_mass) {
    // Narrow the weight's bit pattern from the top byte down.  `prefix` holds the bytes fixed so
    // far; `above` is the mass of all weights whose pattern is larger than any with this prefix.
    if (threadIdx.x == 0) { *s_prefix = 0ull; *s_above = 0.0; }
    __syncthreads();
    for (int byte = 7; byte >= 0; --byte) {
        for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0.0;
        __syncthreads();
        const unsigned long long prefix = *s_prefix;
        const int shift = byte * 8;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const double w = weight_of(row[i], hi, inv_t);
            const unsigned long long bits = (unsigned long long)__double_as_longlong(w);
            const bool match = byte == 7 || ((bits >> (shift + 8)) == (prefix >> (shift + 8)));
            if (match) atomicAdd(&hist[(bits >> shift) & 0xff], w);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            double run = *s_above;
            int pick = -1, last_occupied = 0;
            double run_before_last = run;
            for (int b = 255; b >= 0; --b) {
                if (hist[b] <= 0.0) continue;
                const double next = run + hist[b];
                const bool crossed = strict ? (next > target) : (next >= target);
                if (crossed) { pick = b; break; }
                last_occupied = b;
                run_before_last = run;
                run = next;
            }
            // if nothing crossed (rounding), the walk ends in the smallest occupied bucket
            if (pick < 0) { pick = last_occupied; run = run_before_last; }
            *s_above = run;
            *s_prefix = prefix | ((unsigned long long)pick << shift);
        }
        __syncthreads();
    }
    // All weights equal to the found pattern tie; they are taken in ascending id order.
    const unsigned long long pat = *s_prefix;
    const double wv = __longlong_as_double((long long)pat);
    const double above = *s_above;
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
        if ((unsigned long long)__double_as_longlong(weight_of(row[i], hi, inv_t)) == pat) ++cnt;
    // inclusive scan of cnt over threads (hist reused as int scratch is avoided: use red as doubles)
    __shared__ int s_cnt[SAMPLE_THREADS];
    s_cnt[threadIdx.x] = cnt;
    __syncthreads();
    if (threadIdx.x == 0) {
        long long run = 0, total = 0;
        for (int t = 0; t < (int)blockDim.x; ++t) total += s_cnt[t];
        if (need > total) need = total;          // rounding: take the last tie
        int owner = 0;
        long long before = 0;
        for (int t = 0; t < (int)blockDim.x; ++t) {
            if (run + s_cnt[t] >= need) { owner = t; before = run; break; }
            run += s_cnt[t];
        }
        *s_id = owner;
        *s_mass = above + (double)need * wv;
        red[0] = (double)(need - before);        // rank inside the owner's chunk
    }
    __syncthreads();
    const int owner = *s_id;
    const long long rank = (long long)red[0];
    __syncthreads();
    if ((int)threadIdx.x == owner) {
        long long seen = 0;
        int found = i1 - 1;
        for (int i = i0; i < i1; ++i)
            if ((unsigned long long)__double_as_longlong(weight_of(row[i], hi, inv_t)) == pat) {
                if (++seen == rank) { found = i; break; }
            }
        *s_id = found;
    }
    __syncthreads();
    CrossResult r;
    r.id = *s_id;
    r.mass = *s_mass;
    __syncthreads();
    return r;
}

// One block per row.  u[row] in [0,1).  top_p[row] in (0,1]; temperature[row] > 0.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int V, const double* __restrict__ temperature,
                   const double* __restrict__ top_p, const double* __restrict__ u, int* __restrict__ ids,
                   int* __restrict__ nonfinite) {
    __shared__ double hist[256];
    __shared__ double red[33];
    __shared__ float s_max[33];
    __shared__ unsigned long long s_prefix;
    __shared__ double s_above, s_mass;
    __shared__ int s_id, s_bad;
    const int rowi = blockIdx.x;
    const float* row = logits + (size_t)rowi * V;
    if (threadIdx.x == 0) s_bad = 0;
    __syncthreads();
    float hi = -INFINITY;
    int bad = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
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
    hi = s_max[32];
    if (s_bad) {
        if (threadIdx.x == 0) { nonfinite[rowi] = 1; ids[rowi] = 0; }
        return;
    }
    const double inv_t = 1.0 / temperature[rowi];
    double part = 0.0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) part += weight_of(row[i], hi, inv_t);
    const double total = block_sum_d(part, red);
    const double p = top_p[rowi];
    const double r01 = u[rowi];

    if (p >= 1.0) {
        // walk in id order: thread chunks are contiguous id ranges
        const int chunk = (V + blockDim.x - 1) / blockDim.x;
        const int i0 = threadIdx.x * chunk, i1 = min(V, i0 + chunk);
        double mine = 0.0;
        for (int i = i0; i < i1; ++i) mine += weight_of(row[i], hi, inv_t);
        __shared__ double s_part[SAMPLE_THREADS];
        s_part[threadIdx.x] = mine;
        __syncthreads();
        if (threadIdx.x == 0) {
            const double r = r01 * total;
            double run = 0.0;
            int owner = -1;
            for (int t = 0; t < (int)blockDim.x; ++t) {
                if (r < run + s_part[t]) { owner = t; break; }
                run += s_part[t];
            }
            s_id = owner;
            s_above = run;
        }
        __syncthreads();
        const int owner = s_id;
        if (owner < 0) {
            if (threadIdx.x == 0) { ids[rowi] = V - 1; nonfinite[rowi] = 0; }
            return;
        }
        if ((int)threadIdx.x == owner) {
            const double r = r01 * total;
            double acc = s_above;
            int found = i1 - 1;
            for (int i = i0; i < i1; ++i) {
                acc += weight_of(row[i], hi, inv_t);
                if (r < acc) { found = i; break; }
            }
            ids[rowi] = found;
            nonfinite[rowi] = 0;
        }
        return;
    }
    // nucleus: kept mass = running mass at the first position where it reaches top_p * total
    const CrossResult cut = descending_cross(row, V, hi, inv_t, p * total, false, hist, red, &s_prefix, &s_above,
                                             &s_id, &s_mass);
    const double r = r01 * cut.mass;
    const CrossResult pick = descending_cross(row, V, hi, inv_t, r, true, hist, red, &s_prefix, &s_above, &s_id,
                                              &s_mass);
    if (threadIdx.x == 0) { ids[rowi] = pick.id; nonfinite[rowi] = 0; }
}

GESSO_API int gesso_sample_rows(const float* logits, int n_rows, int V, const double* temperature,
                                const double* top_p, const double* u, int* ids, int* nonfinite,
                                cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (V <= 0) return GESSO_ERR_BAD_SIZE;
    sample_rows_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, V, temperature, top_p, u, ids, nonfinite);
    return launch_status();
}
