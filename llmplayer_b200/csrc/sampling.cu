// Sampling on the device: one block per sequence turns a row of float32 logits into a token.
//
// Stages, in the reference's order (sampler/CompositeSampler.java:33-120):
//   logit edits (DRY subtraction, then repetition penalty: positive / r, else * r)
//   -> first-maximum argmax if greedy (:259-269)
//   -> * 1/temperature -> top-k by threshold, ties at the threshold survive (:70-78)
//   -> softmax (:80-98) -> min-p (:122-139) -> top-p over descending probabilities (:303-352)
//   -> mirostat v2 truncation and draw in descending order (:206-250), or an inverse-CDF
//      walk in index order with the last vocabulary index as fallback (:387-395).
// The reference sorts; here the k-th largest value and the descending-order cut-offs are
// found by a bitwise search over the ordered bit patterns of the floats, and ties at a
// cut-off are resolved in index order, as a stable descending sort would.
#include "common.cuh"

struct LpSampleParams {
    float inv_temperature;     // 0: greedy
    int top_k;                 // <= 0 or >= vocab: off
    float top_p;               // >= 1: off
    float min_p;               // <= 0: off
    float mirostat_threshold;  // < 0: multinomial draw; else keep probabilities >= this (2^-mu)
    float uniform;             // the draw in [0, 1)
    int edit_begin, edit_count;
    int logits_row;
};

namespace {

constexpr int THREADS = 1024;
constexpr int CAP = 2048;      // candidates kept in shared memory after top-k

struct Shared {
    float fscratch[32];
    int iscratch[32];
    float scan[THREADS];
    float cand_val[CAP];
    int cand_idx[CAP];
    int bcast_i;
    float bcast_f;
};

__device__ __forceinline__ unsigned ordered_key(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__device__ int block_sum_int(int v, int* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    int total = 0;
    for (int w = 0; w < THREADS / 32; ++w) total += scratch[w];
    return total;
}

// Exclusive prefix over the threads of the block, in thread order; *total gets the sum.
__device__ float block_exclusive_scan(float v, Shared& sh, float* total) {
    __syncthreads();
    sh.scan[threadIdx.x] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float run = 0.f;
        for (int i = 0; i < THREADS; ++i) {
            const float x = sh.scan[i];
            sh.scan[i] = run;
            run += x;
        }
        sh.bcast_f = run;
    }
    __syncthreads();
    *total = sh.bcast_f;
    return sh.scan[threadIdx.x];
}

__device__ float reduce_max(const float* vals, int n, Shared& sh) {
    float m = -INFINITY;
    for (int i = threadIdx.x; i < n; i += THREADS) m = fmaxf(m, vals[i]);
    return lp_block_max(m, sh.fscratch);
}
__device__ float reduce_sum(const float* vals, int n, Shared& sh) {
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += THREADS) s += vals[i];
    return lp_block_sum(s, sh.fscratch);
}

// Largest key t such that at least k values have key >= t: the key of the k-th largest value.
__device__ unsigned kth_largest_key(const float* vals, int n, int k, Shared& sh) {
    unsigned prefix = 0;
    for (int bit = 31; bit >= 0; --bit) {
        const unsigned cand = prefix | (1u << bit);
        int c = 0;
        for (int i = threadIdx.x; i < n; i += THREADS) c += ordered_key(vals[i]) >= cand;
        if (block_sum_int(c, sh.iscratch) >= k) prefix = cand;
    }
    return prefix;
}

// Walk the values >= floor_value in descending order (equal ones in index order) until the running
// sum exceeds `target`. Returns false if it never does. Otherwise *cut_key is the key of the value
// at which it does, and *ties_kept how many of the values equal to it (in index order) lie up to
// and including that point.
__device__ bool descending_cut(const float* vals, int n, float target, float floor_value, unsigned* cut_key,
                               int* ties_kept, Shared& sh) {
    unsigned prefix = 0;
    bool any = false;
    for (int bit = 31; bit >= 0; --bit) {
        const unsigned cand = prefix | (1u << bit);
        float s = 0.f;
        for (int i = threadIdx.x; i < n; i += THREADS) {
            const float v = vals[i];
            if (v >= floor_value && v > 0.f && ordered_key(v) >= cand) s += v;
        }
        if (lp_block_sum(s, sh.fscratch) > target) { prefix = cand; any = true; }
    }
    if (!any) {
        // no bit could be set: either the whole mass stays below the target, or the cut lies at key 0
        float s = 0.f;
        for (int i = threadIdx.x; i < n; i += THREADS) {
            const float v = vals[i];
            if (v >= floor_value && v > 0.f) s += v;
        }
        if (!(lp_block_sum(s, sh.fscratch) > target)) return false;
    }
    float above = 0.f;
    int equal = 0;
    for (int i = threadIdx.x; i < n; i += THREADS) {
        const float v = vals[i];
        if (v >= floor_value && v > 0.f) {
            const unsigned k = ordered_key(v);
            if (k > prefix) above += v;
            else if (k == prefix) ++equal;
        }
    }
    above = lp_block_sum(above, sh.fscratch);
    equal = block_sum_int(equal, sh.iscratch);
    const float v = key_to_float(prefix);
    int j = 1;
    while (j < equal && !(above + (float)j * v > target)) ++j;
    *cut_key = prefix;
    *ties_kept = j;
    return true;
}

// Index (among 0..n-1) of the tie number `rank` (0-based, in index order) with key == cut_key.
__device__ int nth_tie(const float* vals, int n, unsigned cut_key, float floor_value, int rank, Shared& sh) {
    const int chunk = (n + THREADS - 1) / THREADS;
    const int b = threadIdx.x * chunk, e = min(n, b + chunk);
    int mine = 0;
    for (int i = b; i < e; ++i) mine += (vals[i] >= floor_value && ordered_key(vals[i]) == cut_key);
    float total;
    const int before = (int)block_exclusive_scan((float)mine, sh, &total);
    __syncthreads();
    if (threadIdx.x == 0) sh.bcast_i = -1;
    __syncthreads();
    if (rank >= before && rank < before + mine) {
        int seen = before;
        for (int i = b; i < e; ++i)
            if (vals[i] >= floor_value && ordered_key(vals[i]) == cut_key) {
                if (seen == rank) { sh.bcast_i = i; break; }
                ++seen;
            }
    }
    __syncthreads();
    return sh.bcast_i;
}

// Zero everything after the cut (keeping the first `ties_kept` ties in index order), then renormalise.
__device__ void keep_until_cut(float* vals, int n, unsigned cut_key, int ties_kept, Shared& sh) {
    const int chunk = (n + THREADS - 1) / THREADS;
    const int b = threadIdx.x * chunk, e = min(n, b + chunk);
    int mine = 0;
    for (int i = b; i < e; ++i) mine += (ordered_key(vals[i]) == cut_key);
    float total;
    int seen = (int)block_exclusive_scan((float)mine, sh, &total);
    for (int i = b; i < e; ++i) {
        const unsigned k = ordered_key(vals[i]);
        if (k < cut_key) vals[i] = 0.f;
        else if (k == cut_key) {
            if (seen >= ties_kept) vals[i] = 0.f;
            ++seen;
        }
    }
    __syncthreads();
    const float s = reduce_sum(vals, n, sh);
    if (s > 0.f) {
        const float inv = 1.0f / s;
        for (int i = threadIdx.x; i < n; i += THREADS) vals[i] *= inv;
    }
    __syncthreads();
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, long long logits_stride, float* __restrict__ work, int V,
              const LpSampleParams* __restrict__ params, const int* __restrict__ edit_token,
              const float* __restrict__ edit_subtract, const float* __restrict__ edit_factor,
              int* __restrict__ out_token, float* __restrict__ out_prob) {
    __shared__ Shared sh;
    lp_grid_release();
    lp_grid_wait();
    const int b = blockIdx.x, tid = threadIdx.x;
    const LpSampleParams p = params[b];
    const float* src = logits + (long long)p.logits_row * logits_stride;
    float* w = work + (long long)b * V;

    const bool greedy = p.inv_temperature == 0.f;
    const float* cur = src;
    if (!greedy || p.edit_count > 0) {
        for (int i = tid; i < V; i += THREADS) w[i] = src[i];
        __syncthreads();
        for (int e = tid; e < p.edit_count; e += THREADS) {          // edited tokens are distinct
            const int tok = edit_token[p.edit_begin + e];
            if (tok >= 0 && tok < V) {
                float v = w[tok] - edit_subtract[p.edit_begin + e];
                const float f = edit_factor[p.edit_begin + e];
                v = v > 0.f ? v / f : v * f;
                w[tok] = v;
            }
        }
        __syncthreads();
        cur = w;
    }

    if (greedy) {
        float best = -INFINITY;
        int best_i = 0x7fffffff;
        for (int i = tid; i < V; i += THREADS) {
            const float v = cur[i];
            if (v > best || best_i == 0x7fffffff) { best = v; best_i = i; }
        }
        // reduce (value, index): larger value wins, equal values: lower index
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (oi != 0x7fffffff && (best_i == 0x7fffffff || ov > best || (ov == best && oi < best_i))) {
                best = ov; best_i = oi;
            }
        }
        __syncthreads();
        if ((tid & 31) == 0) { sh.fscratch[tid >> 5] = best; sh.iscratch[tid >> 5] = best_i; }
        __syncthreads();
        if (tid == 0) {
            for (int k = 1; k < THREADS / 32; ++k) {
                const float ov = sh.fscratch[k];
                const int oi = sh.iscratch[k];
                if (oi != 0x7fffffff && (best_i == 0x7fffffff || ov > best || (ov == best && oi < best_i))) {
                    best = ov; best_i = oi;
                }
            }
            out_token[b] = best_i;
            out_prob[b] = 1.f;
        }
        return;
    }

    for (int i = tid; i < V; i += THREADS) w[i] *= p.inv_temperature;
    __syncthreads();

    float* vals = w;
    const int* ids = nullptr;
    int n = V;
    if (p.top_k > 0 && p.top_k < V) {
        const unsigned thr = kth_largest_key(w, V, p.top_k, sh);
        int c = 0;
        for (int i = tid; i < V; i += THREADS) c += ordered_key(w[i]) >= thr;
        const int survivors = block_sum_int(c, sh.iscratch);
        if (survivors <= CAP) {
            // compact the survivors, in index order, into shared memory
            const int chunk = (V + THREADS - 1) / THREADS;
            const int cb = tid * chunk, ce = min(V, cb + chunk);
            int mine = 0;
            for (int i = cb; i < ce; ++i) mine += ordered_key(w[i]) >= thr;
            float total;
            int at = (int)block_exclusive_scan((float)mine, sh, &total);
            for (int i = cb; i < ce; ++i)
                if (ordered_key(w[i]) >= thr) { sh.cand_val[at] = w[i]; sh.cand_idx[at] = i; ++at; }
            __syncthreads();
            vals = sh.cand_val; ids = sh.cand_idx; n = survivors;
        } else {
            for (int i = tid; i < V; i += THREADS) if (ordered_key(w[i]) < thr) w[i] = -INFINITY;
            __syncthreads();
        }
    }

    // softmax
    const float m = reduce_max(vals, n, sh);
    for (int i = tid; i < n; i += THREADS) vals[i] = (vals[i] == -INFINITY) ? 0.f : expf(vals[i] - m);
    __syncthreads();
    float s = reduce_sum(vals, n, sh);
    if (s > 0.f) {
        const float inv = 1.0f / s;
        for (int i = tid; i < n; i += THREADS) vals[i] *= inv;
    }
    __syncthreads();

    if (p.min_p > 0.f) {
        const float mx = reduce_max(vals, n, sh);
        if (mx > 0.f) {
            const float thr = p.min_p * mx;
            for (int i = tid; i < n; i += THREADS) if (vals[i] < thr) vals[i] = 0.f;
            __syncthreads();
            s = reduce_sum(vals, n, sh);
            if (s > 0.f) {
                const float inv = 1.0f / s;
                for (int i = tid; i < n; i += THREADS) vals[i] *= inv;
            }
            __syncthreads();
        }
    }

    if (p.top_p < 1.0f) {
        int c = 0;
        for (int i = tid; i < n; i += THREADS) c += vals[i] > 0.f;
        if (block_sum_int(c, sh.iscratch) > 1) {
            unsigned cut;
            int ties;
            if (descending_cut(vals, n, p.top_p, 0.f, &cut, &ties, sh)) keep_until_cut(vals, n, cut, ties, sh);
        }
    }

    int chosen = -1;          // index into vals
    float observed = 0.f;
    if (p.mirostat_threshold >= 0.f) {
        float floor_value = p.mirostat_threshold;
        const float mx = reduce_max(vals, n, sh);
        if (mx > 0.f) {
            int kept_ties = 0;
            if (mx < floor_value) {
                // nothing reaches the threshold: only the best candidate is kept (the first of equals)
                floor_value = mx;
                kept_ties = 1;
            }
            float kept = 0.f;
            for (int i = tid; i < n; i += THREADS) if (vals[i] >= floor_value) kept += vals[i];
            kept = lp_block_sum(kept, sh.fscratch);
            if (kept_ties == 1) kept = mx;
            const float r = p.uniform * kept;
            unsigned cut;
            int ties;
            if (kept_ties == 1) {
                chosen = nth_tie(vals, n, ordered_key(mx), floor_value, 0, sh);
            } else if (descending_cut(vals, n, r, floor_value, &cut, &ties, sh)) {
                chosen = nth_tie(vals, n, cut, floor_value, ties - 1, sh);
            } else {
                chosen = nth_tie(vals, n, ordered_key(mx), floor_value, 0, sh);
            }
            if (chosen >= 0 && kept > 0.f) observed = vals[chosen] / kept;
        }
    }
    if (chosen < 0) {
        // inverse CDF in index order
        const int chunk = (n + THREADS - 1) / THREADS;
        const int cb = tid * chunk, ce = min(n, cb + chunk);
        float mine = 0.f;
        for (int i = cb; i < ce; ++i) mine += vals[i];
        float total;
        const float before = block_exclusive_scan(mine, sh, &total);
        __syncthreads();
        if (tid == 0) sh.bcast_i = 0x7fffffff;
        __syncthreads();
        if (cb < ce && p.uniform < before + mine) atomicMin(&sh.bcast_i, tid);
        __syncthreads();
        const int owner = sh.bcast_i;
        __syncthreads();
        if (owner == 0x7fffffff) {
            if (tid == 0) { out_token[b] = V - 1; out_prob[b] = 0.f; }
            return;
        }
        if (tid == owner) {
            float cum = before;
            int hit = ce - 1;
            for (int i = cb; i < ce; ++i) {
                cum += vals[i];
                if (p.uniform < cum) { hit = i; break; }
            }
            sh.bcast_i = hit;
        }
        __syncthreads();
        chosen = sh.bcast_i;
        observed = vals[chosen];
    }
    if (tid == 0) {
        out_token[b] = ids ? ids[chosen] : chosen;
        out_prob[b] = observed;
    }
}

}  // namespace

// logits: float32 rows of `vocab` values, `logits_stride` apart; work: [B, vocab] float32 scratch;
// params: [B]; edits: tokens with the amount to subtract and the factor of the repetition penalty.
extern "C" int lp_sample(const float* logits, long long logits_stride, float* work, int vocab, const void* params,
                         int B, const int* edit_token, const float* edit_subtract, const float* edit_factor,
                         int* out_token, float* out_prob, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (vocab <= 0) LP_REFUSE("sample: vocabulary of %d", vocab);
    lp_launch(sample_kernel, B, THREADS, 0, stream, logits, logits_stride, work, vocab, (const LpSampleParams*)params,
              edit_token, edit_subtract, edit_factor, out_token, out_prob);
    return lp_check_launch("sample");
}

extern "C" int lp_sample_params_size() { return (int)sizeof(LpSampleParams); }

// ---------------------------------------------------------------- greedy choice for whole batches
// First-maximum argmax of each row in two stages, so that a few rows still use many SMs:
// grid (ARGMAX_CHUNKS, B) finds the best of each slice, then one block per row picks among them.
namespace {
constexpr int ARGMAX_CHUNKS = 32;

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
    return bi < 0 || v > bv || (v == bv && i < bi);
}

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, long long stride, int V, float* __restrict__ part_val,
                      int* __restrict__ part_idx) {
    __shared__ float sv[8];
    __shared__ int si[8];
    lp_grid_release();
    lp_grid_wait();
    const int b = blockIdx.y, c = blockIdx.x;
    const int per = (V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
    const int begin = c * per, end = min(V, begin + per);
    const float* row = logits + (long long)b * stride;
    float bv = -INFINITY;
    int bi = -1;
    for (int i = begin + threadIdx.x; i < end; i += 256) {
        const float v = row[i];
        if (bi < 0 || v > bv) { bv = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (si[w] >= 0 && better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
        part_val[b * ARGMAX_CHUNKS + c] = bv;
        part_idx[b * ARGMAX_CHUNKS + c] = bi;
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx,
                                    int* __restrict__ out_token) {
    lp_grid_release();
    lp_grid_wait();
    const int b = blockIdx.x, lane = threadIdx.x;       // 32 threads, one per slice
    float bv = part_val[b * ARGMAX_CHUNKS + lane];
    int bi = part_idx[b * ARGMAX_CHUNKS + lane];
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out_token[b] = bi < 0 ? 0 : bi;
}
}  // namespace

// scratch: B * 32 floats followed by B * 32 ints (lp_argmax_scratch_bytes).
extern "C" long long lp_argmax_scratch_bytes(int B) { return (long long)B * ARGMAX_CHUNKS * 8; }

extern "C" int lp_argmax(const float* logits, long long stride, int V, int B, void* scratch, int* out_token,
                         cudaStream_t stream) {
    if (B <= 0) return 0;
    if (V <= 0) LP_REFUSE("argmax: vocabulary of %d", V);
    if (B > 65535) LP_REFUSE("argmax: %d rows exceed the grid", B);
    float* part_val = (float*)scratch;
    int* part_idx = (int*)(part_val + (size_t)B * ARGMAX_CHUNKS);
    lp_launch(argmax_partial_kernel, dim3(ARGMAX_CHUNKS, B), 256, 0, stream, logits, stride, V, part_val, part_idx);
    int rc = lp_check_launch("argmax");
    if (rc) return rc;
    lp_launch(argmax_final_kernel, B, 32, 0, stream, (const float*)part_val, (const int*)part_idx, out_token);
    return lp_check_launch("argmax");
}
