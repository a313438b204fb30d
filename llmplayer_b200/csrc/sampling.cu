// Sampling on the device: a row of float32 logits becomes a token; one block per sequence draws it,
// several blocks per sequence find the candidates of a small top-k beforehand.
//
// Stages, in the reference's order (sampler/CompositeSampler.java:33-120):
//   logit edits (DRY subtraction, then repetition penalty: positive / r, else * r)
//   -> first-maximum argmax if greedy (:259-269)
//   -> * 1/temperature -> top-k by threshold, ties at the threshold survive (:70-78)
//   -> softmax (:80-98) -> min-p (:122-139) -> top-p over descending probabilities (:303-352)
//   -> mirostat v2 truncation and draw in descending order (:206-250), or an inverse-CDF
//      walk in index order with the last vocabulary index as fallback (:387-395).
// The reference sorts the vocabulary. Here the k-th largest value is found by a radix selection over
// the ordered bit patterns of the floats (four passes with a histogram of 8-bit digits), and the
// survivors are gathered into shared memory. A set of at most 1024 candidates is then ranked in
// descending order (equal values in index order, as a stable sort would) and one thread walks
// it, adding the probabilities one by one as the reference does. Larger sets (no top-k, or a very
// wide one) stay in global memory: top-p first looks for its cut among the largest 256 values and
// carries only those on when it lies there; else the key at the cut is searched over the whole row,
// four bits per pass.
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
constexpr int CAP = THREADS;   // candidates kept in shared memory after top-k: one per thread
constexpr int TOP_P_TRY = 256; // top-p without top-k looks for its cut among this many largest values first
constexpr int STAGE = 2048;    // values that the slices of a row may hand over together
constexpr int SLICE_MAX = 8192;   // values of a row that one block of the first stage takes
constexpr int SLICES_MAX = 32;

// Scratch of the radix selection.
struct Select {
    int hist[256];
    int digit, k, above, equal;
};

struct Shared {
    float fscratch[32];
    int iscratch[32];
    float scan[THREADS];
    float cand_val[CAP];       // the candidates in index order ...
    int cand_idx[CAP];         // ... and their places in the vocabulary
    float sorted[CAP];         // a small set in descending order (also the staging area of the gather) ...
    int order[CAP];            // ... and where each of its values lies in the set
    float stage_val[STAGE];    // what the first stage handed over ...
    int stage_idx[STAGE];      // ... with the places in the vocabulary
    int slice_at[SLICES_MAX + 1];
    float many[16][32];        // 15 sums at a time: per warp, and (row 15) over the block
    Select select;
    int bcast_i;
    float bcast_f;
};

// How a row of `vocab` values is cut for the first stage: `slices` blocks take `slice_len` values each and
// hand over at most `capacity` of them. slices == 0: the vocabulary is too large for that.
struct SlicePlan { int slices, slice_len, capacity; };
inline SlicePlan slice_plan(int vocab) {
    SlicePlan plan;
    plan.slices = vocab < 1024 ? 1 : (vocab + 1023) / 1024;
    if (plan.slices > 16) plan.slices = 16;
    plan.slice_len = (vocab + plan.slices - 1) / plan.slices;
    if (plan.slice_len > SLICE_MAX) {
        plan.slices = (vocab + SLICE_MAX - 1) / SLICE_MAX;
        plan.slice_len = (vocab + plan.slices - 1) / plan.slices;
    }
    if (plan.slices > SLICES_MAX) { plan.slices = 0; plan.slice_len = 0; plan.capacity = 0; return plan; }
    plan.capacity = STAGE / plan.slices < CAP ? STAGE / plan.slices : CAP;
    return plan;
}

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
// Warps scan their own 32 values with shuffles, the first warp scans the 32 warp sums.
template <typename T>
__device__ T block_exclusive_scan(T v, Shared& sh, T* total) {
    static_assert(sizeof(T) == 4, "the scan area holds 32-bit values");
    T* area = reinterpret_cast<T*>(sh.scan);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T run = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T up = __shfl_up_sync(0xffffffffu, run, o);
        if (lane >= o) run += up;
    }
    const T lanes_before = __shfl_up_sync(0xffffffffu, run, 1);
    __syncthreads();
    if (lane == 31) area[warp] = run;
    __syncthreads();
    if (warp == 0) {
        const T sum = area[lane];
        T wrun = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const T up = __shfl_up_sync(0xffffffffu, wrun, o);
            if (lane >= o) wrun += up;
        }
        const T wbefore = __shfl_up_sync(0xffffffffu, wrun, 1);
        area[32 + lane] = lane == 0 ? T(0) : wbefore;           // what lies before this warp
        if (lane == 31) area[64] = wrun;
    }
    __syncthreads();
    const T before = area[32 + warp] + (lane == 0 ? T(0) : lanes_before);
    *total = area[64];
    __syncthreads();
    return before;
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

// Largest key t such that at least k values have key >= t: the key of the k-th largest value
// (1 <= k <= n). *at_least gets how many values have a key >= t. Four passes, one per 8-bit digit
// of the keys from the top: a histogram of that digit over the values that agree with the digits
// found so far, then the digit in which the k-th largest lies. Lanes of a warp that meet the same
// digit add to the histogram once, together.
__device__ unsigned kth_largest_key(const float* vals, int n, int k, Select& sel, int* at_least) {
    unsigned prefix = 0;
    int greater = 0, equal = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (threadIdx.x < 256) sel.hist[threadIdx.x] = 0;
        __syncthreads();
        const unsigned settled = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
        // eight values per thread are fetched before any is counted, so that their latencies overlap
        for (int base = 0; base < n; base += 8 * THREADS) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * THREADS + (int)threadIdx.x;
                v[u] = i < n ? vals[i] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * THREADS + (int)threadIdx.x;
                const unsigned key = ordered_key(v[u]);
                const bool in = i < n && (key & settled) == prefix;
                const unsigned takers = __ballot_sync(0xffffffffu, in);
                if (in) {
                    const unsigned digit = (key >> shift) & 0xffu;
                    const unsigned same = __match_any_sync(takers, digit);
                    if ((int)(threadIdx.x & 31) == __ffs(same) - 1) atomicAdd(&sel.hist[digit], __popc(same));
                }
            }
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            const int lane = threadIdx.x;
            const int top = 255 - 8 * lane;            // lane 0 owns the 8 highest digits
            int h[8], mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) { h[j] = sel.hist[top - j]; mine += h[j]; }
            int cum = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, cum, o);
                if (lane >= o) cum += up;
            }
            const unsigned reach = __ballot_sync(0xffffffffu, cum >= k);
            const int owner = reach ? __ffs(reach) - 1 : 31;
            if (lane == owner) {
                int above = cum - mine, digit = top - 7, eq = h[7];
                bool found = false;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (!found) {
                        if (above + h[j] >= k || j == 7) { found = true; digit = top - j; eq = h[j]; }
                        else above += h[j];
                    }
                sel.digit = digit;
                sel.above = above;
                sel.equal = eq;
                sel.k = max(1, k - above);
            }
        }
        __syncthreads();
        prefix |= (unsigned)sel.digit << shift;
        greater += sel.above;
        equal = sel.equal;
        k = sel.k;
    }
    *at_least = greater + equal;
    return prefix;
}

// The `count` (<= CAP) values whose key is >= thr, gathered into cand_val / cand_idx in the order of their
// places in the vocabulary (ids[i], or i itself without ids): first in the order in which the threads find
// them, then each to the rank of its place.
__device__ void gather_candidates(const float* vals, const int* ids, int n, unsigned thr, int count, Shared& sh) {
    if (threadIdx.x == 0) sh.bcast_i = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += THREADS) {
        const float v = vals[i];
        if (ordered_key(v) >= thr) {
            const int at = atomicAdd(&sh.bcast_i, 1);
            if (at < CAP) { sh.sorted[at] = v; sh.order[at] = ids ? ids[i] : i; }
        }
    }
    __syncthreads();
    if ((int)threadIdx.x < count) {
        const int mine = sh.order[threadIdx.x];
        int rank = 0;
        for (int j = 0; j < count; ++j) rank += sh.order[j] < mine;
        sh.cand_val[rank] = sh.sorted[threadIdx.x];
        sh.cand_idx[rank] = mine;
    }
    __syncthreads();
}

// Ranks n <= CAP values in descending order, equal ones in index order: sh.sorted[r] is the r-th
// value and sh.order[r] its place among the values.
__device__ void sort_descending(const float* vals, int n, Shared& sh) {
    __syncthreads();
    if ((int)threadIdx.x < n) {
        const float v = vals[threadIdx.x];
        int rank = 0;
        for (int j = 0; j < n; ++j) {
            const float o = vals[j];
            rank += (o > v) || (o == v && j < (int)threadIdx.x);
        }
        sh.sorted[rank] = v;
        sh.order[rank] = threadIdx.x;
    }
    __syncthreads();
}

// One thread adds list[0], list[1], ... one by one, while they are positive and >= floor_value, and
// stops at the first place where the sum exceeds `target`. Returns that place (-1 if the sum never
// exceeds it); *walked gets how many values were positive and >= floor_value up to there, *sum
// their sum. For thread 0 only; eight values are fetched at a time.
__device__ int walk_until(const float* list, int n, float target, float floor_value, bool stop_at_zero, int* walked,
                          float* sum) {
    float cum = 0.f;
    int hit = -1, count = 0;
    bool done = false;
    for (int r0 = 0; r0 < n && !done; r0 += 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = r0 + j < n ? list[r0 + j] : -1.f;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (!done) {
                if (v[j] < 0.f || (stop_at_zero && !(v[j] > 0.f)) || v[j] < floor_value) done = true;
                else {
                    cum += v[j];
                    ++count;
                    if (cum > target) { hit = r0 + j; done = true; }
                }
            }
    }
    *walked = count;
    *sum = cum;
    return hit;
}

// Walk the values >= floor_value in descending order (equal ones in index order) until the running
// sum exceeds `target`. Returns false if it never does. Otherwise *cut_key is the key of the value
// at which it does, and *ties_kept how many of the values equal to it (in index order) lie up to
// and including that point.
__device__ bool descending_cut(const float* vals, int n, float target, float floor_value, unsigned* cut_key,
                               int* ties_kept, Shared& sh) {
    // The key is settled four bits at a time: for each of the 15 non-zero digits d, the sum of the values
    // whose key is >= prefix | d << shift, and the largest digit whose sum still exceeds the target. Each
    // sum is formed in the order in which a search bit by bit would form it.
    unsigned prefix = 0;
    bool any = false;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int shift = 28; shift >= 0; shift -= 4) {
        const unsigned settled = shift == 28 ? 0u : (0xffffffffu << (shift + 4));
        float acc[15];
#pragma unroll
        for (int j = 0; j < 15; ++j) acc[j] = 0.f;
        for (int i = threadIdx.x; i < n; i += THREADS) {
            const float v = vals[i];
            if (v >= floor_value && v > 0.f) {
                const unsigned key = ordered_key(v);
                const unsigned high = key & settled;
                // how many of the 15 candidates this key reaches
                const int reaches = high > prefix ? 15 : high < prefix ? 0 : (int)((key >> shift) & 15u);
#pragma unroll
                for (int j = 0; j < 15; ++j) acc[j] += reaches > j ? v : 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < 15; ++j) acc[j] = lp_warp_sum(acc[j]);
        __syncthreads();
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < 15; ++j) sh.many[j][warp] = acc[j];
        }
        __syncthreads();
        if (threadIdx.x < 15) {
            float total = 0.f;
            for (int w = 0; w < THREADS / 32; ++w) total += sh.many[threadIdx.x][w];
            sh.many[15][threadIdx.x] = total;
        }
        __syncthreads();
        int digit = 0;
#pragma unroll
        for (int j = 0; j < 15; ++j)
            if (sh.many[15][j] > target) digit = j + 1;
        if (digit > 0) { prefix |= (unsigned)digit << shift; any = true; }
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
    int total;
    const int before = block_exclusive_scan(mine, sh, &total);
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
    int total;
    int seen = block_exclusive_scan(mine, sh, &total);
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

// ---------------------------------------------------------------- top-k in two stages
// A row of a large vocabulary is more than one block reads quickly. When top-k is small, `slices` blocks
// per row each take a slice of it into shared memory (edited, divided by the temperature), find the
// k-th largest of their slice and hand over what reaches it. Every value that reaches the k-th largest
// of the whole row is among those, so the second stage selects among a few hundred values on chip.
struct SliceShared {
    float vals[SLICE_MAX];
    Select select;
    int count;
};

// Per row, in 4-byte words: SLICES_MAX counts (-1: nothing handed over, the second stage reads the whole
// row), then STAGE values, then STAGE places; slice c owns the `capacity` slots from c * capacity.
constexpr int SELECT_WORDS = SLICES_MAX + 2 * STAGE;

__global__ void __launch_bounds__(THREADS)
sample_slices_kernel(const float* __restrict__ logits, long long logits_stride, int V,
                     const LpSampleParams* __restrict__ params, const int* __restrict__ edit_token,
                     const float* __restrict__ edit_subtract, const float* __restrict__ edit_factor,
                     int slice_len, int capacity, int* __restrict__ select) {
    __shared__ SliceShared sh;
    lp_grid_release();
    lp_grid_wait();
    const int b = blockIdx.y, c = blockIdx.x, tid = threadIdx.x;
    const LpSampleParams p = params[b];
    int* row_select = select + (long long)b * SELECT_WORDS;
    int* count_out = row_select + c;
    float* out_val = reinterpret_cast<float*>(row_select + SLICES_MAX) + c * capacity;
    int* out_idx = row_select + SLICES_MAX + STAGE + c * capacity;
    const bool wanted = p.inv_temperature != 0.f && p.top_k > 0 && p.top_k < V && p.top_k <= capacity;
    if (!wanted) {
        if (tid == 0) *count_out = -1;
        return;
    }
    const int begin = c * slice_len;
    const int len = min(V - begin, slice_len);
    if (len <= 0) {
        if (tid == 0) *count_out = 0;
        return;
    }
    const float* row = logits + (long long)p.logits_row * logits_stride;
    for (int i = tid; i < len; i += THREADS) sh.vals[i] = row[begin + i] * p.inv_temperature;
    __syncthreads();
    for (int e = tid; e < p.edit_count; e += THREADS) {          // edited tokens are distinct
        const int tok = edit_token[p.edit_begin + e];
        if (tok >= begin && tok < begin + len) {
            float v = row[tok] - edit_subtract[p.edit_begin + e];
            const float f = edit_factor[p.edit_begin + e];
            v = v > 0.f ? v / f : v * f;
            sh.vals[tok - begin] = v * p.inv_temperature;
        }
    }
    __syncthreads();
    int reach;
    const unsigned thr = kth_largest_key(sh.vals, len, min(p.top_k, len), sh.select, &reach);
    if (reach > capacity) {                                      // many equal values at the threshold
        if (tid == 0) *count_out = -1;
        return;
    }
    if (tid == 0) sh.count = 0;
    __syncthreads();
    for (int i = tid; i < len; i += THREADS) {
        const float v = sh.vals[i];
        if (ordered_key(v) >= thr) {
            const int at = atomicAdd(&sh.count, 1);
            if (at < capacity) { out_val[at] = v; out_idx[at] = begin + i; }
        }
    }
    if (tid == 0) *count_out = reach;
}

// Second stage: take what the slices of this row handed over, find the k-th largest among it and gather
// what reaches it as the candidates. False if a slice handed nothing over, or too much came together.
__device__ bool take_slices(const int* __restrict__ row_select, int slices, int capacity, int top_k, Shared& sh,
                            int* n_out) {
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const int count = lane < slices ? row_select[lane] : 0;
        const bool bad = count < 0 || count > capacity;
        int run = bad ? 0 : count;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, run, o);
            if (lane >= o) run += up;
        }
        const bool any_bad = __any_sync(0xffffffffu, bad);
        sh.slice_at[lane + 1] = run;
        if (lane == 0) { sh.slice_at[0] = 0; sh.bcast_i = any_bad ? 0 : 1; }
    }
    __syncthreads();
    const int total = sh.slice_at[slices];
    const bool usable = sh.bcast_i != 0 && total >= top_k && total <= STAGE;
    __syncthreads();
    if (!usable) return false;
    const float* in_val = reinterpret_cast<const float*>(row_select + SLICES_MAX);
    const int* in_idx = row_select + SLICES_MAX + STAGE;
    for (int pos = threadIdx.x; pos < slices * capacity; pos += THREADS) {
        const int c = pos / capacity, j = pos - c * capacity;
        const int at = sh.slice_at[c];
        if (j < sh.slice_at[c + 1] - at) { sh.stage_val[at + j] = in_val[pos]; sh.stage_idx[at + j] = in_idx[pos]; }
    }
    __syncthreads();
    int reach;
    const unsigned thr = kth_largest_key(sh.stage_val, total, top_k, sh.select, &reach);
    if (reach > CAP) return false;
    gather_candidates(sh.stage_val, sh.stage_idx, total, thr, reach, sh);
    *n_out = reach;
    return true;
}

__global__ void __launch_bounds__(THREADS, 1)
sample_kernel(const float* __restrict__ logits, long long logits_stride, float* __restrict__ work, int V,
              const LpSampleParams* __restrict__ params, const int* __restrict__ edit_token,
              const float* __restrict__ edit_subtract, const float* __restrict__ edit_factor,
              const int* __restrict__ select, int slices, int capacity, int* __restrict__ out_token,
              float* __restrict__ out_prob) {
    __shared__ Shared sh;
    lp_grid_release();
    lp_grid_wait();
    const int b = blockIdx.x, tid = threadIdx.x;
    const LpSampleParams p = params[b];
    const float* src = logits + (long long)p.logits_row * logits_stride;
    float* w = work + (long long)b * V;

    const bool greedy = p.inv_temperature == 0.f;
    float* vals = w;
    const int* ids = nullptr;
    int n = V;
    // the candidates may have been handed over by the first stage; else the whole row is read here
    bool handed = false;
    if (select != nullptr && !greedy && p.top_k > 0 && p.top_k < V && p.top_k <= capacity)
        handed = take_slices(select + (long long)b * SELECT_WORDS, slices, capacity, p.top_k, sh, &n);
    if (handed) { vals = sh.cand_val; ids = sh.cand_idx; }

    const float* cur = src;
    if (!handed && (!greedy || p.edit_count > 0)) {
        // the row, edited and divided by the temperature (an edit comes before the division)
        const float scale = greedy ? 1.f : p.inv_temperature;
        for (int i = tid; i < V; i += THREADS) w[i] = src[i] * scale;
        __syncthreads();
        for (int e = tid; e < p.edit_count; e += THREADS) {          // edited tokens are distinct
            const int tok = edit_token[p.edit_begin + e];
            if (tok >= 0 && tok < V) {
                float v = src[tok] - edit_subtract[p.edit_begin + e];
                const float f = edit_factor[p.edit_begin + e];
                v = v > 0.f ? v / f : v * f;
                w[tok] = v * scale;
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

    if (!handed && p.top_k > 0 && p.top_k < V) {
        int survivors;
        const unsigned thr = kth_largest_key(w, V, p.top_k, sh.select, &survivors);
        if (survivors <= CAP) {
            gather_candidates(w, nullptr, V, thr, survivors, sh);
            vals = sh.cand_val; ids = sh.cand_idx; n = survivors;
        } else {
            for (int i = tid; i < V; i += THREADS) if (ordered_key(w[i]) < thr) w[i] = -INFINITY;
            __syncthreads();
        }
    }
    bool small = n <= CAP;            // ranked and walked by one thread, else searched by all

    // softmax
    const float m = reduce_max(vals, n, sh);
    float part = 0.f;
    for (int i = tid; i < n; i += THREADS) {
        const float e = (vals[i] == -INFINITY) ? 0.f : expf(vals[i] - m);
        vals[i] = e;
        part += e;
    }
    float s = lp_block_sum(part, sh.fscratch);
    float largest = 1.f;
    if (s > 0.f) {
        const float inv = 1.0f / s;
        for (int i = tid; i < n; i += THREADS) vals[i] *= inv;
        largest = inv;
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
        const int positives = block_sum_int(c, sh.iscratch);
        if (positives > 1) {
            // The cut mostly lies among the largest few values: if the TOP_P_TRY largest together exceed
            // top-p, everything else goes, and the candidates alone are carried on. (Before min-p the largest
            // probability is the softmax's exp(0) / sum: that many times it bounds what they hold.)
            if (!small && (p.min_p > 0.f || (float)TOP_P_TRY * largest > p.top_p)) {
                int reach;
                const unsigned thr = kth_largest_key(vals, n, min(TOP_P_TRY, positives), sh.select, &reach);
                if (reach <= CAP) {
                    gather_candidates(vals, nullptr, n, thr, reach, sh);
                    sort_descending(sh.cand_val, reach, sh);
                    if (tid == 0) {
                        int walked;
                        float sum;
                        sh.bcast_i = walk_until(sh.sorted, reach, p.top_p, 0.f, true, &walked, &sum);
                    }
                    __syncthreads();
                    const bool inside = sh.bcast_i >= 0;
                    __syncthreads();
                    if (inside) { vals = sh.cand_val; ids = sh.cand_idx; n = reach; small = true; }
                }
            }
            if (small) {
                sort_descending(vals, n, sh);
                if (tid == 0) {
                    int walked;
                    float sum;
                    sh.bcast_i = walk_until(sh.sorted, n, p.top_p, 0.f, true, &walked, &sum);
                }
                __syncthreads();
                const int cut = sh.bcast_i;
                if (cut >= 0) {
                    if (tid < n && tid > cut) vals[sh.order[tid]] = 0.f;      // this thread takes rank `tid`
                    __syncthreads();
                    s = reduce_sum(vals, n, sh);
                    if (s > 0.f) {
                        const float inv = 1.0f / s;
                        for (int i = tid; i < n; i += THREADS) vals[i] *= inv;
                    }
                }
                __syncthreads();
            } else {
                unsigned cut;
                int ties;
                if (descending_cut(vals, n, p.top_p, 0.f, &cut, &ties, sh)) keep_until_cut(vals, n, cut, ties, sh);
            }
        }
    }

    int chosen = -1;          // index into vals
    float observed = 0.f;
    if (p.mirostat_threshold >= 0.f && small) {
        const float mx = reduce_max(vals, n, sh);
        if (mx > 0.f) {
            sort_descending(vals, n, sh);
            if (tid == 0) {
                // what reaches the threshold is kept, the best candidate at least
                int keep, walked;
                float kept, sum;
                walk_until(sh.sorted, n, INFINITY, p.mirostat_threshold, true, &keep, &kept);
                if (keep == 0) { keep = 1; kept = sh.sorted[0]; }
                int hit = 0;
                if (kept > 0.f) {
                    hit = walk_until(sh.sorted, keep, p.uniform * kept, 0.f, false, &walked, &sum);
                    if (hit < 0) hit = 0;
                }
                sh.bcast_i = sh.order[hit];
                sh.bcast_f = kept;
            }
            __syncthreads();
            chosen = sh.bcast_i;
            const float kept = sh.bcast_f;
            if (kept > 0.f) observed = vals[chosen] / kept;
            __syncthreads();
        }
    } else if (p.mirostat_threshold >= 0.f) {
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
    if (chosen < 0 && small) {
        // inverse CDF in index order, one value after the other
        if (tid == 0) {
            int walked;
            float sum;
            sh.bcast_i = walk_until(vals, n, p.uniform, 0.f, false, &walked, &sum);
        }
        __syncthreads();
        chosen = sh.bcast_i;
        if (chosen < 0) {
            if (tid == 0) { out_token[b] = V - 1; out_prob[b] = 0.f; }
            return;
        }
        observed = vals[chosen];
    } else if (chosen < 0) {
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
// select: nullptr, or [B, lp_sample_select_words()] 4-byte words of scratch: the rows whose top-k is at most
// lp_sample_slice_capacity(vocab) then have their candidates found by several blocks each.
extern "C" int lp_sample(const float* logits, long long logits_stride, float* work, int vocab, const void* params,
                         int B, const int* edit_token, const float* edit_subtract, const float* edit_factor,
                         int* select, int* out_token, float* out_prob, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (vocab <= 0) LP_REFUSE("sample: vocabulary of %d", vocab);
    const SlicePlan plan = slice_plan(vocab);
    if (plan.slices == 0) select = nullptr;
    if (select != nullptr) {
        lp_launch(sample_slices_kernel, dim3(plan.slices, B), THREADS, 0, stream, logits, logits_stride, vocab,
                  (const LpSampleParams*)params, edit_token, edit_subtract, edit_factor, plan.slice_len, plan.capacity,
                  select);
        if (int rc = lp_check_launch("sample (slices)")) return rc;
    }
    lp_launch(sample_kernel, B, THREADS, 0, stream, logits, logits_stride, work, vocab, (const LpSampleParams*)params,
              edit_token, edit_subtract, edit_factor, (const int*)select, plan.slices, plan.capacity, out_token,
              out_prob);
    return lp_check_launch("sample");
}

extern "C" int lp_sample_params_size() { return (int)sizeof(LpSampleParams); }
extern "C" int lp_sample_select_words() { return SELECT_WORDS; }
extern "C" int lp_sample_slice_capacity(int vocab) { return vocab > 0 ? slice_plan(vocab).capacity : 0; }

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

// ---------------------------------------------------------------- the step's sampler block, fetched by a kernel
// A captured decode step whose sampler block lies in page-locked host memory (see lp_decode_loop_sampled in
// host_loop.cu): block i brings record i and as many of sequence i's edits as the record names, so that a step
// moves what it uses and not the whole capacity. host: the page-locked block (device-readable); dev: the same
// layout in device memory (records, then per sequence `cap` tokens, `cap` amounts, `cap` factors).
__global__ void sample_fetch_kernel(const int* __restrict__ host, int* __restrict__ dev, int B, int cap, int record_words,
                                    int field_count) {
    lp_grid_release();
    lp_grid_wait();
    const int i = blockIdx.x;
    for (int w = threadIdx.x; w < record_words; w += blockDim.x) dev[(size_t)i * record_words + w] = host[(size_t)i * record_words + w];
    int count = host[(size_t)i * record_words + field_count];
    count = count < 0 ? 0 : (count > cap ? cap : count);
    const size_t edits = (size_t)B * record_words;
    for (int part = 0; part < 3; ++part) {
        const size_t base = edits + ((size_t)part * B + i) * cap;
        for (int j = threadIdx.x; j < count; j += blockDim.x) dev[base + j] = host[base + j];
    }
}

extern "C" int lp_sample_fetch(const int* host, int* dev, int B, int cap, int record_words, int field_count,
                               cudaStream_t stream) {
    if (B <= 0) return 0;
    if (!host || !dev || cap <= 0 || record_words <= 0 || field_count < 0 || field_count >= record_words)
        LP_REFUSE("sample_fetch: a block of %d records of %d words, %d edits each", B, record_words, cap);
    lp_launch(sample_fetch_kernel, B, 128, 0, stream, host, dev, B, cap, record_words, field_count);
    return lp_check_launch("sample_fetch");
}
