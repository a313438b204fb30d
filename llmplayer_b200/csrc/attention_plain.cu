// Plain attention of a batch of query tokens over the paged key/value cache.
//
// One block per (query token, query head). Keys are visited in blocks of 128
// aligned to absolute positions; within a block one thread scores one key, the
// running maximum and sum are updated (online softmax, all float32), then each
// thread owns output features and adds the block's weighted values in increasing
// key order. The order of every sum depends only on the query's position and the
// window, never on how tokens were cut into steps or batched.
//
// Counterpart in the reference: src/main/resources/kernels/cuda/attention.cu:10-108
// (one query, scores in shared memory) and the online-softmax variant
// inference/Attention.java:161-207.
#include "common.cuh"

namespace {

constexpr int KB = 128;       // keys per block = threads per block
constexpr int MAX_HD = 256;

template <typename TQ, typename TKV>
__global__ void __launch_bounds__(KB)
attention_plain_kernel(const TQ* __restrict__ q, TQ* __restrict__ out, const TKV* __restrict__ pages,
                       const int* __restrict__ page_table, int pt_stride, const int* __restrict__ seq_ids,
                       const int* __restrict__ positions, int H, int G, int hd, int page_size, float scale,
                       int window) {
    __shared__ float qs[MAX_HD];
    __shared__ float prob[KB];
    __shared__ long long row_off[KB];
    __shared__ float scratch[32];

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int g = h / (H / G);
    const int seq = seq_ids[t];
    const int pos = positions[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    const TQ* qr = q + ((long long)t * H + h) * hd;
    for (int i = tid; i < hd; i += KB) qs[i] = lp_to_float(qr[i]);
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc0 = 0.f, acc1 = 0.f;   // features tid and tid + 128
    const int* pt = page_table + (long long)seq * pt_stride;

    for (int c0 = (lo / KB) * KB; c0 <= pos; c0 += KB) {
        const int key = c0 + tid;
        const bool valid = key >= lo && key <= pos;
        float sc = -INFINITY;
        if (valid) {
            const int page = pt[key / page_size];
            const long long off = (((long long)page * 2 * G + g) * page_size + (key % page_size)) * hd;
            row_off[tid] = off;
            const TKV* kr = pages + off;
            float dot = 0.f;
            for (int i = 0; i < hd; ++i) dot = fmaf(qs[i], lp_to_float(kr[i]), dot);
            sc = dot * scale;
        }
        const float cmax = lp_block_max(sc, scratch);
        const float m_new = fmaxf(m, cmax);
        const float pr = valid ? expf(sc - m_new) : 0.f;
        prob[tid] = pr;
        const float csum = lp_block_sum(pr, scratch);   // also publishes prob[] and row_off[]
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * alpha + csum;
        acc0 *= alpha;
        acc1 *= alpha;
        const int nk = (pos - c0 + 1 < KB) ? pos - c0 + 1 : KB;
        const int first = lo > c0 ? lo - c0 : 0;
        const long long v_shift = (long long)G * page_size * hd;    // from a K row to its V row
        if (tid < hd) {
            for (int j = first; j < nk; ++j)
                acc0 = fmaf(prob[j], lp_to_float(pages[row_off[j] + v_shift + tid]), acc0);
        }
        if (tid + KB < hd) {
            for (int j = first; j < nk; ++j)
                acc1 = fmaf(prob[j], lp_to_float(pages[row_off[j] + v_shift + tid + KB]), acc1);
        }
        m = m_new;
        __syncthreads();
    }
    const float inv = 1.0f / l;
    TQ* o = out + ((long long)t * H + h) * hd;
    if (tid < hd) o[tid] = lp_from_float<TQ>(acc0 * inv);
    if (tid + KB < hd) o[tid + KB] = lp_from_float<TQ>(acc1 * inv);
}

}  // namespace

// q, out: [T, H, hd]; pages: [num_pages, 2, G, page_size, hd]; page_table: [B, pt_stride];
// seq_ids, positions: [T]. window <= 0: all keys up to the query's position.
extern "C" int lp_attention_plain(const void* q, void* out, int q_dtype, const void* pages, int kv_dtype,
                                  const int* page_table, int pt_stride, const int* seq_ids, const int* positions,
                                  int T, int H, int G, int hd, int page_size, float scale, int window,
                                  cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G) LP_REFUSE("attention_plain: %d query heads over %d key heads", H, G);
    if (hd <= 0 || hd > MAX_HD) LP_REFUSE("attention_plain: head size %d (supported: 1..%d)", hd, MAX_HD);
    if (page_size <= 0) LP_REFUSE("attention_plain: page size %d", page_size);
    if (H > 65535) LP_REFUSE("attention_plain: %d heads exceed the grid", H);
    dim3 grid(T, H);
#define LP_LAUNCH_ATT(TQ, TKV)                                                                                 \
    attention_plain_kernel<TQ, TKV><<<grid, KB, 0, stream>>>((const TQ*)q, (TQ*)out, (const TKV*)pages,          \
                                                             page_table, pt_stride, seq_ids, positions, H, G,  \
                                                             hd, page_size, scale, window)
    if (q_dtype == LP_F32 && kv_dtype == LP_F32) LP_LAUNCH_ATT(float, float);
    else if (q_dtype == LP_BF16 && kv_dtype == LP_BF16) LP_LAUNCH_ATT(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == LP_F32 && kv_dtype == LP_BF16) LP_LAUNCH_ATT(float, __nv_bfloat16);
    else if (q_dtype == LP_BF16 && kv_dtype == LP_F32) LP_LAUNCH_ATT(__nv_bfloat16, float);
    else LP_REFUSE("attention_plain: dtype codes q=%d kv=%d", q_dtype, kv_dtype);
#undef LP_LAUNCH_ATT
    return lp_check_launch("attention_plain");
}
