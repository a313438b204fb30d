// Tensor-core attention over the paged bfloat16 cache: one kernel for steps that bring
// many tokens per sequence (prefill), one for steps of one token per sequence (decode),
// and the merge of a decode step's partial results.
//
// Both kernels stream pages of 64 keys (and their values) into shared memory with
// cp.async (16-byte chunks, rotated per row so that ldmatrix reads are conflict-free),
// form scores with mma.sync m16n8k16 (bf16 in, fp32 out), keep a running maximum and sum
// per query row in float32 (online softmax, exp2 with the scale folded in) and accumulate
// probabilities times values with a second mma. Masks: a key is seen by a query at
// position p if key <= p and key > p - window (window <= 0: no window).
//
//  * prefill: a CTA takes 64 consecutive new tokens of one sequence and one query head;
//    each of its 4 warps owns 16 query rows and visits the pages its rows can see.
//  * decode:  a CTA takes one sequence, one key/value head and one share of the pages; the keys
//    are the 16 rows of the MMA and the (up to 8) query heads that share the key/value head its
//    columns, so each key and value is read once for all of them; each warp owns 16 of a page's
//    64 keys; the CTA writes an unnormalised partial result (max, sum, output), merged by a
//    second kernel or, in the fused form, by the last CTA of the group.
//
// Reference: src/main/resources/kernels/cuda/attention.cu:10-108 (one block per head,
// scores of one query in shared memory) and the online-softmax form of
// inference/Attention.java:161-207; head mapping kvHead = h / (H/G) (inference/Attention.java:212).
#include "tcgen05_utils.cuh"
#include "attention_decode.cuh"

namespace {


// ============================================================================ prefill
// grid: (tiles of 64 new tokens, H, B); 128 threads.
template <int HD_MAX>
__global__ void __launch_bounds__(128)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                         const __nv_bfloat16* __restrict__ pages, const int* __restrict__ page_table, int pt_stride,
                         const int* __restrict__ q_start, const int* __restrict__ kv_len, int H, int G, int hd,
                         float scale_log2, int window) {
    constexpr int KSTEPS = HD_MAX / 16;
    extern __shared__ __align__(128) uint8_t smem[];
    lp_grid_release();
    lp_grid_wait();
    const int b = blockIdx.z, h = blockIdx.y, tile = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t_begin = q_start[b], n_new = q_start[b + 1] - t_begin;
    if (tile * 64 >= n_new) return;
    const int g = h / (H / G);
    const int len = kv_len[b];
    const int pos0 = len - n_new;                       // position of the sequence's first new token
    const int row0 = tile * 64;                         // first query row of this CTA among the new tokens
    const int rows = min(64, n_new - row0);
    const int first_pos = pos0 + row0, last_pos = pos0 + row0 + rows - 1;
    const int lo = window > 0 ? max(0, first_pos - window + 1) : 0;
    const int page_lo = lo / PAGE, page_hi = last_pos / PAGE;
    const int* table = page_table + (size_t)b * pt_stride;
    const int stage_bytes = 2 * PAGE * hd * 2;

    // query fragments of this warp's 16 rows
    const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
    uint32_t qf[KSTEPS][4];
    {
        const __nv_bfloat16* q_lo = q + ((size_t)(t_begin + row0 + min(r_lo, rows - 1)) * H + h) * hd;
        const __nv_bfloat16* q_hi = q + ((size_t)(t_begin + row0 + min(r_hi, rows - 1)) * H + h) * hd;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            if (kk * 16 < hd) {
                const int c = kk * 16 + (lane & 3) * 2;
                qf[kk][0] = *reinterpret_cast<const uint32_t*>(q_lo + c);
                qf[kk][1] = *reinterpret_cast<const uint32_t*>(q_hi + c);
                qf[kk][2] = *reinterpret_cast<const uint32_t*>(q_lo + c + 8);
                qf[kk][3] = *reinterpret_cast<const uint32_t*>(q_hi + c + 8);
            }
        }
    }
    const int pos_lo = first_pos + min(r_lo, rows - 1), pos_hi = first_pos + min(r_hi, rows - 1);
    const int warp_last_pos = first_pos + min(warp * 16 + 15, rows - 1);
    const int warp_first_pos = first_pos + min(warp * 16, rows - 1);

    float o[KSTEPS * 2][4];
#pragma unroll
    for (int i = 0; i < KSTEPS * 2; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_lo = NEG_BIG, m_hi = NEG_BIG, l_lo = 0.f, l_hi = 0.f;

    load_page(smem, pages, table[page_lo], G, g, hd, tid, 128);
    cp_async_commit();
    for (int p = page_lo; p <= page_hi; ++p) {
        const int cur = (p - page_lo) & 1;
        if (p + 1 <= page_hi) load_page(smem + (cur ^ 1) * stage_bytes, pages, table[p + 1], G, g, hd, tid, 128);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int key_base = p * PAGE;
        // pages wholly after this warp's rows, or wholly before their windows, contribute nothing
        const bool active = key_base <= warp_last_pos &&
                            (window <= 0 || key_base + PAGE - 1 > warp_first_pos - window);
        if (active) {
            const uint32_t k_tile = smem_u32(smem + cur * stage_bytes);
            const uint32_t v_tile = k_tile + PAGE * hd * 2;
            float s[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) scores_16keys<KSTEPS>(&s[ks * 2], qf, k_tile, ks * 16, hd, lane);
            const bool edge = key_base + PAGE - 1 > warp_first_pos ||
                              (window > 0 && key_base <= warp_last_pos - window);
            float mx_lo = NEG_BIG, mx_hi = NEG_BIG;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key_base + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const int pos = (e < 2) ? pos_lo : pos_hi;
                    float v = s[nt][e] * scale_log2;
                    if (edge && (key > pos || (window > 0 && key <= pos - window))) v = NEG_BIG;
                    s[nt][e] = v;
                    if (e < 2) mx_lo = fmaxf(mx_lo, v); else mx_hi = fmaxf(mx_hi, v);
                }
            }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
            const float a_lo = exp2f(m_lo - mn_lo), a_hi = exp2f(m_hi - mn_hi);
            m_lo = mn_lo; m_hi = mn_hi;
            float sum_lo = 0.f, sum_hi = 0.f;
            uint32_t pf[4][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                float e0 = s[nt][0] <= NEG_BIG ? 0.f : exp2f(s[nt][0] - mn_lo);
                float e1 = s[nt][1] <= NEG_BIG ? 0.f : exp2f(s[nt][1] - mn_lo);
                float e2 = s[nt][2] <= NEG_BIG ? 0.f : exp2f(s[nt][2] - mn_hi);
                float e3 = s[nt][3] <= NEG_BIG ? 0.f : exp2f(s[nt][3] - mn_hi);
                sum_lo += e0 + e1; sum_hi += e2 + e3;
                pf[nt >> 1][(nt & 1) * 2] = pack_bf16(e0, e1);
                pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(e2, e3);
            }
            l_lo = l_lo * a_lo + sum_lo; l_hi = l_hi * a_hi + sum_hi;
#pragma unroll
            for (int i = 0; i < KSTEPS * 2; ++i) { o[i][0] *= a_lo; o[i][1] *= a_lo; o[i][2] *= a_hi; o[i][3] *= a_hi; }
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) values_16keys<KSTEPS>(o, pf[ks], v_tile, ks * 16, hd, lane);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = 1.0f / l_lo, inv_hi = 1.0f / l_hi;
#pragma unroll
    for (int dt = 0; dt < KSTEPS * 2; ++dt) {
        const int d = dt * 8 + (lane & 3) * 2;
        if (d < hd) {
            if (r_lo < rows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(t_begin + row0 + r_lo) * H + h) * hd + d) =
                    pack_bf16(o[dt][0] * inv_lo, o[dt][1] * inv_lo);
            if (r_hi < rows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(t_begin + row0 + r_hi) * H + h) * hd + d) =
                    pack_bf16(o[dt][2] * inv_hi, o[dt][3] * inv_hi);
        }
    }
}

// ============================================================================ prefill, head sizes 64 and 128
// The same algorithm with the head size known at compile time: the ldmatrix addresses of a lane
// are computed once, the scale is folded into the exponent's FMA, exp2 is the hardware
// approximation (relative error 2^-22, far below bfloat16's), and the tiles with the most keys
// (the last ones of a prompt) are started first.
template <int HD, int ROWS>
__global__ void __launch_bounds__(ROWS * 2)
attention_prefill_exact_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                               const __nv_bfloat16* __restrict__ pages, const int* __restrict__ page_table,
                               int pt_stride, const int* __restrict__ q_start, const int* __restrict__ kv_len, int H,
                               int G, float scale_log2, int window) {
    constexpr int KSTEPS = HD / 16;
    constexpr int ROW = HD * 2;
    constexpr int TILE = PAGE * ROW;                  // bytes of a K (or V) tile
    constexpr int STAGE = 2 * TILE;
    extern __shared__ __align__(128) uint8_t smem[];
    lp_grid_release();
    lp_grid_wait();
    const int b = blockIdx.z, h = blockIdx.y, tile = gridDim.x - 1 - blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t_begin = q_start[b], n_new = q_start[b + 1] - t_begin;
    if (tile * ROWS >= n_new) return;
    const int g = h / (H / G);
    const int len = kv_len[b];
    const int pos0 = len - n_new;
    const int row0 = tile * ROWS;
    const int rows = min(ROWS, n_new - row0);
    const int first_pos = pos0 + row0, last_pos = pos0 + row0 + rows - 1;
    const int lo = window > 0 ? max(0, first_pos - window + 1) : 0;
    const int page_lo = lo / PAGE, page_hi = last_pos / PAGE;
    const int* table = page_table + (size_t)b * pt_stride;

    const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
    uint32_t qf[KSTEPS][4];
    {
        const __nv_bfloat16* q_lo = q + ((size_t)(t_begin + row0 + min(r_lo, rows - 1)) * H + h) * HD;
        const __nv_bfloat16* q_hi = q + ((size_t)(t_begin + row0 + min(r_hi, rows - 1)) * H + h) * HD;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            const int c = kk * 16 + (lane & 3) * 2;
            qf[kk][0] = *reinterpret_cast<const uint32_t*>(q_lo + c);
            qf[kk][1] = *reinterpret_cast<const uint32_t*>(q_hi + c);
            qf[kk][2] = *reinterpret_cast<const uint32_t*>(q_lo + c + 8);
            qf[kk][3] = *reinterpret_cast<const uint32_t*>(q_hi + c + 8);
        }
    }
    const int pos_lo = first_pos + min(r_lo, rows - 1), pos_hi = first_pos + min(r_hi, rows - 1);
    const int warp_last_pos = first_pos + min(warp * 16 + 15, rows - 1);
    const int warp_first_pos = first_pos + min(warp * 16, rows - 1);

    // byte offsets of this lane's ldmatrix rows inside a slice of 16 keys
    uint32_t k_off[KSTEPS], v_off[KSTEPS];
    {
        const int mat = lane >> 3, row = lane & 7;
        const int kr = (mat >> 1) * 8 + row, vr = (mat & 1) * 8 + row;
#pragma unroll
        for (int i = 0; i < KSTEPS; ++i) {
            k_off[i] = kr * ROW + (((i * 2 + (mat & 1)) ^ (kr & 7)) << 4);
            v_off[i] = vr * ROW + (((i * 2 + (mat >> 1)) ^ (vr & 7)) << 4);
        }
    }

    float o[KSTEPS * 2][4];
#pragma unroll
    for (int i = 0; i < KSTEPS * 2; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_lo = NEG_BIG, m_hi = NEG_BIG, l_lo = 0.f, l_hi = 0.f;      // maxima in scaled log2 units

    load_page(smem, pages, table[page_lo], G, g, HD, tid, ROWS * 2);
    cp_async_commit();
    for (int p = page_lo; p <= page_hi; ++p) {
        const int cur = (p - page_lo) & 1;
        if (p + 1 <= page_hi) load_page(smem + (cur ^ 1) * STAGE, pages, table[p + 1], G, g, HD, tid, ROWS * 2);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int key_base = p * PAGE;
        const bool active = key_base <= warp_last_pos &&
                            (window <= 0 || key_base + PAGE - 1 > warp_first_pos - window);
        if (active) {
            const uint32_t k_tile = smem_u32(smem + cur * STAGE);
            const uint32_t v_tile = k_tile + TILE;
            float s[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(k_tile + ks * 16 * ROW + k_off[kk], b0, b1, b2, b3);
                    mma_bf16(s[ks * 2], qf[kk], b0, b1);
                    mma_bf16(s[ks * 2 + 1], qf[kk], b2, b3);
                }
            }
            const bool edge = key_base + PAGE - 1 > warp_first_pos ||
                              (window > 0 && key_base <= warp_last_pos - window);
            if (edge) {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key_base + nt * 8 + (lane & 3) * 2 + (e & 1);
                        const int pos = (e < 2) ? pos_lo : pos_hi;
                        if (key > pos || (window > 0 && key <= pos - window)) s[nt][e] = -INFINITY;
                    }
            }
            float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                mx_lo = fmaxf(mx_lo, fmaxf(s[nt][0], s[nt][1]));
                mx_hi = fmaxf(mx_hi, fmaxf(s[nt][2], s[nt][3]));
            }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float mn_lo = fmaxf(m_lo, mx_lo * scale_log2), mn_hi = fmaxf(m_hi, mx_hi * scale_log2);
            const float a_lo = fast_exp2(m_lo - mn_lo), a_hi = fast_exp2(m_hi - mn_hi);
            m_lo = mn_lo; m_hi = mn_hi;
            float sum_lo = 0.f, sum_hi = 0.f;
            uint32_t pf[4][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const float e0 = fast_exp2(fmaf(s[nt][0], scale_log2, -mn_lo));      // exp2(-inf) = 0 for masked keys
                const float e1 = fast_exp2(fmaf(s[nt][1], scale_log2, -mn_lo));
                const float e2 = fast_exp2(fmaf(s[nt][2], scale_log2, -mn_hi));
                const float e3 = fast_exp2(fmaf(s[nt][3], scale_log2, -mn_hi));
                sum_lo += e0 + e1; sum_hi += e2 + e3;
                pf[nt >> 1][(nt & 1) * 2] = pack_bf16(e0, e1);
                pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(e2, e3);
            }
            l_lo = l_lo * a_lo + sum_lo; l_hi = l_hi * a_hi + sum_hi;
#pragma unroll
            for (int i = 0; i < KSTEPS * 2; ++i) { o[i][0] *= a_lo; o[i][1] *= a_lo; o[i][2] *= a_hi; o[i][3] *= a_hi; }
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
                for (int dd = 0; dd < KSTEPS; ++dd) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(v_tile + ks * 16 * ROW + v_off[dd], b0, b1, b2, b3);
                    mma_bf16(o[dd * 2], pf[ks], b0, b1);
                    mma_bf16(o[dd * 2 + 1], pf[ks], b2, b3);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = 1.0f / l_lo, inv_hi = 1.0f / l_hi;
#pragma unroll
    for (int dt = 0; dt < KSTEPS * 2; ++dt) {
        const int d = dt * 8 + (lane & 3) * 2;
        if (r_lo < rows)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(t_begin + row0 + r_lo) * H + h) * HD + d) =
                pack_bf16(o[dt][0] * inv_lo, o[dt][1] * inv_lo);
        if (r_hi < rows)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(t_begin + row0 + r_hi) * H + h) * HD + d) =
                pack_bf16(o[dt][2] * inv_hi, o[dt][3] * inv_hi);
    }
}

// ============================================================================ decode
// grid: (splits, G * head_groups, B); 128 threads; one new token per sequence (attention_decode.cuh).
// The fused form that writes the new key and value itself requests its first pages before it waits
// for the previous kernel: within a step nothing writes lengths, page tables or these pages (a kernel that
// moves lengths on belongs to the end of the previous step, and the step's first kernel is launched without
// the early start, so it has finished), and the new row is put into the unit's own copy of the page. Every
// other form waits first (the pages may hold a row that the previous kernel wrote).
template <int HD_MAX, bool FUSED, int HD_EXACT, int STAGES, int NW = 4>
__global__ void __launch_bounds__(32 * NW)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pages,
                        const int* __restrict__ page_table, int pt_stride, const int* __restrict__ kv_len,
                        float* __restrict__ part_o, float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                        int H, int G, int hd_arg, float scale_log2, int window, int pages_per_split, int num_splits,
                        int min_share_pages, int head_groups, FusedDecodeArgs fused) {
    extern __shared__ __align__(128) uint8_t smem[];
    lp_grid_release();
    const bool early = FUSED && fused.pages_rw != nullptr;
    if (!early) lp_grid_wait();
    attention_decode_unit<HD_MAX, FUSED, HD_EXACT, false, STAGES, NW>(
        smem, threadIdx.x, blockIdx.x, blockIdx.y, blockIdx.z, q, pages, page_table, pt_stride, kv_len, part_o, part_ml,
        out, H, G, hd_arg, scale_log2, window, pages_per_split, num_splits, min_share_pages, head_groups, fused,
        [early] { if (early) lp_grid_wait(); });
}

// The fused form with the pages brought by TMA (head sizes 64 and 128; see attention_decode.cuh).
template <int HD, int STAGES, int NW>
__global__ void __launch_bounds__(32 * NW)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap kv_map, const __nv_bfloat16* __restrict__ pages,
                            const int* __restrict__ page_table, int pt_stride, const int* __restrict__ kv_len,
                            float* __restrict__ part_o, float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                            int H, int G, float scale_log2, int window, int pages_per_split, int num_splits,
                            int min_share_pages, int head_groups, FusedDecodeArgs fused, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);     // the swizzle's pattern repeats every 1024 bytes
    if (threadIdx.x == 32) asm volatile("prefetch.tensormap [%0];" ::"l"(&kv_map) : "memory");
    lp_grid_release();
    const bool early = fused.pages_rw != nullptr;
    if (!early) lp_grid_wait();
    attention_decode_unit<HD, true, HD, false, STAGES, NW, true>(
        smem, threadIdx.x, blockIdx.x, blockIdx.y, blockIdx.z, nullptr, pages, page_table, pt_stride, kv_len, part_o,
        part_ml, out, H, G, HD, scale_log2, window, pages_per_split, num_splits, min_share_pages, head_groups, fused,
        [early] { if (early) lp_grid_wait(); }, &kv_map, status);
}

// out[b][head][:] = sum_s part_o * 2^(m_s - m*) / sum_s l_s * 2^(m_s - m*); grid: (H, B), hd threads (<= 256).
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       __nv_bfloat16* __restrict__ out, int H, int hd, int num_splits) {
    lp_grid_release();
    lp_grid_wait();
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const size_t base = ((size_t)b * H + h) * num_splits;
    float m = NEG_BIG;
    for (int s = 0; s < num_splits; ++s) m = fmaxf(m, part_ml[(base + s) * 2]);
    float acc = 0.f, l = 0.f;
    for (int s = 0; s < num_splits; ++s) {
        const float ls = part_ml[(base + s) * 2 + 1];
        if (ls > 0.f) {
            const float f = exp2f(part_ml[(base + s) * 2] - m);
            l += ls * f;
            if (d < hd) acc += part_o[(base + s) * hd + d] * f;
        }
    }
    if (d < hd) out[((size_t)b * H + h) * hd + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
}

// Opt in to `bytes` of dynamic shared memory; remembered per kernel so that later calls
// (also those recorded into a CUDA graph) make no runtime call.
template <typename K> int set_smem(K kernel, int bytes, const char* what) {
    // what each kernel (by its address) has been granted so far; a handful of instantiations are ever used
    constexpr int SLOTS = 64;
    static const void* known[SLOTS];
    static int granted[SLOTS];
    static int used = 0;
    int at = 0;
    while (at < used && known[at] != (const void*)kernel) ++at;
    if (at < used && bytes <= granted[at]) return 0;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) {
        snprintf(lp_error_text, sizeof(lp_error_text), "%s: cannot reserve %d bytes of shared memory: %s", what, bytes,
                 cudaGetErrorString(e));
        return (int)e;
    }
    if (at == used && used < SLOTS) { known[at] = (const void*)kernel; ++used; }
    if (at < used) granted[at] = bytes;
    return 0;
}

int check_geometry(const char* what, int H, int G, int hd) {
    if (H <= 0 || G <= 0 || H % G) LP_REFUSE("%s: %d query heads over %d key heads", what, H, G);
    if (hd < 16 || hd > 256 || hd % 16) LP_REFUSE("%s: head size %d (supported: multiples of 16 up to 256)", what, hd);
    return 0;
}

}  // namespace

// q, out: [T, H, hd] bf16; pages: [num_pages, 2, G, 64, hd] bf16; q_start: [B+1]; kv_len: [B] (after the step).
// max_new: the largest number of new tokens of any sequence of the step.
extern "C" int lp_attention_prefill(const void* q, void* out, const void* pages, const int* page_table, int pt_stride,
                                    const int* q_start, const int* kv_len, int B, int max_new, int H, int G, int hd,
                                    int page_size, float scale, int window, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    int rc = check_geometry("attention_prefill", H, G, hd);
    if (rc) return rc;
    if (page_size != PAGE) LP_REFUSE("attention_prefill: pages of %d positions (built for %d)", page_size, PAGE);
    if (H > 65535 || B > 65535) LP_REFUSE("attention_prefill: %d heads x %d sequences exceed the grid", H, B);
    const int smem = 2 * (2 * PAGE * hd * 2);
    dim3 grid((max_new + 63) / 64, H, B);
    const float scale_log2 = scale * 1.4426950408889634f;
#define LP_PREFILL(HDM)                                                                                          \
    do {                                                                                                         \
        rc = set_smem(attention_prefill_kernel<HDM>, smem, "attention_prefill");                                 \
        if (rc) return rc;                                                                                       \
        lp_launch(attention_prefill_kernel<HDM>, grid, 128, smem, stream,                                        \
            (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)pages, page_table, pt_stride,     \
            q_start, kv_len, H, G, hd, scale_log2, window);                                                      \
    } while (0)
#define LP_PREFILL_EXACT(HD, ROWS)                                                                               \
    do {                                                                                                         \
        rc = set_smem(attention_prefill_exact_kernel<HD, ROWS>, smem, "attention_prefill");    \
        if (rc) return rc;                                                                                       \
        dim3 grid_exact((max_new + ROWS - 1) / ROWS, H, B);                                                      \
        lp_launch(attention_prefill_exact_kernel<HD, ROWS>, grid_exact, ROWS * 2, smem, stream,                  \
                  (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)pages, page_table,         \
                  pt_stride, q_start, kv_len, H, G, scale_log2, window);                                         \
    } while (0)
    // long prompts: 128 query rows share each page of keys; short ones keep 64 rows for more CTAs
    const bool tall = (long long)((max_new + 127) / 128) * H * B >= 8LL * lp_sm_count();
    if (hd == 64 && tall) LP_PREFILL_EXACT(64, 128);
    else if (hd == 64) LP_PREFILL_EXACT(64, 64);
    else if (hd == 128 && tall) LP_PREFILL_EXACT(128, 128);
    else if (hd == 128) LP_PREFILL_EXACT(128, 64);
    else if (hd <= 64) LP_PREFILL(64); else if (hd <= 128) LP_PREFILL(128); else LP_PREFILL(256);
#undef LP_PREFILL_EXACT
#undef LP_PREFILL
    return lp_check_launch("attention_prefill");
}

// Scratch a decode step needs, in floats: part_o [B, H, splits, hd] then part_ml [B, H, splits, 2].
extern "C" long long lp_attention_decode_scratch(int B, int H, int hd, int num_splits) {
    return (long long)B * H * num_splits * (hd + 2);
}

// q, out: [B, H, hd] bf16 (one token per sequence); kv_len: [B] (after the step). The pages of a sequence
// are shared out over `num_splits` CTAs, `pages_per_split` each; scratch as sized above.
// lp_attention_decode_fitted: the same with `min_share_pages` > 0: each sequence's pages are cut into as many
// shares (at most num_splits) as leaves each share that many pages (see attention_decode.cuh).
static int attention_decode_launch(const void* q, void* out, const void* pages, const int* page_table, int pt_stride,
                                   const int* kv_len, float* scratch, int B, int H, int G, int hd, int page_size,
                                   float scale, int window, int pages_per_split, int num_splits, int min_share_pages,
                                   cudaStream_t stream) {
    if (B <= 0) return 0;
    int rc = check_geometry("attention_decode", H, G, hd);
    if (rc) return rc;
    if (page_size != PAGE) LP_REFUSE("attention_decode: pages of %d positions (built for %d)", page_size, PAGE);
    if (pages_per_split <= 0 || num_splits <= 0) LP_REFUSE("attention_decode: %d shares of %d pages", num_splits, pages_per_split);
    const int head_groups = (H / G + HEAD_ROWS - 1) / HEAD_ROWS;
    if (G * head_groups > 65535 || B > 65535) LP_REFUSE("attention_decode: grid too large");
    const int stage = 2 * PAGE * hd * 2;
    const int merge = (2 * 4 * HEAD_ROWS + 4 * HEAD_ROWS * hd) * 4;
    const int smem = 3 * stage > merge ? 3 * stage : merge;
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)B * H * num_splits * hd;
    dim3 grid(num_splits, G * head_groups, B);
    const float scale_log2 = scale * 1.4426950408889634f;
#define LP_DECODE(HDM, EXACT)                                                                                    \
    do {                                                                                                         \
        rc = set_smem(attention_decode_kernel<HDM, false, EXACT, 3>, smem, "attention_decode"); \
        if (rc) return rc;                                                                                       \
        lp_launch(attention_decode_kernel<HDM, false, EXACT, 3>, grid, 128, smem, stream,                           \
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)pages, page_table, pt_stride, kv_len, part_o, part_ml, \
            (__nv_bfloat16*)out, H, G, hd, scale_log2, window, pages_per_split, num_splits, min_share_pages,     \
            head_groups, FusedDecodeArgs{});                                                                     \
    } while (0)
    if (hd == 64) LP_DECODE(64, 64); else if (hd == 128) LP_DECODE(128, 128);
    else if (hd <= 64) LP_DECODE(64, 0); else if (hd <= 128) LP_DECODE(128, 0); else LP_DECODE(256, 0);
#undef LP_DECODE
    rc = lp_check_launch("attention_decode");
    if (rc || num_splits == 1) return rc;
    lp_launch(attention_merge_kernel, dim3(H, B), hd <= 32 ? 32 : (hd + 31) / 32 * 32, 0, stream,
              (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, H, hd, num_splits);
    return lp_check_launch("attention_merge");
}

extern "C" int lp_attention_decode(const void* q, void* out, const void* pages, const int* page_table, int pt_stride,
                                   const int* kv_len, float* scratch, int B, int H, int G, int hd, int page_size,
                                   float scale, int window, int pages_per_split, int num_splits,
                                   cudaStream_t stream) {
    return attention_decode_launch(q, out, pages, page_table, pt_stride, kv_len, scratch, B, H, G, hd, page_size, scale,
                                   window, pages_per_split, num_splits, 0, stream);
}

extern "C" int lp_attention_decode_fitted(const void* q, void* out, const void* pages, const int* page_table,
                                          int pt_stride, const int* kv_len, float* scratch, int B, int H, int G, int hd,
                                          int page_size, float scale, int window, int num_splits, int min_share_pages,
                                          cudaStream_t stream) {
    if (min_share_pages <= 0) LP_REFUSE("attention_decode_fitted: shares of at least %d pages", min_share_pages);
    return attention_decode_launch(q, out, pages, page_table, pt_stride, kv_len, scratch, B, H, G, hd, page_size, scale,
                                   window, pt_stride > 0 ? pt_stride : 1, num_splits, min_share_pages, stream);
}

// Decode attention that starts from the fused projection output: rotation of queries and of the new key,
// the cache write of the new key and value, attention over the pages and the merge of the shares in one
// kernel. qkv: [B, ld] float32 = [H query heads | G key heads | G value heads] x hd (keys and values only
// if `pages_rw` is given: a layer that attends over another run's cache has none). counters: int32
// [B * G * head_groups], zero before the first call; the kernel leaves them zero. row_sumsq (optional, [B]):
// the projection left out the factor of its input's RMS norm; the kernel applies 1 / sqrt(row_sumsq[b] /
// norm_width + norm_eps) to the queries, the key and the value it reads. min_share_pages > 0: shares fitted to each
// sequence's own length (see attention_decode.cuh); pages_per_split then only says how long a share can get.
extern "C" int lp_attention_decode_fused(const float* qkv, int ld, const float* inv_freq, int rd, int interleaved,
                                         void* out, void* pages, int write_kv, const int* page_table, int pt_stride,
                                         const int* kv_len, float* scratch, int* counters, int B, int H, int G,
                                         int hd, int page_size, float scale, int window, int pages_per_split,
                                         int num_splits, int min_share_pages, const float* row_sumsq, float norm_eps,
                                         int norm_width, long long num_pages, int* status, cudaStream_t stream) {
    if (B <= 0) return 0;
    int rc = check_geometry("attention_decode_fused", H, G, hd);
    if (row_sumsq && norm_width <= 0) LP_REFUSE("attention_decode_fused: a row factor over %d values", norm_width);
    if (rc) return rc;
    if (page_size != PAGE) LP_REFUSE("attention_decode_fused: pages of %d positions (built for %d)", page_size, PAGE);
    if (pages_per_split <= 0 || num_splits <= 0) LP_REFUSE("attention_decode_fused: %d shares of %d pages", num_splits, pages_per_split);
    if (rd < 0 || rd > hd || (rd & 1) || rd > 256) LP_REFUSE("attention_decode_fused: rotary width %d of a head of %d", rd, hd);
    if (rd > 0 && !inv_freq) LP_REFUSE("attention_decode_fused: rotation without frequencies");
    if (ld < (write_kv ? H + 2 * G : H) * hd) LP_REFUSE("attention_decode_fused: row of %d values", ld);
    const int head_groups = (H / G + HEAD_ROWS - 1) / HEAD_ROWS;
    if (G * head_groups > 65535 || B > 65535) LP_REFUSE("attention_decode_fused: grid too large");
    const int stage = 2 * PAGE * hd * 2;
    const int extra = (HEAD_ROWS * hd + 2 * hd) * 2 + 256 * 4;
    const int sms = lp_sm_count();
    // With few CTAs altogether (no more than one per SM: measured, batch 24 / 32: 1.01 / 1.02 ms per step against
    // 1.07 / 1.08 when up to two per SM count as few) and small heads a CTA has 16 warps, four pages at a time and
    // eight pages in shared memory; with CTAs enough to hide a page's latency by their number, 4 warps and 3 pages.
    const bool wide = hd <= 64 && pages_per_split > 3 && (long long)num_splits * G * head_groups * B <= sms;
    // up to two CTAs per SM: 8 warps, two pages at a time, six in shared memory (batch 32: 0.96 ms per step against
    // 1.02 with 4 warps; with more CTAs than that, batch 64, the 4-warp form wins: 1.19 against 1.28)
    const bool mid = !wide && hd <= 64 && pages_per_split > 3 && (long long)num_splits * G * head_groups * B <= 2 * sms;
    // heads of 128 (pages of 32 KB): 8 warps, two pages at a time, four in shared memory, one CTA per SM
    const bool wide128 = hd > 64 && hd <= 128 && pages_per_split > 3 && (long long)num_splits * G * head_groups * B <= sms;
    const int stages = wide ? 8 : mid ? 6 : wide128 ? 4 : 3, nw = wide ? 16 : (mid || wide128) ? 8 : 4;
    const int merge = (2 * nw * HEAD_ROWS + nw * HEAD_ROWS * hd) * 4;
    const int smem = (stages * stage > merge ? stages * stage : merge) + extra;
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)B * H * num_splits * hd;
    dim3 grid(num_splits, G * head_groups, B);
    const float scale_log2 = scale * 1.4426950408889634f;
    FusedDecodeArgs fused{qkv, ld, inv_freq, rd, interleaved, write_kv ? (__nv_bfloat16*)pages : nullptr, counters,
                          row_sumsq, norm_eps, norm_width};
    // heads of 64 or 128: the pages come by TMA (num_pages and status given; LLMPLAYER_B200_DECODE_TMA=0 keeps cp.async)
    static int use_tma = -1;
    if (use_tma < 0) { const char* v = getenv("LLMPLAYER_B200_DECODE_TMA"); use_tma = (v && v[0] == '0') ? 0 : 1; }
    if (use_tma && (hd == 64 || hd == 128) && num_pages > 0 && status) {
        CUtensorMap kv_map;
        rc = make_map(&kv_map, pages, num_pages * 2 * G * PAGE, hd, hd, PAGE);
        if (rc) return rc;
        const int smem_tma = smem + 1024 + 64;          // alignment slack and the stages' barriers
#define LP_DECODE_TMA(HDX, ST, NWARPS)                                                                          \
        do {                                                                                                    \
            rc = set_smem(attention_decode_tma_kernel<HDX, ST, NWARPS>, smem_tma, "attention_decode_fused");    \
            if (rc) return rc;                                                                                  \
            lp_launch(attention_decode_tma_kernel<HDX, ST, NWARPS>, grid, 32 * NWARPS, smem_tma, stream, kv_map, \
                      (const __nv_bfloat16*)pages, page_table, pt_stride, kv_len, part_o, part_ml,              \
                      (__nv_bfloat16*)out, H, G, scale_log2, window, pages_per_split, num_splits,               \
                      min_share_pages, head_groups, fused, status);                                             \
        } while (0)
        if (hd == 64) { if (wide) LP_DECODE_TMA(64, 8, 16); else if (mid) LP_DECODE_TMA(64, 6, 8); else LP_DECODE_TMA(64, 3, 4); }
        else { if (wide128) LP_DECODE_TMA(128, 4, 8); else LP_DECODE_TMA(128, 3, 4); }
#undef LP_DECODE_TMA
        return lp_check_launch("attention_decode_fused");
    }
#define LP_DECODE_FUSED(HDM, EXACT, ST, NWARPS)                                                                  \
    do {                                                                                                         \
        rc = set_smem(attention_decode_kernel<HDM, true, EXACT, ST, NWARPS>, smem,  \
                                                   "attention_decode_fused");                                    \
        if (rc) return rc;                                                                                       \
        lp_launch(attention_decode_kernel<HDM, true, EXACT, ST, NWARPS>, grid, 32 * NWARPS, smem, stream,        \
                  (const __nv_bfloat16*)nullptr, (const __nv_bfloat16*)pages, page_table, pt_stride, kv_len,     \
                  part_o, part_ml, (__nv_bfloat16*)out, H, G, hd, scale_log2, window, pages_per_split,           \
                  num_splits, min_share_pages, head_groups, fused);                                              \
    } while (0)
    if (hd == 64) { if (wide) LP_DECODE_FUSED(64, 64, 8, 16); else if (mid) LP_DECODE_FUSED(64, 64, 6, 8); else LP_DECODE_FUSED(64, 64, 3, 4); }
    else if (hd == 128) { if (wide128) LP_DECODE_FUSED(128, 128, 4, 8); else LP_DECODE_FUSED(128, 128, 3, 4); }
    else if (hd <= 64) { if (wide) LP_DECODE_FUSED(64, 0, 8, 16); else if (mid) LP_DECODE_FUSED(64, 0, 6, 8); else LP_DECODE_FUSED(64, 0, 3, 4); }
    else if (hd <= 128) { if (wide128) LP_DECODE_FUSED(128, 0, 4, 8); else LP_DECODE_FUSED(128, 0, 3, 4); }
    else LP_DECODE_FUSED(256, 0, 3, 4);
#undef LP_DECODE_FUSED
    return lp_check_launch("attention_decode_fused");
}

// ---------------------------------------------------------------- decode without allocation
// See attention_noalloc.h. The scratch of lp_attention_decode lives in this file-scope device
// array; host code must not pass the array's name to a kernel (in host code it is only a
// stand-in), so its device address is looked up once per device and kept.
#include "attention_noalloc.h"

static __device__ __align__(256) float lp_decode_static_scratch[LP_NOALLOC_SCRATCH_FLOATS];
static float* lp_decode_static_address[64] = {};

extern "C" int lp_attention_decode_noalloc(const void* q, void* out, const void* pages, const int* page_table,
                                           int pt_stride, const int* kv_len, int B, int H, int G, int hd,
                                           int page_size, float scale, int window, int pages_per_split,
                                           int num_splits, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || hd <= 0 || num_splits <= 0) LP_REFUSE("attention_decode_noalloc: %d heads of %d in %d shares", H, hd, num_splits);
    const long long need = lp_attention_decode_scratch(B, H, hd, num_splits);
    if (need > LP_NOALLOC_SCRATCH_FLOATS)
        LP_REFUSE("attention_decode_noalloc: %d sequences x %d heads x %d shares need %lld floats of scratch, "
                  "the built-in array holds %lld; use fewer shares or lp_attention_decode with your own scratch",
                  B, H, num_splits, need, (long long)LP_NOALLOC_SCRATCH_FLOATS);
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) {
        snprintf(lp_error_text, sizeof(lp_error_text), "attention_decode_noalloc: %s", cudaGetErrorString(err));
        return (int)err;
    }
    if (device < 0 || device >= 64) LP_REFUSE("attention_decode_noalloc: device index %d", device);
    if (!lp_decode_static_address[device]) {
        float* address = nullptr;
        err = cudaGetSymbolAddress((void**)&address, lp_decode_static_scratch);
        if (err != cudaSuccess || !address) {
            snprintf(lp_error_text, sizeof(lp_error_text), "attention_decode_noalloc: cannot find the scratch array: %s",
                     cudaGetErrorString(err));
            return err != cudaSuccess ? (int)err : -1;
        }
        lp_decode_static_address[device] = address;
    }
    return lp_attention_decode(q, out, pages, page_table, pt_stride, kv_len, lp_decode_static_address[device], B, H, G,
                               hd, page_size, scale, window, pages_per_split, num_splits, stream);
}
