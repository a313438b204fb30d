// The decode-step attention unit and the mma.sync / cp.async helpers it shares with the prompt
// kernels: one (sequence, key/value head, share of the pages) handled by 128 threads. Used by the
// stand-alone decode kernels (plain entry, fused entry, entry without allocation).
#pragma once

#include "common.cuh"

namespace {

#ifndef LP_SMEM_U32_DEFINED
#define LP_SMEM_U32_DEFINED
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
#endif
constexpr int PAGE = 64;
constexpr float NEG_BIG = -1.0e30f;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// exp2 by the hardware approximation (relative error about 2^-22, far below bfloat16's rounding)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Position of 16-byte chunk c of row r inside a tile whose rows hold cpr chunks.
__device__ __forceinline__ int swz(int r, int c, int cpr) {
    return (cpr & 7) == 0 ? (c ^ (r & 7)) : (c + r) % cpr;
}

// The same for a tile written by TMA with its 128-byte swizzle (head sizes that are multiples of 64): panels of
// 64 columns, each [64 rows x 128 bytes], chunk c % 8 of a row at (c % 8) xor (r % 8). PANELS = false: the layout
// above (rows of hd elements). Returns the byte offset of chunk c of row r.
template <bool PANELS>
__device__ __forceinline__ uint32_t tile_offset(int r, int c, int hd, int cpr) {
    if (PANELS) return (uint32_t)((c >> 3) * (PAGE * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4));
    return (uint32_t)(r * (hd * 2) + swz(r, c, cpr) * 16);
}

// Copy one page (64 keys and 64 values of one kv head) into a stage: K tile, then V tile.
__device__ __forceinline__ void load_page(uint8_t* stage, const __nv_bfloat16* pages, int page, int G, int g, int hd,
                                          int tid, int nthreads) {
    const int cpr = hd >> 3;
    const int per_tile = PAGE * cpr;
    const uint32_t base = smem_u32(stage);
    const size_t tile_elems = (size_t)PAGE * hd;
    for (int i = tid; i < 2 * per_tile; i += nthreads) {
        const int which = i >= per_tile;
        const int j = which ? i - per_tile : i;
        const int r = j / cpr, c = j - r * cpr;
        const __nv_bfloat16* src = pages + (((size_t)page * 2 + which) * G + g) * tile_elems + (size_t)r * hd + c * 8;
        cp_async16(base + which * (uint32_t)(tile_elems * 2) + r * (hd * 2) + swz(r, c, cpr) * 16, src);
    }
}

// S[16 x 16 keys] += Q[16 x hd] K^T for the keys key0..key0+15 of the K tile (two n-tiles of 8 keys).
template <int KSTEPS>
__device__ __forceinline__ void scores_16keys(float (*s)[4], const uint32_t (*q)[4], uint32_t k_tile, int key0,
                                              int hd, int lane) {
    const int cpr = hd >> 3;
    const int mat = lane >> 3, row = lane & 7;
    const int key = key0 + (mat >> 1) * 8 + row;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
        if (kk * 16 < hd) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(k_tile + key * (hd * 2) + swz(key, kk * 2 + (mat & 1), cpr) * 16, b0, b1, b2, b3);
            mma_bf16(s[0], q[kk], b0, b1);
            mma_bf16(s[1], q[kk], b2, b3);
        }
    }
}

// O[16 x hd] += P[16 x 16 keys] V for the keys key0..key0+15 of the V tile.
template <int KSTEPS>
__device__ __forceinline__ void values_16keys(float (*o)[4], const uint32_t* p, uint32_t v_tile, int key0, int hd,
                                              int lane) {
    const int cpr = hd >> 3;
    const int mat = lane >> 3, row = lane & 7;
    const int key = key0 + (mat & 1) * 8 + row;
#pragma unroll
    for (int dd = 0; dd < KSTEPS; ++dd) {       // 16 output features per step
        if (dd * 16 < hd) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(v_tile + key * (hd * 2) + swz(key, dd * 2 + (mat >> 1), cpr) * 16, b0, b1, b2, b3);
            mma_bf16(o[dd * 2], p, b0, b1);
            mma_bf16(o[dd * 2 + 1], p, b2, b3);
        }
    }
}

// Transpose an 8 x 8 matrix of 16-bit values held as one register per lane (row lane / 4, columns 2 (lane % 4) and
// the next): what turns the accumulator layout of one product into the operand layout of the next when the roles
// of rows and columns swap.
__device__ __forceinline__ uint32_t transpose_8x8(uint32_t v) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}

// A decode step has one query per head, and the handful of query heads that share a key/value head are far fewer
// than the keys. So the keys are the rows (M = 16) of the tensor-core products and the query heads their columns
// (N = 8): S^T[16 keys x 8 heads] = K Q^T and O^T[head size x 8 heads] += V^T P^T. With the query heads as the rows
// of 16-row tiles three quarters of every product and of the softmax's work were padding; this way half is, and
// a page costs half the instructions.
constexpr int HEAD_ROWS = 8;       // query heads per unit (a key/value head with more query heads takes several units)

// ============================================================================ decode
// grid: (splits, G * head_groups, B); 128 threads; one new token per sequence.
// Partial results: part_o[b][head][split][hd] (unnormalised), part_ml[b][head][split][2] = (max, sum),
// both in log2 units of the scaled scores.
//
// FUSED: the kernel starts from the float32 fused projection output qkv[b] = [H q heads | G k heads |
// G v heads] instead of rotated bf16 queries: it rotates the queries of its heads itself, and the CTA
// whose share holds the new token's position rotates the new key, writes key and value into the cache
// and into its own shared-memory copy of that page. The last CTA of a (sequence, kv head) to finish
// merges the shares (a counter per group, zero before the launch and zero again after it).
struct FusedDecodeArgs {
    const float* qkv;          // [B, ld]
    int ld;
    const float* inv_freq;     // [rd / 2] or null
    int rd, interleaved;
    __nv_bfloat16* pages_rw;   // same pages, writable; null: this layer keeps no keys of its own
    int* counters;             // [B * G * head_groups]
    // optional: qkv[b] still lacks the factor of an RMS norm of its input, 1 / sqrt(row_sumsq[b] / norm_width +
    // norm_eps) (the projection took bfloat16(x * gain) and left the row's factor to its reader)
    const float* row_sumsq;
    float norm_eps;
    int norm_width;
};

// The same in two steps, for callers that want the loads of several elements in flight before they combine them.
// (products and sums are rounded one by one, as in the rotation kernels of elementwise.cu: a key must get the
// same bits whichever kernel stores it)
__device__ __forceinline__ int rotation_partner(int e, int rd, int interleaved) {
    const int half = rd >> 1;
    return interleaved ? (e ^ 1) : (e < half ? e + half : e - half);
}
__device__ __forceinline__ float rotate_value(float val, float other, int e, int rd, int interleaved, const float* cs,
                                              const float* sn) {
    if (e >= rd) return val;
    const int half = rd >> 1;
    const bool first = interleaved ? (e & 1) == 0 : e < half;
    const int pair = interleaved ? e >> 1 : (first ? e : e - half);
    return first ? __fsub_rn(__fmul_rn(val, cs[pair]), __fmul_rn(other, sn[pair]))
                 : __fadd_rn(__fmul_rn(other, sn[pair]), __fmul_rn(val, cs[pair]));
}

__device__ __forceinline__ float rotated(const float* head, int e, int rd, int interleaved, const float* cs,
                                         const float* sn) {
    float val = __ldcg(head + e);
    if (e < rd) {
        const int half = rd >> 1;
        int pair, partner;
        bool first;
        if (interleaved) { pair = e >> 1; first = (e & 1) == 0; partner = e ^ 1; }
        else { first = e < half; pair = first ? e : e - half; partner = first ? e + half : e - half; }
        const float other = __ldcg(head + partner);
        val = first ? __fsub_rn(__fmul_rn(val, cs[pair]), __fmul_rn(other, sn[pair]))
                 : __fadd_rn(__fmul_rn(other, sn[pair]), __fmul_rn(val, cs[pair]));
    }
    return val;
}

// HD_EXACT > 0: the head size is that constant (index arithmetic of the copies and of ldmatrix folds
// into shifts and masks); 0: any multiple of 16 up to HD_MAX, taken from `hd_arg`.
// One unit of the decode kernel: share `split` of the pages of sequence `b` for key/value head and head
// group `by` (= g * head_groups + hg), run by 32 NW threads numbered `tid`, with `smem` as their scratch.
// NAMED: the threads are part of a larger CTA and meet at named barrier 1 instead of __syncthreads.
template <bool NAMED, int NT> __device__ __forceinline__ void unit_sync() {
    if (NAMED) asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
    else __syncthreads();
}

// STAGES: pages in flight (the scratch holds STAGES key and value tiles). NW: warps (a multiple of 4): four
// warps share a page, 16 keys each, so NW / 4 pages are worked on at a time and the CTA meets twice per such
// group of pages. With few CTAs on the GPU more warps per CTA hide the latency of a page's short chain
// of dependent steps (copy, scores, softmax, values).
// `before_inputs()` is called once the unit has requested its first pages and computed its angles, right
// before it reads what the step itself produced (the projection output): a caller whose inputs come
// from an earlier operation of the same kernel waits for that operation there, so that the page
// copies (the cache holds nothing the step writes, except the new row this unit patches in itself)
// are already in flight.
// TMA: the pages come as bulk tensor copies (`kv_map`: the cache as a matrix of [pages x 2 x G x 64 rows, hd] with
// boxes of 64 x 64 and the 128-byte swizzle) that one thread requests, two to four instructions per page, and
// each warp awaits its own page at an mbarrier (bounded: `status` is set to 6 if a wait runs out and the page is
// skipped); else every thread copies 16-byte pieces with cp.async, about 120 instructions per page and thread
// at a head size of 64, which was most of what the kernel issued. TMA needs hd % 64 == 0 and `smem` aligned to 1024.
template <int HD_MAX, bool FUSED, int HD_EXACT, bool NAMED, int STAGES, int NW, bool TMA = false, typename Before>
__device__ __forceinline__ void attention_decode_unit(
    uint8_t* smem, const int tid, const int split, const int by, const int b, const __nv_bfloat16* __restrict__ q,
    const __nv_bfloat16* __restrict__ pages, const int* __restrict__ page_table, int pt_stride,
    const int* __restrict__ kv_len, float* __restrict__ part_o, float* __restrict__ part_ml,
    __nv_bfloat16* __restrict__ out, int H, int G, int hd_arg, float scale_log2, int window, int pages_per_split,
    int num_splits, int min_share_pages, int head_groups, const FusedDecodeArgs& fused, Before&& before_inputs,
    const CUtensorMap* kv_map = nullptr, int* status = nullptr) {
    constexpr int KSTEPS = HD_MAX / 16;
    constexpr int NT = 32 * NW, PG = NW / 4, GROUPS = STAGES / PG;
    static_assert(NW % 4 == 0 && STAGES % PG == 0 && GROUPS >= 1, "whole groups of pages in the ring");
    const int hd = HD_EXACT > 0 ? HD_EXACT : hd_arg;
    const int g = by / head_groups, hg = by - g * head_groups;
    const int R = H / G;
    const int head0 = g * R + hg * HEAD_ROWS;
    const int nrows = min(HEAD_ROWS, R - hg * HEAD_ROWS);
    const int warp = tid >> 5, lane = tid & 31;
    const int kw = warp & 3, pg = warp >> 2;       // this warp's quarter of a page's keys, and its page of a group
    const int len = kv_len[b];
    const int pos = len - 1;                       // a length of zero or less is an empty sequence: no page is
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;      // read, nothing is stored, the output is zero
    // Which pages this share takes. Fixed (min_share_pages == 0): share s takes pages s * pages_per_split ... of the
    // table. Fitted to the sequence (min_share_pages > 0): the pages that the sequence really has (within its
    // window) are cut into as many shares as leaves each at least min_share_pages, at most num_splits; the other
    // CTAs of the grid have nothing to do. A share and the merge of shares cost several dependent round trips
    // to memory, so a short sequence is better served by one CTA however wide its page table is.
    int shares = num_splits, page_lo, page_hi;
    if (min_share_pages > 0) {
        const int first = lo / PAGE, last = len > 0 ? pos / PAGE : first - 1;
        const int total = last - first + 1;
        shares = max(1, min(num_splits, total / min_share_pages));
        const int per = (max(total, 1) + shares - 1) / shares;
        page_lo = first + split * per;
        page_hi = min(last, page_lo + per - 1);
        if (split >= shares) {
            if (!FUSED) {                          // the separate merge kernel reads every share: leave an empty one
                for (int r = tid; r < nrows; r += 32 * NW) {
                    const size_t slot = ((size_t)b * H + head0 + r) * num_splits + split;
                    part_ml[slot * 2] = NEG_BIG;
                    part_ml[slot * 2 + 1] = 0.f;
                }
            }
            return;
        }
    } else {
        page_lo = max(lo / PAGE, split * pages_per_split);
        page_hi = len > 0 ? min(pos / PAGE, (split + 1) * pages_per_split - 1) : page_lo - 1;
    }
    const int* table = page_table + (size_t)b * pt_stride;
    const int stage_bytes = 2 * PAGE * hd * 2;
    const int npages = page_hi - page_lo + 1;      // may be <= 0: this share holds nothing of the sequence

    // TMA: one barrier per stage, behind the ring and (FUSED) the extras described below
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * stage_bytes + (HEAD_ROWS * hd + 2 * hd) * 2 + 256 * 4);
    // The first warp keeps 32 entries of the page table in its lanes (entry p of the share in lane p % 32, loaded
    // 32 at a time), so that a request does not begin with a round trip to L2 for the page's number.
    int table_lane = 0, table_base = 0;
    if (TMA && warp == 0 && lane < npages) table_lane = table[page_lo + lane];
    auto page_number = [&](int p) {                // called by the whole first warp
        if (p >= table_base + 32) {
            table_base = p & ~31;
            table_lane = table_base + lane < npages ? table[page_lo + table_base + lane] : 0;
        }
        return __shfl_sync(0xffffffffu, table_lane, p & 31);
    };
    auto request_page = [&](int p, int page) {     // by one thread: the share's page p (number `page`) into stage p % STAGES
        uint8_t* st = smem + (p % STAGES) * stage_bytes;
        uint64_t* bar = &full[p % STAGES];
        mbar_expect_tx(bar, (uint32_t)stage_bytes);
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            const int row = ((page * 2 + which) * G + g) * PAGE;
            for (int x = 0; x < hd; x += 64)
                tma_load_2d(st + which * (PAGE * hd * 2) + (x >> 6) * (PAGE * 128), kv_map, x, row, bar);
        }
    };
    // the ring is requested first; what follows overlaps with the copies
    if (TMA) {
        if (warp == 0) {
            if (lane == 0) {
                for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            }
            for (int p = 0; p < STAGES && p < npages; ++p) {
                const int page = page_number(p);
                if (lane == 0) request_page(p, page);
            }
        }
    } else {
#pragma unroll
        for (int gi = 0; gi < GROUPS; ++gi) {          // one group of copies per group of pages
#pragma unroll
            for (int j = 0; j < PG; ++j) {
                const int p = gi * PG + j;
                if (p < npages) load_page(smem + p * stage_bytes, pages, table[page_lo + p], G, g, hd, tid, NT);
            }
            cp_async_commit();
        }
    }

    const int g8 = lane >> 2, t4 = lane & 3;       // the lane's place in a fragment: row / column group
    uint32_t qf[KSTEPS][2];                        // Q^T as the products' column operand: head g8, features 2 t4 (+8) ...
    // FUSED: extra shared memory behind the ring: rotated queries [8][hd] bf16, the new key and value, cos, sin
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem + STAGES * stage_bytes);
    __nv_bfloat16* new_k = q_s + HEAD_ROWS * hd;
    __nv_bfloat16* new_v = new_k + hd;
    float* cs = reinterpret_cast<float*>(new_v + hd);
    float* sn = cs + 128;
    const bool holds_new = FUSED && fused.pages_rw != nullptr && len > 0 && pos / PAGE >= page_lo && pos / PAGE <= page_hi;
    if (FUSED) {
        const int half = fused.rd >> 1;
        for (int i = tid; i < half; i += NT) sincosf((float)pos * fused.inv_freq[i], &sn[i], &cs[i]);
        unit_sync<NAMED, NT>();
        before_inputs();
        // everything the step itself produced is asked for before any of it is used: the row's sum of squares, the
        // new key and value, the queries. One round trip to L2 instead of three (which was 2 of the 3 us between
        // the end of the projection and the first page's product).
        const float ssq = fused.row_sumsq ? __ldcg(fused.row_sumsq + b) : 0.f;
        const float* row = fused.qkv + (size_t)b * fused.ld;
        constexpr int KV_PER = (HD_MAX + NT - 1) / NT;
        float k_val[KV_PER], k_other[KV_PER], v_val[KV_PER];
        if (holds_new) {
            const float* k_head = row + (size_t)(H + g) * hd;
            const float* v_head = row + (size_t)(H + G + g) * hd;
#pragma unroll
            for (int u = 0; u < KV_PER; ++u) {
                const int e = tid + u * NT;
                k_val[u] = k_other[u] = v_val[u] = 0.f;
                if (e < hd) {
                    k_val[u] = __ldcg(k_head + e);
                    if (e < fused.rd) k_other[u] = __ldcg(k_head + rotation_partner(e, fused.rd, fused.interleaved));
                    v_val[u] = __ldcg(v_head + e);
                }
            }
        }
        // the queries (heads beyond the unit's own are zero): the loads of four elements (each with its partner of
        // the rotation) are in flight together
        for (int idx0 = tid; idx0 < HEAD_ROWS * hd; idx0 += 4 * NT) {
            float val[4], other[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = idx0 + u * NT;
                val[u] = other[u] = 0.f;
                if (idx < HEAD_ROWS * hd) {
                    const int r = idx / hd, e = idx - r * hd;
                    if (r < nrows) {
                        const float* head = row + (size_t)(head0 + r) * hd;
                        val[u] = __ldcg(head + e);
                        if (e < fused.rd) other[u] = __ldcg(head + rotation_partner(e, fused.rd, fused.interleaved));
                    }
                }
            }
            const float in_scale = fused.row_sumsq ? 1.0f / sqrtf(ssq / (float)fused.norm_width + fused.norm_eps) : 1.0f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = idx0 + u * NT;
                if (idx < HEAD_ROWS * hd) {
                    const int e = idx % hd;
                    q_s[idx] = __float2bfloat16_rn(rotate_value(val[u], other[u], e, fused.rd, fused.interleaved, cs, sn) * in_scale);
                }
            }
        }
        if (holds_new) {
            const float in_scale = fused.row_sumsq ? 1.0f / sqrtf(ssq / (float)fused.norm_width + fused.norm_eps) : 1.0f;
#pragma unroll
            for (int u = 0; u < KV_PER; ++u) {
                const int e = tid + u * NT;
                if (e < hd) {
                    new_k[e] = __float2bfloat16_rn(rotate_value(k_val[u], k_other[u], e, fused.rd, fused.interleaved, cs, sn) * in_scale);
                    new_v[e] = __float2bfloat16_rn(v_val[u] * in_scale);
                }
            }
        }
        unit_sync<NAMED, NT>();
        if (holds_new && hg == 0) {           // one CTA per (sequence, kv head) stores the new row
            const size_t base = ((size_t)table[pos / PAGE] * 2 * G + g) * PAGE * hd + (size_t)(pos % PAGE) * hd;
            for (int e = tid; e < hd; e += NT) {
                fused.pages_rw[base + e] = new_k[e];
                fused.pages_rw[base + (size_t)G * PAGE * hd + e] = new_v[e];
            }
        }
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            if (kk * 16 < hd) {
                const int c = kk * 16 + t4 * 2;
                qf[kk][0] = *reinterpret_cast<const uint32_t*>(q_s + g8 * hd + c);
                qf[kk][1] = *reinterpret_cast<const uint32_t*>(q_s + g8 * hd + c + 8);
            }
        }
    } else {
        before_inputs();
        // heads beyond the unit's own repeat its last one (finite values; their results are never stored)
        const __nv_bfloat16* q_row = q + ((size_t)b * H + head0 + min(g8, nrows - 1)) * hd;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            if (kk * 16 < hd) {
                const int c = kk * 16 + t4 * 2;
                qf[kk][0] = *reinterpret_cast<const uint32_t*>(q_row + c);
                qf[kk][1] = *reinterpret_cast<const uint32_t*>(q_row + c + 8);
            }
        }
    }
    // O^T: tile mt holds features 16 mt + g8 (o[mt][0..1]) and 16 mt + 8 + g8 (o[mt][2..3]) of heads 2 t4, 2 t4 + 1
    float o[KSTEPS][4];
#pragma unroll
    for (int i = 0; i < KSTEPS; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = NEG_BIG, m1 = NEG_BIG, l0 = 0.f, l1 = 0.f;       // running maximum and sum of heads 2 t4 and 2 t4 + 1

    const int ngroups = (npages + PG - 1) / PG;
    const int new_at = pos / PAGE - page_lo;         // which of the share's pages holds the new token
    const int cpr = hd >> 3;
    const int frag_row = (lane & 7) + ((lane >> 3) & 1) * 8, frag_chunk = lane >> 4;      // ldmatrix.x4 for a 16 x 16 row operand
    for (int gi = 0; gi < ngroups; ++gi) {
        const bool patch = FUSED && holds_new && new_at >= gi * PG && new_at < (gi + 1) * PG;
        if (!TMA) {
            cp_async_wait<GROUPS - 1>();             // all but the newest groups of copies: this group's pages are there
            unit_sync<NAMED, NT>();
        } else if (patch) {
            mbar_wait(&full[new_at % STAGES], (uint32_t)(new_at / STAGES) & 1u);      // its owners check the outcome below
        }
        if (patch) {
            // the copy of this page predates the new token: put its key and value in place
            const int row = pos % PAGE;
            uint8_t* tile = smem + (new_at % STAGES) * stage_bytes;
            for (int c = tid; c < 2 * cpr; c += NT) {
                const int which = c >= cpr, cc = which ? c - cpr : c;
                const uint4 v = *reinterpret_cast<const uint4*>((which ? new_v : new_k) + cc * 8);
                *reinterpret_cast<uint4*>(tile + which * (PAGE * hd * 2) + tile_offset<TMA>(row, cc, hd, cpr)) = v;
            }
            unit_sync<NAMED, NT>();
        }
        const int i = gi * PG + pg;                  // this warp's page
        bool arrived = true;
        if (TMA && i < npages) {
            arrived = mbar_wait(&full[i % STAGES], (uint32_t)(i / STAGES) & 1u);
            if (!arrived && lane == 0) atomicExch(status, 6);
        }
        if (i < npages && arrived) {
            const int key_base = (page_lo + i) * PAGE;
            const uint32_t k_tile = smem_u32(smem + (i % STAGES) * stage_bytes);
            const uint32_t v_tile = k_tile + PAGE * hd * 2;
            const int key0 = kw * 16;                    // this warp's 16 keys of its page
            if (key_base + key0 <= pos && key_base + key0 + 15 >= lo) {
                // S^T: s[0], s[1] = key g8 with heads 2 t4, 2 t4 + 1; s[2], s[3] = key g8 + 8 with the same heads
                float s[4] = {0.f, 0.f, 0.f, 0.f};
                const int k_row = key0 + frag_row;
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk) {
                    if (kk * 16 < hd) {
                        uint32_t a[4];
                        ldmatrix_x4(k_tile + tile_offset<TMA>(k_row, kk * 2 + frag_chunk, hd, cpr), a[0], a[1], a[2], a[3]);
                        mma_bf16(s, a, qf[kk][0], qf[kk][1]);
                    }
                }
                const int key_a = key_base + key0 + g8, key_b = key_a + 8;
                const bool out_a = key_a > pos || key_a < lo, out_b = key_b > pos || key_b < lo;
                s[0] = out_a ? NEG_BIG : s[0] * scale_log2; s[1] = out_a ? NEG_BIG : s[1] * scale_log2;
                s[2] = out_b ? NEG_BIG : s[2] * scale_log2; s[3] = out_b ? NEG_BIG : s[3] * scale_log2;
                float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);        // over the 16 keys: the lanes of equal t4
#pragma unroll
                for (int sh = 4; sh < 32; sh <<= 1) {
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
                }
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
                const float a0 = fast_exp2(m0 - mn0), a1 = fast_exp2(m1 - mn1);
                m0 = mn0; m1 = mn1;
                const float e0 = out_a ? 0.f : fast_exp2(s[0] - mn0), e1 = out_a ? 0.f : fast_exp2(s[1] - mn1);
                const float e2 = out_b ? 0.f : fast_exp2(s[2] - mn0), e3 = out_b ? 0.f : fast_exp2(s[3] - mn1);
                l0 = l0 * a0 + (e0 + e2);
                l1 = l1 * a1 + (e1 + e3);
                // P^T as the column operand of the second product: (keys 2 t4, 2 t4 + 1 | + 8, head g8)
                const uint32_t p0 = transpose_8x8(pack_bf16(e0, e1)), p1 = transpose_8x8(pack_bf16(e2, e3));
                const int v_row = key0 + (lane & 7) + (lane >> 4) * 8;          // ldmatrix.x4.trans for V^T, 16 features x 16 keys
                const int v_chunk = (lane >> 3) & 1;
#pragma unroll
                for (int mt = 0; mt < KSTEPS; ++mt) {
                    if (mt * 16 < hd) {
                        o[mt][0] *= a0; o[mt][1] *= a1; o[mt][2] *= a0; o[mt][3] *= a1;
                        uint32_t a[4];
                        ldmatrix_x4_trans(v_tile + tile_offset<TMA>(v_row, mt * 2 + v_chunk, hd, cpr), a[0], a[1], a[2], a[3]);
                        mma_bf16(o[mt], a, p0, p1);
                    }
                }
            }
        }
        unit_sync<NAMED, NT>();
        // the group's stages are free: the group that comes GROUPS later goes there
        if (TMA) {
            if (warp == 0) {
                for (int j = 0; j < PG; ++j) {
                    const int nxt = (gi + GROUPS) * PG + j;
                    if (nxt < npages) {
                        const int page = page_number(nxt);
                        if (lane == 0) request_page(nxt, page);
                    }
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < PG; ++j) {
                const int nxt = (gi + GROUPS) * PG + j;
                if (nxt < npages)
                    load_page(smem + (nxt % STAGES) * stage_bytes, pages, table[page_lo + nxt], G, g, hd, tid, NT);
            }
            cp_async_commit();
        }
    }
    if (!TMA) {
        cp_async_wait<0>();
        unit_sync<NAMED, NT>();
    }

    // merge the warps (each saw a quarter of some pages) through shared memory; a head's sum over the keys lies in
    // the lanes of equal t4
#pragma unroll
    for (int sh = 4; sh < 32; sh <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
        l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
    }
    float* sm_m = reinterpret_cast<float*>(smem);            // [NW][8]
    float* sm_l = sm_m + NW * HEAD_ROWS;                     // [NW][8]
    float* sm_o = sm_l + NW * HEAD_ROWS;                     // [NW][8][hd]
    if (g8 == 0) {
        sm_m[warp * HEAD_ROWS + 2 * t4] = m0; sm_m[warp * HEAD_ROWS + 2 * t4 + 1] = m1;
        sm_l[warp * HEAD_ROWS + 2 * t4] = l0; sm_l[warp * HEAD_ROWS + 2 * t4 + 1] = l1;
    }
#pragma unroll
    for (int mt = 0; mt < KSTEPS; ++mt) {
        const int d = mt * 16 + g8;
        if (d < hd) {
            float* head_a = sm_o + ((size_t)warp * HEAD_ROWS + 2 * t4) * hd;
            float* head_b = head_a + hd;
            head_a[d] = o[mt][0]; head_b[d] = o[mt][1];
            head_a[d + 8] = o[mt][2]; head_b[d + 8] = o[mt][3];
        }
    }
    unit_sync<NAMED, NT>();
    for (int idx = tid; idx < nrows * hd; idx += NT) {
        const int r = idx / hd, d = idx - r * hd;
        float m = NEG_BIG;
#pragma unroll
        for (int w = 0; w < NW; ++w) m = fmaxf(m, sm_m[w * HEAD_ROWS + r]);
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float f = fast_exp2(sm_m[w * HEAD_ROWS + r] - m);
            acc += sm_o[((size_t)w * HEAD_ROWS + r) * hd + d] * f;
            l += sm_l[w * HEAD_ROWS + r] * f;
        }
        if ((FUSED ? shares : num_splits) == 1) {   // the only share: this is the result
            out[((size_t)b * H + head0 + r) * hd + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        } else {
            const size_t slot = ((size_t)b * H + head0 + r) * num_splits + split;
            part_o[slot * hd + d] = acc;
            if (d == 0) { part_ml[slot * 2] = m; part_ml[slot * 2 + 1] = l; }
        }
    }
    if (FUSED && shares > 1) {
        // the last share of this (sequence, kv head, head group) to arrive merges them all
        __shared__ int last;
        __threadfence();
        unit_sync<NAMED, NT>();
        int* counter = fused.counters + ((size_t)b * G + g) * head_groups + hg;
        if (tid == 0) {
            const int ticket = atomicAdd(counter, 1);
            last = ticket == shares - 1;
            if (last) *counter = 0;                 // ready for the next launch
        }
        unit_sync<NAMED, NT>();
        if (last) {
            __threadfence();
            for (int idx = tid; idx < nrows * hd; idx += NT) {
                const int r = idx / hd, d = idx - r * hd;
                const size_t base = ((size_t)b * H + head0 + r) * num_splits;
                // the shares' (max, sum, output) are requested eight shares at a time, then combined
                float m = NEG_BIG;
                for (int s0 = 0; s0 < shares; s0 += 8) {
                    float mm[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) mm[u] = s0 + u < shares ? __ldcg(part_ml + (base + s0 + u) * 2) : NEG_BIG;
#pragma unroll
                    for (int u = 0; u < 8; ++u) m = fmaxf(m, mm[u]);
                }
                float acc = 0.f, l = 0.f;
                for (int s0 = 0; s0 < shares; s0 += 8) {
                    float mm[8], ll[8], oo[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const bool in = s0 + u < shares;
                        mm[u] = in ? __ldcg(part_ml + (base + s0 + u) * 2) : NEG_BIG;
                        ll[u] = in ? __ldcg(part_ml + (base + s0 + u) * 2 + 1) : 0.f;
                        oo[u] = in ? __ldcg(part_o + (base + s0 + u) * hd + d) : 0.f;
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        if (ll[u] > 0.f) {
                            const float f = fast_exp2(mm[u] - m);
                            l += ll[u] * f;
                            acc += oo[u] * f;
                        }
                    }
                }
                out[((size_t)b * H + head0 + r) * hd + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
            }
        }
    }
    unit_sync<NAMED, NT>();          // the scratch may be reused by the caller's next unit
}

}  // namespace
