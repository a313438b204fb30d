// Prefill attention on the Blackwell tensor cores, head size 64: scores and the
// probabilities-times-values product run as tcgen05.mma with accumulators in tensor memory.
//
// A CTA takes 128 consecutive new tokens of one sequence and one query head. Per page of 64
// keys of the sequence's cache:
//   loader warp   TMA brings the page's K tile and V tile (64 x 64 bf16 each, 128-byte swizzle)
//                 into a ring of stages; the Q tile (128 x 64) is loaded once
//   MMA warp      S[128 x 64] = Q K^T into tensor memory (both operands K-major), and, once the
//                 probabilities are in shared memory, O_page[128 x 64] = P V (V is the N operand
//                 with N contiguous: the "MN-major" form of the same 128-byte-swizzled tile)
//   8 softmax warps  two threads per query row, each with half of the page's keys and half of the
//                 output features: read S from tensor memory, mask (causal, window), exchange the
//                 halves' maxima through shared memory, running maximum and sum in float32 with
//                 exp2, write P as bf16 into the swizzled shared-memory tile that feeds the second
//                 MMA, and add the previous page's O_page into the row's output held in registers
//                 (rescaled by the change of the maximum)
// S, P and O_page are double-buffered: the scores of page i+1 are formed while the softmax of
// page i runs, and P V of page i is collected one iteration later, so that no MMA latency lies
// between two softmax passes. Two CTAs fit an SM.
//
// Reference counterpart: src/main/resources/kernels/cuda/attention.cu:10-108 (one query at a
// time, SIMT); the online-softmax recurrence is that of inference/Attention.java:161-207.
// Every mbarrier wait is bounded; a wait that runs out sets *status and the CTA winds down.
#include "tcgen05_utils.cuh"

namespace {

constexpr int HD = 64;
constexpr int ROWS = 128;          // query rows per CTA = MMA M
constexpr int PAGE = 64;           // keys per page = MMA N of the scores
constexpr int STAGES = 3;
constexpr int Q_BYTES = ROWS * HD * 2;            // 16 KB
constexpr int KV_BYTES = PAGE * HD * 2;           // 8 KB each
constexpr int STAGE_BYTES = 2 * KV_BYTES;
constexpr int P_BYTES = ROWS * PAGE * 2;          // 16 KB
constexpr int XCHG_BYTES = 2 * 2 * ROWS * 4;      // row maxima of the two halves, double-buffered
constexpr int SMEM_BYTES = Q_BYTES + STAGES * STAGE_BYTES + 2 * P_BYTES + XCHG_BYTES + 1024 + 256;
// Two float32 operations in one instruction (Blackwell's packed f32x2 forms): the softmax warps are bound by
// how many instructions they issue.
__device__ __forceinline__ void fma2(float& x0, float& x1, float a, float b) {            // x = x * a + b
    uint64_t vx, va, vb;
    asm("mov.b64 %0, {%1, %2};" : "=l"(vx) : "f"(x0), "f"(x1));
    asm("mov.b64 %0, {%1, %1};" : "=l"(va) : "f"(a));
    asm("mov.b64 %0, {%1, %1};" : "=l"(vb) : "f"(b));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(vx) : "l"(vx), "l"(va), "l"(vb));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(vx));
}
__device__ __forceinline__ void addmul2(float& x0, float& x1, float y0, float y1, float a) {   // x = (x + y) * a
    uint64_t vx, vy, va;
    asm("mov.b64 %0, {%1, %2};" : "=l"(vx) : "f"(x0), "f"(x1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(vy) : "f"(y0), "f"(y1));
    asm("mov.b64 %0, {%1, %1};" : "=l"(va) : "f"(a));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(vx) : "l"(vx), "l"(vy));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(vx) : "l"(vx), "l"(va));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(vx));
}

__device__ __forceinline__ void add2(float& x0, float& x1, float y0, float y1) {              // x += y
    uint64_t vx, vy;
    asm("mov.b64 %0, {%1, %2};" : "=l"(vx) : "f"(x0), "f"(x1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(vy) : "f"(y0), "f"(y1));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(vx) : "l"(vx), "l"(vy));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(vx));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

constexpr int THREADS = 320;       // warp 0: loader, warp 1: MMA, warps 2-9: softmax
constexpr int TMEM_COLS = 256;     // S[2]: 0..127, O_page[2]: 128..255

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            __nv_bfloat16* __restrict__ out, const int* __restrict__ page_table, int pt_stride,
                            const int* __restrict__ q_start, const int* __restrict__ kv_len, int H, int G,
                            float scale_log2, int window, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_tile = smem;
    uint8_t* ring = smem + Q_BYTES;
    uint8_t* p_tile = ring + STAGES * STAGE_BYTES;
    float* xchg = (float*)(p_tile + 2 * P_BYTES);            // [2 buffers][2 halves][ROWS]
    uint64_t* bars = (uint64_t*)((uint8_t*)xchg + XCHG_BYTES);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;                  // [STAGES]
    uint64_t* kv_empty = kv_full + STAGES;         // [STAGES]
    uint64_t* s_ready = kv_empty + STAGES;         // [2] scores of a page are in tensor memory
    uint64_t* p_ready = s_ready + 2;               // [2] probabilities of a page are in shared memory
    uint64_t* o_ready = p_ready + 2;               // [2] P V of a page is in tensor memory
    uint32_t* tmem_slot = (uint32_t*)(o_ready + 2);
    volatile uint32_t* failed = tmem_slot + 1;

    lp_grid_release();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y, tile = gridDim.x - 1 - blockIdx.x;     // heavy tiles first

    if (threadIdx.x == 0) {
        *failed = 0;
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kv) : "memory");
        mbar_init(q_full, 1);
        for (int s = 0; s < STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
        for (int k = 0; k < 2; ++k) {
            mbar_init(&s_ready[k], 1);
            mbar_init(&p_ready[k], 8);             // one arrival per softmax warp
            mbar_init(&o_ready[k], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    lp_grid_wait();                                // everything below reads what earlier kernels wrote
    const int t_begin = q_start[b], n_new = q_start[b + 1] - t_begin;
    const bool has_work = tile * ROWS < n_new;     // uniform over the CTA
    const int g = h / (H / G);
    const int len = kv_len[b];
    const int pos0 = len - n_new;
    const int row0 = tile * ROWS;
    const int rows = has_work ? min(ROWS, n_new - row0) : 0;
    const int first_pos = pos0 + row0, last_pos = pos0 + row0 + rows - 1;
    const int lo = window > 0 ? max(0, first_pos - window + 1) : 0;
    const int page_lo = lo / PAGE, page_hi = last_pos / PAGE;
    const int npages = has_work ? page_hi - page_lo + 1 : 0;
    const int* table = page_table + (size_t)b * pt_stride;

    if (warp == 0) {
        // ------------------------------------------------------------ loader
        if (lane == 0 && has_work) {
            mbar_expect_tx(q_full, Q_BYTES);
            tma_load_2d(q_tile, &map_q, h * HD, t_begin + row0, q_full);
            for (int i = 0; i < npages; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (i / STAGES) & 1;
                if (!mbar_wait(&kv_empty[s], phase ^ 1)) { atomicExch(status, 11); *failed = 1; break; }
                const int page = table[page_lo + i];
                const int row = ((page * 2) * G + g) * PAGE;          // K rows; V rows lie G * PAGE further
                mbar_expect_tx(&kv_full[s], STAGE_BYTES);
                tma_load_2d(ring + s * STAGE_BYTES, &map_kv, 0, row, &kv_full[s]);
                tma_load_2d(ring + s * STAGE_BYTES + KV_BYTES, &map_kv, 0, row + G * PAGE, &kv_full[s]);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && has_work) {
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PAGE >> 3) << 17) |
                                         ((uint32_t)(ROWS >> 4) << 24);
            constexpr uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |      // B is MN-major
                                          ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) { atomicExch(status, 12); *failed = 1; }
            const uint64_t dq = smem_desc(smem_u32(q_tile));
            auto scores = [&](int i) -> bool {          // S(i) into buffer i & 1
                const int s = i % STAGES;
                if (!mbar_wait(&kv_full[s], (i / STAGES) & 1)) { atomicExch(status, 13); *failed = 1; return false; }
                tcgen05_fence_after();
                const uint64_t dk = smem_desc(smem_u32(ring + s * STAGE_BYTES));
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    tcgen05_mma(tmem_base + (i & 1) * PAGE, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_s,
                                k > 0 ? 1u : 0u);
                tcgen05_commit(&s_ready[i & 1]);
                return true;
            };
            if (ok) ok = scores(0);
            for (int i = 0; i < npages && ok; ++i) {
                // the scores of the next page are formed while the softmax of this one runs
                // (their buffer was released by p_ready of page i - 1, awaited one iteration ago)
                if (i + 1 < npages && !scores(i + 1)) { ok = false; break; }
                if (!mbar_wait(&p_ready[i & 1], (i >> 1) & 1)) { atomicExch(status, 14); *failed = 1; ok = false; break; }
                tcgen05_fence_after();
                const int s = i % STAGES;
                const uint32_t v_addr = smem_u32(ring + s * STAGE_BYTES + KV_BYTES);
                const uint64_t dp = smem_desc(smem_u32(p_tile + (i & 1) * P_BYTES));
#pragma unroll
                for (int k = 0; k < PAGE / 16; ++k)          // 16 keys = two groups of 8 rows of the V tile
                    tcgen05_mma(tmem_base + 2 * PAGE + (i & 1) * HD, dp + (uint64_t)(k * 2),
                                smem_desc_mn(v_addr + k * 2048, 0), idesc_pv, k > 0 ? 1u : 0u);
                tcgen05_commit(&kv_empty[s]);                // the stage is free once both products have read it
                tcgen05_commit(&o_ready[i & 1]);
            }
        }
        __syncwarp();
    } else if (has_work) {
        // ------------------------------------------------------------ softmax, two threads per row
        constexpr int HALF = PAGE / 2;                       // keys of a page, and output features, per thread
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;                    // warps 2-5: first half, warps 6-9: second half
        const int r = quarter * 32 + lane;                   // row of the tile = TMEM lane
        const int pos = first_pos + min(r, rows - 1);
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float o[HALF];
#pragma unroll
        for (int d = 0; d < HALF; ++d) o[d] = 0.f;
        float m = -1.0e30f, l = 0.f;
        bool ok = true;
        for (int i = 0; i < npages; ++i) {
            uint32_t sreg[HALF];
            if (ok && !mbar_wait(&s_ready[i & 1], (i >> 1) & 1)) { if (lane == 0) atomicExch(status, 15); *failed = 1; ok = false; }
            tcgen05_fence_after();
            if (ok) {
                tmem_ld32(lane_addr + (i & 1) * PAGE + half * HALF, sreg);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < HALF; ++j) sreg[j] = 0;
            }
            const int key_base = (page_lo + i) * PAGE + half * HALF;
            const bool edge = key_base + HALF - 1 > first_pos || (window > 0 && key_base <= last_pos - window);
            if (edge) {
#pragma unroll
                for (int j = 0; j < HALF; ++j) {
                    const int key = key_base + j;
                    if (key > pos || (window > 0 && key <= pos - window)) sreg[j] = 0xff800000u;      // -inf
                }
            }
            // independent chains for the maximum (and below for the sum): one chain of dependent
            // operations would cost its full latency on a warp that has little else to issue
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < HALF; j += 8) {             // three-input maximum: two scores per instruction
                mx4[0] = max3(mx4[0], __uint_as_float(sreg[j]), __uint_as_float(sreg[j + 1]));
                mx4[1] = max3(mx4[1], __uint_as_float(sreg[j + 2]), __uint_as_float(sreg[j + 3]));
                mx4[2] = max3(mx4[2], __uint_as_float(sreg[j + 4]), __uint_as_float(sreg[j + 5]));
                mx4[3] = max3(mx4[3], __uint_as_float(sreg[j + 6]), __uint_as_float(sreg[j + 7]));
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            float* mine = xchg + ((i & 1) * 2 + half) * ROWS;
            const float* other = xchg + ((i & 1) * 2 + (half ^ 1)) * ROWS;
            mine[r] = mx;
            // the two warps that share these 32 rows (each has half of the keys) meet; the other six go on
            asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");
            mx = fmaxf(mx, other[r]);
            const float m_new = fmaxf(m, mx * scale_log2);
            const float alpha = ex2(m - m_new);
            m = m_new;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint8_t* p_row = p_tile + (i & 1) * P_BYTES + r * 128;
#pragma unroll
            for (int c = 0; c < HALF / 8; ++c) {
                float e[8];
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    e[j] = __uint_as_float(sreg[c * 8 + j]);
                    e[j + 1] = __uint_as_float(sreg[c * 8 + j + 1]);
                    fma2(e[j], e[j + 1], scale_log2, -m_new);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) e[j] = ex2(e[j]);
                add2(sum4[0], sum4[1], e[0], e[1]);
                add2(sum4[2], sum4[3], e[2], e[3]);
                add2(sum4[0], sum4[1], e[4], e[5]);
                add2(sum4[2], sum4[3], e[6], e[7]);
                uint4 packed;
                __nv_bfloat162 t0 = __floats2bfloat162_rn(e[0], e[1]), t1 = __floats2bfloat162_rn(e[2], e[3]);
                __nv_bfloat162 t2 = __floats2bfloat162_rn(e[4], e[5]), t3 = __floats2bfloat162_rn(e[6], e[7]);
                packed.x = *reinterpret_cast<uint32_t*>(&t0); packed.y = *reinterpret_cast<uint32_t*>(&t1);
                packed.z = *reinterpret_cast<uint32_t*>(&t2); packed.w = *reinterpret_cast<uint32_t*>(&t3);
                *reinterpret_cast<uint4*>(p_row + (((half * (HALF / 8) + c) ^ (r & 7)) << 4)) = packed;
            }
            l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            // the probabilities were written through the generic proxy; the MMA reads through the async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[i & 1]);
            // collect P V of the previous page (long finished) and bring the sum to this page's maximum
            if (i > 0) {
                const int pi = i - 1;
                if (ok && !mbar_wait(&o_ready[pi & 1], (pi >> 1) & 1)) { if (lane == 0) atomicExch(status, 16); *failed = 1; ok = false; }
                tcgen05_fence_after();
                if (ok) {
                    uint32_t oreg[HALF];
                    tmem_ld32(lane_addr + 2 * PAGE + (pi & 1) * HD + half * HALF, oreg);
                    tmem_ld_wait();
#pragma unroll
                    for (int d = 0; d < HALF; d += 2)
                        addmul2(o[d], o[d + 1], __uint_as_float(oreg[d]), __uint_as_float(oreg[d + 1]), alpha);
                }
                tcgen05_fence_before();
            }
        }
        if (npages > 0) {
            const int pi = npages - 1;
            if (ok && !mbar_wait(&o_ready[pi & 1], (pi >> 1) & 1)) { if (lane == 0) atomicExch(status, 16); *failed = 1; ok = false; }
            tcgen05_fence_after();
            if (ok) {
                uint32_t oreg[HALF];
                tmem_ld32(lane_addr + 2 * PAGE + (pi & 1) * HD + half * HALF, oreg);
                tmem_ld_wait();
#pragma unroll
                for (int d = 0; d < HALF; ++d) o[d] += __uint_as_float(oreg[d]);
            }
            tcgen05_fence_before();
        }
        // the two halves of a row add their sums
        float* mine = xchg + half * ROWS;
        const float* other = xchg + (half ^ 1) * ROWS;
        asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");       // both are past the last maximum exchange
        mine[r] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");
        l += other[r];
        if (ok && *failed == 0 && r < rows) {
            const float inv = 1.0f / l;
            __nv_bfloat16* dst = out + ((size_t)(t_begin + row0 + r) * H + h) * HD + half * HALF;
#pragma unroll
            for (int c = 0; c < HALF / 8; ++c) {
                uint4 packed;
                __nv_bfloat162 t0 = __floats2bfloat162_rn(o[c * 8] * inv, o[c * 8 + 1] * inv);
                __nv_bfloat162 t1 = __floats2bfloat162_rn(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
                __nv_bfloat162 t2 = __floats2bfloat162_rn(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv);
                __nv_bfloat162 t3 = __floats2bfloat162_rn(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
                packed.x = *reinterpret_cast<uint32_t*>(&t0); packed.y = *reinterpret_cast<uint32_t*>(&t1);
                packed.z = *reinterpret_cast<uint32_t*>(&t2); packed.w = *reinterpret_cast<uint32_t*>(&t3);
                reinterpret_cast<uint4*>(dst)[c] = packed;
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS));
    }
}

}  // namespace

// q, out: [T, H, 64] bf16 (T = all new tokens of the step); pages: [num_pages, 2, G, 64, 64] bf16;
// q_start: [B+1]; kv_len: [B] (after the step). status: one int in device memory.
extern "C" int lp_attention_prefill_tc(const void* q, void* out, const void* pages, long long num_pages,
                                       const int* page_table, int pt_stride, const int* q_start, const int* kv_len,
                                       int B, int T, int max_new, int H, int G, int hd, int page_size, float scale,
                                       int window, int* status, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (hd != HD) LP_REFUSE("attention_prefill_tc: head size %d (this kernel is built for %d)", hd, HD);
    if (page_size != PAGE) LP_REFUSE("attention_prefill_tc: pages of %d positions (built for %d)", page_size, PAGE);
    if (H <= 0 || G <= 0 || H % G) LP_REFUSE("attention_prefill_tc: %d query heads over %d key heads", H, G);
    if (H > 65535 || B > 65535) LP_REFUSE("attention_prefill_tc: %d heads x %d sequences exceed the grid", H, B);
    if (((uintptr_t)q | (uintptr_t)pages) & 15) LP_REFUSE("attention_prefill_tc: operands must be 16-byte aligned");
    CUtensorMap mq, mkv;
    int rc = make_map(&mq, q, T, (long long)H * HD, (long long)H * HD, ROWS);
    if (rc) return rc;
    rc = make_map(&mkv, pages, num_pages * 2 * G * PAGE, HD, HD, PAGE);
    if (rc) return rc;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             SMEM_BYTES);
        if (e != cudaSuccess) LP_REFUSE("attention_prefill_tc: cannot reserve %d bytes of shared memory: %s", SMEM_BYTES,
                                        cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid((max_new + ROWS - 1) / ROWS, H, B);
    cudaError_t err = lp_launch(attention_prefill_tc_kernel, grid, THREADS, SMEM_BYTES, stream, mq, mkv,
                                (__nv_bfloat16*)out, page_table, pt_stride, q_start, kv_len, H, G,
                                scale * 1.4426950408889634f, window, status);
    if (err != cudaSuccess) {
        snprintf(lp_error_text, sizeof(lp_error_text), "attention_prefill_tc: %s", cudaGetErrorString(err));
        return (int)err;
    }
    return lp_check_launch("attention_prefill_tc");
}
