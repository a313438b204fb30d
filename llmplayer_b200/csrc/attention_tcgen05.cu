// Prefill attention on the Blackwell tensor cores, head sizes 64 and 128: scores and the
// probabilities-times-values product run as tcgen05.mma with accumulators in tensor memory.
//
// A CTA takes 128 consecutive new tokens of one sequence and one query head. Per page of 64
// keys of the sequence's cache:
//   loader warp   TMA brings the page's K tile and V tile (64 keys x head size bf16 each, 128-byte swizzle,
//                 in blocks of 64 features) into a ring of stages; the Q tile (128 rows) is loaded once
//   MMA warp      S[128 x 64] = Q K^T into tensor memory (both operands K-major), and, once the
//                 probabilities are in shared memory, O[128 x head size] += P V (V is the N operand
//                 with N contiguous: the "MN-major" form of the same 128-byte-swizzled tile)
//   8 softmax warps  two threads per query row, each with half of the page's keys and half of the
//                 output features: read S from tensor memory, mask (causal, window), exchange the
//                 halves' maxima through shared memory, keep the row's sum in float32 with exp2, and
//                 write P as bf16 into the swizzled shared-memory tile that feeds the second MMA
// The output accumulates in tensor memory over all pages and is read once at the end. The exponentials
// of a row are taken relative to a reference maximum that only moves when the row's true maximum has
// outgrown it by more than 2^8 (the probabilities then still fit bfloat16 and the sums float32 with
// room to spare); only then does the thread bring its half of the row's output in tensor memory and
// its sum down to the new reference. With random scores this happens in a row's first pages and
// hardly ever after, so the softmax warps, which are bound by the instructions they issue, no longer
// read and rescale a page's product on every page.
// S and P are double-buffered: the scores of page i+1 are formed while the softmax of page i runs.
// Two CTAs fit an SM at head size 64, one at head size 128.
//
// Reference counterpart: src/main/resources/kernels/cuda/attention.cu:10-108 (one query at a
// time, SIMT); the online-softmax recurrence is that of inference/Attention.java:161-207.
// Every mbarrier wait is bounded; a wait that runs out sets *status and the CTA winds down.
#include "tcgen05_utils.cuh"

namespace {

constexpr int ROWS = 128;          // query rows per CTA = MMA M
constexpr int PAGE = 64;           // keys per page = MMA N of the scores
constexpr int P_BYTES = ROWS * PAGE * 2;          // 16 KB
constexpr int XCHG_BYTES = 2 * 2 * ROWS * 4;      // row maxima of the two halves, double-buffered
constexpr float RESCALE_ABOVE = 8.0f;             // in log2 units: the reference maximum may lag by a factor of 256

template <int HD> struct Shape {
    static constexpr int BLOCKS = HD / 64;                   // blocks of 64 features (one swizzle row each)
    static constexpr int STAGES = 3;
    static constexpr int Q_BYTES = ROWS * HD * 2;
    static constexpr int KV_BYTES = PAGE * HD * 2;           // a K tile, or a V tile
    static constexpr int STAGE_BYTES = 2 * KV_BYTES;
    static constexpr int SMEM_BYTES = Q_BYTES + STAGES * STAGE_BYTES + 2 * P_BYTES + XCHG_BYTES + 1024 + 256;
    static constexpr int TMEM_COLS = 256;                    // S[2]: 0..127, O: 128 .. 128 + HD
    static constexpr int CTAS_PER_SM = HD == 64 ? 2 : 1;
};
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

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <int HD>
__global__ void __launch_bounds__(THREADS, Shape<HD>::CTAS_PER_SM)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            __nv_bfloat16* __restrict__ out, const int* __restrict__ page_table, int pt_stride,
                            const int* __restrict__ q_start, const int* __restrict__ kv_len, int H, int G,
                            float scale_log2, int window, int* __restrict__ status) {
    using SH = Shape<HD>;
    constexpr int STAGES = SH::STAGES, STAGE_BYTES = SH::STAGE_BYTES, KV_BYTES = SH::KV_BYTES, BLOCKS = SH::BLOCKS;
    constexpr int O_COL = 2 * PAGE;                          // the output's first column of tensor memory
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_tile = smem;                                  // BLOCKS tiles of [ROWS x 64]
    uint8_t* ring = smem + SH::Q_BYTES;                      // per stage: K (BLOCKS tiles of [PAGE x 64]), then V likewise
    uint8_t* p_tile = ring + STAGES * STAGE_BYTES;
    float* xchg = (float*)(p_tile + 2 * P_BYTES);            // [2 buffers][2 halves][ROWS]
    uint64_t* bars = (uint64_t*)((uint8_t*)xchg + XCHG_BYTES);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;                  // [STAGES]
    uint64_t* kv_empty = kv_full + STAGES;         // [STAGES]
    uint64_t* s_ready = kv_empty + STAGES;         // [2] scores of a page are in tensor memory
    uint64_t* p_ready = s_ready + 2;               // [2] probabilities of a page are in shared memory
    uint64_t* o_ready = p_ready + 2;               // [2] P V of a page has been added to the output
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
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)SH::TMEM_COLS) : "memory");
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
            mbar_expect_tx(q_full, SH::Q_BYTES);
#pragma unroll
            for (int c = 0; c < BLOCKS; ++c)
                tma_load_2d(q_tile + c * (ROWS * 128), &map_q, h * HD + c * 64, t_begin + row0, q_full);
            for (int i = 0; i < npages; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (i / STAGES) & 1;
                if (!mbar_wait(&kv_empty[s], phase ^ 1)) { atomicExch(status, 11); *failed = 1; break; }
                const int page = table[page_lo + i];
                const int row = ((page * 2) * G + g) * PAGE;          // K rows; V rows lie G * PAGE further
                mbar_expect_tx(&kv_full[s], STAGE_BYTES);
#pragma unroll
                for (int c = 0; c < BLOCKS; ++c) {
                    tma_load_2d(ring + s * STAGE_BYTES + c * (PAGE * 128), &map_kv, c * 64, row, &kv_full[s]);
                    tma_load_2d(ring + s * STAGE_BYTES + KV_BYTES + c * (PAGE * 128), &map_kv, c * 64, row + G * PAGE,
                                &kv_full[s]);
                }
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
            const uint32_t q_addr = smem_u32(q_tile);
            auto scores = [&](int i) -> bool {          // S(i) into buffer i & 1
                const int s = i % STAGES;
                if (!mbar_wait(&kv_full[s], (i / STAGES) & 1)) { atomicExch(status, 13); *failed = 1; return false; }
                tcgen05_fence_after();
                const uint32_t k_addr = smem_u32(ring + s * STAGE_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {          // 16 features per instruction; 4 instructions per block of 64
                    const uint64_t dq = smem_desc(q_addr + (k >> 2) * (ROWS * 128)) + (uint64_t)((k & 3) * 2);
                    const uint64_t dk = smem_desc(k_addr + (k >> 2) * (PAGE * 128)) + (uint64_t)((k & 3) * 2);
                    tcgen05_mma(tmem_base + (i & 1) * PAGE, dq, dk, idesc_s, k > 0 ? 1u : 0u);
                }
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
                    tcgen05_mma(tmem_base + O_COL, dp + (uint64_t)(k * 2),
                                smem_desc_mn(v_addr + k * 2048, PAGE * 128), idesc_pv, (i > 0 || k > 0) ? 1u : 0u);
                tcgen05_commit(&kv_empty[s]);                // the stage is free once both products have read it
                tcgen05_commit(&o_ready[i & 1]);
            }
        }
        __syncwarp();
    } else if (has_work) {
        // ------------------------------------------------------------ softmax, two threads per row
        constexpr int HALF = PAGE / 2;                       // keys of a page per thread
        constexpr int OHALF = HD / 2;                        // output features per thread
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;                    // warps 2-5: first half, warps 6-9: second half
        const int r = quarter * 32 + lane;                   // row of the tile = TMEM lane
        const int pos = first_pos + min(r, rows - 1);
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t o_addr = lane_addr + O_COL + half * OHALF;
        float m = -1.0e30f, l = 0.f;                         // m: the reference maximum the exponentials are taken against
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
            mx = fmaxf(mx, other[r]) * scale_log2;
            // The reference maximum follows only when the row's maximum has outgrown it by more than a factor of
            // 2^8. Then the sum so far and this thread's half of the output in tensor memory come down to the new
            // reference; the product of the previous page must have arrived there first, and the product of this
            // page is issued only after all eight warps have passed p_ready below.
            const bool moves = mx > m + RESCALE_ABOVE;
            if (__any_sync(0xffffffffu, moves && i > 0)) {
                const int pi = i - 1;
                if (ok && !mbar_wait(&o_ready[pi & 1], (pi >> 1) & 1)) { if (lane == 0) atomicExch(status, 16); *failed = 1; ok = false; }
                tcgen05_fence_after();
                const float factor = moves ? ex2(m - mx) : 1.0f;
                if (ok) {
#pragma unroll
                    for (int c = 0; c < OHALF; c += 32) {
                        uint32_t oreg[32];
                        tmem_ld32(o_addr + c, oreg);
                        tmem_ld_wait();
#pragma unroll
                        for (int d = 0; d < 32; ++d) oreg[d] = __float_as_uint(__uint_as_float(oreg[d]) * factor);
                        tmem_st32(o_addr + c, oreg);
                    }
                    tmem_st_wait();
                }
                tcgen05_fence_before();
            }
            if (moves) {
                l *= ex2(m - mx);
                m = mx;
            }
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint8_t* p_row = p_tile + (i & 1) * P_BYTES + r * 128;
#pragma unroll
            for (int c = 0; c < HALF / 8; ++c) {
                float e[8];
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    e[j] = __uint_as_float(sreg[c * 8 + j]);
                    e[j + 1] = __uint_as_float(sreg[c * 8 + j + 1]);
                    fma2(e[j], e[j + 1], scale_log2, -m);
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
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            // the probabilities were written through the generic proxy; the MMA reads through the async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[i & 1]);
        }
        // the two halves of a row add their sums (both are past the last maximum exchange)
        float* mine = xchg + half * ROWS;
        const float* other = xchg + (half ^ 1) * ROWS;
        asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");
        mine[r] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");
        l += other[r];
        if (npages > 0) {
            const int pi = npages - 1;
            if (ok && !mbar_wait(&o_ready[pi & 1], (pi >> 1) & 1)) { if (lane == 0) atomicExch(status, 16); *failed = 1; ok = false; }
            tcgen05_fence_after();
            const bool store = ok && *failed == 0 && r < rows;
            const float inv = 1.0f / l;
            __nv_bfloat16* dst = out + ((size_t)(t_begin + row0 + min(r, rows - 1)) * H + h) * HD + half * OHALF;
#pragma unroll
            for (int c0 = 0; c0 < OHALF; c0 += 32) {
                uint32_t oreg[32];
                if (ok) {                                    // warp-uniform: the loads are collective
                    tmem_ld32(o_addr + c0, oreg);
                    tmem_ld_wait();
                }
                if (store) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint4 packed;
                        __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(oreg[c * 8]) * inv, __uint_as_float(oreg[c * 8 + 1]) * inv);
                        __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(oreg[c * 8 + 2]) * inv, __uint_as_float(oreg[c * 8 + 3]) * inv);
                        __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(oreg[c * 8 + 4]) * inv, __uint_as_float(oreg[c * 8 + 5]) * inv);
                        __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(oreg[c * 8 + 6]) * inv, __uint_as_float(oreg[c * 8 + 7]) * inv);
                        packed.x = *reinterpret_cast<uint32_t*>(&t0); packed.y = *reinterpret_cast<uint32_t*>(&t1);
                        packed.z = *reinterpret_cast<uint32_t*>(&t2); packed.w = *reinterpret_cast<uint32_t*>(&t3);
                        reinterpret_cast<uint4*>(dst + c0)[c] = packed;
                    }
                }
            }
            tcgen05_fence_before();
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)SH::TMEM_COLS));
    }
}

template <int HD>
int launch_prefill_tc(const void* q, void* out, const void* pages, long long num_pages, const int* page_table,
                      int pt_stride, const int* q_start, const int* kv_len, int B, int T, int max_new, int H, int G,
                      float scale, int window, int* status, cudaStream_t stream) {
    using SH = Shape<HD>;
    CUtensorMap mq, mkv;
    int rc = make_map(&mq, q, T, (long long)H * HD, (long long)H * HD, ROWS);
    if (rc) return rc;
    rc = make_map(&mkv, pages, num_pages * 2 * G * PAGE, HD, HD, PAGE);
    if (rc) return rc;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             SH::SMEM_BYTES);
        if (e != cudaSuccess) LP_REFUSE("attention_prefill_tc: cannot reserve %d bytes of shared memory: %s", SH::SMEM_BYTES,
                                        cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid((max_new + ROWS - 1) / ROWS, H, B);
    cudaError_t err = lp_launch(attention_prefill_tc_kernel<HD>, grid, THREADS, SH::SMEM_BYTES, stream, mq, mkv,
                                (__nv_bfloat16*)out, page_table, pt_stride, q_start, kv_len, H, G,
                                scale * 1.4426950408889634f, window, status);
    if (err != cudaSuccess) {
        snprintf(lp_error_text, sizeof(lp_error_text), "attention_prefill_tc: %s", cudaGetErrorString(err));
        return (int)err;
    }
    return lp_check_launch("attention_prefill_tc");
}

}  // namespace

// q, out: [T, H, hd] bf16 (T = all new tokens of the step), hd 64 or 128; pages: [num_pages, 2, G, 64, hd] bf16;
// q_start: [B+1]; kv_len: [B] (after the step). status: one int in device memory.
extern "C" int lp_attention_prefill_tc(const void* q, void* out, const void* pages, long long num_pages,
                                       const int* page_table, int pt_stride, const int* q_start, const int* kv_len,
                                       int B, int T, int max_new, int H, int G, int hd, int page_size, float scale,
                                       int window, int* status, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (hd != 64 && hd != 128) LP_REFUSE("attention_prefill_tc: head size %d (this kernel is built for 64 and 128)", hd);
    if (page_size != PAGE) LP_REFUSE("attention_prefill_tc: pages of %d positions (built for %d)", page_size, PAGE);
    if (H <= 0 || G <= 0 || H % G) LP_REFUSE("attention_prefill_tc: %d query heads over %d key heads", H, G);
    if (H > 65535 || B > 65535) LP_REFUSE("attention_prefill_tc: %d heads x %d sequences exceed the grid", H, B);
    if (((uintptr_t)q | (uintptr_t)pages) & 15) LP_REFUSE("attention_prefill_tc: operands must be 16-byte aligned");
    if (hd == 64)
        return launch_prefill_tc<64>(q, out, pages, num_pages, page_table, pt_stride, q_start, kv_len, B, T, max_new, H, G,
                                     scale, window, status, stream);
    return launch_prefill_tc<128>(q, out, pages, num_pages, page_table, pt_stride, q_start, kv_len, B, T, max_new, H, G,
                                  scale, window, status, stream);
}
