// Tensor-core matrix product for bfloat16 weights stored [out, in]:
//   C[tokens, features] (=|+=) X[tokens, K] * W[features, K]^T          (float32 accumulation)
//
// Blackwell path: TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) brings
// tiles of W and X into a ring of shared-memory stages; one thread issues tcgen05.mma
// (kind::f16, bf16 in, fp32 out) with the accumulator in tensor memory; four warps read
// the accumulator back with tcgen05.ld and run the epilogue. The weights are the MMA's
// 128-row operand and the tokens its N operand (16..256), so the same kernel streams
// weights for a handful of decoding sequences and tiles a long prompt. A K range can be
// split over CTAs (grid.z); partial sums then meet in float32 atomics.
//
// Epilogues: store (float32 or bfloat16), add into a float32 output (the residual
// stream, or split-K partial sums), or the gated activation silu(gate) * up. For the
// latter W interleaves gate and up rows in blocks of 64 (rows 128t..128t+63 = gate features
// 64t..64t+63, rows 128t+64..128t+127 = the same features of up), so one accumulator tile
// holds both halves of 64 output features; the gate half crosses to the warps that hold
// the up half through shared memory. For large token tiles (prompts) a second form keeps a
// gate and an up accumulator of 128 features each, filled from 64-row boxes of the same
// layout, so that the activation needs no exchange.
//
// Three forms live in this file, chosen by the number of tokens of a step:
//   * gemm_tcgen05_kernel: one output tile per CTA, token tiles of 16..256 (what is described above);
//     serves 17 to some hundred tokens. gemm_tcgen05_normed_kernel: the same for 9 to 32 tokens with the RMS
//     norm of its input applied on the way in.
//   * gemm_fewtok_kernel: at most 16 tokens. The same TMA ring, but four warps of ldmatrix + mma.sync consume
//     it: the sums stay in registers and the epilogue, which nothing hides in a one-tile kernel, is a few
//     stores per thread. Can apply the RMS norm of its input itself (8 tokens at most).
//   * gemm_persistent_kernel: prompts. One CTA per SM walks over the tiles with two accumulators in tensor
//     memory; for the gated product the tokens are the MMA's M and 256 weight rows its N.
//
// Counterparts in the reference are its one-warp-per-row SIMT kernels
// (src/main/resources/kernels/cuda/matmul_bf16.cu:6-37, silu_mul.cu:6-15).
//
// Every wait on an mbarrier is bounded: after too many polls the waiting thread records
// an error code in *status, and the CTA winds down (outstanding copies are awaited,
// tensor memory is freed) instead of spinning forever.
#include "tcgen05_utils.cuh"

#define LP_GEMM_STORE 0
#define LP_GEMM_ACCUMULATE 1
#define LP_GEMM_SWIGLU 2
#define LP_GEMM_SWIGLU_WIDE 3   // same result and weight layout; two accumulators, 128 output features per CTA
#define LP_GEMM_SWIGLU_TOKM 4   // same again, persistent form only: 128 tokens are the MMA's M, 256 weight rows its N
#define LP_GEMM_QKV_TOKM 5      // persistent form only: the fused q|k|v projection with tokens as M; the epilogue rotates
                                // queries and keys and writes queries to their buffer, keys and values into the cache

namespace {

constexpr int BLOCK_FEAT = 128;   // weight rows per CTA = MMA M
constexpr int UMMA_K = 16;
// The weight tile(s) of one k-block. WIDE: gate rows of two neighbouring 64-feature blocks form the
// first 128-row tile, their up rows the second (the tensor map's box is 64 rows then).
template <int MODE>
__device__ __forceinline__ void load_weights(uint8_t* stage, const CUtensorMap* map_w, int k, int cta, uint64_t* bar,
                                             uint64_t read_once = 0) {
    if (MODE == LP_GEMM_SWIGLU_TOKM || MODE == LP_GEMM_QKV_TOKM) {
        tma_load_2d(stage, map_w, k, cta * 256, bar);            // one box of 256 rows (gated: gate | up | gate | up of 128 features)
    } else if (MODE == LP_GEMM_SWIGLU_WIDE) {
        const int row = cta * 256;
        tma_load_2d(stage, map_w, k, row, bar);                  // gate, features 128 cta ..
        tma_load_2d(stage + 8192, map_w, k, row + 128, bar);     // gate, features 128 cta + 64 ..
        tma_load_2d(stage + 16384, map_w, k, row + 64, bar);     // up
        tma_load_2d(stage + 24576, map_w, k, row + 192, bar);    // up
    } else if (read_once != 0) {
        tma_load_2d_hint(stage, map_w, k, cta * BLOCK_FEAT, bar, read_once);
    } else {
        tma_load_2d(stage, map_w, k, cta * BLOCK_FEAT, bar);
    }
}

// An RMS norm of the (float32) output rows, done by the last CTA to finish once every CTA has added
// its part: out_norm[t, i] = out[t, i] / sqrt(mean_i out[t]^2 + eps) * weight[i] in bfloat16. For
// products that add into the residual stream of a few decoding sequences, where the norm would
// otherwise be a kernel of its own between two products. `counter` is zero before the launch and zero
// again after it; `clear` (optional) is a float32 buffer the same CTA sets to zero.
struct NormAfter {
    const float* weight;       // null: no norm
    __nv_bfloat16* out_norm;
    float eps;
    int* counter;
    float* clear;
    long long clear_count;
};

// The tail of a product that adds into `out` with atomics: the last CTA to get here writes the norm (see NormAfter).
// Called by all threads of the CTA after their additions and a __threadfence().
template <int NTHREADS>
__device__ __forceinline__ void norm_after_tail(const NormAfter& norm, const void* out, int tokens, int features, int ldc) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int THREADS = NTHREADS;
    if (norm.weight != nullptr) {
        __shared__ int is_last;
        if (threadIdx.x == 0) {
            const int total = gridDim.x * gridDim.y * gridDim.z;
            const int ticket = atomicAdd(norm.counter, 1);
            is_last = ticket == total - 1;
            if (is_last) *norm.counter = 0;
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            // one warp per row; a lane takes the float4 chunks lane, lane + 32, ... (features % 128 == 0),
            // eight independent loads at a time
            const float* sums = (const float*)out;
            const int chunks = features >> 7;                            // float4 chunks per lane
            for (int t = warp; t < tokens; t += THREADS / 32) {
                const float4* row = reinterpret_cast<const float4*>(sums + (size_t)t * ldc);
                float ss = 0.f;
                for (int c0 = 0; c0 < chunks; c0 += 8) {
                    float4 v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        v[u] = c0 + u < chunks ? __ldcg(row + (c0 + u) * 32 + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < 8; ++u) ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
                }
                ss = lp_warp_sum(ss);
                const float scale = 1.0f / sqrtf(ss / (float)features + norm.eps);
                const float4* gain = reinterpret_cast<const float4*>(norm.weight);
                uint2* dst = reinterpret_cast<uint2*>(norm.out_norm + (size_t)t * features);
                for (int c0 = 0; c0 < chunks; c0 += 8) {
                    float4 v[8], g[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (c0 + u < chunks) { v[u] = __ldcg(row + (c0 + u) * 32 + lane); g[u] = gain[(c0 + u) * 32 + lane]; }
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (c0 + u < chunks) {
                            __nv_bfloat162 lo = __floats2bfloat162_rn(v[u].x * scale * g[u].x, v[u].y * scale * g[u].y);
                            __nv_bfloat162 hi = __floats2bfloat162_rn(v[u].z * scale * g[u].z, v[u].w * scale * g[u].w);
                            uint2 packed;
                            packed.x = *reinterpret_cast<uint32_t*>(&lo);
                            packed.y = *reinterpret_cast<uint32_t*>(&hi);
                            dst[(c0 + u) * 32 + lane] = packed;
                        }
                }
            }
            for (long long i = threadIdx.x; i < norm.clear_count; i += THREADS) norm.clear[i] = 0.f;
        }
    }
}

template <int BLOCK_TOK, int MODE>
struct Tile {
    static constexpr int W_TILES = MODE == LP_GEMM_SWIGLU_WIDE ? 2 : 1;
    static constexpr int W_BYTES = BLOCK_FEAT * BLOCK_K * 2;
    static constexpr int X_BYTES = BLOCK_TOK * BLOCK_K * 2;
    static constexpr int STAGE_BYTES = W_TILES * W_BYTES + X_BYTES;
    // token tiles up to 64 stream weights for a few sequences: two such CTAs fit an SM, so the next
    // product's CTAs can set up and prefetch weights while the current one drains; larger tiles
    // (prompts) take the whole shared memory for a deeper ring
    static constexpr int BUDGET = BLOCK_TOK <= 128 ? 110 * 1024 : 196 * 1024;
    static constexpr int STAGES = (BUDGET / STAGE_BYTES) > 8 ? 8 : (BUDGET / STAGE_BYTES);
    // a CTA that has an SM to itself (a grid of no more CTAs than SMs) may take a deeper ring: streaming weights
    // for a few dozen tokens is bound by how many bytes an SM has in flight
    static constexpr int STAGES_ALONE = ((196 * 1024) / STAGE_BYTES) > 8 ? 8 : ((196 * 1024) / STAGE_BYTES);
    static constexpr int TAIL_BYTES = 1024 /* alignment slack */ + 256 /* barriers */;
    static constexpr int ACC_COLS = BLOCK_TOK * W_TILES;
    static constexpr int TMEM_COLS = ACC_COLS < 32 ? 32 : ACC_COLS;       // power of two by construction
    // Token tiles of 32 and 64 belong to decode steps, where the epilogue is not hidden under another tile's main
    // loop: two warps per quarter of the tensor memory's lanes share its columns (measured at 64 tokens: the
    // epilogue of four warps took 5 of the gated product's 21 us, 2 of the output projection's 6).
    static constexpr int EPI_WARPS = (BLOCK_TOK == 32 || BLOCK_TOK == 64) ? 8 : 4;
    static constexpr int NTHREADS = 64 + 32 * EPI_WARPS;
};

// out: [tokens, ldc]; OUT_BF16 selects the element type of a STORE / SWIGLU output.
// TAIL: the product is followed by a norm that its last CTA writes (NormAfter); a kernel of its own, since the
// tail's registers (116 against 48) would otherwise keep the next kernel's CTAs from starting beside this one.
template <int BLOCK_TOK, int MODE, bool OUT_BF16, bool ATOMIC, bool TAIL = false>
__global__ void __launch_bounds__(Tile<BLOCK_TOK, MODE>::NTHREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    void* __restrict__ out, int tokens, int features, int ldc, int k_blocks, int k_blocks_per_split,
                    int withheld_kblock, int num_stages, int* __restrict__ status, NormAfter norm) {
    // withheld_kblock >= 0 (tests of the bounded waits only, see lp_gemm_withhold_next): the loader never brings
    // that k-block, so the waits for it run out, the roles report through *status and the CTA winds down.
    using T = Tile<BLOCK_TOK, MODE>;
    const uint32_t wait_limit = withheld_kblock >= 0 ? (1u << 14) : SPIN_LIMIT;     // a test need not wait long
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + num_stages * T::STAGE_BYTES);
    uint64_t* empty = full + num_stages;
    uint64_t* acc_ready = empty + num_stages;
    uint32_t* tmem_slot = (uint32_t*)(acc_ready + 1);
    volatile uint32_t* failed = tmem_slot + 1;     // set by a role whose wait ran out; read by the epilogue

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int feat0 = blockIdx.x * BLOCK_FEAT;          // first weight row of this CTA
    const int tok0 = blockIdx.y * BLOCK_TOK;
    const int kb_begin = blockIdx.z * k_blocks_per_split;
    const int kb_end = min(k_blocks, kb_begin + k_blocks_per_split);
    const int nkb = kb_end - kb_begin;            // > 0 by the launcher's choice of grid.z

    lp_grid_release();          // the next kernel on the stream may set itself up behind this one

    if (threadIdx.x == 0) {
        *failed = 0;
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        for (int s = 0; s < num_stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)T::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            // with one token tile each weight is read once: its lines need not stay in L2
            const uint64_t read_once = gridDim.y == 1 ? l2_policy_evict_first() : 0;
            // Weights are written by no kernel of a step: the first ring of weight tiles is requested
            // before waiting for the previous kernel, the activation tiles only after it.
            const int early = min(nkb, num_stages);
            for (int i = 0; i < early; ++i) {
                if (kb_begin + i == withheld_kblock) continue;
                uint8_t* stage = smem + i * T::STAGE_BYTES;
                mbar_expect_tx(&full[i], T::STAGE_BYTES);
                const int k = (kb_begin + i) * BLOCK_K;
                load_weights<MODE>(stage, &map_w, k, blockIdx.x, &full[i], read_once);
            }
            lp_grid_wait();
            for (int i = 0; i < early; ++i) {
                if (kb_begin + i == withheld_kblock) continue;
                tma_load_2d(smem + i * T::STAGE_BYTES + T::W_TILES * T::W_BYTES, &map_x, (kb_begin + i) * BLOCK_K, tok0,
                            &full[i]);
            }
            issued = early;
            int s = early == num_stages ? 0 : early;          // stage and phase of k-block i, kept by counting (a
            uint32_t phase = early == num_stages ? 1 : 0;     // division per k-block is felt in a one-thread loop)
            for (int i = early; i < nkb && ok; ++i) {
                if (!mbar_wait(&empty[s], phase ^ 1, wait_limit)) { atomicExch(status, 1); *failed = 1; ok = false; break; }
                issued = i + 1;
                if (kb_begin + i != withheld_kblock) {
                    uint8_t* stage = smem + s * T::STAGE_BYTES;
                    mbar_expect_tx(&full[s], T::STAGE_BYTES);
                    const int k = (kb_begin + i) * BLOCK_K;
                    load_weights<MODE>(stage, &map_w, k, blockIdx.x, &full[s], read_once);
                    tma_load_2d(stage + T::W_TILES * T::W_BYTES, &map_x, k, tok0, &full[s]);
                }
                if (++s == num_stages) { s = 0; phase ^= 1; }
            }
            if (!ok || *failed) {
                // consumers may be gone: await the copies still in flight before the CTA's memory is released
                // (a withheld k-block has no copy in flight and is not waited for)
                for (int i = max(0, issued - num_stages); i < issued; ++i)
                    if (kb_begin + i != withheld_kblock) mbar_wait(&full[i % num_stages], (i / num_stages) & 1, wait_limit);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BLOCK_TOK >> 3) << 17) |
                                       ((uint32_t)(BLOCK_FEAT >> 4) << 24);
            bool ok = true;
            int s = 0;
            uint32_t phase = 0;
            for (int i = 0; i < nkb; ++i) {
                if (!mbar_wait(&full[s], phase, wait_limit)) { atomicExch(status, 2); *failed = 1; ok = false; break; }
                tcgen05_fence_after();
                const uint32_t w_addr = smem_u32(smem + s * T::STAGE_BYTES);
                const uint32_t x_addr = w_addr + T::W_TILES * T::W_BYTES;
                const uint64_t dw = smem_desc(w_addr), dx = smem_desc(x_addr);
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    const uint64_t step = (uint64_t)((k * UMMA_K * 2) >> 4);
                    tcgen05_mma(tmem_base, dw + step, dx + step, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    if (MODE == LP_GEMM_SWIGLU_WIDE) {
                        const uint64_t du = smem_desc(w_addr + T::W_BYTES);
                        tcgen05_mma(tmem_base + BLOCK_TOK, du + step, dx + step, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    }
                }
                tcgen05_commit(&empty[s]);        // the stage is free once these MMAs have read it
                if (++s == num_stages) { s = 0; phase ^= 1; }
            }
            (void)ok;
            tcgen05_commit(acc_ready);            // arrives when every MMA issued so far is complete
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2 ..)
        const int quarter = warp & 3;             // TMEM lanes 32*quarter .. +31 belong to this warp
        // with eight epilogue warps, warps 2-5 take the lower half of the columns (tokens) and warps 6-9 the upper
        constexpr int EPI = T::EPI_WARPS, COLS = BLOCK_TOK / (EPI / 4);
        const int col_lo = ((warp - 2) >> 2) * COLS;
        const bool ready = mbar_wait(acc_ready, 0, wait_limit);
        if (!ready && lane == 0) atomicExch(status, 3);
        tcgen05_fence_after();
        const bool go = __all_sync(0xffffffffu, ready && *failed == 0);
        if (norm.weight == nullptr && norm.clear != nullptr && ready) {
            // no norm to follow, only a buffer to clear on the side: all CTAs share it (the x tiles have arrived,
            // so the kernel before this one, the buffer's last reader, has ended)
            const long long cta = ((long long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
            const long long ctas = (long long)gridDim.x * gridDim.y * gridDim.z;
            for (long long i = cta * (32 * EPI) + threadIdx.x - 64; i < norm.clear_count; i += ctas * (32 * EPI)) norm.clear[i] = 0.f;
        }
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        constexpr int CHUNK = COLS >= 32 ? 32 : 16;
        if constexpr (MODE != LP_GEMM_SWIGLU) {
            if (go) {
                const int f = feat0 + quarter * 32 + lane;
#pragma unroll 1
                for (int c0 = col_lo; c0 < col_lo + COLS; c0 += CHUNK) {
                    uint32_t g[CHUNK], u[MODE == LP_GEMM_SWIGLU_WIDE ? CHUNK : 1];
                    if (CHUNK == 32) tmem_ld32(lane_addr + c0, g); else tmem_ld16(lane_addr + c0, g);
                    if (MODE == LP_GEMM_SWIGLU_WIDE) {
                        if (CHUNK == 32) tmem_ld32(lane_addr + BLOCK_TOK + c0, u);
                        else tmem_ld16(lane_addr + BLOCK_TOK + c0, u);
                    }
                    tmem_ld_wait();
                    if (f < features) {
#pragma unroll
                        for (int j = 0; j < CHUNK; ++j) {
                            const int t = tok0 + c0 + j;
                            if (t >= tokens) break;
                            float v = __uint_as_float(g[j]);
                            if (MODE == LP_GEMM_SWIGLU_WIDE) v = __fdividef(v, 1.0f + __expf(-v)) * __uint_as_float(u[j]);
                            const size_t at = (size_t)t * ldc + f;
                            if (ATOMIC) atomicAdd((float*)out + at, v);
                            else if (OUT_BF16) ((__nv_bfloat16*)out)[at] = __float2bfloat16_rn(v);
                            else ((float*)out)[at] = v;
                        }
                    }
                }
            }
        } else {
            // Rows 0..63 of the tile are gate, rows 64..127 up, of the same 64 output features, and a warp reaches
            // only its own quarter of the lanes: of its columns, a gate warp hands the upper half of its gates
            // to the up warp of the same feature and takes that warp's lower half of the ups, so that all warps
            // share the activation and the stores. Every load has been consumed by now: the ring's memory carries
            // the halves across.
            float* cross = reinterpret_cast<float*>(smem);            // [EPI / 4][2][64][COLS / 2 + 1]
            constexpr int HALF = COLS / 2, LD = HALF + 1;
            const int local = (quarter & 1) * 32 + lane;              // feature within the 64
            const bool is_gate = quarter < 2;
            float* mine = cross + (((warp - 2) >> 2) * 2 + (is_gate ? 0 : 1)) * 64 * LD + local * LD;     // what this warp hands over
            float* theirs = cross + (((warp - 2) >> 2) * 2 + (is_gate ? 1 : 0)) * 64 * LD + local * LD;
            // the half this warp keeps: gate warps the lower half of their columns, up warps the upper
            const int keep_lo = col_lo + (is_gate ? 0 : HALF), give_lo = col_lo + (is_gate ? HALF : 0);
            uint32_t kept[HALF];
            if (go) {
                uint32_t given[HALF];
                static_assert(HALF == 8 || HALF == 16, "the gated epilogue serves token tiles of 16, 32 and 64");
                if constexpr (HALF == 16) { tmem_ld16(lane_addr + give_lo, given); tmem_ld16(lane_addr + keep_lo, kept); }
                else { tmem_ld8(lane_addr + give_lo, given); tmem_ld8(lane_addr + keep_lo, kept); }
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < HALF; ++j) mine[j] = __uint_as_float(given[j]);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI) : "memory");            // the epilogue warps
            if (go) {
                const int f = blockIdx.x * (BLOCK_FEAT / 2) + local;
                if (f < features) {
#pragma unroll
                    for (int j = 0; j < HALF; ++j) {
                        const int t = tok0 + keep_lo + j;
                        if (t >= tokens) break;
                        const float gate = is_gate ? __uint_as_float(kept[j]) : theirs[j];
                        const float up = is_gate ? theirs[j] : __uint_as_float(kept[j]);
                        const float v = __fdividef(gate, 1.0f + __expf(-gate)) * up;
                        const size_t at = (size_t)t * ldc + f;
                        if (OUT_BF16) ((__nv_bfloat16*)out)[at] = __float2bfloat16_rn(v);
                        else ((float*)out)[at] = v;
                    }
                }
            }
        }
        tcgen05_fence_before();
        if (ATOMIC) __threadfence();          // this thread's additions are out before the CTA is counted below
    }
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)T::TMEM_COLS));
    }
    if constexpr (ATOMIC && TAIL) norm_after_tail<T::NTHREADS>(norm, out, tokens, features, ldc);
}

// ------------------------------------------------------------------ a handful of tokens: mma.sync consumers
// For up to 16 tokens the one-tile tcgen05 kernel measured slower (8 tokens: 0.80 against 0.69 ms per step at
// the 1B shape): what it does after its last MMA (accumulator ready, tensor memory to registers, the exchange of
// the gated halves, stores) is not hidden by anything, and the main loop gains nothing from the tensor memory at
// these sizes. (A tcgen05.mma of 128 x N x 16 issues every 55 cycles for N <= 64; an earlier figure of 142
// cycles for any shape came from a probe whose loop divided by a run-time number in the issuing thread.)
// Here the same ring of TMA stages feeds four warps that read the swizzled tiles with ldmatrix and
// multiply with mma.sync m16n8k16: the 8 tokens of an n-tile are exactly the instruction's N, nothing
// is issued by a single thread, and the sums stay in registers (no tensor memory, no accumulator
// hand-over). Warp w owns weight rows 16 w .. 16 w + 15 and 64 + 16 w .. 64 + 16 w + 15 of the
// 128-row tile: in the interleaved gate/up layout those are the gate and the up rows of the same 16
// features, so the gated activation needs no exchange.
//
// XNORM: the activations are the float32 residual stream and the product applies an RMS norm on the way in.
// The tile of x comes as float32 (two boxes of rows x 32 values per k-block) with the gain's 64 values, and every
// consumer warp forms its own column operand bfloat16(x * gain) from it in registers (a pair of float2 and a pair
// of gains per k-step and token tile; the first warp also sums x^2). A fifth warp that made one bfloat16 tile
// for all four was measured first: at 8 tokens the gated product took 15.6 us with it against 12.2 without the
// norm, at 16 tokens 20.3 against 12.5 (one warp's conversions and the hand-over were in the way). The row's factor
// 1 / sqrt(mean x^2 + eps) is a scalar per token, so it is applied to the sums at the end: by this kernel when
// a CTA sees the whole K range, else (K shared out over CTAs, partial sums meeting in atomics) the CTAs
// with blockIdx.x == 0 add their share of the sum of squares to `sumsq_out` and the reader of the output
// applies the factor. `zero` (optional) is cleared on the side, a slice by every CTA.
constexpr int FEW_THREADS = 160;          // warp 0: TMA; warps 1-4: consumers
constexpr int FEW_W_BYTES = BLOCK_FEAT * BLOCK_K * 2;
// The ring has as many stages as the launch gives it (`stages`): what lets two CTAs share an SM (up to six,
// LLMPLAYER_B200_RING_SHARED), or, for a grid of no more than one CTA per SM whose K range is longer than that,
// up to ten (LLMPLAYER_B200_RING_ALONE): such a CTA requests that much more of its weights before it waits
// for the previous kernel. The shared size also leaves room for the next kernel's CTAs to start beside it.
template <bool XNORM, int NT> struct FewTile {
    static constexpr int X_ROWS = NT <= 2 ? 16 : 8 * NT;          // rows of the activation tile (tokens, padded)
    static constexpr int X_BOX_BYTES = X_ROWS * 128;              // one box: X_ROWS x 128 bytes
    static constexpr int X_BYTES = XNORM ? 2 * X_BOX_BYTES : X_BOX_BYTES;
    static constexpr int GAIN_BYTES = XNORM ? 1024 : 0;           // 64 floats of gain per k-block, padded to the tiles' alignment
    static constexpr int STAGE_BYTES = FEW_W_BYTES + X_BYTES + GAIN_BYTES;
    static constexpr int TAIL_BYTES = 1024 + 512;                 // alignment slack, barriers, row factors
    static constexpr int MAX_SHARED = (110 * 1024 - TAIL_BYTES) / STAGE_BYTES;      // two CTAs per SM
    static constexpr int MAX_ALONE = (224 * 1024 - TAIL_BYTES) / STAGE_BYTES;
};

struct NormBefore {
    const float* gain;        // [K]
    float eps;
    int K;
    float* sumsq_out;         // [tokens]: used when K is shared out over CTAs
    float* zero;              // optional buffer cleared on the side
    int zero_count;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_m16n8k16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// NT: n-tiles of 8 tokens (1, 2, 4 or 8). MODE: STORE or SWIGLU (interleaved rows). out as in the tcgen05 kernel.
template <int NT, int MODE, bool OUT_BF16, bool ATOMIC, bool XNORM, bool TAIL = false>
__global__ void __launch_bounds__(FEW_THREADS, 2)
gemm_fewtok_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   void* __restrict__ out, int tokens, int features, int ldc, int k_blocks, int k_blocks_per_split,
                   int FEW_STAGES, int* __restrict__ status, NormAfter norm, NormBefore before) {
    using FT = FewTile<XNORM, NT>;
    constexpr int FEW_STAGE_BYTES = FT::STAGE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + FEW_STAGES * FEW_STAGE_BYTES);
    uint64_t* empty = full + FEW_STAGES;
    volatile uint32_t* failed = (volatile uint32_t*)(empty + FEW_STAGES);
    float* row_scale = (float*)(failed + 1);          // [8 NT], XNORM
    constexpr int NTHREADS = FEW_THREADS;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kb_begin = blockIdx.z * k_blocks_per_split;
    const int kb_end = min(k_blocks, kb_begin + k_blocks_per_split);
    const int nkb = kb_end - kb_begin;

    lp_grid_release();
    if (threadIdx.x == 0) {
        *failed = 0;
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        for (int s = 0; s < FEW_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == 0) {
        if (lane == 0) {
            // weights are written by no kernel of a step: the first ring is requested before waiting for
            // the previous kernel, the activation tiles only after it
            constexpr int TILE_BYTES = FEW_W_BYTES + FT::X_BYTES;
            const uint64_t read_once = l2_policy_evict_first();      // a decode step reads each weight once
            // what nothing in the step writes (weights, the norm's gain) ...
            auto load_constants = [&](int i, int s) {
                uint8_t* stage = smem + s * FEW_STAGE_BYTES;
                const int k = (kb_begin + i) * BLOCK_K;
                uint32_t gain_bytes = 0;
                if (XNORM) gain_bytes = (uint32_t)min(BLOCK_K, before.K - k) * 4u;
                mbar_expect_tx(&full[s], TILE_BYTES + gain_bytes);
                tma_load_2d_hint(stage, &map_w, k, blockIdx.x * BLOCK_FEAT, &full[s], read_once);
                if (XNORM) bulk_load(stage + TILE_BYTES, before.gain + k, gain_bytes, &full[s]);
            };
            // ... and the activations, which the previous kernel produced
            auto load_activations = [&](int i, int s) {
                uint8_t* xs = smem + s * FEW_STAGE_BYTES + FEW_W_BYTES;
                const int k = (kb_begin + i) * BLOCK_K;
                tma_load_2d(xs, &map_x, k, 0, &full[s]);
                if (XNORM) tma_load_2d(xs + FT::X_BOX_BYTES, &map_x, k + 32, 0, &full[s]);
            };
            const int early = min(nkb, FEW_STAGES);
            for (int i = 0; i < early; ++i) load_constants(i, i);
            lp_grid_wait();
            for (int i = 0; i < early; ++i) load_activations(i, i);
            int issued = early;
            bool ok = true;
            // stage and phase of k-block i: i mod stages, (i / stages) & 1, kept by counting
            int s = early == FEW_STAGES ? 0 : early;
            uint32_t phase = early == FEW_STAGES ? 1 : 0;
            for (int i = early; i < nkb; ++i, s = (s + 1 == FEW_STAGES ? 0 : s + 1), phase ^= (s == 0)) {
                if (!mbar_wait(&empty[s], phase ^ 1)) { atomicExch(status, 1); *failed = 1; ok = false; break; }
                load_constants(i, s);
                load_activations(i, s);
                issued = i + 1;
            }
            if (!ok) {
                for (int i = max(0, issued - FEW_STAGES); i < issued; ++i)
                    mbar_wait(&full[i % FEW_STAGES], (i / FEW_STAGES) & 1);
            }
        }
        __syncwarp();
    } else {
        lp_grid_wait();                        // the epilogue adds into / overwrites what earlier kernels use
        const int w = warp - 1;
        const int g = lane >> 2, t = lane & 3;
        if (before.zero != nullptr) {          // all CTAs share the clearing
            const int cta = blockIdx.z * gridDim.x + blockIdx.x, ctas = gridDim.x * gridDim.z;
            for (int i = cta * 128 + threadIdx.x - 32; i < before.zero_count; i += ctas * 128) before.zero[i] = 0.f;
        }
        float acc[2][NT][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;
        // ldmatrix.x4: lane l gives the address of row (l & 7) + 8 * ((l >> 3) & 1), 16-byte chunk (l >> 4) of the 16 x 16 tile
        const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8;
        const int a_chunk = lane >> 4;
        bool ok = true;
        int s = 0;
        uint32_t phase = 0;
        float ss[NT];                                  // XNORM, first consumer warp: sum x^2 of tokens g + 8 nt over this lane's k
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) ss[nt] = 0.f;
        for (int i = 0; i < nkb; ++i, s = (s + 1 == FEW_STAGES ? 0 : s + 1), phase ^= (s == 0)) {
            if (!mbar_wait(&full[s], phase)) { if (lane == 0) atomicExch(status, 2); *failed = 1; ok = false; }
            const uint32_t w_tile = smem_u32(smem + s * FEW_STAGE_BYTES);
            const uint8_t* x_tile = smem + s * FEW_STAGE_BYTES + FEW_W_BYTES;
            if (!ok) break;
            const float* gain_tile = reinterpret_cast<const float*>(x_tile + FT::X_BYTES);
            const int k_abs = (kb_begin + i) * BLOCK_K;
#pragma unroll
            for (int ks = 0; ks < BLOCK_K / 16; ++ks) {
                uint32_t b[NT][2];
                if (XNORM) {
                    // float32 tile: value k of the k-block lies in box k / 32, 16-byte chunk (k % 32) / 4 of its row
                    // (swizzled with the row). This lane's k: 16 ks + 2 t, + 1 and the same + 8. The gain beyond K
                    // is unset (and x is zero there).
                    const int k0 = ks * 16 + 2 * t;
                    float2 g0 = make_float2(0.f, 0.f), g1 = g0;
                    if (k_abs + k0 < before.K) g0 = *reinterpret_cast<const float2*>(gain_tile + k0);
                    if (k_abs + k0 + 8 < before.K) g1 = *reinterpret_cast<const float2*>(gain_tile + k0 + 8);
                    const int c0 = 4 * (ks & 1) + (t >> 1);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const int row = g + 8 * nt;                // token; row & 7 == g
                        const uint8_t* xr = x_tile + (ks >> 1) * FT::X_BOX_BYTES + row * 128 + (t & 1) * 8;
                        const float2 v0 = *reinterpret_cast<const float2*>(xr + ((c0 ^ g) << 4));
                        const float2 v1 = *reinterpret_cast<const float2*>(xr + (((c0 + 2) ^ g) << 4));
                        if (w == 0) ss[nt] += v0.x * v0.x + v0.y * v0.y + v1.x * v1.x + v1.y * v1.y;
                        __nv_bfloat162 lo = __floats2bfloat162_rn(v0.x * g0.x, v0.y * g0.y);
                        __nv_bfloat162 hi = __floats2bfloat162_rn(v1.x * g1.x, v1.y * g1.y);
                        b[nt][0] = *reinterpret_cast<uint32_t*>(&lo);
                        b[nt][1] = *reinterpret_cast<uint32_t*>(&hi);
                    }
                } else {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const int row = g + 8 * nt;                    // token; row & 7 == g
                        const uint8_t* xr = x_tile + row * 128 + t * 4;
                        b[nt][0] = *reinterpret_cast<const uint32_t*>(xr + (((2 * ks) ^ g) << 4));
                        b[nt][1] = *reinterpret_cast<const uint32_t*>(xr + (((2 * ks + 1) ^ g) << 4));
                    }
                }
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    const int row = (w + 4 * mt) * 16 + a_row;
                    uint32_t a[4];
                    ldmatrix_x4(w_tile + row * 128 + (((2 * ks + a_chunk) ^ (row & 7)) << 4), a[0], a[1], a[2], a[3]);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) mma_m16n8k16(acc[mt][nt], a, b[nt][0], b[nt][1]);
                }
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&empty[s])) : "memory");
        }
        ok = ok && *failed == 0;
        if (XNORM && w == 0) {
            // a token's sum of x^2: over the four lanes that shared its row
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                ss[nt] += __shfl_xor_sync(0xffffffffu, ss[nt], 1);
                ss[nt] += __shfl_xor_sync(0xffffffffu, ss[nt], 2);
                const int row = g + 8 * nt;
                if (t == 0) {
                    if (gridDim.z == 1) row_scale[row] = 1.0f / sqrtf(ss[nt] / (float)before.K + before.eps);
                    else if (blockIdx.x == 0 && ok && row < tokens) atomicAdd(before.sumsq_out + row, ss[nt]);
                }
            }
        }
        if (XNORM && gridDim.z == 1) {
            asm volatile("bar.sync 1, 128;" ::: "memory");             // the first consumer warp has written the rows' factors
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[mt][nt][e] *= row_scale[nt * 8 + 2 * t + (e & 1)];
        }
        // c fragment: c0, c1 = (row g, tokens 2t, 2t + 1); c2, c3 = (row g + 8, same tokens)
        if (ok) {
            if (MODE == LP_GEMM_SWIGLU) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int f = blockIdx.x * (BLOCK_FEAT / 2) + w * 16 + g + (e >> 1) * 8;
                        const int tok = nt * 8 + 2 * t + (e & 1);
                        if (f < features && tok < tokens) {
                            const float gate = acc[0][nt][e], up = acc[1][nt][e];
                            const float v = __fdividef(gate, 1.0f + __expf(-gate)) * up;
                            const size_t at = (size_t)tok * ldc + f;
                            if (OUT_BF16) ((__nv_bfloat16*)out)[at] = __float2bfloat16_rn(v);
                            else ((float*)out)[at] = v;
                        }
                    }
            } else {
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int f = blockIdx.x * BLOCK_FEAT + (w + 4 * mt) * 16 + g + (e >> 1) * 8;
                            const int tok = nt * 8 + 2 * t + (e & 1);
                            if (f < features && tok < tokens) {
                                const float v = acc[mt][nt][e];
                                const size_t at = (size_t)tok * ldc + f;
                                if (ATOMIC) atomicAdd((float*)out + at, v);
                                else if (OUT_BF16) ((__nv_bfloat16*)out)[at] = __float2bfloat16_rn(v);
                                else ((float*)out)[at] = v;
                            }
                        }
            }
        }
        if (ATOMIC) __threadfence();
    }
    __syncthreads();
    if constexpr (ATOMIC && TAIL) norm_after_tail<NTHREADS>(norm, out, tokens, features, ldc);
}

// Settings of the few-token product (lp_gemm_configure; until that is called, the environment's
// LLMPLAYER_B200_FEWTOK / _RING_SHARED / _RING_ALONE or the defaults 1 / 6 / 10).
struct FewSettings { int enabled, ring_shared, ring_alone, ring_alone_tile, ring_normed; bool decided; };
static FewSettings& few_settings() {
    static FewSettings st = {1, 6, 10, 0, 6, false};
    if (!st.decided) {
        const char* v = getenv("LLMPLAYER_B200_FEWTOK");
        st.enabled = (v && v[0] == '0') ? 0 : 1;
        v = getenv("LLMPLAYER_B200_RING_ALONE");
        st.ring_alone = v ? atoi(v) : 10;
        v = getenv("LLMPLAYER_B200_RING_SHARED");
        st.ring_shared = v ? atoi(v) : 6;
        if (st.ring_alone < 2) st.ring_alone = 2;
        if (st.ring_shared < 2) st.ring_shared = 2;
        v = getenv("LLMPLAYER_B200_RING_ALONE_TILE");
        st.ring_alone_tile = v ? atoi(v) : 0;
        v = getenv("LLMPLAYER_B200_RING_NORMED");
        st.ring_normed = v ? atoi(v) : 6;
        st.decided = true;
    }
    return st;
}

template <int NT, int MODE, bool OUT_BF16, bool ATOMIC, bool XNORM, bool TAIL = false>
int launch_fewtok(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int tokens, int features, int ldc, int k_blocks,
                  int splits, int* status, const NormAfter& norm, const NormBefore& before, cudaStream_t stream) {
    using FT = FewTile<XNORM, NT>;
    auto kernel = gemm_fewtok_kernel<NT, MODE, OUT_BF16, ATOMIC, XNORM, TAIL>;
    static bool configured = false;
    if (!configured) {
        const int most = FT::MAX_ALONE * FT::STAGE_BYTES + FT::TAIL_BYTES;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e != cudaSuccess) LP_REFUSE("gemm: cannot reserve %d bytes of shared memory: %s", most, cudaGetErrorString(e));
        configured = true;
    }
    const int per_split = (k_blocks + splits - 1) / splits;
    const int grid_z = (k_blocks + per_split - 1) / per_split;
    const int per_cta = MODE == LP_GEMM_SWIGLU ? BLOCK_FEAT / 2 : BLOCK_FEAT;
    dim3 grid((features + per_cta - 1) / per_cta, 1, grid_z);
    const int ring_alone = few_settings().ring_alone, ring_shared = few_settings().ring_shared;
    const int shared_stages = ring_shared < FT::MAX_SHARED ? ring_shared : FT::MAX_SHARED;
    const bool alone = (long long)grid.x * grid.z <= lp_sm_count() && per_split > shared_stages + 2;
    int stages = alone ? (ring_alone < FT::MAX_ALONE ? ring_alone : FT::MAX_ALONE) : shared_stages;
    // (measured at the 1B shape, 8 tokens: 0.73 ms per step with 7 to 10 stages for the two long products, 0.80 ms
    // with 6; giving the short products no more stages than they have k-blocks changed nothing; a q|k|v product
    // with more than the shared ring keeps the attention kernel's CTAs from starting beside it: 0.81 ms)
    const int smem = stages * FT::STAGE_BYTES + FT::TAIL_BYTES;
    cudaError_t err = lp_launch(kernel, grid, FEW_THREADS, smem, stream, mw, mx, out, tokens, features,
                                ldc, k_blocks, per_split, stages, status, norm, before);
    if (err != cudaSuccess) {
        snprintf(lp_error_text, sizeof(lp_error_text), "gemm_fewtok: %s", cudaGetErrorString(err));
        return (int)err;
    }
    return lp_check_launch("gemm_fewtok");
}

template <int NT, bool XNORM>
int dispatch_fewtok(int mode, bool out_bf16, bool atomic, const CUtensorMap& mw, const CUtensorMap& mx, void* out,
                    int tokens, int features, int ldc, int k_blocks, int splits, int* status, const NormAfter& norm,
                    const NormBefore& before, cudaStream_t stream) {
#define LP_GO(MODE, BF, AT) \
    return launch_fewtok<NT, MODE, BF, AT, XNORM>(mw, mx, out, tokens, features, ldc, k_blocks, splits, status, norm, before, stream)
    if (mode == LP_GEMM_SWIGLU) {
        if (out_bf16) LP_GO(LP_GEMM_SWIGLU, true, false);
        LP_GO(LP_GEMM_SWIGLU, false, false);
    }
    if (atomic && norm.weight != nullptr)
        return launch_fewtok<NT, LP_GEMM_STORE, false, true, XNORM, true>(mw, mx, out, tokens, features, ldc, k_blocks, splits,
                                                                       status, norm, before, stream);
    if (atomic) LP_GO(LP_GEMM_STORE, false, true);
    if (out_bf16) LP_GO(LP_GEMM_STORE, true, false);
    LP_GO(LP_GEMM_STORE, false, false);
#undef LP_GO
}

static bool fewtok_enabled() { return few_settings().enabled != 0; }

// ------------------------------------------------------------------ 9 to 64 tokens with the norm on the way in
// The one-tile tcgen05 product for a decode batch beyond what the mma.sync kernel above serves, taking the
// float32 residual stream and applying an RMS norm on the way in, as that kernel does: the tile of x comes as
// float32 (two boxes of rows x 32 values per k-block) with the gain's 64 values; four "maker" warps turn it into
// the bfloat16 operand bfloat16(x * gain) in place of the first box (every value is read before any is written),
// sum x^2 per row, and hand the stage to the MMA thread through a barrier of their own. The row factor
// 1 / sqrt(mean x^2 + eps) is applied to the sums in the epilogue when the CTA sees the whole K range; else the
// CTAs of the first feature tile add their shares of the sums of squares to `sumsq_out` and the reader of the
// output applies the factor. Saves the norm kernels in front of the q|k|v and the gated products of a layer.
//
// Once the last operand is made, the makers join the epilogue: eight warps share its columns.
//
// Measured at the 1B shape (ms per decode step, this kernel against norm kernels of their own): 20 tokens
// 0.840 / 0.887, 32 tokens 0.858 / 0.939; with the 64-token tile 48 tokens 1.068 / 0.991 and 64 tokens
// 1.138 / 1.059: there the float32 tile makes 80 KB of shared-memory traffic per k-block against 48 KB, and the
// callers keep the norm kernels. A variant whose makers read x from L2 with plain loads, two k-blocks ahead
// (no float32 tile in shared memory), was slower at every size (1.17 ms at 24 tokens): TMA keeps as many
// k-blocks of x in flight as the ring has stages, the makers' registers cannot.
constexpr int NORMED_THREADS = 320;       // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue, warps 6-9: operand makers, then epilogue

template <int BLOCK_TOK> struct NormedTile {
    static constexpr int W_BYTES = BLOCK_FEAT * BLOCK_K * 2;
    static constexpr int X_BOX_BYTES = BLOCK_TOK * 128;            // BLOCK_TOK rows x 32 float32
    static constexpr int X_BYTES = 2 * X_BOX_BYTES;
    static constexpr int GAIN_BYTES = 1024;                        // 64 float32 of gain, padded to the tiles' alignment
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES + GAIN_BYTES;
    static constexpr int TAIL_BYTES = 1024 + 768;                  // alignment slack, barriers, row factors
    static constexpr int MAX_STAGES = 8;
    static constexpr int STAGES_SHARED = (110 * 1024 - TAIL_BYTES) / STAGE_BYTES;          // two CTAs on an SM
    static constexpr int STAGES_ALONE =
        (227 * 1024 - TAIL_BYTES) / STAGE_BYTES < MAX_STAGES ? (227 * 1024 - TAIL_BYTES) / STAGE_BYTES : MAX_STAGES;
    static constexpr int TMEM_COLS = BLOCK_TOK < 32 ? 32 : BLOCK_TOK;
    static_assert(BLOCK_TOK == 32 || BLOCK_TOK == 64, "token tiles of 32 or 64");
    static_assert(STAGES_SHARED >= 2, "at least two stages");
};

// MODE: STORE or SWIGLU (interleaved rows, 64 output features per CTA). tokens <= BLOCK_TOK (one token tile).
template <int BLOCK_TOK, int MODE, bool OUT_BF16, bool ATOMIC>
__global__ void __launch_bounds__(NORMED_THREADS, 1)
gemm_tcgen05_normed_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                           void* __restrict__ out, int tokens, int features, int ldc, int k_blocks,
                           int k_blocks_per_split, int num_stages, int* __restrict__ status, NormBefore before) {
    using T = NormedTile<BLOCK_TOK>;
    constexpr int MAXS = T::MAX_STAGES;
    const int STAGES = num_stages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + STAGES * T::STAGE_BYTES);
    uint64_t* empty = full + MAXS;
    uint64_t* made = empty + MAXS;                 // the bfloat16 operand of the stage is ready
    uint64_t* acc_ready = made + MAXS;
    uint32_t* tmem_slot = (uint32_t*)(acc_ready + 1);
    volatile uint32_t* failed = tmem_slot + 1;
    float* row_scale = (float*)(tmem_slot + 4);    // [BLOCK_TOK]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int feat0 = blockIdx.x * BLOCK_FEAT;
    const int kb_begin = blockIdx.z * k_blocks_per_split;
    const int kb_end = min(k_blocks, kb_begin + k_blocks_per_split);
    const int nkb = kb_end - kb_begin;
    const bool whole_k = gridDim.z == 1;

    lp_grid_release();
    if (threadIdx.x == 0) {
        *failed = 0;
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&made[s], 4); }
        mbar_init(acc_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)T::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            constexpr int TILE_BYTES = T::W_BYTES + T::X_BYTES;
            const uint64_t read_once = l2_policy_evict_first();      // a decode step reads each weight once
            auto load_constants = [&](int i, int s) {            // what nothing in the step writes: weights, gain
                uint8_t* stage = smem + s * T::STAGE_BYTES;
                const int k = (kb_begin + i) * BLOCK_K;
                const uint32_t gain_bytes = (uint32_t)min(BLOCK_K, before.K - k) * 4u;
                mbar_expect_tx(&full[s], TILE_BYTES + gain_bytes);
                tma_load_2d_hint(stage, &map_w, k, blockIdx.x * BLOCK_FEAT, &full[s], read_once);
                bulk_load(stage + TILE_BYTES, before.gain + k, gain_bytes, &full[s]);
            };
            auto load_activations = [&](int i, int s) {          // what the previous kernel produced
                uint8_t* xs = smem + s * T::STAGE_BYTES + T::W_BYTES;
                const int k = (kb_begin + i) * BLOCK_K;
                tma_load_2d(xs, &map_x, k, 0, &full[s]);
                tma_load_2d(xs + T::X_BOX_BYTES, &map_x, k + 32, 0, &full[s]);
            };
            const int early = min(nkb, STAGES);
            for (int i = 0; i < early; ++i) load_constants(i, i);
            lp_grid_wait();
            for (int i = 0; i < early; ++i) load_activations(i, i);
            int issued = early;
            bool ok = true;
            int s = early == STAGES ? 0 : early;              // stage and phase of k-block i, kept by counting
            uint32_t phase = early == STAGES ? 1 : 0;
            for (int i = early; i < nkb; ++i) {
                if (!mbar_wait(&empty[s], phase ^ 1)) { atomicExch(status, 1); *failed = 1; ok = false; break; }
                load_constants(i, s);
                load_activations(i, s);
                issued = i + 1;
                if (++s == STAGES) { s = 0; phase ^= 1; }
            }
            if (!ok) {
                for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(&full[i % STAGES], (i / STAGES) & 1);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BLOCK_TOK >> 3) << 17) |
                                       ((uint32_t)(BLOCK_FEAT >> 4) << 24);
            int s = 0;
            uint32_t phase = 0;
            for (int i = 0; i < nkb; ++i) {
                if (!mbar_wait(&made[s], phase)) { atomicExch(status, 2); *failed = 1; break; }
                tcgen05_fence_after();
                const uint32_t w_addr = smem_u32(smem + s * T::STAGE_BYTES);
                const uint64_t dw = smem_desc(w_addr), dx = smem_desc(w_addr + T::W_BYTES);
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    const uint64_t step = (uint64_t)((k * UMMA_K * 2) >> 4);
                    tcgen05_mma(tmem_base, dw + step, dx + step, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                tcgen05_commit(&empty[s]);
                if (++s == STAGES) { s = 0; phase ^= 1; }
            }
            tcgen05_commit(acc_ready);
        }
        __syncwarp();
    } else {
      if (warp >= 6) {
        // ------------------------------------------------------------ operand makers (128 threads)
        // float4 q of the k-block: row q / 16, values 4 (q % 16) ..; thread c takes q = c, c + 128, ...: a fixed
        // place in the row, rows 8 apart, so sixteen neighbouring threads share a row
        const int c = threadIdx.x - 192;
        constexpr int PASSES = BLOCK_TOK / 8;
        const int kq = c & 15, k = kq * 4;
        float ss[PASSES];
#pragma unroll
        for (int it = 0; it < PASSES; ++it) ss[it] = 0.f;
        bool ok = true;
        int s = 0;
        uint32_t phase = 0;
        for (int i = 0; i < nkb && ok; ++i) {
            if (!mbar_wait(&full[s], phase)) { if (lane == 0) atomicExch(status, 4); *failed = 1; ok = false; }
            uint8_t* x_tile = smem + s * T::STAGE_BYTES + T::W_BYTES;
            const float* gain_tile = reinterpret_cast<const float*>(x_tile + T::X_BYTES);
            const int k_abs = (kb_begin + i) * BLOCK_K;
            float4 gn = make_float4(0.f, 0.f, 0.f, 0.f);           // the gain beyond K is unset (and x is zero there)
            if (ok && k_abs + k < before.K) gn = *reinterpret_cast<const float4*>(gain_tile + k);
            uint2 packed[PASSES];
#pragma unroll
            for (int it = 0; it < PASSES; ++it) {
                const int row = (c >> 4) + it * 8;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (ok) v = *reinterpret_cast<const float4*>(
                    x_tile + (kq >> 3) * T::X_BOX_BYTES + row * 128 + (((kq & 7) ^ (row & 7)) << 4));
                ss[it] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * gn.x, v.y * gn.y);
                __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * gn.z, v.w * gn.w);
                packed[it].x = *reinterpret_cast<uint32_t*>(&lo);
                packed[it].y = *reinterpret_cast<uint32_t*>(&hi);
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");        // every maker has read its share of the float32 tile
#pragma unroll
            for (int it = 0; it < PASSES; ++it) {
                const int row = (c >> 4) + it * 8;
                *reinterpret_cast<uint2*>(x_tile + row * 128 + (((k >> 3) ^ (row & 7)) << 4) + (k & 7) * 2) = packed[it];
            }
            // written through the generic proxy, read by the MMA through the async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&made[s])) : "memory");
            if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        // a row's sum of x^2: over the sixteen threads that shared it
#pragma unroll
        for (int it = 0; it < PASSES; ++it) {
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) ss[it] += __shfl_xor_sync(0xffffffffu, ss[it], o);
        }
        if (kq == 0) {
#pragma unroll
            for (int it = 0; it < PASSES; ++it) {
                const int row = (c >> 4) + it * 8;
                if (whole_k) row_scale[row] = 1.0f / sqrtf(ss[it] / (float)before.K + before.eps);
                else if (blockIdx.x == 0 && ok && row < tokens) atomicAdd(before.sumsq_out + row, ss[it]);
            }
        }
        lp_grid_wait();
      } else {
        lp_grid_wait();
        if (before.zero != nullptr) {              // all CTAs share the clearing
            const int cta = blockIdx.z * gridDim.x + blockIdx.x, ctas = gridDim.x * gridDim.z;
            for (int i = cta * 128 + threadIdx.x - 64; i < before.zero_count; i += ctas * 128) before.zero[i] = 0.f;
        }
      }
        // ------------------------------------------------------------ epilogue (warps 2..9: the makers, their work done,
        // take the upper half of the columns)
        const int quarter = warp & 3;
        constexpr int COLS = BLOCK_TOK / 2, CHUNK = COLS >= 32 ? 32 : 16;
        const int col_lo = ((warp - 2) >> 2) * COLS;
        const bool ready = mbar_wait(acc_ready, 0);
        if (!ready && lane == 0) atomicExch(status, 3);
        tcgen05_fence_after();
        if (whole_k) asm volatile("bar.sync 1, 256;" ::: "memory");     // the makers have written the rows' factors
        const bool go = __all_sync(0xffffffffu, ready && *failed == 0);
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        if constexpr (MODE != LP_GEMM_SWIGLU) {
            if (go) {
                const int f = feat0 + quarter * 32 + lane;
#pragma unroll 1
                for (int c0 = col_lo; c0 < col_lo + COLS; c0 += CHUNK) {
                    uint32_t g[CHUNK];
                    if (CHUNK == 32) tmem_ld32(lane_addr + c0, g); else tmem_ld16(lane_addr + c0, g);
                    tmem_ld_wait();
                    if (f < features) {
#pragma unroll
                        for (int j = 0; j < CHUNK; ++j) {
                            const int t = c0 + j;
                            if (t >= tokens) break;
                            float v = __uint_as_float(g[j]);
                            if (whole_k) v *= row_scale[t];
                            const size_t at = (size_t)t * ldc + f;
                            if (ATOMIC) atomicAdd((float*)out + at, v);
                            else if (OUT_BF16) ((__nv_bfloat16*)out)[at] = __float2bfloat16_rn(v);
                            else ((float*)out)[at] = v;
                        }
                    }
                }
            }
        } else {
            // rows 0..63 of the tile are gate, rows 64..127 up, of the same 64 output features, and a warp reaches
            // only its own quarter of the lanes: of its columns, a gate warp hands the upper half of its gates to the
            // up warp of the same feature and takes that warp's lower half of the ups (as in the kernel above); the
            // ring's memory (every load has been consumed) carries the halves across
            float* cross = reinterpret_cast<float*>(smem);            // [2][2][64][COLS / 2 + 1]
            constexpr int HALF = COLS / 2, LD = HALF + 1;
            static_assert(HALF == 8 || HALF == 16, "token tiles of 32 and 64");
            const int local = (quarter & 1) * 32 + lane;
            const bool is_gate = quarter < 2;
            float* mine = cross + (((warp - 2) >> 2) * 2 + (is_gate ? 0 : 1)) * 64 * LD + local * LD;
            float* theirs = cross + (((warp - 2) >> 2) * 2 + (is_gate ? 1 : 0)) * 64 * LD + local * LD;
            const int keep_lo = col_lo + (is_gate ? 0 : HALF), give_lo = col_lo + (is_gate ? HALF : 0);
            uint32_t kept[HALF];
            if (go) {
                uint32_t given[HALF];
                if constexpr (HALF == 16) { tmem_ld16(lane_addr + give_lo, given); tmem_ld16(lane_addr + keep_lo, kept); }
                else { tmem_ld8(lane_addr + give_lo, given); tmem_ld8(lane_addr + keep_lo, kept); }
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < HALF; ++j) mine[j] = __uint_as_float(given[j]);
            }
            asm volatile("bar.sync 3, 256;" ::: "memory");            // the eight epilogue warps
            if (go) {
                const int f = blockIdx.x * (BLOCK_FEAT / 2) + local;
                if (f < features) {
#pragma unroll
                    for (int j = 0; j < HALF; ++j) {
                        const int t = keep_lo + j;
                        if (t >= tokens) break;
                        const float rs = row_scale[t];                   // the gated product is never split along K
                        const float gate = (is_gate ? __uint_as_float(kept[j]) : theirs[j]) * rs;
                        const float up = (is_gate ? theirs[j] : __uint_as_float(kept[j])) * rs;
                        const float v = __fdividef(gate, 1.0f + __expf(-gate)) * up;
                        const size_t at = (size_t)t * ldc + f;
                        if (OUT_BF16) ((__nv_bfloat16*)out)[at] = __float2bfloat16_rn(v);
                        else ((float*)out)[at] = v;
                    }
                }
            }
        }
        tcgen05_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)T::TMEM_COLS));
    }
}

template <int BLOCK_TOK, int MODE, bool OUT_BF16, bool ATOMIC>
int launch_normed(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int tokens, int features, int ldc, int k_blocks,
                  int splits, int* status, const NormBefore& before, cudaStream_t stream) {
    using T = NormedTile<BLOCK_TOK>;
    auto kernel = gemm_tcgen05_normed_kernel<BLOCK_TOK, MODE, OUT_BF16, ATOMIC>;
    static bool configured = false;
    if (!configured) {
        const int most = T::STAGES_ALONE * T::STAGE_BYTES + T::TAIL_BYTES;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e != cudaSuccess) LP_REFUSE("gemm: cannot reserve %d bytes of shared memory: %s", most, cudaGetErrorString(e));
        configured = true;
    }
    const int per_split = (k_blocks + splits - 1) / splits;
    const int grid_z = (k_blocks + per_split - 1) / per_split;
    const int per_cta = MODE == LP_GEMM_SWIGLU ? BLOCK_FEAT / 2 : BLOCK_FEAT;
    dim3 grid((features + per_cta - 1) / per_cta, 1, grid_z);
    // a float32 tile of x beside each tile of weights shrinks what a ring of a given size keeps in flight: a grid
    // of at most one CTA per SM takes up to lp_gemm_configure's ring_normed stages (0: never more than what lets
    // two CTAs share an SM)
    int stages = T::STAGES_SHARED;
    const int wanted = few_settings().ring_normed;
    if ((long long)grid.x * grid.z <= lp_sm_count() && wanted > stages) stages = wanted < T::STAGES_ALONE ? wanted : T::STAGES_ALONE;
    if (stages > per_split) stages = per_split > T::STAGES_SHARED ? per_split : T::STAGES_SHARED;
    const int smem = stages * T::STAGE_BYTES + T::TAIL_BYTES;
    cudaError_t err = lp_launch(kernel, grid, NORMED_THREADS, smem, stream, mw, mx, out, tokens, features, ldc,
                                k_blocks, per_split, stages, status, before);
    if (err != cudaSuccess) {
        snprintf(lp_error_text, sizeof(lp_error_text), "gemm_tcgen05_normed: %s", cudaGetErrorString(err));
        return (int)err;
    }
    return lp_check_launch("gemm_tcgen05_normed");
}

template <int BLOCK_TOK>
int dispatch_normed(int mode, bool out_bf16, bool atomic, const CUtensorMap& mw, const CUtensorMap& mx, void* out, int tokens,
                    int features, int ldc, int k_blocks, int splits, int* status, const NormBefore& before,
                    cudaStream_t stream) {
#define LP_GO(MODE, BF, AT) \
    return launch_normed<BLOCK_TOK, MODE, BF, AT>(mw, mx, out, tokens, features, ldc, k_blocks, splits, status, before, stream)
    if (mode == LP_GEMM_SWIGLU) {
        if (out_bf16) LP_GO(LP_GEMM_SWIGLU, true, false);
        LP_GO(LP_GEMM_SWIGLU, false, false);
    }
    if (atomic) LP_GO(LP_GEMM_STORE, false, true);
    if (out_bf16) LP_GO(LP_GEMM_STORE, true, false);
    LP_GO(LP_GEMM_STORE, false, false);
#undef LP_GO
}

// ------------------------------------------------------------------ persistent form for prompts
// One CTA per SM walks over output tiles (tile = blockIdx.x, + gridDim.x, ...). Tensor memory holds two
// accumulators: while the epilogue warps read tile i out of one, the MMA thread fills the other with
// tile i + 1, and the loader keeps the ring of stages full across tile boundaries. No split of K, no
// norm fusion: this form serves steps with hundreds of tokens.
// What the epilogue of the fused q|k|v projection needs (LP_GEMM_QKV_TOKM): a token is a row of the accumulator, so
// a thread holds whole heads of its token and a rotation pair never leaves the thread.
struct QkvEpilogue {
    const float2* angles;       // [tokens, half] (cos, sin) of position x frequency; null: no rotation
    int half;                   // rotary width / 2 (the rotary width is the head size, or 0)
    int interleaved;            // pairs (2i, 2i + 1) instead of (i, i + head size / 2)
    const int* positions;       // [tokens]
    const int* seq_ids;         // [tokens]
    const int* page_table;      // [sequences, pt_stride]
    int pt_stride;
    __nv_bfloat16* q_out;       // [tokens, H * hd]
    __nv_bfloat16* pages;       // [num_pages, 2, G, page_size, hd]; null: this layer keeps no keys of its own
    int H, G, hd, page_size;
};

// 16 float32 values of a token -> 16 bfloat16 at dst (16-byte aligned)
__device__ __forceinline__ void store_row16(__nv_bfloat16* dst, const float* v) {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        uint4 packed;
        __nv_bfloat162 t0 = __floats2bfloat162_rn(v[q * 8], v[q * 8 + 1]), t1 = __floats2bfloat162_rn(v[q * 8 + 2], v[q * 8 + 3]);
        __nv_bfloat162 t2 = __floats2bfloat162_rn(v[q * 8 + 4], v[q * 8 + 5]), t3 = __floats2bfloat162_rn(v[q * 8 + 6], v[q * 8 + 7]);
        packed.x = *reinterpret_cast<uint32_t*>(&t0); packed.y = *reinterpret_cast<uint32_t*>(&t1);
        packed.z = *reinterpret_cast<uint32_t*>(&t2); packed.w = *reinterpret_cast<uint32_t*>(&t3);
        reinterpret_cast<uint4*>(dst)[q] = packed;
    }
}

template <int BLOCK_TOK, int MODE>
struct PersistentTile {
    static constexpr bool TOKM = MODE == LP_GEMM_SWIGLU_TOKM || MODE == LP_GEMM_QKV_TOKM;
    static constexpr int FEAT_PER_TILE = MODE == LP_GEMM_QKV_TOKM ? 256 : BLOCK_FEAT;
    static constexpr int W_TILES = MODE == LP_GEMM_SWIGLU_WIDE ? 2 : 1;
    static constexpr int W_BYTES = (TOKM ? 256 : BLOCK_FEAT) * BLOCK_K * 2;
    static constexpr int X_BYTES = BLOCK_TOK * BLOCK_K * 2;
    static constexpr int STAGE_BYTES = W_TILES * W_BYTES + X_BYTES;
    static constexpr int STAGES = (196 * 1024) / STAGE_BYTES;
    static constexpr int ACC_COLS = TOKM ? 256 : BLOCK_TOK * W_TILES;
    static constexpr int TMEM_COLS = 2 * ACC_COLS;                // 512 for all uses below
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
    static_assert(TMEM_COLS == 512 || TMEM_COLS == 256, "two accumulators must fit tensor memory");
    static_assert(!TOKM || BLOCK_TOK == 128, "tokens are the MMA's M");
};

// Eight epilogue warps: two per quarter of the tensor memory's lanes, each with half of the accumulator's columns.
// The products of a prompt with about one tile per CTA (output and down projection: 128 tiles, q|k|v: 192) have
// no next tile under whose MMAs the epilogue could run.
constexpr int PERSIST_THREADS = 64 + 32 * 8;
template <int BLOCK_TOK, int MODE, bool OUT_BF16, bool ATOMIC>
__global__ void __launch_bounds__(PERSIST_THREADS, 1)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                       void* __restrict__ out, int tokens, int features, int ldc, int k_blocks, int feat_tiles,
                       int num_tiles, int group_tok, int* __restrict__ status, QkvEpilogue qkv) {
    using T = PersistentTile<BLOCK_TOK, MODE>;
    // Tiles are numbered in bands of `group_tok` token tiles, token tile first within a band: the CTAs that run
    // at the same time then share a few weight tiles and a few activation tiles, which stay in L2 (feature
    // tile first has every CTA on a weight tile of its own).
    const int tok_tiles = num_tiles / feat_tiles;
    auto tile_at = [&](int tile, int& ft, int& tt) {
        const int per_band = group_tok * feat_tiles;
        const int band = tile / per_band, r = tile - band * per_band;
        const int rows = min(group_tok, tok_tiles - band * group_tok);     // token tiles of this band
        ft = r / rows;
        tt = band * group_tok + (r - ft * rows);
    };
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + T::STAGES * T::STAGE_BYTES);
    uint64_t* empty = full + T::STAGES;
    uint64_t* acc_full = empty + T::STAGES;       // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile uint32_t* failed = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    lp_grid_release();
    if (threadIdx.x == 0) {
        *failed = 0;
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        for (int s = 0; s < T::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int k = 0; k < 2; ++k) { mbar_init(&acc_full[k], 1); mbar_init(&acc_empty[k], 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)T::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ loader: one ring across all tiles
        if (lane == 0) {
            lp_grid_wait();
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int ft, tt;
                tile_at(tile, ft, tt);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % T::STAGES;
                    if (!mbar_wait(&empty[s], ((it / T::STAGES) & 1) ^ 1)) { atomicExch(status, 21); *failed = 1; ok = false; break; }
                    uint8_t* stage = smem + s * T::STAGE_BYTES;
                    mbar_expect_tx(&full[s], T::STAGE_BYTES);
                    load_weights<MODE>(stage, &map_w, kb * BLOCK_K, ft, &full[s]);
                    tma_load_2d(stage + T::W_TILES * T::W_BYTES, &map_x, kb * BLOCK_K, tt * BLOCK_TOK, &full[s]);
                }
            }
            if (!ok) {
                for (int i = max(0, it - T::STAGES); i < it; ++i) mbar_wait(&full[i % T::STAGES], (i / T::STAGES) & 1);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer: alternating accumulators
        if (lane == 0) {
            // TOKM: M = 128 tokens (A = the activation tile), N = 256 weight rows (B = the weight tile)
            constexpr uint32_t idesc = T::TOKM
                ? ((1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24))
                : ((1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BLOCK_TOK >> 3) << 17) |
                   ((uint32_t)(BLOCK_FEAT >> 4) << 24));
            int it = 0, j = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++j) {
                const int ab = j & 1;
                if (!mbar_wait(&acc_empty[ab], ((j >> 1) & 1) ^ 1)) { atomicExch(status, 22); *failed = 1; ok = false; break; }
                tcgen05_fence_after();
                const uint32_t acc = tmem_base + ab * T::ACC_COLS;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % T::STAGES;
                    if (!mbar_wait(&full[s], (it / T::STAGES) & 1)) { atomicExch(status, 23); *failed = 1; ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t w_addr = smem_u32(smem + s * T::STAGE_BYTES);
                    const uint32_t x_addr = w_addr + T::W_TILES * T::W_BYTES;
                    const uint64_t dw = smem_desc(w_addr), dx = smem_desc(x_addr);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t step = (uint64_t)((k * UMMA_K * 2) >> 4);
                        if (T::TOKM) tcgen05_mma(acc, dx + step, dw + step, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        else tcgen05_mma(acc, dw + step, dx + step, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        if (MODE == LP_GEMM_SWIGLU_WIDE) {
                            const uint64_t du = smem_desc(w_addr + T::W_BYTES);
                            tcgen05_mma(acc + BLOCK_TOK, du + step, dx + step, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                    tcgen05_commit(&empty[s]);
                }
                tcgen05_commit(&acc_full[ab]);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue: drains one accumulator at a time
        const int quarter = warp & 3;
        const int ehalf = (warp - 2) >> 2;                 // which half of the columns this warp drains
        constexpr int CHUNK = 32;
        int j = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++j) {
            const int ab = j & 1;
            int ft, tt;
            tile_at(tile, ft, tt);
            if (ok && !mbar_wait(&acc_full[ab], (j >> 1) & 1)) { if (lane == 0) atomicExch(status, 24); *failed = 1; ok = false; }
            tcgen05_fence_after();
            const bool go = __all_sync(0xffffffffu, ok && *failed == 0);
            if (go && MODE == LP_GEMM_QKV_TOKM) {
                // lanes are tokens, columns the tile's 256 features = whole heads. Queries and keys: every pair of
                // a head is rotated by the token's angle (products and sums rounded one by one, as the rotation
                // kernels do); queries go to their buffer, keys and values to the token's place in the cache.
                const uint32_t lane_addr = tmem_base + ab * T::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
                const int t = tt * BLOCK_TOK + quarter * 32 + lane;
                const bool live = t < tokens;
                const int hd = qkv.hd, chunks = hd >> 5;             // 32 columns per chunk
                long long page_base = 0;
                if (live && qkv.pages) {
                    const int pos = qkv.positions[t];
                    const int page = qkv.page_table[(long long)qkv.seq_ids[t] * qkv.pt_stride + pos / qkv.page_size];
                    page_base = (long long)page * 2 * qkv.G * qkv.page_size * hd + (long long)(pos % qkv.page_size) * hd;
                }
                const float2* ang = qkv.angles ? qkv.angles + (size_t)(live ? t : 0) * qkv.half : nullptr;
                const int heads_per_tile = 256 / hd, total_heads = qkv.pages ? qkv.H + 2 * qkv.G : qkv.H;
                auto dest = [&](int head) -> __nv_bfloat16* {
                    if (head < qkv.H) return qkv.q_out + ((size_t)(live ? t : 0) * qkv.H + head) * hd;
                    const bool is_v = head >= qkv.H + qkv.G;
                    return qkv.pages + page_base + (size_t)(is_v ? head - qkv.H : head - qkv.H) * qkv.page_size * hd;
                };
                const int rotated_heads = ang == nullptr ? 0 : (qkv.pages ? qkv.H + qkv.G : qkv.H);     // heads below this index are rotated
                const bool split_half = ang != nullptr && !qkv.interleaved;
                // Of every chunk of 32 columns this warp takes 16 (the two warps of a quarter of the lanes share
                // each head, so that neither fetches the token's angles twice).
                const int sub = ehalf * 16;
                // heads that pass through (values; everything when there is no rotation) and interleaved pairs: chunk by chunk
#pragma unroll 1
                for (int hh = 0; hh < heads_per_tile; ++hh) {
                    const int head = ft * heads_per_tile + hh;
                    if (head >= total_heads) break;
                    const bool rotate = head < rotated_heads;
                    if (rotate && split_half) continue;
                    __nv_bfloat16* dst = dest(head);
                    const uint32_t col0 = lane_addr + hh * hd;
#pragma unroll 1
                    for (int c = 0; c < chunks; ++c) {
                        uint32_t g[16];
                        float v[16];
                        tmem_ld16(col0 + c * 32 + sub, g);
                        tmem_ld_wait();
                        if (rotate) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float2 cs = live ? ang[c * 16 + ehalf * 8 + i] : make_float2(1.f, 0.f);
                                const float xa = __uint_as_float(g[2 * i]), xb = __uint_as_float(g[2 * i + 1]);
                                v[2 * i] = __fsub_rn(__fmul_rn(xa, cs.x), __fmul_rn(xb, cs.y));
                                v[2 * i + 1] = __fadd_rn(__fmul_rn(xa, cs.y), __fmul_rn(xb, cs.x));
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(g[i]);
                        }
                        if (live) store_row16(dst + c * 32 + sub, v);
                    }
                }
                // pairs (i, i + hd / 2): chunk c of a head with its chunk c + half_chunks; the token's angles of a
                // chunk are fetched once and serve every rotated head of the tile
                if (split_half) {
                    const int half_chunks = chunks >> 1;
#pragma unroll 1
                    for (int c = 0; c < half_chunks; ++c) {
                        float2 cs[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) cs[i] = live ? ang[c * 32 + sub + i] : make_float2(1.f, 0.f);
#pragma unroll 1
                        for (int hh = 0; hh < heads_per_tile; ++hh) {
                            const int head = ft * heads_per_tile + hh;
                            if (head >= rotated_heads) break;
                            __nv_bfloat16* dst = dest(head);
                            const uint32_t col0 = lane_addr + hh * hd;
                            uint32_t g[16], u[16];
                            float va[16], vb[16];
                            tmem_ld16(col0 + c * 32 + sub, g);
                            tmem_ld16(col0 + (c + half_chunks) * 32 + sub, u);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const float xa = __uint_as_float(g[i]), xb = __uint_as_float(u[i]);
                                va[i] = __fsub_rn(__fmul_rn(xa, cs[i].x), __fmul_rn(xb, cs[i].y));
                                vb[i] = __fadd_rn(__fmul_rn(xa, cs[i].y), __fmul_rn(xb, cs[i].x));
                            }
                            if (live) {
                                store_row16(dst + c * 32 + sub, va);
                                store_row16(dst + (c + half_chunks) * 32 + sub, vb);
                            }
                        }
                    }
                }
            } else if (go && T::TOKM) {
                // lanes are tokens; columns 0..63 gate, 64..127 up of features 128 ft .. + 63, columns 128..255 the
                // same for the next 64 features: a thread forms 32 outputs of its token at a time
                const uint32_t lane_addr = tmem_base + ab * T::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
                const int t = tt * BLOCK_TOK + quarter * 32 + lane;
#pragma unroll 1
                for (int part = 2 * ehalf; part < 2 * ehalf + 2; ++part) {
                    const int half = part >> 1, c0 = (part & 1) * 32;
                    uint32_t g[CHUNK], u[CHUNK];
                    tmem_ld32(lane_addr + half * 128 + c0, g);
                    tmem_ld32(lane_addr + half * 128 + 64 + c0, u);
                    tmem_ld_wait();
                    const int f0 = ft * 128 + half * 64 + c0;
                    if (t < tokens && f0 < features) {
                        uint32_t packed[CHUNK / 2];
                        float vals[CHUNK];
#pragma unroll
                        for (int jj = 0; jj < CHUNK; ++jj) {
                            const float gate = __uint_as_float(g[jj]);
                            vals[jj] = __fdividef(gate, 1.0f + __expf(-gate)) * __uint_as_float(u[jj]);
                        }
                        const size_t at = (size_t)t * ldc + f0;
                        if (OUT_BF16 && f0 + CHUNK <= features && (ldc & 7) == 0) {
#pragma unroll
                            for (int jj = 0; jj < CHUNK / 2; ++jj) {
                                __nv_bfloat162 p = __floats2bfloat162_rn(vals[2 * jj], vals[2 * jj + 1]);
                                packed[jj] = *reinterpret_cast<uint32_t*>(&p);
                            }
                            uint4* dst = reinterpret_cast<uint4*>((__nv_bfloat16*)out + at);
#pragma unroll
                            for (int q = 0; q < CHUNK / 8; ++q)
                                dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                        } else {
#pragma unroll
                            for (int jj = 0; jj < CHUNK; ++jj) {
                                if (f0 + jj < features) {
                                    if (OUT_BF16) ((__nv_bfloat16*)out)[at + jj] = __float2bfloat16_rn(vals[jj]);
                                    else ((float*)out)[at + jj] = vals[jj];
                                }
                            }
                        }
                    }
                }
            } else if (go) {
                const uint32_t lane_addr = tmem_base + ab * T::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
                const int f = ft * BLOCK_FEAT + quarter * 32 + lane;
                const int tok0 = tt * BLOCK_TOK;
#pragma unroll 1
                for (int c0 = ehalf * (BLOCK_TOK / 2); c0 < (ehalf + 1) * (BLOCK_TOK / 2); c0 += CHUNK) {
                    uint32_t g[CHUNK], u[MODE == LP_GEMM_SWIGLU_WIDE ? CHUNK : 1];
                    tmem_ld32(lane_addr + c0, g);
                    if (MODE == LP_GEMM_SWIGLU_WIDE) tmem_ld32(lane_addr + BLOCK_TOK + c0, u);
                    tmem_ld_wait();
                    if (f < features) {
#pragma unroll
                        for (int jj = 0; jj < CHUNK; ++jj) {
                            const int t = tok0 + c0 + jj;
                            if (t >= tokens) break;
                            float v = __uint_as_float(g[jj]);
                            if (MODE == LP_GEMM_SWIGLU_WIDE) v = __fdividef(v, 1.0f + __expf(-v)) * __uint_as_float(u[jj]);
                            const size_t at = (size_t)t * ldc + f;
                            if (ATOMIC) atomicAdd((float*)out + at, v);
                            else if (OUT_BF16) ((__nv_bfloat16*)out)[at] = __float2bfloat16_rn(v);
                            else ((float*)out)[at] = v;
                        }
                    }
                }
            }
            // hand the accumulator back to the MMA thread
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[ab])) : "memory");
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)T::TMEM_COLS));
    }
}

template <int BLOCK_TOK, int MODE, bool OUT_BF16, bool ATOMIC>
int launch_persistent(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int tokens, int features, int ldc,
                      int k_blocks, int* status, cudaStream_t stream, const QkvEpilogue& qkv = QkvEpilogue{}) {
    using T = PersistentTile<BLOCK_TOK, MODE>;
    auto kernel = gemm_persistent_kernel<BLOCK_TOK, MODE, OUT_BF16, ATOMIC>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES);
        if (e != cudaSuccess) LP_REFUSE("gemm: cannot reserve %d bytes of shared memory: %s", T::SMEM_BYTES,
                                        cudaGetErrorString(e));
        configured = true;
    }
    const int sms = lp_sm_count();
    const int feat_tiles = (features + T::FEAT_PER_TILE - 1) / T::FEAT_PER_TILE;
    const int tok_tiles = (tokens + BLOCK_TOK - 1) / BLOCK_TOK;
    const int num_tiles = feat_tiles * tok_tiles;
    const int grid = num_tiles < sms ? num_tiles : sms;
    // how many token tiles a band has: the CTAs of one wave should touch as few distinct rows of X and W as possible
    const int w_rows = T::TOKM ? 256 : BLOCK_FEAT * T::W_TILES;
    int group_tok = 1;
    long long best = -1;
    for (int gt = 1; gt <= tok_tiles; ++gt) {
        const int gf = (grid + gt - 1) / gt;
        const long long cost = (long long)gt * BLOCK_TOK + (long long)(gf < feat_tiles ? gf : feat_tiles) * w_rows;
        if (best < 0 || cost <= best) { best = cost; group_tok = gt; }       // ties: the larger band
    }
    cudaError_t err = lp_launch(kernel, dim3(grid), PERSIST_THREADS, T::SMEM_BYTES, stream, mw, mx, out, tokens, features, ldc,
                                k_blocks, feat_tiles, num_tiles, group_tok, status, qkv);
    if (err != cudaSuccess) {
        snprintf(lp_error_text, sizeof(lp_error_text), "gemm_persistent: %s", cudaGetErrorString(err));
        return (int)err;
    }
    return lp_check_launch("gemm_persistent");
}

// For tests of the bounded waits: the next launch of the one-tile kernel gets this k-block withheld (then -1 again).
static int withhold_next_kblock = -1;

template <int BLOCK_TOK, int MODE, bool OUT_BF16, bool ATOMIC, bool TAIL = false>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int tokens, int features, int ldc, int k_blocks,
           int splits, int up_offset, int* status, const NormAfter& norm, cudaStream_t stream) {
    (void)up_offset;
    const int withheld = withhold_next_kblock;
    withhold_next_kblock = -1;
    using T = Tile<BLOCK_TOK, MODE>;
    auto kernel = gemm_tcgen05_kernel<BLOCK_TOK, MODE, OUT_BF16, ATOMIC, TAIL>;
    static bool configured = false;
    if (!configured) {
        const int most = T::STAGES_ALONE * T::STAGE_BYTES + T::TAIL_BYTES;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e != cudaSuccess) LP_REFUSE("gemm: cannot reserve %d bytes of shared memory: %s", most, cudaGetErrorString(e));
        configured = true;
    }
    const int per_split = (k_blocks + splits - 1) / splits;
    const int grid_z = (k_blocks + per_split - 1) / per_split;
    const int per_cta = MODE == LP_GEMM_SWIGLU ? BLOCK_FEAT / 2 : BLOCK_FEAT;     // output features per CTA
    dim3 grid((features + per_cta - 1) / per_cta, (tokens + BLOCK_TOK - 1) / BLOCK_TOK, grid_z);
    // the ring: what lets two CTAs share an SM, or, for a grid of at most one CTA per SM and when lp_gemm_configure's
    // ring_alone_tile allows it, up to the whole shared memory. Off by default: measured at the 1B shape, batches of
    // 32 / 64, a ring of 8 stages gave 1.101 / 1.340 ms per step against 1.078 / 1.320 with the shared ring (the
    // next kernel's CTAs can no longer start beside a CTA that holds the whole shared memory)
    int stages = T::STAGES;
    const bool alone = (long long)grid.x * grid.y * grid.z <= lp_sm_count();
    if (alone && few_settings().ring_alone_tile > stages) {
        stages = few_settings().ring_alone_tile < T::STAGES_ALONE ? few_settings().ring_alone_tile : T::STAGES_ALONE;
        if (stages > per_split) stages = per_split > T::STAGES ? per_split : T::STAGES;
    }
    const int smem = stages * T::STAGE_BYTES + T::TAIL_BYTES;
    cudaError_t err = lp_launch(kernel, grid, T::NTHREADS, smem, stream, mw, mx, out, tokens, features, ldc,
                                k_blocks, per_split, withheld, stages, status, norm);
    if (err != cudaSuccess) {
        snprintf(lp_error_text, sizeof(lp_error_text), "gemm_tcgen05: %s", cudaGetErrorString(err));
        return (int)err;
    }
    return lp_check_launch("gemm_tcgen05");
}

template <int BLOCK_TOK>
int dispatch(int mode, bool out_bf16, bool atomic, const CUtensorMap& mw, const CUtensorMap& mx, void* out, int tokens,
             int features, int ldc, int k_blocks, int splits, int up_offset, int* status, const NormAfter& norm,
             cudaStream_t stream) {
#define LP_GO(MODE, BF, AT) \
    return launch<BLOCK_TOK, MODE, BF, AT>(mw, mx, out, tokens, features, ldc, k_blocks, splits, up_offset, status, norm, stream)
    if (mode == LP_GEMM_SWIGLU) {
        if constexpr (BLOCK_TOK >= 128) {
            if (out_bf16) LP_GO(LP_GEMM_SWIGLU_WIDE, true, false);
            LP_GO(LP_GEMM_SWIGLU_WIDE, false, false);
        } else {
            if (out_bf16) LP_GO(LP_GEMM_SWIGLU, true, false);
            LP_GO(LP_GEMM_SWIGLU, false, false);
        }
    }
    if (atomic && norm.weight != nullptr)
        return launch<BLOCK_TOK, LP_GEMM_STORE, false, true, true>(mw, mx, out, tokens, features, ldc, k_blocks, splits,
                                                                  up_offset, status, norm, stream);
    if (atomic) LP_GO(LP_GEMM_STORE, false, true);
    if (out_bf16) LP_GO(LP_GEMM_STORE, true, false);
    LP_GO(LP_GEMM_STORE, false, false);
#undef LP_GO
}

}  // namespace

// Tests only: the next launch of the one-tile tcgen05 kernel (lp_gemm_tcgen05 with more than 16 tokens) never loads
// k-block `kblock`. The waits for it run out after their limit, the kernel sets *status and returns by itself
// with nothing left in flight; its output is not written. Exercises what the host does after such a report.
extern "C" int lp_gemm_withhold_next(int kblock) {
    withhold_next_kblock = kblock;
    return 0;
}

// fewtok: whether lp_gemm_tcgen05 hands 16-token tiles to the few-token kernel; ring_shared / ring_alone: stages of
// that kernel's ring when two CTAs share an SM / when a CTA has an SM to itself (at least 2 each); ring_alone_tile:
// the most stages the one-tile tcgen05 kernel takes when its grid has no more CTAs than there are SMs (0: never
// more than what lets two CTAs share an SM).
extern "C" int lp_gemm_configure(int fewtok, int ring_shared, int ring_alone, int ring_alone_tile, int ring_normed) {
    FewSettings& st = few_settings();
    st.enabled = fewtok ? 1 : 0;
    st.ring_shared = ring_shared < 2 ? 2 : ring_shared;
    st.ring_alone = ring_alone < 2 ? 2 : ring_alone;
    st.ring_alone_tile = ring_alone_tile;
    st.ring_normed = ring_normed;
    return 0;
}

// X: [tokens, K] bf16 (row stride ldx); W: [features, K] bf16 (row stride ldw); for SWIGLU, W holds
// 128 rows per 64 output features (64 gate rows, then the 64 up rows), features rounded up to 64;
// out: [tokens, ldc] float32 or bfloat16. mode: STORE / ACCUMULATE / SWIGLU. block_tok: 16..256 (a power of two).
// splits > 1 or ACCUMULATE adds into a float32 `out` with atomics (a STORE with splits needs `out` zeroed before).
// status: one int in device memory, set non-zero if a wait inside the kernel ran out.
// The persistent form (see above) for steps with many tokens: STORE (float32 / bfloat16), ACCUMULATE
// (float32, atomics) with 256-token tiles, SWIGLU (interleaved gate/up rows) with 128-token tiles.
extern "C" int lp_gemm_persistent(const void* X, const void* W, void* out, int out_dtype, int tokens, int features,
                                  int K, int ldx, int ldw, int ldc, int mode, int* status, cudaStream_t stream) {
    if (tokens <= 0 || features <= 0) return 0;
    if (K <= 0 || K % 8) LP_REFUSE("gemm: inner size %d must be a positive multiple of 8 for the tensor-core path", K);
    if (ldx % 8 || ldw % 8) LP_REFUSE("gemm: row strides %d / %d must be multiples of 8 elements", ldx, ldw);
    if (((uintptr_t)X | (uintptr_t)W) & 15) LP_REFUSE("gemm: operands must be 16-byte aligned");
    if (mode < 0 || mode > 2) LP_REFUSE("gemm: mode %d", mode);
    if (out_dtype != LP_F32 && out_dtype != LP_BF16) LP_REFUSE("gemm: output dtype code %d", out_dtype);
    if (mode == LP_GEMM_ACCUMULATE && out_dtype != LP_F32) LP_REFUSE("gemm: sums across CTAs need a float32 output");
    const int k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
    const bool gated = mode == LP_GEMM_SWIGLU;
    const long long w_rows = gated ? 128LL * ((features + 63) / 64) : features;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, W, w_rows, K, ldw, gated ? 256 : BLOCK_FEAT);
    if (rc) return rc;
    rc = make_map(&mx, X, tokens, K, ldx, gated ? 128 : 256);
    if (rc) return rc;
    const bool bf = out_dtype == LP_BF16;
    if (gated) {
        if (bf) return launch_persistent<128, LP_GEMM_SWIGLU_TOKM, true, false>(mw, mx, out, tokens, features, ldc, k_blocks, status, stream);
        return launch_persistent<128, LP_GEMM_SWIGLU_TOKM, false, false>(mw, mx, out, tokens, features, ldc, k_blocks, status, stream);
    }
    if (mode == LP_GEMM_ACCUMULATE)
        return launch_persistent<256, LP_GEMM_STORE, false, true>(mw, mx, out, tokens, features, ldc, k_blocks, status, stream);
    if (bf) return launch_persistent<256, LP_GEMM_STORE, true, false>(mw, mx, out, tokens, features, ldc, k_blocks, status, stream);
    return launch_persistent<256, LP_GEMM_STORE, false, false>(mw, mx, out, tokens, features, ldc, k_blocks, status, stream);
}

// The fused q|k|v projection of a step with many tokens: [tokens, K] x W[(H + 2G) * hd, K]^T (or H * hd rows when the
// layer keeps no keys of its own: pages null), whose epilogue rotates queries and keys by `angles` ([tokens, half]
// (cos, sin) pairs from lp_rope_angles; half = hd / 2, or 0 with angles null for no rotation), writes the queries to
// q_out [tokens, H * hd] and keys and values into pages [num_pages, 2, G, page_size, hd] at the tokens' positions,
// all bfloat16. Head sizes 32 (interleaved pairs or no rotation only), 64, 128, 256.
extern "C" int lp_gemm_qkv_rope(const void* X, const void* W, int tokens, int K, int ldx, int ldw, const float* angles,
                                int half, int interleaved, const int* positions, const int* seq_ids,
                                const int* page_table, int pt_stride, void* q_out, void* pages, int H, int G, int hd,
                                int page_size, int* status, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (K <= 0 || K % 8) LP_REFUSE("gemm_qkv_rope: inner size %d must be a positive multiple of 8", K);
    if (ldx % 8 || ldw % 8) LP_REFUSE("gemm_qkv_rope: row strides %d / %d must be multiples of 8 elements", ldx, ldw);
    if ((((uintptr_t)X | (uintptr_t)W | (uintptr_t)q_out | (uintptr_t)pages) & 15)) LP_REFUSE("gemm_qkv_rope: operands must be 16-byte aligned");
    if (H <= 0 || G < 0 || hd < 32 || hd > 256 || 256 % hd) LP_REFUSE("gemm_qkv_rope: heads %d/%d of %d (head sizes 32, 64, 128, 256)", H, G, hd);
    if (half != 0 && half * 2 != hd) LP_REFUSE("gemm_qkv_rope: rotary width %d of a head of %d (all of it, or none)", 2 * half, hd);
    if (half != 0 && !angles) LP_REFUSE("gemm_qkv_rope: rotation without angles");
    if (half != 0 && !interleaved && hd < 64) LP_REFUSE("gemm_qkv_rope: split-half pairs need heads of at least 64");
    if (pages && (page_size <= 0 || !page_table || !seq_ids)) LP_REFUSE("gemm_qkv_rope: a cache without page tables");
    if (!positions || !q_out) LP_REFUSE("gemm_qkv_rope: a null argument");
    const int features = (pages ? H + 2 * G : H) * hd;
    const int k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, W, features, K, ldw, 256);
    if (rc) return rc;
    rc = make_map(&mx, X, tokens, K, ldx, 128);
    if (rc) return rc;
    const QkvEpilogue qkv{half ? (const float2*)angles : nullptr, half, interleaved, positions, seq_ids, page_table, pt_stride,
                          (__nv_bfloat16*)q_out, (__nv_bfloat16*)pages, H, G, hd, page_size};
    return launch_persistent<128, LP_GEMM_QKV_TOKM, true, false>(mw, mx, nullptr, tokens, features, features, k_blocks,
                                                                 status, stream, qkv);
}

// norm_weight (optional, ACCUMULATE only, ldc == features): after the sums are complete, the last CTA writes
// the RMS norm of every output row to norm_out (bf16 [tokens, features]) and zeroes norm_clear; norm_counter
// is one int32, zero before the call.
extern "C" int lp_gemm_tcgen05(const void* X, const void* W, void* out, int out_dtype, int tokens, int features, int K,
                               int ldx, int ldw, int ldc, int mode, int block_tok, int splits, int* status,
                               const float* norm_weight, float norm_eps, void* norm_out, float* norm_clear,
                               long long norm_clear_count, int* norm_counter, cudaStream_t stream) {
    if (tokens <= 0 || features <= 0) return 0;
    if (K <= 0 || K % 8) LP_REFUSE("gemm: inner size %d must be a positive multiple of 8 for the tensor-core path", K);
    if (ldx % 8 || ldw % 8) LP_REFUSE("gemm: row strides %d / %d must be multiples of 8 elements", ldx, ldw);
    if (((uintptr_t)X | (uintptr_t)W) & 15) LP_REFUSE("gemm: operands must be 16-byte aligned");
    if (mode < 0 || mode > 2) LP_REFUSE("gemm: mode %d", mode);
    const int k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
    if (splits < 1) splits = 1;
    if (splits > k_blocks) splits = k_blocks;
    const bool atomic = mode == LP_GEMM_ACCUMULATE || (mode == LP_GEMM_STORE && splits > 1);
    if (mode == LP_GEMM_SWIGLU && splits > 1) LP_REFUSE("gemm: the gated epilogue cannot be split along K");
    if (atomic && out_dtype != LP_F32) LP_REFUSE("gemm: sums across CTAs need a float32 output");
    if (out_dtype != LP_F32 && out_dtype != LP_BF16) LP_REFUSE("gemm: output dtype code %d", out_dtype);
    const long long w_rows = mode == LP_GEMM_SWIGLU ? 128LL * ((features + 63) / 64) : features;
    CUtensorMap mw, mx;
    const bool wide = mode == LP_GEMM_SWIGLU && block_tok >= 128;
    int rc = make_map(&mw, W, w_rows, K, ldw, wide ? 64 : BLOCK_FEAT);
    if (rc) return rc;
    rc = make_map(&mx, X, tokens, K, ldx, block_tok);
    if (rc) return rc;
    NormAfter norm{};
    if (norm_weight) {
        if (mode != LP_GEMM_ACCUMULATE || ldc != features || features % 128 || !norm_out || !norm_counter)
            LP_REFUSE("gemm: a following norm needs an accumulating product over whole rows of a multiple of 128");
        norm = NormAfter{norm_weight, (__nv_bfloat16*)norm_out, norm_eps, norm_counter, norm_clear,
                         norm_clear ? norm_clear_count : 0};
    }
    const bool bf = out_dtype == LP_BF16;
    const int mmode = mode == LP_GEMM_SWIGLU ? LP_GEMM_SWIGLU : LP_GEMM_STORE;
    if (block_tok == 16 && tokens <= 16 && fewtok_enabled()) {
        // a handful of tokens: the mma.sync consumers (LLMPLAYER_B200_FEWTOK=0 keeps the tcgen05 kernel)
        const NormBefore none{};
        if (tokens <= 8) return dispatch_fewtok<1, false>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, status, norm, none, stream);
        return dispatch_fewtok<2, false>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, status, norm, none, stream);
    }
    switch (block_tok) {
        case 16: return dispatch<16>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, features, status, norm, stream);
        case 32: return dispatch<32>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, features, status, norm, stream);
        case 64: return dispatch<64>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, features, status, norm, stream);
        case 128: return dispatch<128>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, features, status, norm, stream);
        case 256: return dispatch<256>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, features, status, norm, stream);
        default: LP_REFUSE("gemm: token tile %d (supported: 16, 32, 64, 128, 256)", block_tok);
    }
}

// A product for at most 64 tokens with what a decode step fuses around it: the mma.sync kernel above up to 16
// tokens (8 with the norm on the way in), the one-tile tcgen05 kernels (with the norm on the way in, or plain) beyond.
// x_dtype LP_F32: X is the float32 residual stream and the product applies the RMS norm (gain, eps) on the
// way in; with splits > 1 the output then still lacks the rows' factors and `sumsq_out` [tokens] (zero before
// the call) receives sum x^2 per token for the reader to apply them. x_dtype LP_BF16: X as in lp_gemm_tcgen05.
// `zero` (optional): zero_count floats cleared on the side (nothing else in flight may use them).
extern "C" int lp_gemm_fewtok(const void* X, int x_dtype, const void* W, void* out, int out_dtype, int tokens,
                              int features, int K, int ldx, int ldw, int ldc, int mode, int splits, int* status,
                              const float* gain, float eps, float* sumsq_out, float* zero, int zero_count,
                              cudaStream_t stream) {
    if (tokens <= 0 || features <= 0) return 0;
    if (tokens > 64) LP_REFUSE("gemm_fewtok: %d tokens (at most 64)", tokens);
    if (K <= 0 || K % 8) LP_REFUSE("gemm: inner size %d must be a positive multiple of 8 for the tensor-core path", K);
    const bool xnorm = x_dtype == LP_F32;
    if (x_dtype != LP_F32 && x_dtype != LP_BF16) LP_REFUSE("gemm_fewtok: activation dtype code %d", x_dtype);
    if (ldw % 8 || ldx % (xnorm ? 4 : 8)) LP_REFUSE("gemm: row strides %d / %d must be multiples of 16 bytes", ldx, ldw);
    if (((uintptr_t)X | (uintptr_t)W) & 15) LP_REFUSE("gemm: operands must be 16-byte aligned");
    if (mode < 0 || mode > 2) LP_REFUSE("gemm: mode %d", mode);
    if (xnorm && (!gain || ((uintptr_t)gain & 15))) LP_REFUSE("gemm_fewtok: a float32 input needs the norm's gain, 16-byte aligned");
    const int k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
    if (splits < 1) splits = 1;
    if (splits > k_blocks) splits = k_blocks;
    const bool atomic = mode == LP_GEMM_ACCUMULATE || (mode == LP_GEMM_STORE && splits > 1);
    if (mode == LP_GEMM_SWIGLU && splits > 1) LP_REFUSE("gemm: the gated epilogue cannot be split along K");
    if (atomic && out_dtype != LP_F32) LP_REFUSE("gemm: sums across CTAs need a float32 output");
    if (out_dtype != LP_F32 && out_dtype != LP_BF16) LP_REFUSE("gemm: output dtype code %d", out_dtype);
    const int per_split = (k_blocks + splits - 1) / splits;
    if (xnorm && (k_blocks + per_split - 1) / per_split > 1 && !sumsq_out)
        LP_REFUSE("gemm_fewtok: a normed input shared out over %d CTAs needs a place for the sums of squares", splits);
    const long long w_rows = mode == LP_GEMM_SWIGLU ? 128LL * ((features + 63) / 64) : features;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, W, w_rows, K, ldw, BLOCK_FEAT);
    if (rc) return rc;
    const NormAfter after{};
    const NormBefore before{gain, eps, K, sumsq_out, zero, zero ? zero_count : 0};
    const bool bf = out_dtype == LP_BF16;
    const int mmode = mode == LP_GEMM_SWIGLU ? LP_GEMM_SWIGLU : LP_GEMM_STORE;
    // Beyond what the mma.sync consumers serve well: the tcgen05 kernels. With the norm on the way in that is beyond
    // 8 tokens (two token tiles double what every consumer warp converts; measured at the 1B shape, ms per step
    // with the mma.sync kernel against the tcgen05 kernel: 9 tokens 0.803 / 0.796, 12 tokens 0.840 / 0.790,
    // 16 tokens 0.842 / 0.797), without it beyond 16 (12 tokens: 0.790 against 0.807 with the tcgen05 kernel).
    if (tokens > (xnorm ? 8 : 16)) {
        const int tile = tokens <= 32 ? 32 : 64;
        if (xnorm) {
            rc = make_map_f32(&mx, X, tokens, K, ldx, tile);
            if (rc) return rc;
            if (tile == 32) return dispatch_normed<32>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, status, before, stream);
            return dispatch_normed<64>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, status, before, stream);
        }
        rc = make_map(&mx, X, tokens, K, ldx, tile);
        if (rc) return rc;
        const NormAfter side{nullptr, nullptr, 0.f, nullptr, zero, zero ? zero_count : 0};
        if (tile == 32) return dispatch<32>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, features, status, side, stream);
        return dispatch<64>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, features, status, side, stream);
    }
    // at most 16 tokens: the mma.sync consumers, one or two tiles of 8 tokens
    rc = xnorm ? make_map_f32(&mx, X, tokens, K, ldx, 16) : make_map(&mx, X, tokens, K, ldx, 16);
    if (rc) return rc;
#define LP_FEW(NT, XN) dispatch_fewtok<NT, XN>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, status, after, before, stream)
    if (xnorm) return LP_FEW(1, true);
    return tokens <= 8 ? LP_FEW(1, false) : LP_FEW(2, false);
#undef LP_FEW
}
