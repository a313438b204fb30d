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

namespace {

constexpr int BLOCK_FEAT = 128;   // weight rows per CTA = MMA M
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;      // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue
// The weight tile(s) of one k-block. WIDE: gate rows of two neighbouring 64-feature blocks form the
// first 128-row tile, their up rows the second (the tensor map's box is 64 rows then).
template <int MODE>
__device__ __forceinline__ void load_weights(uint8_t* stage, const CUtensorMap* map_w, int k, int cta, uint64_t* bar) {
    if (MODE == LP_GEMM_SWIGLU_WIDE) {
        const int row = cta * 256;
        tma_load_2d(stage, map_w, k, row, bar);                  // gate, features 128 cta ..
        tma_load_2d(stage + 8192, map_w, k, row + 128, bar);     // gate, features 128 cta + 64 ..
        tma_load_2d(stage + 16384, map_w, k, row + 64, bar);     // up
        tma_load_2d(stage + 24576, map_w, k, row + 192, bar);    // up
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
    static constexpr int ACC_COLS = BLOCK_TOK * W_TILES;
    static constexpr int TMEM_COLS = ACC_COLS < 32 ? 32 : ACC_COLS;       // power of two by construction
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};

// out: [tokens, ldc]; OUT_BF16 selects the element type of a STORE / SWIGLU output.
template <int BLOCK_TOK, int MODE, bool OUT_BF16, bool ATOMIC>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    void* __restrict__ out, int tokens, int features, int ldc, int k_blocks, int k_blocks_per_split,
                    int up_row_offset, int* __restrict__ status, NormAfter norm) {
    using T = Tile<BLOCK_TOK, MODE>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + T::STAGES * T::STAGE_BYTES);
    uint64_t* empty = full + T::STAGES;
    uint64_t* acc_ready = empty + T::STAGES;
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
        for (int s = 0; s < T::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
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
            // Weights are written by no kernel of a step: the first ring of weight tiles is requested
            // before waiting for the previous kernel, the activation tiles only after it.
            const int early = min(nkb, T::STAGES);
            for (int i = 0; i < early; ++i) {
                uint8_t* stage = smem + i * T::STAGE_BYTES;
                mbar_expect_tx(&full[i], T::STAGE_BYTES);
                const int k = (kb_begin + i) * BLOCK_K;
                load_weights<MODE>(stage, &map_w, k, blockIdx.x, &full[i]);
            }
            lp_grid_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d(smem + i * T::STAGE_BYTES + T::W_TILES * T::W_BYTES, &map_x, (kb_begin + i) * BLOCK_K, tok0,
                            &full[i]);
            issued = early;
            for (int i = early; i < nkb && ok; ++i) {
                const int s = i % T::STAGES;
                const uint32_t phase = (i / T::STAGES) & 1;
                if (!mbar_wait(&empty[s], phase ^ 1)) { atomicExch(status, 1); *failed = 1; ok = false; break; }
                uint8_t* stage = smem + s * T::STAGE_BYTES;
                mbar_expect_tx(&full[s], T::STAGE_BYTES);
                const int k = (kb_begin + i) * BLOCK_K;
                load_weights<MODE>(stage, &map_w, k, blockIdx.x, &full[s]);
                tma_load_2d(stage + T::W_TILES * T::W_BYTES, &map_x, k, tok0, &full[s]);
                issued = i + 1;
            }
            if (!ok) {
                // consumers may be gone: await the copies still in flight before the CTA's memory is released
                for (int i = max(0, issued - T::STAGES); i < issued; ++i)
                    mbar_wait(&full[i % T::STAGES], (i / T::STAGES) & 1);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BLOCK_TOK >> 3) << 17) |
                                       ((uint32_t)(BLOCK_FEAT >> 4) << 24);
            bool ok = true;
            for (int i = 0; i < nkb; ++i) {
                const int s = i % T::STAGES;
                const uint32_t phase = (i / T::STAGES) & 1;
                if (!mbar_wait(&full[s], phase)) { atomicExch(status, 2); *failed = 1; ok = false; break; }
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
            }
            (void)ok;
            tcgen05_commit(acc_ready);            // arrives when every MMA issued so far is complete
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;             // TMEM lanes 32*quarter .. +31 belong to this warp
        const bool ready = mbar_wait(acc_ready, 0);
        if (!ready && lane == 0) atomicExch(status, 3);
        tcgen05_fence_after();
        const bool go = __all_sync(0xffffffffu, ready && *failed == 0);
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        constexpr int CHUNK = BLOCK_TOK >= 32 ? 32 : 16;
        if (MODE != LP_GEMM_SWIGLU) {
            if (go) {
                const int f = feat0 + quarter * 32 + lane;
#pragma unroll 1
                for (int c0 = 0; c0 < BLOCK_TOK; c0 += CHUNK) {
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
            // rows 0..63 of the tile are gate, rows 64..127 up, of the same 64 output features. Every load
            // has been consumed by now, so the ring's memory carries the gate half across.
            float* cross = reinterpret_cast<float*>(smem);            // [64][BLOCK_TOK + 1]
            constexpr int LD = BLOCK_TOK + 1;
            const int local = (quarter & 1) * 32 + lane;              // feature within the 64
            if (go && quarter < 2) {
#pragma unroll 1
                for (int c0 = 0; c0 < BLOCK_TOK; c0 += CHUNK) {
                    uint32_t g[CHUNK];
                    if (CHUNK == 32) tmem_ld32(lane_addr + c0, g); else tmem_ld16(lane_addr + c0, g);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < CHUNK; ++j) cross[local * LD + c0 + j] = __uint_as_float(g[j]);
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");            // the four epilogue warps
            if (go && quarter >= 2) {
                const int f = blockIdx.x * (BLOCK_FEAT / 2) + local;
#pragma unroll 1
                for (int c0 = 0; c0 < BLOCK_TOK; c0 += CHUNK) {
                    uint32_t u[CHUNK];
                    if (CHUNK == 32) tmem_ld32(lane_addr + c0, u); else tmem_ld16(lane_addr + c0, u);
                    tmem_ld_wait();
                    if (f < features) {
#pragma unroll
                        for (int j = 0; j < CHUNK; ++j) {
                            const int t = tok0 + c0 + j;
                            if (t >= tokens) break;
                            const float gate = cross[local * LD + c0 + j];
                            const float v = __fdividef(gate, 1.0f + __expf(-gate)) * __uint_as_float(u[j]);
                            const size_t at = (size_t)t * ldc + f;
                            if (OUT_BF16) ((__nv_bfloat16*)out)[at] = __float2bfloat16_rn(v);
                            else ((float*)out)[at] = v;
                        }
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
    if (ATOMIC && norm.weight != nullptr) {
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

// ------------------------------------------------------------------ persistent form for prompts
// One CTA per SM walks over output tiles (tile = blockIdx.x, + gridDim.x, ...). Tensor memory holds two
// accumulators: while the epilogue warps read tile i out of one, the MMA thread fills the other with
// tile i + 1, and the loader keeps the ring of stages full across tile boundaries. No split of K, no
// norm fusion: this form serves steps with hundreds of tokens.
template <int BLOCK_TOK, int MODE>
struct PersistentTile {
    static constexpr int W_TILES = MODE == LP_GEMM_SWIGLU_WIDE ? 2 : 1;
    static constexpr int W_BYTES = BLOCK_FEAT * BLOCK_K * 2;
    static constexpr int X_BYTES = BLOCK_TOK * BLOCK_K * 2;
    static constexpr int STAGE_BYTES = W_TILES * W_BYTES + X_BYTES;
    static constexpr int STAGES = (196 * 1024) / STAGE_BYTES;
    static constexpr int ACC_COLS = BLOCK_TOK * W_TILES;
    static constexpr int TMEM_COLS = 2 * ACC_COLS;                // 512 for both uses below
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
    static_assert(TMEM_COLS == 512 || TMEM_COLS == 256, "two accumulators must fit tensor memory");
};

template <int BLOCK_TOK, int MODE, bool OUT_BF16, bool ATOMIC>
__global__ void __launch_bounds__(THREADS, 1)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                       void* __restrict__ out, int tokens, int features, int ldc, int k_blocks, int feat_tiles,
                       int num_tiles, int* __restrict__ status) {
    using T = PersistentTile<BLOCK_TOK, MODE>;
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
        for (int k = 0; k < 2; ++k) { mbar_init(&acc_full[k], 1); mbar_init(&acc_empty[k], 4); }
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
                const int ft = tile % feat_tiles, tt = tile / feat_tiles;
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
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BLOCK_TOK >> 3) << 17) |
                                       ((uint32_t)(BLOCK_FEAT >> 4) << 24);
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
                        tcgen05_mma(acc, dw + step, dx + step, idesc, (kb > 0 || k > 0) ? 1u : 0u);
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
        constexpr int CHUNK = 32;
        int j = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++j) {
            const int ab = j & 1;
            const int ft = tile % feat_tiles, tt = tile / feat_tiles;
            if (ok && !mbar_wait(&acc_full[ab], (j >> 1) & 1)) { if (lane == 0) atomicExch(status, 24); *failed = 1; ok = false; }
            tcgen05_fence_after();
            const bool go = __all_sync(0xffffffffu, ok && *failed == 0);
            if (go) {
                const uint32_t lane_addr = tmem_base + ab * T::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
                const int f = ft * BLOCK_FEAT + quarter * 32 + lane;
                const int tok0 = tt * BLOCK_TOK;
#pragma unroll 1
                for (int c0 = 0; c0 < BLOCK_TOK; c0 += CHUNK) {
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
                      int k_blocks, int* status, cudaStream_t stream) {
    using T = PersistentTile<BLOCK_TOK, MODE>;
    auto kernel = gemm_persistent_kernel<BLOCK_TOK, MODE, OUT_BF16, ATOMIC>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES);
        if (e != cudaSuccess) LP_REFUSE("gemm: cannot reserve %d bytes of shared memory: %s", T::SMEM_BYTES,
                                        cudaGetErrorString(e));
        configured = true;
    }
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const int feat_tiles = (features + BLOCK_FEAT - 1) / BLOCK_FEAT;
    const int num_tiles = feat_tiles * ((tokens + BLOCK_TOK - 1) / BLOCK_TOK);
    const int grid = num_tiles < sms ? num_tiles : sms;
    cudaError_t err = lp_launch(kernel, dim3(grid), THREADS, T::SMEM_BYTES, stream, mw, mx, out, tokens, features, ldc,
                                k_blocks, feat_tiles, num_tiles, status);
    if (err != cudaSuccess) {
        snprintf(lp_error_text, sizeof(lp_error_text), "gemm_persistent: %s", cudaGetErrorString(err));
        return (int)err;
    }
    return lp_check_launch("gemm_persistent");
}

template <int BLOCK_TOK, int MODE, bool OUT_BF16, bool ATOMIC>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int tokens, int features, int ldc, int k_blocks,
           int splits, int up_offset, int* status, const NormAfter& norm, cudaStream_t stream) {
    using T = Tile<BLOCK_TOK, MODE>;
    auto kernel = gemm_tcgen05_kernel<BLOCK_TOK, MODE, OUT_BF16, ATOMIC>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES);
        if (e != cudaSuccess) LP_REFUSE("gemm: cannot reserve %d bytes of shared memory: %s", T::SMEM_BYTES,
                                        cudaGetErrorString(e));
        configured = true;
    }
    const int per_split = (k_blocks + splits - 1) / splits;
    const int grid_z = (k_blocks + per_split - 1) / per_split;
    const int per_cta = MODE == LP_GEMM_SWIGLU ? BLOCK_FEAT / 2 : BLOCK_FEAT;     // output features per CTA
    dim3 grid((features + per_cta - 1) / per_cta, (tokens + BLOCK_TOK - 1) / BLOCK_TOK, grid_z);
    cudaError_t err = lp_launch(kernel, grid, THREADS, T::SMEM_BYTES, stream, mw, mx, out, tokens, features, ldc,
                                k_blocks, per_split, up_offset, status, norm);
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
    if (atomic) LP_GO(LP_GEMM_STORE, false, true);
    if (out_bf16) LP_GO(LP_GEMM_STORE, true, false);
    LP_GO(LP_GEMM_STORE, false, false);
#undef LP_GO
}

}  // namespace

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
    int rc = make_map(&mw, W, w_rows, K, ldw, gated ? 64 : BLOCK_FEAT);
    if (rc) return rc;
    rc = make_map(&mx, X, tokens, K, ldx, gated ? 128 : 256);
    if (rc) return rc;
    const bool bf = out_dtype == LP_BF16;
    if (gated) {
        if (bf) return launch_persistent<128, LP_GEMM_SWIGLU_WIDE, true, false>(mw, mx, out, tokens, features, ldc, k_blocks, status, stream);
        return launch_persistent<128, LP_GEMM_SWIGLU_WIDE, false, false>(mw, mx, out, tokens, features, ldc, k_blocks, status, stream);
    }
    if (mode == LP_GEMM_ACCUMULATE)
        return launch_persistent<256, LP_GEMM_STORE, false, true>(mw, mx, out, tokens, features, ldc, k_blocks, status, stream);
    if (bf) return launch_persistent<256, LP_GEMM_STORE, true, false>(mw, mx, out, tokens, features, ldc, k_blocks, status, stream);
    return launch_persistent<256, LP_GEMM_STORE, false, false>(mw, mx, out, tokens, features, ldc, k_blocks, status, stream);
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
    switch (block_tok) {
        case 16: return dispatch<16>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, features, status, norm, stream);
        case 32: return dispatch<32>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, features, status, norm, stream);
        case 64: return dispatch<64>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, features, status, norm, stream);
        case 128: return dispatch<128>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, features, status, norm, stream);
        case 256: return dispatch<256>(mmode, bf, atomic, mw, mx, out, tokens, features, ldc, k_blocks, splits, features, status, norm, stream);
        default: LP_REFUSE("gemm: token tile %d (supported: 16, 32, 64, 128, 256)", block_tok);
    }
}
