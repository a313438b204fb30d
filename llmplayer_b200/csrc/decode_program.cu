// A whole decode step (one new token for each of up to 16 sequences) as ONE persistent kernel
// that walks a list of operations: matrix products over bfloat16 weights (tcgen05 MMA, weights
// by TMA, accumulators in tensor memory) and attention over the paged cache (mma.sync units of
// attention_decode.cuh). One CTA per SM, launched cooperatively; between two operations all CTAs
// meet at a barrier in global memory.
//
// Why one kernel: a step of a small model is a chain of some hundred products that each stream a
// few megabytes; as separate kernels each pays its launch, set-up and first-load latency. Here the
// loader warp of every CTA runs ahead through the list and keeps its ring of weight tiles full across
// the barriers (weights depend on nothing), so HBM keeps streaming while the CTAs synchronise.
//
// Roles in a CTA of 192 threads: warp 0 loads weight tiles (TMA, 128-byte swizzle, no multicast),
// warp 1 issues the MMAs, warps 2..5 (the workers) build the activation operand in shared memory,
// drain the accumulators and run the attention units.
//   * activation operand: the workers read the activations from global memory (L2; other CTAs of
//     this kernel wrote them), optionally apply an RMS norm over the whole row (float32), round to
//     bfloat16 and write the 16 x K tile in the swizzled layout the MMA wants. A product whose input
//     is the normed residual stream therefore needs no norm kernel and no barrier for it.
//   * epilogues: store float32, add into float32 (atomics: the residual stream, or split-K partial
//     sums), or silu(gate) * up to bfloat16 from the interleaved gate/up weight layout.
//   * a product is cut into units of (128 features) x (a share of K); unit u belongs to CTA u mod grid.
//
// The reference runs a captured chain of one kernel per operation for the same step
// (java21 inference/CudaForwardPass.java:1760-1812); it has no counterpart of this kernel.
//
// Every wait (mbarrier, grid barrier) is bounded. A wait that runs out records a code in *status,
// raises a flag that all roles and all CTAs poll, and the kernel winds down: copies in flight are
// awaited, tensor memory is freed, every CTA returns.
#include "tcgen05_utils.cuh"
#include "attention_decode.cuh"

#define LP_OP_PRODUCT 0
#define LP_OP_ATTENTION 1
#define LP_X_BF16 0
#define LP_X_RMSNORM 1
#define LP_EPI_STORE 0
#define LP_EPI_ADD 1
#define LP_EPI_SWIGLU 2

namespace {

constexpr int TOK = 16;                         // MMA N: the step's tokens, padded
constexpr int ACC_WAYS = 4;                     // the four k-steps of a k-block add into accumulators of their own:
                                                // MMAs into one accumulator wait for one another, these do not
constexpr int ACC_COLS = TOK * ACC_WAYS;        // tensor-memory columns of a unit
constexpr int TMEM_COLS = 2 * ACC_COLS;         // two units in flight
constexpr int FEAT = 128;                       // MMA M: weight rows per unit
constexpr int UMMA_K = 16;
constexpr int W_BYTES = FEAT * BLOCK_K * 2;     // one ring stage: a 128 x 64 weight tile
constexpr int X_KB_BYTES = TOK * BLOCK_K * 2;   // the activation tile of one k-block
constexpr int THREADS = 192;
constexpr int MAX_STAGES = 12;
constexpr int CROSS_BYTES = 64 * (TOK + 1) * 4; // gate half on its way to the warps that hold the up half
constexpr uint32_t GRID_SPIN_LIMIT = 1u << 22;

struct AttentionOp {
    FusedDecodeArgs fused;
    const __nv_bfloat16* pages;
    const int* page_table;
    const int* kv_len;
    float* part_o;
    float* part_ml;
    __nv_bfloat16* out;
    int pt_stride, H, G, hd, window, pages_per_split, num_splits, head_groups, batch;
    float scale_log2;
};

struct ProductArgs {
    int units;                // work units of this operation over all CTAs
    int features;             // output features (for SWIGLU: of the activation, half the weight rows)
    int K, k_blocks, splits;
    int x_kind, epilogue;
    int tokens;               // rows of the activation operand that are real (<= 16)
    int ldx, ldc;
    int clear_count;
    float eps;
    const void* x;            // [*, ldx] bfloat16, or float32 when x_kind is RMSNORM
    const int* x_rows;        // optional: operand row i is row x_rows[i] of x
    const float* gain;        // RMSNORM: [K]
    void* out;                // [tokens, ldc]
    float* clear;             // optional float32 buffer that the CTAs zero while they work on this operation
};

struct alignas(128) ProgramOp {
    CUtensorMap map_w;        // [rows, K] bfloat16 weights, boxes of 128 x 64
    int type;
    int units;                // = p.units or the attention's
    ProductArgs p;
    AttentionOp at;
};

struct Shared {
    uint64_t full[MAX_STAGES], empty[MAX_STAGES];
    uint64_t acc_full[2], acc_empty[2], x_full[2];
    uint32_t tmem_slot;
    volatile uint32_t failed;
    float scale[TOK];
};

__device__ __forceinline__ void unit_range(int splits, int k_blocks, int u, int& tile, int& kb0, int& nkb) {
    const int split = u % splits;
    tile = u / splits;
    const int base = k_blocks / splits, extra = k_blocks % splits;
    kb0 = split * base + min(split, extra);
    nkb = base + (split < extra ? 1 : 0);
}

__device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// True for all 128 workers if `flag` is true for any of them: decisions that lead to different barriers
// must be the same in every worker.
__device__ __forceinline__ bool workers_any(bool flag) {
    uint32_t any;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 p, %1, 0;\n\t"
        "barrier.cta.red.or.pred q, 1, 128, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(any) : "r"((uint32_t)flag) : "memory");
    return any != 0;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// The 16 x (nkb * 64) activation operand of a unit, written by the 128 workers. With an RMS norm the
// operand is bfloat16(x * gain); the row's factor 1 / sqrt(mean x^2 + eps) is applied to the sums in the
// epilogue (it is a scalar per row, so it commutes with the product). A thread owns 16-byte columns
// (8 features) of the operand and fills them for every row: the gain is fetched once per column and the
// loads of eight rows are in flight together.
__device__ __forceinline__ void produce_x(const ProductArgs& a_, int kb0, int nkb, uint8_t* xs, int tid) {
    const ProductArgs* op = &a_;
    const int n = op->tokens, K = op->K, ldx = op->ldx;
    const int* rows = op->x_rows;
    const bool normed = op->x_kind == LP_X_RMSNORM;
    const int cols = nkb * 8;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    // every CTA reads the same rows at the same time: each starts at a column of its own, so that their
    // requests spread over the L2 instead of queueing at one line after the other
    const int rot = (int)((blockIdx.x * 40u) % (uint32_t)cols) & ~7;
    for (int c0 = tid; c0 < cols; c0 += 128) {
        int cc = c0 + rot;
        if (cc >= cols) cc -= cols;
        const int kb = cc >> 3, j = cc & 7;
        const int k = (kb0 + kb) * BLOCK_K + j * 8;
        uint8_t* col = xs + kb * X_KB_BYTES;
        const bool inside = k < K;                    // K is a multiple of 8: a column is inside or outside
        float4 ga = make_float4(1.f, 1.f, 1.f, 1.f), gb = ga;
        if (normed && inside) {
            ga = __ldg(reinterpret_cast<const float4*>(op->gain + k));
            gb = __ldg(reinterpret_cast<const float4*>(op->gain + k) + 1);
        }
#pragma unroll 1
        for (int r0 = 0; r0 < TOK; r0 += 8) {
            float4 a[8], b[8];                        // a bfloat16 operand's 16 bytes travel in a[]
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int r = r0 + u;
                if (r < n && inside) {
                    const size_t src = (size_t)(rows ? rows[r] : r) * ldx + k;
                    if (normed) {
                        const float4* p = reinterpret_cast<const float4*>((const float*)op->x + src);
                        a[u] = __ldcg(p);
                        b[u] = __ldcg(p + 1);
                    } else {
                        const uint4 h = __ldcg(reinterpret_cast<const uint4*>((const __nv_bfloat16*)op->x + src));
                        a[u] = make_float4(__uint_as_float(h.x), __uint_as_float(h.y), __uint_as_float(h.z), __uint_as_float(h.w));
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int r = r0 + u;                 // r & 7 == u
                uint4 packed = zero4;
                if (r < n && inside) {
                    if (normed) {
                        packed.x = pack_bf16(a[u].x * ga.x, a[u].y * ga.y);
                        packed.y = pack_bf16(a[u].z * ga.z, a[u].w * ga.w);
                        packed.z = pack_bf16(b[u].x * gb.x, b[u].y * gb.y);
                        packed.w = pack_bf16(b[u].z * gb.z, b[u].w * gb.w);
                    } else {
                        packed = make_uint4(__float_as_uint(a[u].x), __float_as_uint(a[u].y), __float_as_uint(a[u].z),
                                            __float_as_uint(a[u].w));
                    }
                }
                *reinterpret_cast<uint4*>(col + (r >> 3) * 1024 + u * 128 + ((j ^ u) << 4)) = packed;
            }
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the MMA reads through the async proxy
    workers_sync();

}

// scale[t] = 1 / sqrt(mean of x[t]^2 + eps) for the operand rows of a normed product: warp w takes rows w,
// w + 4, ...; a fixed order of additions, so every CTA gets the same factors.
__device__ __forceinline__ void row_scales(const ProductArgs& a_, float* scale_s, int tid) {
    const ProductArgs* op = &a_;
    const int n = op->tokens, K = op->K;
    const int warp = tid >> 5, lane = tid & 31;
    const int quads = K >> 2;
    for (int t = warp; t < n; t += 4) {
        const float4* row = reinterpret_cast<const float4*>((const float*)op->x +
                                                            (size_t)(op->x_rows ? op->x_rows[t] : t) * op->ldx);
        float ss = 0.f;
        const int rot = (int)((blockIdx.x * 40u) % (uint32_t)quads);      // see produce_x
        for (int i0 = lane; i0 < quads; i0 += 32 * 16) {
            float4 v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                int i = i0 + u * 32;
                const bool in = i < quads;
                i += rot;
                if (i >= quads) i -= quads;
                v[u] = in ? __ldcg(row + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 16; ++u) ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
        }
        ss = lp_warp_sum(ss);
        if (lane == 0) scale_s[t] = 1.0f / sqrtf(ss / (float)K + op->eps);
    }
    workers_sync();
}

struct PendingUnit {
    int tile;
    uint32_t count;           // running number of the unit: accumulator count & 1, use count >> 1
};

// Drain the accumulator of a finished unit. False when the wait for the MMAs ran out.
__device__ __forceinline__ bool epilogue(const ProductArgs& a_, const PendingUnit& p, Shared* sh, uint32_t tmem_base,
                                         float* cross, int tid, int* status) {
    const int warp = tid >> 5, lane = tid & 31;
    const int quarter = ((tid >> 5) + 2) & 3;          // worker warp w is CTA warp w + 2: TMEM lanes 32 * ((w + 2) % 4)
    const uint32_t buf = p.count & 1, use = p.count >> 1;
    const bool ready = mbar_wait(&sh->acc_full[buf], use & 1);
    if (!ready) { if (lane == 0) atomicCAS(status, 0, 33); sh->failed = 1; }
    tcgen05_fence_after();
    const bool go = !workers_any(!ready || sh->failed != 0);
    const ProductArgs* op = &a_;
    const int n = op->tokens, ldc = op->ldc;
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * ACC_COLS;
    uint32_t r[TOK];
    if (go) {
        uint32_t w[ACC_COLS];
        tmem_ld64(taddr, w);
        tmem_ld_wait();
        const bool normed = op->x_kind == LP_X_RMSNORM;
#pragma unroll
        for (int j = 0; j < TOK; ++j) {
            float v = (__uint_as_float(w[j]) + __uint_as_float(w[TOK + j])) +
                      (__uint_as_float(w[2 * TOK + j]) + __uint_as_float(w[3 * TOK + j]));
            if (normed) v *= sh->scale[j];
            r[j] = __float_as_uint(v);
        }
    }
    if (op->epilogue != LP_EPI_SWIGLU) {
        const int f = p.tile * FEAT + quarter * 32 + lane;
        if (go && f < op->features) {
            float* out = (float*)op->out + f;
            if (op->epilogue == LP_EPI_ADD) {
#pragma unroll
                for (int j = 0; j < TOK; ++j) if (j < n) atomicAdd(out + (size_t)j * ldc, __uint_as_float(r[j]));
            } else {
#pragma unroll
                for (int j = 0; j < TOK; ++j) if (j < n) out[(size_t)j * ldc] = __uint_as_float(r[j]);
            }
        }
    } else {
        // weight rows 0..63 of the tile are gate, 64..127 up, of the same 64 features
        constexpr int LD = TOK + 1;
        const int local = (quarter & 1) * 32 + lane;
        if (go && quarter < 2) {
#pragma unroll
            for (int j = 0; j < TOK; ++j) cross[local * LD + j] = __uint_as_float(r[j]);
        }
        workers_sync();
        const int f = p.tile * (FEAT / 2) + local;
        if (go && quarter >= 2 && f < op->features) {
            __nv_bfloat16* out = (__nv_bfloat16*)op->out + f;
#pragma unroll
            for (int j = 0; j < TOK; ++j) {
                if (j < n) {
                    const float gate = cross[local * LD + j];
                    out[(size_t)j * ldc] = __float2bfloat16_rn(__fdividef(gate, 1.0f + __expf(-gate)) * __uint_as_float(r[j]));
                }
            }
        }
        workers_sync();                                // `cross` is free for the next unit
    }
    (void)warp;
    tcgen05_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&sh->acc_empty[buf]);
    return go;
}

// All CTAs have finished the operations before `op_index` (each adds 1 per operation).
__device__ __forceinline__ bool grid_wait(uint32_t* counter, uint32_t target, Shared* sh, int* status, int tid) {
    if (tid == 0) {
        bool ok = false;
        for (uint32_t i = 0; i < GRID_SPIN_LIMIT; ++i) {
            if (load_acquire(counter) >= target) { ok = true; break; }
            if ((i & 255) == 255 && *(volatile int*)status != 0) break;     // another CTA gave up
            if (i > 32) __nanosleep(32);
        }
        if (!ok) { atomicCAS(status, 0, 40); sh->failed = 1; }
        __threadfence();
    }
    return !workers_any(sh->failed != 0);
}
__device__ __forceinline__ void grid_arrive(uint32_t* counter, int tid) {
    workers_sync();                  // every worker's writes precede ...
    if (tid == 0) {
        __threadfence();             // ... this fence, which precedes the count
        atomicAdd(counter, 1u);
    }
}

// Out of line: the unit's registers are its own, not the product path's.
template <int HD, int STAGES, typename Before>
__device__ __noinline__ void attention_unit(uint8_t* scratch, int tid, int split, int by, int b, const AttentionOp& a,
                                            Before& before_inputs) {
    attention_decode_unit<HD, true, HD, true, STAGES, 4>(
        scratch, tid, split, by, b, nullptr, a.pages, a.page_table, a.pt_stride, a.kv_len, a.part_o, a.part_ml, a.out, a.H,
        a.G, a.hd, a.scale_log2, a.window, a.pages_per_split, a.num_splits, a.head_groups, a.fused, before_inputs);
}

__global__ void __launch_bounds__(THREADS, 1)
decode_program_kernel(const ProgramOp* __restrict__ ops, int num_ops, uint32_t* __restrict__ counter,
                      int* __restrict__ status, int stages, int region_bytes, long long* __restrict__ timing) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* ring = smem;
    uint8_t* region = ring + (size_t)stages * W_BYTES;            // activation operand, or attention scratch
    float* cross = reinterpret_cast<float*>(region + region_bytes);
    Shared* sh = reinterpret_cast<Shared*>(region + region_bytes + CROSS_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        sh->failed = 0;
        for (int s = 0; s < stages; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
        for (int k = 0; k < 2; ++k) {
            mbar_init(&sh->acc_full[k], 1); mbar_init(&sh->acc_empty[k], 4); mbar_init(&sh->x_full[k], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&sh->tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = sh->tmem_slot;
    const int cta = blockIdx.x, grid = gridDim.x;

    if (warp == 0) {
        // ------------------------------------------------------------ weight loader: runs ahead through the list
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int o = 0; o < num_ops && ok; ++o) {
                const ProgramOp* op = ops + o;
                if (op->type != LP_OP_PRODUCT) continue;
                const int units = op->units, splits = op->p.splits, k_blocks = op->p.k_blocks;
                if (cta < units) asm volatile("prefetch.tensormap [%0];" ::"l"(&op->map_w) : "memory");
                for (int u = cta; u < units && ok; u += grid) {
                    int tile, kb0, nkb;
                    unit_range(splits, k_blocks, u, tile, kb0, nkb);
                    for (int i = 0; i < nkb; ++i, ++it) {
                        const uint32_t s = it % stages, phase = (it / stages) & 1;
                        if (sh->failed || !mbar_wait(&sh->empty[s], phase ^ 1)) {
                            if (!sh->failed) { atomicCAS(status, 0, 31); sh->failed = 1; }
                            ok = false;
                            break;
                        }
                        mbar_expect_tx(&sh->full[s], W_BYTES);
                        tma_load_2d(ring + (size_t)s * W_BYTES, &op->map_w, (kb0 + i) * BLOCK_K, tile * FEAT, &sh->full[s]);
                    }
                }
            }
            if (!ok) {
                // consumers may be gone: await the copies still in flight before the CTA's memory is released
                const uint32_t first = it > (uint32_t)stages ? it - stages : 0;
                for (uint32_t i = first; i < it; ++i) mbar_wait(&sh->full[i % stages], (i / stages) & 1);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TOK >> 3) << 17) |
                                       ((uint32_t)(FEAT >> 4) << 24);
            uint32_t it = 0, count = 0;
            bool ok = true;
            for (int o = 0; o < num_ops && ok; ++o) {
                const ProgramOp* op = ops + o;
                if (op->type != LP_OP_PRODUCT) continue;
                const int units = op->units, splits = op->p.splits, k_blocks = op->p.k_blocks;
                for (int u = cta; u < units && ok; u += grid, ++count) {
                    int tile, kb0, nkb;
                    unit_range(splits, k_blocks, u, tile, kb0, nkb);
                    const uint32_t buf = count & 1, use = count >> 1;
                    if (!mbar_wait(&sh->acc_empty[buf], (use & 1) ^ 1) || !mbar_wait(&sh->x_full[buf], use & 1) ||
                        sh->failed) {
                        if (!sh->failed) { atomicCAS(status, 0, 32); sh->failed = 1; }
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t acc = tmem_base + buf * ACC_COLS;
                    for (int i = 0; i < nkb; ++i, ++it) {
                        const uint32_t s = it % stages, phase = (it / stages) & 1;
                        if (!mbar_wait(&sh->full[s], phase)) { atomicCAS(status, 0, 34); sh->failed = 1; ok = false; break; }
                        tcgen05_fence_after();
                        const uint64_t dw = smem_desc(smem_u32(ring + (size_t)s * W_BYTES));
                        const uint64_t dx = smem_desc(smem_u32(region + (size_t)i * X_KB_BYTES));
#pragma unroll
                        for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                            const uint64_t step = (uint64_t)((k * UMMA_K * 2) >> 4);
                            tcgen05_mma(acc + k * TOK, dw + step, dx + step, idesc, i > 0 ? 1u : 0u);
                        }
                        tcgen05_commit(&sh->empty[s]);
                    }
                    tcgen05_commit(&sh->acc_full[buf]);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ workers
        static_assert(BLOCK_K / UMMA_K == ACC_WAYS, "one accumulator per k-step of a k-block");
        const int tid = threadIdx.x - 64;
        uint32_t count = 0;
        bool ok = true;
        for (int o = 0; o < num_ops && ok; ++o) {
            const ProgramOp* op = ops + o;
            const bool timed = timing != nullptr && cta == 0 && tid == 0;    // clock stamps of CTA 0, four per operation
            if (timed) { timing[o * 4] = clock64(); timing[o * 4 + 2] = 0; }
            const uint32_t target = (uint32_t)o * (uint32_t)grid;
            if (op->type == LP_OP_PRODUCT) {
                // what does not depend on earlier operations comes before the barrier: the operation's
                // description (into registers) and the gain of this thread's operand columns (into L1)
                const ProductArgs pa = op->p;
                if (cta < pa.units && pa.x_kind == LP_X_RMSNORM) {
                    int tile, kb0, nkb;
                    unit_range(pa.splits, pa.k_blocks, cta, tile, kb0, nkb);
                    for (int cc = tid; cc < nkb * 8; cc += 128) {
                        const int k = (kb0 + (cc >> 3)) * BLOCK_K + (cc & 7) * 8;
                        if (k < pa.K) asm volatile("prefetch.global.L1 [%0];" ::"l"(pa.gain + k));
                    }
                }
                if (o > 0) ok = grid_wait(counter, target, sh, status, tid);
                if (!ok) break;
                if (timed) timing[o * 4 + 1] = clock64();
                if (pa.clear) {
                    for (int i = cta * 128 + tid; i < pa.clear_count; i += grid * 128) __stcg(pa.clear + i, 0.f);
                }
                PendingUnit pending;
                bool have_pending = false;
                bool scales_known = pa.x_kind != LP_X_RMSNORM;
                int res_kb0 = -1, res_nkb = -1;           // the k range of the operand that is in shared memory
                for (int u = cta; u < pa.units && ok; u += grid, ++count) {
                    int tile, kb0, nkb;
                    unit_range(pa.splits, pa.k_blocks, u, tile, kb0, nkb);
                    const bool same = kb0 == res_kb0 && nkb == res_nkb;
                    if (!same) {
                        // the MMAs that read the old operand must be complete: drain their unit first
                        if (have_pending) { ok = epilogue(pa, pending, sh, tmem_base, cross, tid, status); have_pending = false; }
                        if (!ok) break;
                        produce_x(pa, kb0, nkb, region, tid);
                        res_kb0 = kb0; res_nkb = nkb;
                        if (timed && timing[o * 4 + 2] == 0) timing[o * 4 + 2] = clock64();
                    }
                    if (tid == 0) mbar_arrive(&sh->x_full[count & 1]);
                    if (!scales_known) {               // while the MMAs of the first unit run
                        row_scales(pa, sh->scale, tid);
                        scales_known = true;
                    }
                    if (have_pending) ok = epilogue(pa, pending, sh, tmem_base, cross, tid, status);
                    pending.tile = tile; pending.count = count;
                    have_pending = true;
                }
                if (have_pending && ok) ok = epilogue(pa, pending, sh, tmem_base, cross, tid, status);
            } else {
                const AttentionOp a = op->at;
                const int units = op->units;
                const int per_seq = a.G * a.head_groups;
                bool waited = o == 0;
                // the unit requests its pages first and waits for the projection (the previous operation) only then
                auto before_inputs = [&]() {
                    if (!waited) {
                        ok = grid_wait(counter, target, sh, status, tid);
                        waited = true;
                        if (timed) timing[o * 4 + 1] = clock64();
                    }
                };
                for (int u = cta; u < units; u += grid) {
                    const int split = u % a.num_splits, rest = u / a.num_splits;
                    const int by = rest % per_seq, b = rest / per_seq;
                    if (a.hd == 64) attention_unit<64, 6>(region, tid, split, by, b, a, before_inputs);
                    else attention_unit<128, 3>(region, tid, split, by, b, a, before_inputs);
                }
                before_inputs();                       // a CTA without a unit keeps in step all the same
            }
            if (!ok) break;
            if (timed) timing[o * 4 + 3] = clock64();
            if (o + 1 < num_ops) grid_arrive(counter, tid);
        }
        if (!ok && tid == 0) sh->failed = 1;
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS));
    }
}

// The step's first kernel: x[t] = embedding[token[t]] in float32, and the buffers the program wants
// zero at its start (the barrier count; the partial sums of the first split-K product).
template <typename TEmb>
__global__ void program_prologue_kernel(const TEmb* __restrict__ table, const int* __restrict__ tokens,
                                        float* __restrict__ x, int d, int vocab, float* __restrict__ zero,
                                        int zero_count, uint32_t* __restrict__ counter) {
    lp_grid_release();
    lp_grid_wait();
    const int t = blockIdx.x;
    int token = tokens[t];
    token = min(max(token, 0), vocab - 1);
    for (int i = threadIdx.x; i < d; i += blockDim.x) x[(size_t)t * d + i] = lp_to_float(table[(size_t)token * d + i]);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < zero_count; i += gridDim.x * blockDim.x) zero[i] = 0.f;
    if (t == 0 && threadIdx.x == 0) *counter = 0u;
}

int shared_bytes(int stages, int region_bytes) {
    return stages * W_BYTES + region_bytes + CROSS_BYTES + (int)sizeof(Shared) + 1024;
}

}  // namespace

extern "C" int lp_program_op_bytes() { return (int)sizeof(ProgramOp); }
extern "C" int lp_program_max_tokens() { return TOK; }

// Bytes of the shared-memory region a product unit of `k_blocks` k-blocks needs for its operand.
extern "C" int lp_program_operand_bytes(int k_blocks) { return k_blocks * X_KB_BYTES; }
// ... and an attention unit for heads of `hd`.
extern "C" int lp_program_attention_bytes(int hd) {
    return (hd == 64 ? 6 : 3) * 2 * PAGE * hd * 2 + 16 * hd * 2 + 2 * hd * 2 + 2 * 128 * 4;
}

// Fill one product operation at `op_host` (host memory, lp_program_op_bytes() bytes).
extern "C" int lp_program_product(void* op_host, const void* W, long long w_rows, int K, long long ldw, int features,
                                  int splits, int x_kind, const void* x, int ldx, const int* x_rows, const float* gain,
                                  float eps, int tokens, int epilogue, void* out, int ldc, float* clear,
                                  int clear_count) {
    if (tokens < 1 || tokens > TOK) LP_REFUSE("program: %d tokens in a step (1..%d)", tokens, TOK);
    if (K <= 0 || K % 8 || ldw % 8) LP_REFUSE("program: K = %d, row stride %lld (multiples of 8 wanted)", K, ldw);
    if ((uintptr_t)W % 16) LP_REFUSE("program: weights not 16-byte aligned");
    if (x_kind == LP_X_RMSNORM ? (ldx % 4 || (uintptr_t)x % 16 || (uintptr_t)gain % 16)
                               : (ldx % 8 || (uintptr_t)x % 16))
        LP_REFUSE("program: activation rows are not 16-byte aligned (stride %d)", ldx);
    const int k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
    if (splits < 1 || splits > k_blocks) LP_REFUSE("program: %d shares of %d k-blocks", splits, k_blocks);
    if (epilogue != LP_EPI_ADD && splits != 1) LP_REFUSE("program: only an adding product can share out K");
    if (epilogue == LP_EPI_SWIGLU && w_rows % 128) LP_REFUSE("program: interleaved gate/up rows %lld", w_rows);
    ProgramOp op;
    memset(&op, 0, sizeof(op));
    if (make_map(&op.map_w, W, w_rows, K, ldw, FEAT)) return -1;
    op.type = LP_OP_PRODUCT;
    ProductArgs& p = op.p;
    p.features = features;
    p.K = K; p.k_blocks = k_blocks; p.splits = splits;
    const int feat_tiles = (int)((w_rows + FEAT - 1) / FEAT);
    p.units = op.units = feat_tiles * splits;
    p.x_kind = x_kind; p.epilogue = epilogue; p.tokens = tokens;
    p.ldx = ldx; p.ldc = ldc; p.eps = eps;
    p.x = x; p.x_rows = x_rows; p.gain = gain; p.out = out;
    p.clear = clear; p.clear_count = clear_count;
    memcpy(op_host, &op, sizeof(op));
    return 0;
}

extern "C" int lp_program_attention(void* op_host, const float* qkv, int ld, const float* inv_freq, int rd,
                                    int interleaved, void* out, void* pages, int write_kv, const int* page_table,
                                    int pt_stride, const int* kv_len, float* partials, int* counters, int B, int H, int G,
                                    int hd, int page_size, float scale, int window, int pages_per_split, int num_splits) {
    if (page_size != PAGE) LP_REFUSE("program: pages of %d positions (64 wanted)", page_size);
    if (hd != 64 && hd != 128) LP_REFUSE("program: head size %d (64 or 128)", hd);
    if (H <= 0 || G <= 0 || H % G) LP_REFUSE("program: %d query heads over %d key/value heads", H, G);
    if (rd < 0 || rd > hd || rd % 2 || rd > 256) LP_REFUSE("program: rotary width %d for heads of %d", rd, hd);
    if (num_splits < 1 || pages_per_split < 1) LP_REFUSE("program: %d shares of %d pages", num_splits, pages_per_split);
    ProgramOp op;
    memset(&op, 0, sizeof(op));
    op.type = LP_OP_ATTENTION;
    AttentionOp& a = op.at;
    a.fused.qkv = qkv; a.fused.ld = ld; a.fused.inv_freq = inv_freq; a.fused.rd = rd; a.fused.interleaved = interleaved;
    a.fused.pages_rw = write_kv ? (__nv_bfloat16*)pages : nullptr;
    a.fused.counters = counters;
    a.pages = (const __nv_bfloat16*)pages; a.page_table = page_table; a.kv_len = kv_len;
    a.part_o = partials;
    a.part_ml = partials + (size_t)B * H * num_splits * hd;
    a.out = (__nv_bfloat16*)out;
    a.pt_stride = pt_stride; a.H = H; a.G = G; a.hd = hd; a.window = window;
    a.pages_per_split = pages_per_split; a.num_splits = num_splits;
    a.head_groups = (H / G + 15) / 16;
    a.batch = B;
    a.scale_log2 = scale * 1.4426950408889634f;
    op.units = num_splits * G * a.head_groups * B;
    memcpy(op_host, &op, sizeof(op));
    return 0;
}

// Embedding rows into the float32 residual stream, and the zeroes the program starts from.
extern "C" int lp_program_prologue(const void* table, int table_dtype, const int* tokens, float* x, int T, int d,
                                   int vocab, float* zero, int zero_count, unsigned* counter, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (table_dtype == LP_BF16)
        lp_launch(program_prologue_kernel<__nv_bfloat16>, T, 256, 0, stream, (const __nv_bfloat16*)table, tokens, x, d,
                  vocab, zero, zero_count, counter);
    else if (table_dtype == LP_F32)
        lp_launch(program_prologue_kernel<float>, T, 256, 0, stream, (const float*)table, tokens, x, d, vocab, zero,
                  zero_count, counter);
    else LP_REFUSE("program: embedding dtype code %d", table_dtype);
    return lp_check_launch("program prologue");
}

// Run `num_ops` operations (device memory, as filled above) with one CTA on each of `grid` SMs.
// `region_bytes`: the largest operand or attention scratch any unit needs.
// `timing` (optional, 4 * num_ops int64 in device memory): SM clock stamps of CTA 0 per operation: start, after
// the barrier, after its first operand was built, end.
extern "C" int lp_program_launch(const void* ops_device, int num_ops, int grid, int region_bytes, unsigned* counter,
                                 int* status, long long* timing, cudaStream_t stream) {
    if (num_ops <= 0) return 0;
    if ((uintptr_t)ops_device % 128) LP_REFUSE("program: the operation list is not 128-byte aligned");
    region_bytes = (region_bytes + 1023) / 1024 * 1024;
    static int max_smem = 0, num_sms = 0;
    if (!max_smem) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    }
    if (grid < 1 || grid > num_sms) LP_REFUSE("program: a grid of %d CTAs on %d SMs", grid, num_sms);
    int stages = (max_smem - shared_bytes(0, region_bytes)) / W_BYTES;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) LP_REFUSE("program: %d bytes of operand leave no room for a ring of weight tiles", region_bytes);
    const int bytes = shared_bytes(stages, region_bytes);
    static int granted = 0;
    if (bytes > granted) {
        cudaError_t e = cudaFuncSetAttribute(decode_program_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) LP_REFUSE("program: cannot reserve %d bytes of shared memory: %s", bytes, cudaGetErrorString(e));
        granted = bytes;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // all CTAs resident at once: they wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_program_kernel, (const ProgramOp*)ops_device, num_ops,
                                       (uint32_t*)counter, status, stages, region_bytes, timing);
    if (e != cudaSuccess) {
        snprintf(lp_error_text, sizeof(lp_error_text), "program launch: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}
