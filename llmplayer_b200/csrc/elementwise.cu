// Small memory-bound kernels of the step: embedding rows, RMS norm, and the
// rotation of queries and keys together with the write of keys and values into
// the paged cache. All arithmetic is float32; only loads and stores convert.
//
// Counterparts in the reference (src/main/resources/kernels/cuda/): rmsnorm.cu:6-46,
// rope.cu:11-52, attention.cu:114-128 (kv_cache_update); the embedding row is
// gathered on the host there (inference/InferenceEngine.java:199-201).
#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int d) {
    lp_grid_release();
    lp_grid_wait();
    const int t = blockIdx.x;
    const long long row = tokens[t];
    const TW* src = table + row * d;
    float* dst = out + (long long)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = lp_to_float(src[i]);
}

extern "C" int lp_embed(const void* table, int table_dtype, const int* tokens, float* out, int T, int d,
                        cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0) LP_REFUSE("embed: width %d", d);
    const int threads = d >= 1024 ? 256 : 128;
    // the embedding opens a step: it is launched without the early start (see lp_launch_first)
    if (table_dtype == LP_F32)
        lp_launch_first(embed_kernel<float>, T, threads, 0, stream, (const float*)table, tokens, out, d);
    else if (table_dtype == LP_BF16)
        lp_launch_first(embed_kernel<__nv_bfloat16>, T, threads, 0, stream, (const __nv_bfloat16*)table, tokens, out, d);
    else
        LP_REFUSE("embed: table dtype code %d", table_dtype);
    return lp_check_launch("embed");
}

// ---------------------------------------------------------------- RMS norm
// out[r, i] = x[row(r), i] * (1 / sqrt(sum_i x^2 / d + eps)) * w[i]; one block per row.
// When `add` is given, x[row] += add[row] first (in float32) and the sum is stored back:
// the residual sum and the norm that follows it in one pass. The row is read once and kept
// in registers (up to PER * 256 values; wider rows take the two-pass kernel below).
// `zero` (optional): a float32 buffer that the blocks clear on the side, for the product that
// follows the norm and sums its partial results with atomics.
constexpr int NORM_THREADS = 256;
constexpr int NORM_PER = 16;

__device__ __forceinline__ void clear_on_the_side(float* zero, long long zero_count) {
    if (zero) {
        const long long stride = (long long)gridDim.x * blockDim.x;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < zero_count; i += stride) zero[i] = 0.f;
    }
}

template <typename TOut, typename TAdd>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_kernel(float* __restrict__ x, const TAdd* __restrict__ add, const int* __restrict__ rows,
               const float* __restrict__ w, TOut* __restrict__ out, int d, float eps, float* __restrict__ zero,
               long long zero_count) {
    __shared__ float scratch[32];
    lp_grid_release();
    lp_grid_wait();
    const int r = blockIdx.x;
    const long long src = rows ? rows[r] : r;
    float* xr = x + src * d;
    float v[NORM_PER];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_PER; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        v[k] = 0.f;
        if (i < d) {
            float t = xr[i];
            if (add) { t += lp_to_float(add[src * d + i]); xr[i] = t; }
            v[k] = t;
            ss += t * t;
        }
    }
    clear_on_the_side(zero, zero_count);
    ss = lp_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    TOut* o = out + (long long)r * d;
#pragma unroll
    for (int k = 0; k < NORM_PER; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < d) o[i] = lp_from_float<TOut>(v[k] * scale * w[i]);
    }
}

// The same for rows of a multiple of 4 values without a residual add: four values per load and store.
constexpr int NORM_VEC_PER = 4;          // float4 per thread: rows up to 256 * 4 * 4 = 4096 values
template <typename TOut>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_vec4_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                    TOut* __restrict__ out, int d, float eps, float* __restrict__ zero, long long zero_count) {
    __shared__ float scratch[32];
    lp_grid_release();
    lp_grid_wait();
    const int r = blockIdx.x;
    const long long src = rows ? rows[r] : r;
    const float4* xr = reinterpret_cast<const float4*>(x + src * d);
    const int quads = d >> 2;
    float4 v[NORM_VEC_PER];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_VEC_PER; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < quads) v[k] = xr[i];
    }
#pragma unroll
    for (int k = 0; k < NORM_VEC_PER; ++k) ss += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    clear_on_the_side(zero, zero_count);
    ss = lp_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    const float4* wq = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int k = 0; k < NORM_VEC_PER; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < quads) {
            const float4 g = wq[i];
            const float a = v[k].x * scale * g.x, b = v[k].y * scale * g.y, c = v[k].z * scale * g.z, e = v[k].w * scale * g.w;
            if (sizeof(TOut) == 2) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, e);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t*>(&lo);
                packed.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>(out + (long long)r * d)[i] = packed;
            } else {
                reinterpret_cast<float4*>(out + (long long)r * d)[i] = make_float4(a, b, c, e);
            }
        }
    }
}

template <typename TOut, typename TAdd>
__global__ void rmsnorm_wide_kernel(float* __restrict__ x, const TAdd* __restrict__ add,
                                    const int* __restrict__ rows, const float* __restrict__ w,
                                    TOut* __restrict__ out, int d, float eps, float* __restrict__ zero,
                                    long long zero_count) {
    __shared__ float scratch[32];
    lp_grid_release();
    lp_grid_wait();
    const int r = blockIdx.x;
    const long long src = rows ? rows[r] : r;
    float* xr = x + src * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float t = xr[i];
        if (add) { t += lp_to_float(add[src * d + i]); xr[i] = t; }
        ss += t * t;
    }
    clear_on_the_side(zero, zero_count);
    ss = lp_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    TOut* o = out + (long long)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = lp_from_float<TOut>(xr[i] * scale * w[i]);
}

extern "C" int lp_rmsnorm(float* x, const void* add, int add_dtype, const int* rows, const float* w, void* out,
                          int out_dtype, int R, int d, float eps, float* zero, long long zero_count,
                          cudaStream_t stream) {
    if (R <= 0) return 0;
    if (d <= 0) LP_REFUSE("rmsnorm: width %d", d);
    if (add && rows) LP_REFUSE("rmsnorm: a fused residual add cannot be combined with a row selection");
    const bool wide = d > NORM_THREADS * NORM_PER;
    if (!add && d % 4 == 0 && d <= NORM_THREADS * 4 * NORM_VEC_PER &&
        ((((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0)) {
        if (out_dtype == LP_BF16)
            lp_launch(rmsnorm_vec4_kernel<__nv_bfloat16>, R, NORM_THREADS, 0, stream, (const float*)x, rows, w,
                      (__nv_bfloat16*)out, d, eps, zero, zero_count);
        else if (out_dtype == LP_F32)
            lp_launch(rmsnorm_vec4_kernel<float>, R, NORM_THREADS, 0, stream, (const float*)x, rows, w, (float*)out, d,
                      eps, zero, zero_count);
        else LP_REFUSE("rmsnorm: dtype code out=%d", out_dtype);
        return lp_check_launch("rmsnorm");
    }
#define LP_LAUNCH_NORM(TOUT, TADD)                                                                              \
    do {                                                                                                        \
        if (wide)                                                                                               \
            lp_launch(rmsnorm_wide_kernel<TOUT, TADD>, R, 512, 0, stream, x, (const TADD*)add, rows, w,          \
                      (TOUT*)out, d, eps, zero, zero_count);                                                    \
        else                                                                                                    \
            lp_launch(rmsnorm_kernel<TOUT, TADD>, R, NORM_THREADS, 0, stream, x, (const TADD*)add, rows, w,      \
                      (TOUT*)out, d, eps, zero, zero_count);                                                    \
    } while (0)
    if (out_dtype == LP_F32 && add_dtype == LP_F32) LP_LAUNCH_NORM(float, float);
    else if (out_dtype == LP_F32 && add_dtype == LP_BF16) LP_LAUNCH_NORM(float, __nv_bfloat16);
    else if (out_dtype == LP_BF16 && add_dtype == LP_F32) LP_LAUNCH_NORM(__nv_bfloat16, float);
    else if (out_dtype == LP_BF16 && add_dtype == LP_BF16) LP_LAUNCH_NORM(__nv_bfloat16, __nv_bfloat16);
    else LP_REFUSE("rmsnorm: dtype codes out=%d add=%d", out_dtype, add_dtype);
#undef LP_LAUNCH_NORM
    return lp_check_launch("rmsnorm");
}

// ---------------------------------------------------------------- rotation + cache write
// One block per token of the fused projection output
//   qkv[t] = [ H query heads | G key heads | G value heads ] x head_dim   (float32).
// Queries and keys: the first `rd` features of a head are rotated by
// angle = float(position) * inv_freq[pair] (cosine and sine are formed once per token and
// shared by all its heads); the rest pass through. Queries go to q_out[t, h, :]; keys and
// values go to the page of the token's sequence that holds its position:
//   pages[page][0|1][g][position % page_size][:].
template <typename TQ, typename TKV>
__global__ void __launch_bounds__(256)
rope_cache_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ inv_freq,
                  const int* __restrict__ positions, const int* __restrict__ seq_ids,
                  const int* __restrict__ page_table, int pt_stride, TQ* __restrict__ q_out,
                  TKV* __restrict__ pages, int H, int G, int hd, int rd, int interleaved, int page_size,
                  int heads_per_block) {
    __shared__ float cs[128], sn[128];          // rd / 2 <= 128
    lp_grid_release();
    lp_grid_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rd >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float angle = (float)pos * inv_freq[i];
        sincosf(angle, &sn[i], &cs[i]);
    }
    __syncthreads();
    const float* src = qkv + (long long)t * ld;
    const int heads = pages ? H + 2 * G : H;
    long long page_base = 0;
    if (pages) {
        const int page = page_table[(long long)seq_ids[t] * pt_stride + pos / page_size];
        page_base = (long long)page * 2 * G * page_size * hd + (long long)(pos % page_size) * hd;
    }
    const int head_begin = blockIdx.y * heads_per_block;
    const int head_end = min(heads, head_begin + heads_per_block);
    // A warp takes whole heads. Rotated heads go pair by pair (each value is read once, both results of a
    // pair are written by the lane that read them); several heads are in flight per lane.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int rot_end = min(head_end, pages ? H + G : H);          // queries and keys are rotated, values are not
    auto dest = [&](int head, int e) -> long long {
        if (head < H) return ((long long)t * H + head) * hd + e;
        const bool is_v = head >= H + G;
        const int g = is_v ? head - H - G : head - H;
        return page_base + ((long long)(is_v ? G : 0) + g) * page_size * hd + e;
    };
    for (int p = lane; p < half; p += 32) {
        const int a = interleaved ? 2 * p : p, b = interleaved ? 2 * p + 1 : p + half;
        const float c = cs[p], sv = sn[p];
#pragma unroll 4
        for (int head = head_begin + warp; head < rot_end; head += nwarps) {
            const float* hsrc = src + (long long)head * hd;
            const float xa = hsrc[a], xb = hsrc[b];
            // products and sums rounded one by one (no contraction into FMAs): the same bits as the kernel in fours
            const float ra = __fsub_rn(__fmul_rn(xa, c), __fmul_rn(xb, sv)), rb = __fadd_rn(__fmul_rn(xa, sv), __fmul_rn(xb, c));
            if (head < H) {
                q_out[dest(head, a)] = lp_from_float<TQ>(ra);
                q_out[dest(head, b)] = lp_from_float<TQ>(rb);
            } else {
                pages[dest(head, a)] = lp_from_float<TKV>(ra);
                pages[dest(head, b)] = lp_from_float<TKV>(rb);
            }
        }
    }
    // what lies beyond the rotary width passes through
    for (int e = rd + lane; e < hd; e += 32) {
#pragma unroll 4
        for (int head = head_begin + warp; head < rot_end; head += nwarps) {
            const float val = src[(long long)head * hd + e];
            if (head < H) q_out[dest(head, e)] = lp_from_float<TQ>(val);
            else pages[dest(head, e)] = lp_from_float<TKV>(val);
        }
    }
    // values
    const int v_first = max(head_begin, H + G);
    for (int head = v_first + warp; head < head_end; head += nwarps) {
#pragma unroll 4
        for (int e = lane; e < hd; e += 32) pages[dest(head, e)] = lp_from_float<TKV>(src[(long long)head * hd + e]);
    }
}

// The common case in fours: split-half pairs over the whole head (rd == hd, hd a multiple of 8). An item is four
// neighbouring pairs of one head: two float4 loads, one float4 of cosines and of sines, two stores of four values.
template <typename T> __device__ __forceinline__ void store4(T* dst, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* dst, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = packed;
}

template <typename TQ, typename TKV>
__global__ void __launch_bounds__(256)
rope_cache_vec_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ inv_freq,
                      const int* __restrict__ positions, const int* __restrict__ seq_ids,
                      const int* __restrict__ page_table, int pt_stride, TQ* __restrict__ q_out,
                      TKV* __restrict__ pages, int H, int G, int hd, int page_size) {
    __shared__ __align__(16) float cs[128], sn[128];
    lp_grid_release();
    lp_grid_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = hd >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sn[i], &cs[i]);
    __syncthreads();
    const float* src = qkv + (long long)t * ld;
    long long page_base = 0;
    if (pages) {
        const int page = page_table[(long long)seq_ids[t] * pt_stride + pos / page_size];
        page_base = (long long)page * 2 * G * page_size * hd + (long long)(pos % page_size) * hd;
    }
    const int qph = half >> 2;                                   // items per rotated head
    const int rot_heads = pages ? H + G : H;
    for (int it = threadIdx.x; it < rot_heads * qph; it += blockDim.x) {
        const int head = it / qph, a = (it - head * qph) * 4;
        const float* hsrc = src + (long long)head * hd;
        const float4 xa = *reinterpret_cast<const float4*>(hsrc + a);
        const float4 xb = *reinterpret_cast<const float4*>(hsrc + a + half);
        const float4 c = *reinterpret_cast<const float4*>(cs + a);
        const float4 sv = *reinterpret_cast<const float4*>(sn + a);
        // products and sums rounded one by one (no contraction into FMAs): the same bits as the kernel above,
        // whichever of the two a step's size selects
#define LP_ROT_A(u) __fsub_rn(__fmul_rn(xa.u, c.u), __fmul_rn(xb.u, sv.u))
#define LP_ROT_B(u) __fadd_rn(__fmul_rn(xa.u, sv.u), __fmul_rn(xb.u, c.u))
        const float ra0 = LP_ROT_A(x), ra1 = LP_ROT_A(y), ra2 = LP_ROT_A(z), ra3 = LP_ROT_A(w);
        const float rb0 = LP_ROT_B(x), rb1 = LP_ROT_B(y), rb2 = LP_ROT_B(z), rb3 = LP_ROT_B(w);
#undef LP_ROT_A
#undef LP_ROT_B
        if (head < H) {
            TQ* dst = q_out + ((long long)t * H + head) * hd + a;
            store4<TQ>(dst, ra0, ra1, ra2, ra3);
            store4<TQ>(dst + half, rb0, rb1, rb2, rb3);
        } else {
            TKV* dst = pages + page_base + (long long)(head - H) * page_size * hd + a;
            store4<TKV>(dst, ra0, ra1, ra2, ra3);
            store4<TKV>(dst + half, rb0, rb1, rb2, rb3);
        }
    }
    if (pages) {                                                 // values: copied as they are
        const int per = hd >> 2;
        for (int it = threadIdx.x; it < G * per; it += blockDim.x) {
            const int g = it / per, e = (it - g * per) * 4;
            const float4 v = *reinterpret_cast<const float4*>(src + (long long)(H + G + g) * hd + e);
            store4<TKV>(pages + page_base + ((long long)G + g) * page_size * hd + e, v.x, v.y, v.z, v.w);
        }
    }
}

extern "C" int lp_rope_cache_write(const float* qkv, int ld, const float* inv_freq, const int* positions,
                                   const int* seq_ids, const int* page_table, int pt_stride, void* q_out,
                                   int q_dtype, void* pages, int kv_dtype, int T, int H, int G, int hd, int rd,
                                   int interleaved, int page_size, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || H <= 0 || G < 0) LP_REFUSE("rope_cache_write: heads %d/%d of %d", H, G, hd);
    if (rd < 0 || rd > hd || (rd & 1)) LP_REFUSE("rope_cache_write: rotary width %d of a head of %d", rd, hd);
    if (rd > 256) LP_REFUSE("rope_cache_write: rotary width %d (supported: up to 256)", rd);
    if (rd > 0 && !inv_freq) LP_REFUSE("rope_cache_write: rotation without frequencies");
    const int heads = pages ? H + 2 * G : H;
    if (ld < heads * hd) LP_REFUSE("rope_cache_write: row of %d values for %d heads of %d", ld, heads, hd);
    if (pages && page_size <= 0) LP_REFUSE("rope_cache_write: page size %d", page_size);
    // many tokens, split-half pairs over whole heads of a multiple of 8, everything 16-byte aligned: in fours
    if (T >= 256 && !interleaved && rd == hd && hd % 8 == 0 && ld % 4 == 0 &&
        ((((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)pages) & 15) == 0)) {
#define LP_LAUNCH_ROPE_VEC(TQ, TKV)                                                                         \
    lp_launch(rope_cache_vec_kernel<TQ, TKV>, T, 256, 0, stream, qkv, ld, inv_freq, positions, seq_ids,      \
              page_table, pt_stride, (TQ*)q_out, (TKV*)pages, H, G, hd, page_size)
        if (q_dtype == LP_F32 && kv_dtype == LP_F32) LP_LAUNCH_ROPE_VEC(float, float);
        else if (q_dtype == LP_BF16 && kv_dtype == LP_BF16) LP_LAUNCH_ROPE_VEC(__nv_bfloat16, __nv_bfloat16);
        else if (q_dtype == LP_F32 && kv_dtype == LP_BF16) LP_LAUNCH_ROPE_VEC(float, __nv_bfloat16);
        else if (q_dtype == LP_BF16 && kv_dtype == LP_F32) LP_LAUNCH_ROPE_VEC(__nv_bfloat16, float);
        else LP_REFUSE("rope_cache_write: dtype codes q=%d kv=%d", q_dtype, kv_dtype);
#undef LP_LAUNCH_ROPE_VEC
        return lp_check_launch("rope_cache_write");
    }
    // many tokens: one block per token takes all its heads; few tokens: the heads are shared out
    int heads_per_block = heads;
    if (T < 256) {
        heads_per_block = (512 + hd - 1) / hd;
        if (heads_per_block < 1) heads_per_block = 1;
        if (heads_per_block > heads) heads_per_block = heads;
    }
    const int parts = (heads + heads_per_block - 1) / heads_per_block;
    const int threads = heads_per_block * hd >= 1024 ? 256 : 128;
    dim3 grid(T, parts);
#define LP_LAUNCH_ROPE(TQ, TKV)                                                                          \
    lp_launch(rope_cache_kernel<TQ, TKV>, grid, threads, 0, stream, qkv, ld, inv_freq, positions, seq_ids, \
              page_table, pt_stride, (TQ*)q_out, (TKV*)pages, H, G, hd, rd, interleaved, page_size,       \
              heads_per_block)
    if (q_dtype == LP_F32 && kv_dtype == LP_F32) LP_LAUNCH_ROPE(float, float);
    else if (q_dtype == LP_BF16 && kv_dtype == LP_BF16) LP_LAUNCH_ROPE(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == LP_F32 && kv_dtype == LP_BF16) LP_LAUNCH_ROPE(float, __nv_bfloat16);
    else if (q_dtype == LP_BF16 && kv_dtype == LP_F32) LP_LAUNCH_ROPE(__nv_bfloat16, float);
    else LP_REFUSE("rope_cache_write: dtype codes q=%d kv=%d", q_dtype, kv_dtype);
#undef LP_LAUNCH_ROPE
    return lp_check_launch("rope_cache_write");
}

// ---------------------------------------------------------------- rotation angles of a step's tokens
// out[t][i] = (cos, sin) of float(positions[t]) * inv_freq[i]: the same float32 product and the same sincosf as
// the rotation kernels above, formed once per step for a product whose epilogue rotates (gemm_tcgen05.cu).
__global__ void __launch_bounds__(128)
rope_angles_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, float2* __restrict__ out,
                   int T, int half) {
    lp_grid_release();
    lp_grid_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)T * half) return;
    const int t = (int)(i / half), p = (int)(i - (long long)t * half);
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[p], &sn, &cs);
    out[i] = make_float2(cs, sn);
}

extern "C" int lp_rope_angles(const int* positions, const float* inv_freq, float* out, int T, int half,
                              cudaStream_t stream) {
    if (T <= 0 || half <= 0) return 0;
    const long long n = (long long)T * half;
    lp_launch(rope_angles_kernel, (unsigned)((n + 127) / 128), 128, 0, stream, positions, inv_freq, (float2*)out, T, half);
    return lp_check_launch("rope_angles");
}

// ---------------------------------------------------------------- advancing a decoding batch on the device
// After a decode step whose sampler left one token per sequence: that token becomes the next
// step's input, and every sequence moves on by one position. Lets decode steps follow one
// another without the host (the reference keeps position and length on the device for the
// same reason: java21 inference/CudaForwardPass.java:138-141).
__global__ void advance_kernel(int* __restrict__ tokens, int* __restrict__ positions, int* __restrict__ kv_len,
                               const int* __restrict__ sampled, int B) {
    lp_grid_release();
    lp_grid_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < B) {
        tokens[i] = sampled[i];
        positions[i] += 1;
        kv_len[i] += 1;
    }
}

extern "C" int lp_advance(int* tokens, int* positions, int* kv_len, const int* sampled, int B, cudaStream_t stream) {
    if (B <= 0) return 0;
    lp_launch(advance_kernel, (B + 127) / 128, 128, 0, stream, tokens, positions, kv_len, sampled, B);
    return lp_check_launch("advance");
}
