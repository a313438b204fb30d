// Plain matrix product for weights stored [out, in]:  C[M, N] = A[M, K] * W[N, K]^T.
// No tensor cores, float32 multiply-add only, and each output element sums its K
// products in increasing k whatever M is, so a row's result does not depend on
// which other rows share the launch. It is the product of the float32 path and
// the comparison twin of the tensor-core kernels.
//
// Counterparts in the reference (src/main/resources/kernels/cuda/): matmul_f32.cu:6-39,
// matmul_bf16.cu:6-37 (one warp per output row, one input vector), silu_mul.cu:6-15,
// and the add-to-output mode the reference uses for the residual
// (java21 inference/CudaForwardPass.java:1012-1017).
#include "common.cuh"

#define LP_GEMM_STORE 0      // C = A W^T
#define LP_GEMM_ACCUMULATE 1 // C += A W^T         (C float32: the residual stream)
#define LP_GEMM_SWIGLU 2     // C = silu(A Wg^T) * (A Wu^T), W = [gate rows | up rows], N = rows of each

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW, typename TC, int MODE>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C, int M, int N, int K,
                  int lda, int ldw, int ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ float Us[MODE == LP_GEMM_SWIGLU ? BK : 1][BN + 4];

    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

    float acc[TM][TN];
    float acu[MODE == LP_GEMM_SWIGLU ? TM : 1][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            acc[i][j] = 0.f;
            if (MODE == LP_GEMM_SWIGLU) acu[i][j] = 0.f;
        }

    // each thread loads 4 elements of each 64x16 tile: row = tid / 4, k = (tid % 4) * 4 .. +3
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int am = m0 + lr, wn = n0 + lr;
            As[lk + j][lr] = (am < M && k < K) ? lp_to_float(A[(long long)am * lda + k]) : 0.f;
            Ws[lk + j][lr] = (wn < N && k < K) ? lp_to_float(W[(long long)wn * ldw + k]) : 0.f;
            if (MODE == LP_GEMM_SWIGLU)
                Us[lk + j][lr] = (wn < N && k < K) ? lp_to_float(W[(long long)(wn + N) * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], w[TN], u[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                w[j] = Ws[k][tx * TN + j];
                if (MODE == LP_GEMM_SWIGLU) u[j] = Us[k][tx * TN + j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
                    if (MODE == LP_GEMM_SWIGLU) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
                }
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            TC* c = C + (long long)m * ldc + n;
            if (MODE == LP_GEMM_STORE) {
                *c = lp_from_float<TC>(acc[i][j]);
            } else if (MODE == LP_GEMM_ACCUMULATE) {
                *c = lp_from_float<TC>(lp_to_float(*c) + acc[i][j]);
            } else {
                const float g = acc[i][j];
                *c = lp_from_float<TC>(g / (1.0f + expf(-g)) * acu[i][j]);
            }
        }
    }
}

template <typename TA, typename TW, typename TC>
int launch_mode(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc, int mode,
                cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (mode == LP_GEMM_STORE)
        gemm_plain_kernel<TA, TW, TC, LP_GEMM_STORE><<<grid, 256, 0, stream>>>(
            (const TA*)A, (const TW*)W, (TC*)C, M, N, K, lda, ldw, ldc);
    else if (mode == LP_GEMM_ACCUMULATE)
        gemm_plain_kernel<TA, TW, TC, LP_GEMM_ACCUMULATE><<<grid, 256, 0, stream>>>(
            (const TA*)A, (const TW*)W, (TC*)C, M, N, K, lda, ldw, ldc);
    else
        gemm_plain_kernel<TA, TW, TC, LP_GEMM_SWIGLU><<<grid, 256, 0, stream>>>(
            (const TA*)A, (const TW*)W, (TC*)C, M, N, K, lda, ldw, ldc);
    return lp_check_launch("gemm_plain");
}

template <typename TA, typename TW>
int launch_out(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int lda, int ldw, int ldc,
               int mode, cudaStream_t stream) {
    if (c_dtype == LP_F32) return launch_mode<TA, TW, float>(A, W, C, M, N, K, lda, ldw, ldc, mode, stream);
    return launch_mode<TA, TW, __nv_bfloat16>(A, W, C, M, N, K, lda, ldw, ldc, mode, stream);
}

}  // namespace

// A: [M, K] row stride lda; W: [N, K] (or [2N, K] in SWIGLU mode) row stride ldw; C: [M, N] row stride ldc.
extern "C" int lp_gemm_plain(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype, int M,
                             int N, int K, int lda, int ldw, int ldc, int mode, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) LP_REFUSE("gemm_plain: inner size %d", K);
    if (mode < 0 || mode > 2) LP_REFUSE("gemm_plain: mode %d", mode);
    if (c_dtype != LP_F32 && c_dtype != LP_BF16) LP_REFUSE("gemm_plain: output dtype code %d", c_dtype);
    if (mode == LP_GEMM_ACCUMULATE && c_dtype != LP_F32)
        LP_REFUSE("gemm_plain: accumulation needs a float32 output");
    if ((N + BN - 1) / BN > 2147483647 || (M + BM - 1) / BM > 65535)
        LP_REFUSE("gemm_plain: %d rows exceed the grid", M);
    if (a_dtype == LP_F32 && w_dtype == LP_F32)
        return launch_out<float, float>(A, W, C, c_dtype, M, N, K, lda, ldw, ldc, mode, stream);
    if (a_dtype == LP_BF16 && w_dtype == LP_BF16)
        return launch_out<__nv_bfloat16, __nv_bfloat16>(A, W, C, c_dtype, M, N, K, lda, ldw, ldc, mode, stream);
    if (a_dtype == LP_BF16 && w_dtype == LP_F32)
        return launch_out<__nv_bfloat16, float>(A, W, C, c_dtype, M, N, K, lda, ldw, ldc, mode, stream);
    if (a_dtype == LP_F32 && w_dtype == LP_BF16)
        return launch_out<float, __nv_bfloat16>(A, W, C, c_dtype, M, N, K, lda, ldw, ldc, mode, stream);
    LP_REFUSE("gemm_plain: dtype codes a=%d w=%d", a_dtype, w_dtype);
}
