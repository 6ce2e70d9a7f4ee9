// A plain tiled matrix product on the FMA units: C[M, N] = A[M, K] . W[N, K]^T.
//
// This is the 32-bit path's product (no tensor cores, no reduced-precision mode) and
// the fallback for shapes the tensor-core kernel refuses.  Every output element is
// accumulated by one thread over k = 0 .. K-1 in ascending order, so a row's result
// does not depend on M, on the other rows, or on which tile it falls in.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TC>
__global__ void __launch_bounds__(256) gemm_plain_kernel(const TA* __restrict__ A, const TA* __restrict__ W,
                                                         TC* __restrict__ C, int M, int N, int K, int lda,
                                                         int ldw, int ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // each thread loads 4 elements of A and 4 of W per k-tile: row = tid / 4, k = (tid % 4) * 4 ..
    const int lrow = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + i][lrow] = (am < M && k < K) ? to_float(A[(size_t)am * lda + k]) : 0.f;
            Ws[lk + i][lrow] = (wn < N && k < K) ? to_float(W[(size_t)wn * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = from_float<TC>(acc[i][j]);
        }
    }
}
}  // namespace

// in_dtype: type of A and W; out_dtype: type of C (float logits from bfloat16 operands are allowed).
RMX_API int rmx_gemm_plain(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw,
                           int ldc, int in_dtype, int out_dtype, void* stream) {
    if (M == 0 || N == 0) return 0;
    RMX_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_plain: bad sizes M=%d N=%d K=%d", M, N, K);
    RMX_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_plain: leading dimensions too small");
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    RMX_REQUIRE(grid.y <= 65535, "gemm_plain: M=%d is beyond 65535 row tiles", M);
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == RMX_F32 && out_dtype == RMX_F32)
        gemm_plain_kernel<float, float><<<grid, 256, 0, s>>>((const float*)A, (const float*)W, (float*)C, M, N, K, lda, ldw, ldc);
    else if (in_dtype == RMX_BF16 && out_dtype == RMX_BF16)
        gemm_plain_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, s>>>(
            (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (__nv_bfloat16*)C, M, N, K, lda, ldw, ldc);
    else if (in_dtype == RMX_BF16 && out_dtype == RMX_F32)
        gemm_plain_kernel<__nv_bfloat16, float><<<grid, 256, 0, s>>>((const __nv_bfloat16*)A, (const __nv_bfloat16*)W,
                                                                  (float*)C, M, N, K, lda, ldw, ldc);
    else
        RMX_FAIL("gemm_plain: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
    RMX_CHECK_LAUNCH("gemm_plain");
    return 0;
}
