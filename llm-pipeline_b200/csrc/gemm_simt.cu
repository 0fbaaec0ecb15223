// C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) on the CUDA cores with float32 accumulation.
// This is the matrix product of the true 32-bit path (no tensor core, no reduced-precision
// mode) and accepts every size. Each output element adds its K products in ascending k, so a
// row's result does not depend on how many other rows are in the call.
#include "common.cuh"

#define GT_BM 64
#define GT_BN 64
#define GT_BK 16

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gemm_nt_kernel(const TI* __restrict__ A, const TI* __restrict__ W, const void* __restrict__ bias, int bias_bf16,
               TO* __restrict__ C, int M, int N, int K, long lda, long ldw, long ldc) {
    __shared__ float As[GT_BK][GT_BM + 4];
    __shared__ float Ws[GT_BK][GT_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * GT_BM, n0 = blockIdx.x * GT_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GT_BK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int e = tid + 256 * r;
            const int row = e >> 4, col = e & 15;
            const int k = k0 + col;
            const int m = m0 + row, n = n0 + row;
            As[col][row] = (m < M && k < K) ? to_float(A[(size_t)m * lda + k]) : 0.f;
            Ws[col][row] = (n < N && k < K) ? to_float(W[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GT_BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
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
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += load_as_float(bias, bias_bf16, n);
            C[(size_t)m * ldc + n] = from_float<TO>(v);
        }
    }
}

// in_dtype: type of A and W.  out_dtype: type of C (float32, or the input type).
LLMP_API int llmp_gemm_simt(const void* A, const void* W, const void* bias, int bias_dtype, void* C, int in_dtype,
                            int out_dtype, int M, int N, int K, long lda, long ldw, long ldc, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    LLMP_REQUIRE(K > 0, "gemm: bad K %d", K);
    LLMP_REQUIRE((M + GT_BM - 1) / GT_BM <= 65535, "gemm: too many rows %d", M);
    dim3 grid((N + GT_BN - 1) / GT_BN, (M + GT_BM - 1) / GT_BM);
    const int bb = bias_dtype == LLMP_BF16;
    if (in_dtype == LLMP_F32 && out_dtype == LLMP_F32)
        gemm_nt_kernel<float, float><<<grid, 256, 0, stream>>>((const float*)A, (const float*)W, bias, bb, (float*)C,
                                                               M, N, K, lda, ldw, ldc);
    else if (in_dtype == LLMP_BF16 && out_dtype == LLMP_BF16)
        gemm_nt_kernel<bf16, bf16><<<grid, 256, 0, stream>>>((const bf16*)A, (const bf16*)W, bias, bb, (bf16*)C, M, N,
                                                             K, lda, ldw, ldc);
    else if (in_dtype == LLMP_BF16 && out_dtype == LLMP_F32)
        gemm_nt_kernel<bf16, float><<<grid, 256, 0, stream>>>((const bf16*)A, (const bf16*)W, bias, bb, (float*)C, M,
                                                              N, K, lda, ldw, ldc);
    else {
        llmp_set_error("gemm: unsupported type combination in=%d out=%d", in_dtype, out_dtype);
        return 1;
    }
    return llmp_check_launch("gemm_simt");
}
