// Y[M, N] = X[M, K] * W[N, K]^T for few rows of X (M <= 64): the matrix products of a decode step.
//
// The product is bound by reading W once from HBM, so the kernel is built as a stream: a block owns
// ROWS rows of W and walks K in chunks; every chunk of W (and the matching chunk of X) travels to
// shared memory as 16-byte cp.async copies through a ring of STAGES buffers, so several chunks are
// in flight per block while the tensor cores (mma.sync m16n8k16, bf16 in, float32 accumulate) work
// on the oldest one. The MMA tile has the rows of W on its 16-row side and the rows of X on its
// 8-column side, so no tensor-core work is wasted on padding M. The four warps of a block split
// each chunk along K; their partial sums are added in warp order 0..3 in shared memory, so the
// result does not depend on timing, and a row of X gives the same result whatever else is in X.
#include "common.cuh"

#define SK_THREADS 128
#define SK_WARPS 4
#define SK_STAGES 4
#define SK_PAD 8             // bf16 elements of padding per shared-memory row (16 bytes)

__device__ __forceinline__ void sk_cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void sk_ldmatrix_x4(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void sk_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ROWS: rows of W per block (16 or 32). NT: 8-row tiles of X (M <= 8 * NT). KC: K elements per chunk.
template <int ROWS, int NT, int KC, typename TO>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, TO* __restrict__ Y, int M, int N, int K,
                   long ldx, long ldw, long ldy) {
    extern __shared__ __align__(16) unsigned char sk_smem[];
    constexpr int STRIDE = KC + SK_PAD;                  // elements per shared-memory row
    constexpr int MT = ROWS / 16;                        // 16-row MMA tiles of W
    constexpr int XROWS = NT * 8;
    constexpr int STAGE_ELEMS = (ROWS + XROWS) * STRIDE;
    constexpr int CPR = KC / 8;                          // 16-byte chunks per row
    constexpr int ROWS_PER_PASS = SK_THREADS / CPR;
    bf16* ring = reinterpret_cast<bf16*>(sk_smem);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * ROWS;
    const int chunks = (K + KC - 1) / KC;
    const int cc = (tid % CPR) * 8;                      // this thread's column inside a chunk
    const int r0 = tid / CPR;

    auto issue = [&](int chunk, int stage) {
        bf16* Ws = ring + (size_t)stage * STAGE_ELEMS;
        bf16* Xs = Ws + ROWS * STRIDE;
        const int k = chunk * KC + cc;
        const bool kin = k < K;
#pragma unroll
        for (int row = r0; row < ROWS; row += ROWS_PER_PASS) {
            const bool ok = kin && (n0 + row) < N;
            sk_cp_async_16(Ws + row * STRIDE + cc, ok ? W + (size_t)(n0 + row) * ldw + k : W, ok);
        }
#pragma unroll
        for (int row = r0; row < XROWS; row += ROWS_PER_PASS) {
            const bool ok = kin && row < M;
            sk_cp_async_16(Xs + row * STRIDE + cc, ok ? X + (size_t)row * ldx + k : X, ok);
        }
    };

    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

#pragma unroll
    for (int s = 0; s < SK_STAGES - 1; ++s) {
        if (s < chunks) issue(s, s);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    constexpr int KW = KC / SK_WARPS;                    // this warp's share of a chunk along K
    for (int chunk = 0; chunk < chunks; ++chunk) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(SK_STAGES - 2) : "memory");
        __syncthreads();                                 // chunk has landed for all threads; the oldest buffer is free
        {
            const int next = chunk + SK_STAGES - 1;
            if (next < chunks) issue(next, next % SK_STAGES);
            asm volatile("cp.async.commit_group;\n" ::: "memory");
        }
        const bf16* Ws = ring + (size_t)(chunk % SK_STAGES) * STAGE_ELEMS;
        const bf16* Xs = Ws + ROWS * STRIDE;
#pragma unroll
        for (int ks = 0; ks < KW / 16; ++ks) {
            const int kk = warp * KW + ks * 16;
            unsigned a[MT][4];
#pragma unroll
            for (int i = 0; i < MT; ++i)
                sk_ldmatrix_x4(a[i], Ws + (size_t)(i * 16 + (lane & 15)) * STRIDE + kk + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const bf16* xrow = Xs + (size_t)(j * 8 + g) * STRIDE + kk + 2 * t;
                const unsigned b0 = *reinterpret_cast<const unsigned*>(xrow);
                const unsigned b1 = *reinterpret_cast<const unsigned*>(xrow + 8);
#pragma unroll
                for (int i = 0; i < MT; ++i) sk_mma(acc[i][j], a[i], b0, b1);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();                                     // the ring is free: reuse it for the warps' partial sums

    // partial[warp][x row][w row]; acc[i][j] holds W rows i*16 + g (+8), X rows j*8 + 2t (+1)
    float* part = reinterpret_cast<float*>(sk_smem);
    constexpr int PSTRIDE = ROWS + 1;
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            float* base = part + ((size_t)warp * XROWS + j * 8 + 2 * t) * PSTRIDE + i * 16 + g;
            base[0] = acc[i][j][0];
            base[PSTRIDE] = acc[i][j][1];
            base[8] = acc[i][j][2];
            base[PSTRIDE + 8] = acc[i][j][3];
        }
    __syncthreads();
    for (int e = tid; e < XROWS * ROWS; e += SK_THREADS) {
        const int m = e / ROWS, row = e % ROWS;
        if (m < M && n0 + row < N) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < SK_WARPS; ++w) v += part[((size_t)w * XROWS + m) * PSTRIDE + row];
            Y[(size_t)m * ldy + n0 + row] = from_float<TO>(v);
        }
    }
}

template <int ROWS, int NT, int KC, typename TO>
static int launch_skinny(const bf16* X, const bf16* W, TO* Y, int M, int N, int K, long ldx, long ldw, long ldy,
                         cudaStream_t stream) {
    constexpr size_t ring = (size_t)SK_STAGES * (ROWS + NT * 8) * (KC + SK_PAD) * sizeof(bf16);
    constexpr size_t part = (size_t)SK_WARPS * NT * 8 * (ROWS + 1) * sizeof(float);
    constexpr size_t smem = ring > part ? ring : part;
    auto kernel = gemm_skinny_kernel<ROWS, NT, KC, TO>;
    LLMP_ALLOW_SMEM(kernel, smem);
    kernel<<<(N + ROWS - 1) / ROWS, SK_THREADS, smem, stream>>>(X, W, Y, M, N, K, ldx, ldw, ldy);
    return llmp_check_launch("gemm_skinny");
}

template <typename TO>
static int dispatch_skinny(const bf16* X, const bf16* W, TO* Y, int M, int N, int K, long ldx, long ldw, long ldy,
                           cudaStream_t stream) {
    // 32 rows of W per block where that still gives every SM a block; 16 rows for narrow outputs
    const bool wide = N >= 32 * 120;
    if (M <= 8)
        return wide ? launch_skinny<32, 1, 256, TO>(X, W, Y, M, N, K, ldx, ldw, ldy, stream)
                    : launch_skinny<16, 1, 256, TO>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
    if (M <= 16)
        return wide ? launch_skinny<32, 2, 256, TO>(X, W, Y, M, N, K, ldx, ldw, ldy, stream)
                    : launch_skinny<16, 2, 256, TO>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
    if (M <= 32)
        return wide ? launch_skinny<32, 4, 128, TO>(X, W, Y, M, N, K, ldx, ldw, ldy, stream)
                    : launch_skinny<16, 4, 128, TO>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
    return wide ? launch_skinny<32, 8, 128, TO>(X, W, Y, M, N, K, ldx, ldw, ldy, stream)
                : launch_skinny<16, 8, 128, TO>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
}

// X and W bfloat16, rows 16-byte aligned (K, ldx, ldw multiples of 8); out_dtype bfloat16 or float32; M <= 64.
LLMP_API int llmp_gemm_skinny(const void* X, const void* W, void* Y, int out_dtype, int M, int N, int K, long ldx,
                              long ldw, long ldy, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    LLMP_REQUIRE(M <= 64, "gemm_skinny: %d rows, at most 64 are taken", M);
    LLMP_REQUIRE(K > 0 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0,
                 "gemm_skinny: K=%d and the row strides (%ld, %ld) must be multiples of 8", K, ldx, ldw);
    LLMP_REQUIRE(((size_t)X % 16) == 0 && ((size_t)W % 16) == 0, "gemm_skinny: operands must be 16-byte aligned");
    if (out_dtype == LLMP_F32)
        return dispatch_skinny<float>((const bf16*)X, (const bf16*)W, (float*)Y, M, N, K, ldx, ldw, ldy, stream);
    return dispatch_skinny<bf16>((const bf16*)X, (const bf16*)W, (bf16*)Y, M, N, K, ldx, ldw, ldy, stream);
}
