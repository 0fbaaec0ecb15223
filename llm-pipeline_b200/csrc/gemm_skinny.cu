// Y[M, N] = X[M, K] * W[N, K]^T for few rows of X (M <= 16): the matrix products of a decode step.
//
// The product is bound by reading W once from HBM, so the kernel is built as a stream. A tile is
// ROWS rows of W; a block walks its tiles (block b takes tiles b, b + grid, ...) and each tile's K
// in chunks of KC. Every chunk of W, with the matching chunk of X, travels to shared memory as
// 16-byte cp.async copies through a ring of STAGES buffers that keeps running across tile
// boundaries, so a block always has STAGES - 1 chunks in flight while the tensor cores (mma.sync
// m16n8k16, bf16 in, float32 accumulate) work on the oldest one. The MMA tile has the rows of W on
// its 16-row side and the rows of X on its 8-column side, so no tensor-core work is spent on
// padding M. The four warps split each chunk along K (warp w takes the w-th quarter); their partial
// sums are added in warp order in shared memory, so the result does not depend on timing, and a
// row of X gives the same result whatever else is in X.
#include "common.cuh"

#define SK_THREADS 128
#define SK_WARPS 4
#define SK_KC 256            // K elements per chunk
#define SK_PAD 8             // bf16 elements of padding per shared-memory row (16 bytes)

__device__ __forceinline__ void sk_cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;       // 0: nothing is read, the 16 bytes are filled with zeros
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

// ROWS: rows of W per tile (16 or 32). NT: 8-row tiles of X (M <= 8 * NT). STAGES: ring depth.
template <int ROWS, int NT, int STAGES, typename TO>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, TO* __restrict__ Y, int M, int N, int K,
                   long ldx, long ldw, long ldy) {
    extern __shared__ __align__(16) unsigned char sk_smem[];
    pdl_trigger();                                       // the kernel after this one may take its places
    constexpr int STRIDE = SK_KC + SK_PAD;               // elements per shared-memory row
    constexpr int MT = ROWS / 16;                        // 16-row MMA tiles of W
    constexpr int XROWS = NT * 8;
    constexpr int STAGE_ELEMS = (ROWS + XROWS) * STRIDE;
    constexpr int CPR = SK_KC / 8;                       // 16-byte pieces per row
    constexpr int ROWS_PER_PASS = SK_THREADS / CPR;
    constexpr int PSTRIDE = ROWS + 1;
    bf16* ring = reinterpret_cast<bf16*>(sk_smem);
    float* part = reinterpret_cast<float*>(ring + (size_t)STAGES * STAGE_ELEMS);   // [warps][XROWS][PSTRIDE]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tiles = (N + ROWS - 1) / ROWS;
    const int chunks = (K + SK_KC - 1) / SK_KC;
    const int my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int total = my_tiles * chunks;
    const int cc = (tid % CPR) * 8;                      // this thread's column inside a chunk
    const int r0 = tid / CPR;

    // the copies of step (tile, chunk) into a ring buffer: the rows of W, and the rows of X
    auto issue_w = [&](int tile, int chunk, int stage) {
        bf16* Ws = ring + (size_t)stage * STAGE_ELEMS;
        const int n0 = tile * ROWS;
        const int k = chunk * SK_KC + cc;
        const bool kin = k < K;
#pragma unroll
        for (int row = r0; row < ROWS; row += ROWS_PER_PASS) {
            const bool ok = kin && (n0 + row) < N;
            sk_cp_async_16(Ws + row * STRIDE + cc, ok ? W + (size_t)(n0 + row) * ldw + k : W, ok);
        }
    };
    auto issue_x = [&](int chunk, int stage) {
        bf16* Xs = ring + (size_t)stage * STAGE_ELEMS + ROWS * STRIDE;
        const int k = chunk * SK_KC + cc;
        const bool kin = k < K;
#pragma unroll
        for (int row = r0; row < XROWS; row += ROWS_PER_PASS) {
            const bool ok = kin && row < M;
            sk_cp_async_16(Xs + row * STRIDE + cc, ok ? X + (size_t)row * ldx + k : X, ok);
        }
    };
    auto issue = [&](int tile, int chunk, int stage) {
        issue_w(tile, chunk, stage);
        issue_x(chunk, stage);
    };

    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

    // The first STAGES - 1 steps: their rows of W are asked for at once; X may still be in the making by the
    // kernel before this one, so its rows follow after pdl_wait(). The first copy group then holds all of
    // these rows of W, which were asked for first.
    int issue_tile = blockIdx.x, issue_chunk = 0, issued = 0;
    {
        int t = issue_tile, c = issue_chunk;
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (s < total) {
                issue_w(t, c, s);
                if (++c == chunks) {
                    c = 0;
                    t += gridDim.x;
                }
            }
        }
    }
    pdl_wait();
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (issued < total) {
            issue_x(issue_chunk, s);
            ++issued;
            if (++issue_chunk == chunks) {
                issue_chunk = 0;
                issue_tile += gridDim.x;
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    constexpr int KW = SK_KC / SK_WARPS;                 // this warp's share of a chunk along K
    int tile = blockIdx.x, chunk = 0, stage = 0, issue_stage = STAGES - 1;
    for (int step = 0; step < total; ++step) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2) : "memory");
        __syncthreads();                                 // this step has landed for all threads; the oldest buffer is free
        if (issued < total) {
            issue(issue_tile, issue_chunk, issue_stage);
            ++issued;
            if (++issue_chunk == chunks) {
                issue_chunk = 0;
                issue_tile += gridDim.x;
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        if (++issue_stage == STAGES) issue_stage = 0;

        const bf16* Ws = ring + (size_t)stage * STAGE_ELEMS;
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
        if (++stage == STAGES) stage = 0;

        if (++chunk == chunks) {
            // the tile is complete: add the four warps' sums in warp order and store
            // part[warp][x row][w row]; acc[i][j] holds W rows i*16 + g (+8), X rows j*8 + 2t (+1)
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    float* base = part + ((size_t)warp * XROWS + j * 8 + 2 * t) * PSTRIDE + i * 16 + g;
                    base[0] = acc[i][j][0];
                    base[PSTRIDE] = acc[i][j][1];
                    base[8] = acc[i][j][2];
                    base[PSTRIDE + 8] = acc[i][j][3];
                    acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
                }
            __syncthreads();
            const int n0 = tile * ROWS;
            for (int e = tid; e < XROWS * ROWS; e += SK_THREADS) {
                const int m = e / ROWS, row = e % ROWS;
                if (m < M && n0 + row < N) {
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < SK_WARPS; ++w) v += part[((size_t)w * XROWS + m) * PSTRIDE + row];
                    Y[(size_t)m * ldy + n0 + row] = from_float<TO>(v);
                }
            }
            chunk = 0;
            tile += gridDim.x;
            // the next write to part comes after the barrier at the top of a later step
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

template <int ROWS, int NT, int STAGES, typename TO>
static int launch_skinny(const bf16* X, const bf16* W, TO* Y, int M, int N, int K, long ldx, long ldw, long ldy,
                         cudaStream_t stream) {
    constexpr size_t ring = (size_t)STAGES * (ROWS + NT * 8) * (SK_KC + SK_PAD) * sizeof(bf16);
    constexpr size_t part = (size_t)SK_WARPS * NT * 8 * (ROWS + 1) * sizeof(float);
    constexpr size_t smem = ring + part;
    auto kernel = gemm_skinny_kernel<ROWS, NT, STAGES, TO>;
    LLMP_ALLOW_SMEM(kernel, smem);
    static int sms = 0, per_sm = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, SK_THREADS, smem);
        if (per_sm < 1) per_sm = 1;
    }
    const int tiles = (N + ROWS - 1) / ROWS;
    const int resident = sms * per_sm;
    const int grid = tiles < resident ? tiles : resident;
    const cudaError_t launched = llmp_launch_dependent(kernel, dim3(grid), dim3(SK_THREADS), smem, stream, X, W, Y, M, N, K,
                                                       ldx, ldw, ldy);
    if (launched != cudaSuccess) {
        llmp_set_error("gemm_skinny: launch failed: %s", cudaGetErrorString(launched));
        return 2;
    }
    return llmp_check_launch("gemm_skinny");
}

template <typename TO>
static int dispatch_skinny(const bf16* X, const bf16* W, TO* Y, int M, int N, int K, long ldx, long ldw, long ldy,
                           cudaStream_t stream) {
    // 16 rows of W per tile unless the output is so wide that 32-row tiles still outnumber the blocks
    const bool wide = N >= 16384;
    if (M <= 8)
        return wide ? launch_skinny<32, 1, 5, TO>(X, W, Y, M, N, K, ldx, ldw, ldy, stream)
                    : launch_skinny<16, 1, 6, TO>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
    return wide ? launch_skinny<32, 2, 4, TO>(X, W, Y, M, N, K, ldx, ldw, ldy, stream)
                : launch_skinny<16, 2, 5, TO>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
}

// X and W bfloat16, rows 16-byte aligned (K, ldx, ldw multiples of 8); out_dtype bfloat16 or float32; M <= 16.
LLMP_API int llmp_gemm_skinny(const void* X, const void* W, void* Y, int out_dtype, int M, int N, int K, long ldx,
                              long ldw, long ldy, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    LLMP_REQUIRE(M <= 16, "gemm_skinny: %d rows, at most 16 are taken", M);
    LLMP_REQUIRE(K > 0 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0,
                 "gemm_skinny: K=%d and the row strides (%ld, %ld) must be multiples of 8", K, ldx, ldw);
    LLMP_REQUIRE(((size_t)X % 16) == 0 && ((size_t)W % 16) == 0, "gemm_skinny: operands must be 16-byte aligned");
    if (out_dtype == LLMP_F32)
        return dispatch_skinny<float>((const bf16*)X, (const bf16*)W, (float*)Y, M, N, K, ldx, ldw, ldy, stream);
    return dispatch_skinny<bf16>((const bf16*)X, (const bf16*)W, (bf16*)Y, M, N, K, ldx, ldw, ldy, stream);
}
