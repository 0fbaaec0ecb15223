// Y[M, N] = X[M, K] * W[N, K]^T for the rows of a larger decode step (M <= 64), bound by reading W once from HBM:
// the stream of gemm_stream.cu with the products on the fifth-generation tensor cores.
//
// As there, one persistent block per SM owns the contiguous rows [b * per, (b + 1) * per) of W, walks them in
// chunks of RB <= 128 rows and each chunk's K in steps of KB blocks of 64 elements; a ring stage holds the box of
// X (NB = 16, 32 or 64 rows, rows beyond M read as zeros) and the box of W (RB rows) of one step, each as KB planes
// of lines of 128 bytes in the 128-byte swizzle, filled by one TMA box each. One thread issues the loads, one
// thread the tcgen05.mma (the 128-row side takes the plane of W, of which the first RB rows count; the N side
// the plane of X; float32 accumulator of 128 lanes x NB columns in tensor memory over the whole K of a chunk)
// and frees a stage with tcgen05.commit; four warps read the finished accumulator with tcgen05.ld and store the
// transpose. A plane of W starts wherever the plane before it ends, not on a 1024-byte boundary: TMA and MMA both
// take the swizzle from the bits of the shared-memory address itself, so the plain descriptor of the plane's
// first line is right (measured: with the line's phase in the descriptor's base-offset field the products were
// wrong). The K order of the additions is the same for every row of X, so a row's result does not depend on the
// other rows.
//
// As a dependent launch: the load thread fills the ring with boxes of W, waits for the kernel before this one,
// then adds the boxes of X.
//
// Every wait on an mbarrier is bounded: when one runs out the kernel records 1 in *error_flag and goes on without
// waiting (its output is then wrong; the host reads the flag); the tensor memory is always freed.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"

#define GT_THREADS 192
#define GT_MAX_RB 128
#define GT_MAX_STAGES 24
#define GT_SMEM_BUDGET (207 * 1024)               // the ring; 16 KB more follow it, which a plane's 128-line read may reach
#define GT_TAIL_BYTES (16 * 1024)
#define GT_STAGE_LIMIT (48 * 1024)

struct StreamTcParams {
    void* Y;
    long ldy;
    int M, N, K;
    int per;              // rows of W per block
    int RB;               // rows of W per chunk and box
    int KB;               // 64-element blocks of K per stage
    int stages;
    int out_f32;
    int* error_flag;
};

// NB: rows of the X box, the N of the MMA.
template <int NB>
__global__ void __launch_bounds__(GT_THREADS, 1)
gemm_stream_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const StreamTcParams p) {
    extern __shared__ unsigned char gt_raw[];
    __shared__ __align__(8) uint64_t full_bar[GT_MAX_STAGES], empty_bar[GT_MAX_STAGES], acc_full, acc_empty;
    __shared__ uint32_t tmem_slot;
    constexpr uint32_t COLS = NB < 32 ? 32 : NB;                // tensor-memory columns (a power of two >= 32)
    const uint32_t raw_addr = tc_smem_u32(gt_raw);
    unsigned char* ring = gt_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);      // 1024-byte aligned stages
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // a stage: KB planes of NB lines of X, then KB planes of RB lines of W, rounded up to 1024 bytes
    const uint32_t x_bytes = (uint32_t)NB * 128 * p.KB, w_bytes = (uint32_t)p.RB * 128 * p.KB;
    const uint32_t stage_bytes = (x_bytes + w_bytes + 1023u) & ~1023u;

    const int row_begin = blockIdx.x * p.per;
    int row_end = row_begin + p.per;
    if (row_end > p.N) row_end = p.N;
    const int chunks = row_begin < row_end ? (row_end - row_begin + p.RB - 1) / p.RB : 0;
    const int ksteps = p.K / (64 * p.KB);                       // stages per chunk
    const int total = chunks * ksteps;

    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_empty, 4);                               // one arrival per epilogue warp
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_x) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem_u32(&tmem_slot)), "r"(COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    pdl_trigger();                                              // the kernel after this one may take its places

    if (warp == 0) {
        if (lane == 0) {
            // the ring is filled with boxes of W at once; the boxes of X follow after pdl_wait()
            const int ahead = total < p.stages ? total : p.stages;
            for (int i = 0; i < ahead; ++i) {
                const int chunk = i / ksteps, ks = i - chunk * ksteps;
                mbar_expect_tx(&full_bar[i], x_bytes + w_bytes);
                tma_load_3d(ring + (size_t)i * stage_bytes + x_bytes, &map_w, 0, row_begin + chunk * p.RB, ks * p.KB, &full_bar[i]);
            }
            pdl_wait();
            for (int i = 0; i < ahead; ++i) {
                const int chunk = i / ksteps, ks = i - chunk * ksteps;
                tma_load_3d(ring + (size_t)i * stage_bytes, &map_x, 0, 0, ks * p.KB, &full_bar[i]);
            }
            for (int i = ahead; i < total; ++i) {
                const int slot = i % p.stages;
                const int chunk = i / ksteps, ks = i - chunk * ksteps;
                mbar_wait(&empty_bar[slot], (uint32_t)(((i / p.stages) - 1) & 1), p.error_flag);
                mbar_expect_tx(&full_bar[slot], x_bytes + w_bytes);
                unsigned char* stage = ring + (size_t)slot * stage_bytes;
                tma_load_3d(stage + x_bytes, &map_w, 0, row_begin + chunk * p.RB, ks * p.KB, &full_bar[slot]);
                tma_load_3d(stage, &map_x, 0, 0, ks * p.KB, &full_bar[slot]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(128, NB);
            int i = 0;
            for (int chunk = 0; chunk < chunks; ++chunk) {
                if (chunk > 0) {                                // the accumulator of the chunk before has been read
                    mbar_wait(&acc_empty, (uint32_t)((chunk - 1) & 1), p.error_flag);
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                }
                for (int ks = 0; ks < ksteps; ++ks, ++i) {
                    const int slot = i % p.stages;
                    mbar_wait(&full_bar[slot], (uint32_t)((i / p.stages) & 1), p.error_flag);
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t stage = tc_smem_u32(ring + (size_t)slot * stage_bytes);
                    for (int j = 0; j < p.KB; ++j) {
                        const uint32_t x_plane = stage + (uint32_t)j * NB * 128;                 // 1024-byte aligned
                        const uint32_t w_line = (x_bytes >> 7) + (uint32_t)j * p.RB;             // first line of the plane of W
                        const uint32_t w_plane = stage + (w_line << 7);
#pragma unroll
                        for (int k = 0; k < 4; ++k)             // 16 elements of K (32 bytes) per MMA
                            umma_f16(tmem_base, umma_desc(w_plane + k * 32), umma_desc(x_plane + k * 32), idesc,
                                     (ks | j | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[slot]);              // the stage is free when these MMAs have read it
                }
                umma_commit(&acc_full);                         // the chunk's accumulator is complete
            }
        }
    } else {
        // epilogue: warp w reads the 32 tensor-memory lanes of its quarter (w % 4): lane = row of W, column = row of X
        const int quarter = warp & 3;
        for (int chunk = 0; chunk < chunks; ++chunk) {
            mbar_wait(&acc_full, (uint32_t)(chunk & 1), p.error_flag);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int n0 = row_begin + chunk * p.RB;
            int rows = row_end - n0;
            if (rows > p.RB) rows = p.RB;
            const int row = quarter * 32 + lane;
#pragma unroll
            for (int c0 = 0; c0 < NB; c0 += 16) {
                float v[16];
                tmem_ld_16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                if (row < rows) {
#pragma unroll
                    for (int m = 0; m < 16; ++m) {
                        if (c0 + m < p.M) {
                            if (p.out_f32) reinterpret_cast<float*>(p.Y)[(size_t)(c0 + m) * p.ldy + n0 + row] = v[m];
                            else reinterpret_cast<bf16*>(p.Y)[(size_t)(c0 + m) * p.ldy + n0 + row] = __float2bfloat16_rn(v[m]);
                        }
                    }
                }
            }
            // this warp has read its part of the accumulator
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem_u32(&acc_empty)) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(COLS) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------------------
struct StreamTcPlan {
    int per, grid, rb, nb, kb, stages;
    size_t smem;
};

static bool stream_tc_plan(int M, int N, int K, long ldx, long ldw, StreamTcPlan* out) {
    if (!(M > 0 && M <= 64 && N > 0 && K >= 64 && K % 64 == 0 && ldx % 8 == 0 && ldw % 8 == 0)) return false;
    const int sms = llmp_sm_count();
    StreamTcPlan q;
    q.per = (N + sms - 1) / sms;                                 // rows per block: an even share
    if (q.per < 8) q.per = 8;
    q.grid = (N + q.per - 1) / q.per;
    const int chunks = (q.per + GT_MAX_RB - 1) / GT_MAX_RB;
    q.rb = (q.per + chunks - 1) / chunks;
    q.nb = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    // blocks of K per stage: as in gemm_stream.cu, chosen from N and K alone
    q.kb = 1;
    while (q.kb < 8 && (long)(q.rb + 16) * 128 * q.kb * 2 <= GT_STAGE_LIMIT && (K / 64) % (q.kb * 2) == 0) q.kb *= 2;
    const size_t stage_bytes = ((size_t)(q.rb + q.nb) * 128 * q.kb + 1023) / 1024 * 1024;
    int stages = (int)(GT_SMEM_BUDGET / stage_bytes);
    if (stages > GT_MAX_STAGES) stages = GT_MAX_STAGES;
    if (stages < 2) return false;
    q.stages = stages;
    q.smem = (size_t)stages * stage_bytes + GT_TAIL_BYTES + 1024;
    *out = q;
    return true;
}

// Shapes this kernel takes: M <= 64 rows of X, K a multiple of 64, rows of 16 bytes' alignment.
LLMP_API int llmp_gemm_stream_tc_supports(int M, int N, int K, long ldx, long ldw) {
    StreamTcPlan q;
    return stream_tc_plan(M, N, K, ldx, ldw, &q) ? 1 : 0;
}

// X and W bfloat16, rows 16-byte aligned; out_dtype bfloat16 or float32; shapes as llmp_gemm_stream_tc_supports says.
LLMP_API int llmp_gemm_stream_tc(const void* X, const void* W, void* Y, int out_dtype, int M, int N, int K, long ldx,
                                 long ldw, long ldy, int* error_flag, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    StreamTcPlan q;
    LLMP_REQUIRE(stream_tc_plan(M, N, K, ldx, ldw, &q), "gemm_stream_tc: M=%d, N=%d, K=%d (a multiple of 64) or the row strides are not taken", M, N, K);
    LLMP_REQUIRE(((size_t)X % 16) == 0 && ((size_t)W % 16) == 0, "gemm_stream_tc: operands must be 16-byte aligned");
    LLMP_REQUIRE(error_flag != nullptr, "gemm_stream_tc: an error flag in device memory is required");
    StreamTcParams p;
    p.Y = Y; p.ldy = ldy; p.M = M; p.N = N; p.K = K; p.out_f32 = out_dtype == LLMP_F32; p.error_flag = error_flag;
    p.per = q.per; p.RB = q.rb; p.KB = q.kb; p.stages = q.stages;
    CUtensorMap map_w, map_x;
    if (llmp_stream_tensor_map(W, N, K, ldw, q.rb, q.kb, &map_w) || llmp_stream_tensor_map(X, M, K, ldx, q.nb, q.kb, &map_x)) return 1;
    cudaError_t launched = cudaSuccess;
#define GT_LAUNCH(NB)                                                                                              \
    do {                                                                                                           \
        LLMP_ALLOW_SMEM(gemm_stream_tc_kernel<NB>, q.smem);                                                        \
        launched = llmp_launch_dependent(gemm_stream_tc_kernel<NB>, dim3(q.grid), dim3(GT_THREADS), q.smem, stream, \
                                         map_w, map_x, p);                                                         \
    } while (0)
    if (q.nb == 16) GT_LAUNCH(16); else if (q.nb == 32) GT_LAUNCH(32); else GT_LAUNCH(64);
#undef GT_LAUNCH
    if (launched != cudaSuccess) {
        llmp_set_error("gemm_stream_tc: launch failed: %s", cudaGetErrorString(launched));
        return 2;
    }
    return llmp_check_launch("gemm_stream_tc");
}
