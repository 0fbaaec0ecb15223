// C = A * B^T on the fifth-generation tensor cores: TMA loads, tcgen05.mma with the accumulator in
// tensor memory, tcgen05.ld for the epilogue. bfloat16 operands, float32 accumulation.
//
// Both operands are K-major ([rows, K] row-major). A tile of 128 rows of A and BN rows of B is
// multiplied per block; K is walked in blocks of 64 elements (128 bytes, one swizzle span). One
// thread issues the TMA loads of a K block into a ring of STAGES shared-memory buffers (128-byte
// swizzle), one thread issues four tcgen05.mma (K = 16 each) per K block and frees the buffer with
// tcgen05.commit, four warps read the finished accumulator from tensor memory and store it.
// For the few rows of a decode step the roles are swapped: A is the weight matrix (its rows fill the
// 128-row side of the MMA), B is the activations (BN = 16, 32 or 64 rows, rows beyond M read as
// zeros by the TMA unit) and the epilogue stores the transpose; nothing is padded in memory and
// every weight byte is read once. The K order of the additions is the same for every row, so a
// row's result does not depend on the other rows of the call.
//
// Every wait on an mbarrier is bounded: when a wait runs out, the kernel records 1 in *error_flag,
// leaves its loops, frees its tensor memory and returns; the host reads the flag.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

#define TC_THREADS 192
#define TC_BM 128
#define TC_BK 64

// BN: rows of B per tile (the N of the MMA). SWAP: store the transpose (Y[b row, a row]).
template <int BN, int STAGES, bool SWAP, typename TO>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TO* __restrict__ Y,
               int rows_a, int rows_b, int K, long ldy, int* __restrict__ error_flag) {
    extern __shared__ unsigned char tc_raw[];
    constexpr uint32_t A_BYTES = TC_BM * 128, B_BYTES = BN * 128, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t COLS = BN < 32 ? 32 : BN;               // tensor-memory columns (a power of two >= 32)
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], accum_bar;
    __shared__ uint32_t tmem_slot;

    // the swizzled tiles want 1024-byte alignment
    const uint32_t raw_addr = tc_smem_u32(tc_raw);
    unsigned char* tiles = tc_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a0 = blockIdx.x * TC_BM, b0 = blockIdx.y * BN;
    const int kblocks = (K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem_u32(&tmem_slot)), "r"(COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // producer: TMA loads of K block kb into buffer kb % STAGES
            for (int kb = 0; kb < kblocks; ++kb) {
                const int s = kb % STAGES;
                if (kb >= STAGES && !mbar_wait(&empty_bar[s], ((kb / STAGES) - 1) & 1, error_flag)) break;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
                tma_load_2d(stage, &map_a, kb * TC_BK, a0, &full_bar[s]);
                tma_load_2d(stage + A_BYTES, &map_b, kb * TC_BK, b0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // MMA issuer
            constexpr uint32_t idesc = umma_idesc(TC_BM, BN);
            bool ok = true;
            for (int kb = 0; kb < kblocks && ok; ++kb) {
                const int s = kb % STAGES;
                ok = mbar_wait(&full_bar[s], (kb / STAGES) & 1, error_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t a_addr = tc_smem_u32(tiles + (size_t)s * STAGE_BYTES);
                const uint64_t desc_a = umma_desc(a_addr), desc_b = umma_desc(a_addr + A_BYTES);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)     // 32 bytes along K per MMA: 2 units of 16 bytes
                    umma_f16(tmem_base, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                umma_commit(&empty_bar[s]);              // the buffer is free when these MMAs have read it
            }
            if (ok) umma_commit(&accum_bar);             // the accumulator is complete
        }
    } else {
        // epilogue: warp w reads the 32 tensor-memory lanes of its quarter (w % 4)
        const int quarter = warp & 3;
        if (mbar_wait(&accum_bar, 0, error_flag)) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int arow = a0 + quarter * 32 + lane;
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float v[16];
                tmem_ld_16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                if (SWAP) {
                    // Y[b row, a row]: the lanes of a warp hold consecutive a rows
                    if (arow < rows_a) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (b0 + c0 + j < rows_b) Y[(size_t)(b0 + c0 + j) * ldy + arow] = from_float<TO>(v[j]);
                    }
                } else if (arow < rows_a) {
                    TO* dst = Y + (size_t)arow * ldy + b0 + c0;
                    if (b0 + c0 + 16 <= rows_b && ((size_t)dst % 16) == 0) {
                        if (sizeof(TO) == 4) {
#pragma unroll
                            for (int j = 0; j < 16; j += 4)
                                *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; j += 8) {
                                uint4 pack;
                                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]), h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                                pack.x = *reinterpret_cast<unsigned*>(&h0);
                                pack.y = *reinterpret_cast<unsigned*>(&h1);
                                pack.z = *reinterpret_cast<unsigned*>(&h2);
                                pack.w = *reinterpret_cast<unsigned*>(&h3);
                                *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dst) + j) = pack;
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (b0 + c0 + j < rows_b) dst[j] = from_float<TO>(v[j]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(COLS) : "memory");
    }
}

// ---- split-K for the few rows of a decode step ----------------------------------------------------------
// With fewer 128-row tiles of the weight matrix than SMs, one tile per block would leave most of the
// GPU without work and every working SM with more bytes to pull than it can. The blocks of a
// thread-block cluster (1, 1, splits) therefore share one output tile and each takes a contiguous
// share of the K blocks. When all of them are done, the blocks of rank 1.. write their float32
// partial tiles into the shared memory of the rank-0 block (distributed shared memory; its TMA ring
// is free by then), and rank 0 adds them in rank order and stores. No scratch in global memory, no
// atomics, and a fixed order of additions.
template <int BN, int STAGES, typename TO>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_splitk_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      TO* __restrict__ Y, int rows_a, int rows_b, int K, long ldy, int splits,
                      int* __restrict__ error_flag) {
    extern __shared__ unsigned char tc_raw[];
    constexpr uint32_t A_BYTES = TC_BM * 128, B_BYTES = BN * 128, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t COLS = BN < 32 ? 32 : BN;
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], accum_bar;
    __shared__ uint32_t tmem_slot;
    const uint32_t raw_addr = tc_smem_u32(tc_raw);
    unsigned char* tiles = tc_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a0 = blockIdx.x * TC_BM, b0 = blockIdx.y * BN;
    const int rank = (int)cluster_ctarank();
    pdl_trigger();                                   // the kernel after this one may take its places
    const int kblocks = (K + TC_BK - 1) / TC_BK;
    const int per = (kblocks + splits - 1) / splits;
    const int kb0 = rank * per;
    const int count = kb0 >= kblocks ? 0 : (kb0 + per <= kblocks ? per : kblocks - kb0);

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem_u32(&tmem_slot)), "r"(COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_slot;

    float v[BN];                     // this thread's row of the partial tile (epilogue warps only)
    bool have = false;
    const int quarter = warp & 3;
    if (warp == 0) {
        if (lane == 0) {
            // A holds the weights: the ring is filled with them at once. B, the activations, may still be in the
            // making by the kernel before this one: its loads follow after pdl_wait().
            const int ahead = count < STAGES ? count : STAGES;
            for (int i = 0; i < ahead; ++i) {
                mbar_expect_tx(&full_bar[i], STAGE_BYTES);
                tma_load_2d(tiles + (size_t)i * STAGE_BYTES, &map_a, (kb0 + i) * TC_BK, a0, &full_bar[i]);
            }
            pdl_wait();
            for (int i = 0; i < ahead; ++i)
                tma_load_2d(tiles + (size_t)i * STAGE_BYTES + A_BYTES, &map_b, (kb0 + i) * TC_BK, b0, &full_bar[i]);
            for (int i = ahead; i < count; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1, error_flag)) break;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
                tma_load_2d(stage, &map_a, (kb0 + i) * TC_BK, a0, &full_bar[s]);
                tma_load_2d(stage + A_BYTES, &map_b, (kb0 + i) * TC_BK, b0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(TC_BM, BN);
            bool ok = true;
            for (int i = 0; i < count; ++i) {
                const int s = i % STAGES;
                ok = mbar_wait(&full_bar[s], (i / STAGES) & 1, error_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t a_addr = tc_smem_u32(tiles + (size_t)s * STAGE_BYTES);
                const uint64_t desc_a = umma_desc(a_addr), desc_b = umma_desc(a_addr + A_BYTES);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)
                    umma_f16(tmem_base, desc_a + 2 * k, desc_b + 2 * k, idesc, (i | k) != 0 ? 1u : 0u);
                umma_commit(&empty_bar[s]);
            }
            if (ok && count > 0) umma_commit(&accum_bar);
        }
    } else if (count > 0) {
        if (mbar_wait(&accum_bar, 0, error_flag)) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float part[16];
                tmem_ld_16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, part);
#pragma unroll
                for (int j = 0; j < 16; ++j) v[c0 + j] = part[j];
            }
            have = true;
        }
    }
    // every block of the cluster has finished reading its ring: rank 0's ring may now receive partial tiles
    cluster_sync_all();
    const int row = quarter * 32 + lane;                 // row of the tile held by an epilogue thread
    if (warp >= 2 && rank != 0 && have) {
        const uint32_t base = tc_smem_u32(tiles) + (uint32_t)((rank - 1) * BN * TC_BM + row) * 4u;
#pragma unroll
        for (int j = 0; j < BN; ++j) st_cluster_f32(base + (uint32_t)(j * TC_BM) * 4u, 0u, v[j]);
    }
    cluster_sync_all();
    if (warp >= 2 && rank == 0 && have) {
        const float* slots = reinterpret_cast<const float*>(tiles);
        const int arow = a0 + row;
        if (arow < rows_a) {
#pragma unroll
            for (int j = 0; j < BN; ++j) {
                float sum = v[j];
                for (int r = 1; r < splits; ++r) {
                    const int rk0 = r * per;
                    if (rk0 < kblocks) sum += slots[((size_t)(r - 1) * BN + j) * TC_BM + row];     // rank order
                }
                if (b0 + j < rows_b) Y[(size_t)(b0 + j) * ldy + arow] = from_float<TO>(sum);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(COLS) : "memory");
    }
}

// ---- persistent kernel for many rows (prompt portions) -------------------------------------------------
// One block per SM walks output tiles of 128 x BN (tile t: column block t / m_tiles, row block
// t % m_tiles, so blocks that run side by side share a weight tile through L2). The TMA ring keeps
// running across tiles. Two accumulators live in tensor memory: while the four epilogue warps read
// tile i out of one (tcgen05.ld, convert, store), the MMA thread already fills the other with tile
// i + 1. Barriers: full/empty per ring stage, accumulator-full/accumulator-empty per accumulator.
template <int BN, int STAGES, typename TO>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          TO* __restrict__ Y, int rows_a, int rows_b, int K, long ldy, int* __restrict__ error_flag) {
    extern __shared__ unsigned char tc_raw[];
    constexpr uint32_t A_BYTES = TC_BM * 128, B_BYTES = BN * 128, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t COLS = 2 * BN;                          // two accumulators (BN = 128 or 256: a power of two)
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    const uint32_t raw_addr = tc_smem_u32(tc_raw);
    unsigned char* tiles = tc_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (K + TC_BK - 1) / TC_BK;
    const int m_tiles = (rows_a + TC_BM - 1) / TC_BM, n_tiles = (rows_b + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_full[0], 1);
        mbar_init(&acc_full[1], 1);
        mbar_init(&acc_empty[0], 4);       // one arrival per epilogue warp
        mbar_init(&acc_empty[1], 4);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem_u32(&tmem_slot)), "r"(COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;                                          // K blocks issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int a0 = (tile % m_tiles) * TC_BM, b0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) - 1) & 1, error_flag)) { ok = false; break; }
                    mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                    unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
                    tma_load_2d(stage, &map_a, kb * TC_BK, a0, &full_bar[s]);
                    tma_load_2d(stage + A_BYTES, &map_b, kb * TC_BK, b0, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(TC_BM, BN);
            int it = 0, n = 0;                                   // K blocks consumed, tiles done
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++n) {
                const int acc = n & 1;
                // the epilogue must have drained this accumulator (its use n / 2 - 1)
                if (n >= 2 && !mbar_wait(&acc_empty[acc], ((n >> 1) - 1) & 1, error_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t d_addr = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full_bar[s], (it / STAGES) & 1, error_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t a_addr = tc_smem_u32(tiles + (size_t)s * STAGE_BYTES);
                    const uint64_t desc_a = umma_desc(a_addr), desc_b = umma_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        umma_f16(d_addr, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    umma_commit(&empty_bar[s]);
                }
                if (ok) umma_commit(&acc_full[acc]);
            }
        }
    } else {
        const int quarter = warp & 3;
        int n = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++n) {
            const int acc = n & 1;
            if (!mbar_wait(&acc_full[acc], (n >> 1) & 1, error_flag)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int a0 = (tile % m_tiles) * TC_BM, b0 = (tile / m_tiles) * BN;
            const int arow = a0 + quarter * 32 + lane;
#pragma unroll 4
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float v[16];
                tmem_ld_16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN + c0), v);
                if (arow < rows_a) {
                    TO* dst = Y + (size_t)arow * ldy + b0 + c0;
                    if (b0 + c0 + 16 <= rows_b && ((size_t)dst % 16) == 0) {
                        if (sizeof(TO) == 4) {
#pragma unroll
                            for (int j = 0; j < 16; j += 4)
                                *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; j += 8) {
                                uint4 pack;
                                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]), h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                                pack.x = *reinterpret_cast<unsigned*>(&h0);
                                pack.y = *reinterpret_cast<unsigned*>(&h1);
                                pack.z = *reinterpret_cast<unsigned*>(&h2);
                                pack.w = *reinterpret_cast<unsigned*>(&h3);
                                *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dst) + j) = pack;
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (b0 + c0 + j < rows_b) dst[j] = from_float<TO>(v[j]);
                    }
                }
            }
            // this warp has read its part of the accumulator: one arrival per warp frees it for the MMA thread
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem_u32(&acc_empty[acc])) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(COLS) : "memory");
    }
}

// ---- host side: tensor maps ------------------------------------------------------------------------
EncodeTiledFn llmp_tensor_map_encoder() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &status) == cudaSuccess &&
            status == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

struct MapKey {
    const void* ptr;
    long rows, k, ld;
    int box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && k == o.k && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& m) const {
        size_t h = (size_t)m.ptr;
        h = h * 1000003u ^ (size_t)m.rows;
        h = h * 1000003u ^ (size_t)m.k;
        h = h * 1000003u ^ (size_t)m.ld;
        return h * 1000003u ^ (size_t)m.box_rows;
    }
};

// A [rows, K] bfloat16 row-major matrix with row pitch ld, read in boxes of box_rows x 64 elements.
static int make_map(const void* ptr, long rows, long k, long ld, int box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex lock;
    const MapKey key{ptr, rows, k, ld, box_rows};
    std::lock_guard<std::mutex> guard(lock);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return 0;
    }
    EncodeTiledFn fn = llmp_tensor_map_encoder();
    LLMP_REQUIRE(fn != nullptr, "gemm_tc: the driver does not provide cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(bf16)};
    const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    LLMP_REQUIRE(rc == CUDA_SUCCESS, "gemm_tc: cuTensorMapEncodeTiled failed with code %d", (int)rc);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

template <int BN, int STAGES, bool SWAP, typename TO>
static int launch_tc(const void* A, long rows_a, long lda, const void* B, long rows_b, long ldb, TO* Y, int K, long ldy,
                     int* error_flag, cudaStream_t stream) {
    CUtensorMap map_a, map_b;
    if (make_map(A, rows_a, K, lda, TC_BM, &map_a) || make_map(B, rows_b, K, ldb, BN, &map_b)) return 1;
    constexpr size_t smem = (size_t)STAGES * (TC_BM * 128 + BN * 128) + 1024;
    auto kernel = gemm_tc_kernel<BN, STAGES, SWAP, TO>;
    LLMP_ALLOW_SMEM(kernel, smem);
    dim3 grid((unsigned)((rows_a + TC_BM - 1) / TC_BM), (unsigned)((rows_b + BN - 1) / BN));
    LLMP_REQUIRE(grid.y <= 65535, "gemm_tc: too many column tiles");
    kernel<<<grid, TC_THREADS, smem, stream>>>(map_a, map_b, Y, (int)rows_a, (int)rows_b, K, ldy, error_flag);
    return llmp_check_launch("gemm_tc");
}

// Number of K shares for an output with `tiles` 128-row tiles: the one that fills whole waves of SMs
// best, with at least 8 K blocks per share, at most 8 shares (portable cluster size) and no more
// than fit the rank-0 ring as float32 partial tiles.
static int choose_splits(int tiles, int kblocks, int bn, size_t ring_bytes) {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    int best = 1;
    double best_score = -1.0;
    for (int s = 1; s <= 8; ++s) {
        if (s > 1 && (kblocks / s < 8 || (size_t)(s - 1) * bn * TC_BM * 4 > ring_bytes)) break;
        const int per = (kblocks + s - 1) / s;
        if ((s - 1) * per >= kblocks) continue;          // the last share would be empty
        const long ctas = (long)tiles * s;
        const long waves = (ctas + sms - 1) / sms;
        const double score = (double)ctas / (double)(waves * sms) - 0.01 * (s - 1);
        if (score > best_score) {
            best_score = score;
            best = s;
        }
    }
    return best;
}

template <int BN, int STAGES, typename TO>
static int launch_tc_splitk(const void* A, long rows_a, long lda, const void* B, long rows_b, long ldb, TO* Y, int K,
                            long ldy, int* error_flag, cudaStream_t stream) {
    CUtensorMap map_a, map_b;
    if (make_map(A, rows_a, K, lda, TC_BM, &map_a) || make_map(B, rows_b, K, ldb, BN, &map_b)) return 1;
    constexpr size_t ring = (size_t)STAGES * (TC_BM * 128 + BN * 128);
    constexpr size_t smem = ring + 1024;
    auto kernel = gemm_tc_splitk_kernel<BN, STAGES, TO>;
    LLMP_ALLOW_SMEM(kernel, smem);
    const int tiles = (int)((rows_a + TC_BM - 1) / TC_BM);
    const int splits = choose_splits(tiles, (K + TC_BK - 1) / TC_BK, BN, ring);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)tiles, (unsigned)((rows_b + BN - 1) / BN), (unsigned)splits);
    config.blockDim = dim3(TC_THREADS, 1, 1);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = (unsigned)splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // see pdl_wait() in the kernel
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = llmp_pdl_enabled() ? 2 : 1;
    const cudaError_t err = cudaLaunchKernelEx(&config, kernel, map_a, map_b, Y, (int)rows_a, (int)rows_b, K, ldy, splits,
                                               error_flag);
    if (err != cudaSuccess) {
        llmp_set_error("gemm_tc: cluster launch failed: %s", cudaGetErrorString(err));
        return 2;
    }
    return llmp_check_launch("gemm_tc_splitk");
}

template <int BN, int STAGES, typename TO>
static int launch_tc_persistent(const void* A, long rows_a, long lda, const void* B, long rows_b, long ldb, TO* Y, int K,
                                long ldy, int* error_flag, cudaStream_t stream) {
    CUtensorMap map_a, map_b;
    if (make_map(A, rows_a, K, lda, TC_BM, &map_a) || make_map(B, rows_b, K, ldb, BN, &map_b)) return 1;
    constexpr size_t smem = (size_t)STAGES * (TC_BM * 128 + BN * 128) + 1024;
    auto kernel = gemm_tc_persistent_kernel<BN, STAGES, TO>;
    LLMP_ALLOW_SMEM(kernel, smem);
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const long tiles = ((rows_a + TC_BM - 1) / TC_BM) * ((rows_b + BN - 1) / BN);
    const int grid = (int)(tiles < sms ? tiles : sms);
    kernel<<<grid, TC_THREADS, smem, stream>>>(map_a, map_b, Y, (int)rows_a, (int)rows_b, K, ldy, error_flag);
    return llmp_check_launch("gemm_tc_persistent");
}

template <typename TO>
static int dispatch_tc(const void* X, const void* W, TO* Y, int M, int N, int K, long ldx, long ldw, long ldy,
                       int* error_flag, cudaStream_t stream) {
    if (M <= 16) return launch_tc_splitk<16, 10, TO>(W, N, ldw, X, M, ldx, Y, K, ldy, error_flag, stream);
    if (M <= 32) return launch_tc_splitk<32, 9, TO>(W, N, ldw, X, M, ldx, Y, K, ldy, error_flag, stream);
    if (M <= 64) return launch_tc_splitk<64, 8, TO>(W, N, ldw, X, M, ldx, Y, K, ldy, error_flag, stream);
    // 128 x 256 tiles do twice the work per byte read from shared memory; 128 x 128 only for narrow outputs
    if (N >= 256) return launch_tc_persistent<256, 4, TO>(X, M, ldx, W, N, ldw, Y, K, ldy, error_flag, stream);
    return launch_tc_persistent<128, 6, TO>(X, M, ldx, W, N, ldw, Y, K, ldy, error_flag, stream);
}

// Y[M, N] = X[M, K] * W[N, K]^T, bfloat16 operands with 16-byte aligned rows (K, ldx, ldw multiples of 8),
// Y bfloat16 or float32. error_flag: one int in device memory that the kernel sets to 1 when a wait
// ran out (the host checks it after synchronising).
LLMP_API int llmp_gemm_tc(const void* X, const void* W, void* Y, int out_dtype, int M, int N, int K, long ldx, long ldw,
                          long ldy, int* error_flag, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    LLMP_REQUIRE(K > 0 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0,
                 "gemm_tc: K=%d and the row strides (%ld, %ld) must be multiples of 8", K, ldx, ldw);
    LLMP_REQUIRE(((size_t)X % 16) == 0 && ((size_t)W % 16) == 0, "gemm_tc: operands must be 16-byte aligned");
    LLMP_REQUIRE(error_flag != nullptr, "gemm_tc: an error flag in device memory is required");
    if (out_dtype == LLMP_F32) return dispatch_tc<float>(X, W, (float*)Y, M, N, K, ldx, ldw, ldy, error_flag, stream);
    return dispatch_tc<bf16>(X, W, (bf16*)Y, M, N, K, ldx, ldw, ldy, error_flag, stream);
}
