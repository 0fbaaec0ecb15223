// Shared by the weight-streaming products (gemm_stream.cu: one product per launch; gemm_stream_chain.cu: several
// products in one persistent launch): ring geometry, the mma.sync and ldmatrix helpers, and the plan of a product.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"

#define GS_CWARPS 4
#define GS_THREADS ((GS_CWARPS + 1) * 32)
#define GS_MAX_RB 128
#define GS_MAX_STAGES 24
#define GS_SMEM_BUDGET (223 * 1024)                // ring and partial sums; 2 KB more go to alignment and over-reads
#define GS_STAGE_LIMIT (48 * 1024)                // a stage may grow to half of this before KB stops doubling

__device__ __forceinline__ void gs_tma_load_3d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
        ::"r"(tc_smem_u32(smem_dst)), "l"(map), "r"(tc_smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}

__device__ __forceinline__ void gs_ldmatrix_x4(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void gs_ldmatrix_x2(unsigned (&r)[2], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}

__device__ __forceinline__ void gs_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 16 bytes of line `line` of a stage (lines of 128 bytes, counted from the stage's 1024-byte aligned start)
// starting at 16-byte chunk `chunk`: the 128-byte swizzle exchanges the chunk index with the low bits of the line.
__device__ __forceinline__ const unsigned char* gs_at(const unsigned char* stage, int line, int chunk) {
    return stage + line * 128 + ((chunk ^ (line & 7)) << 4);
}

// How a product is laid out: rows per block and chunk, blocks of K per stage, ring depth. False when the shape is
// not taken.
struct StreamPlan {
    int per, grid, rb, nt, mt, kb, stages;
    size_t stage_bytes, part_bytes, smem;
};

// The plan of Y[M, N] = X[M, K] W[N, K]^T (glu_rows = N / 2 for a [gate rows; up rows] matrix, else 0) on this
// device; false when the shape is not taken. per, rb and kb follow from N and K alone.
bool llmp_stream_plan(int M, int N, int K, long ldx, long ldw, int glu_rows, StreamPlan* out);
