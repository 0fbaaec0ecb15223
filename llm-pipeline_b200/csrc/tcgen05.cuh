// Device helpers for the fifth-generation tensor cores: mbarriers with bounded waits, TMA tile loads,
// shared-memory matrix descriptors, tcgen05.mma issue and commit, tensor-memory loads.
#pragma once
#include <cuda.h>

#include "common.cuh"

#define TC_WAIT_LIMIT (1u << 20)

__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(tc_smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(tc_smem_u32(bar)), "r"(bytes) : "memory");
}

// Bounded wait: false (and *error_flag = 1) when the phase did not complete within ``limit`` tries. The kernels wait
// with TC_WAIT_LIMIT (mbar_wait below); the self-check of bounded_wait_check.cu passes a small limit to the same code.
__device__ __forceinline__ bool mbar_wait_limited(uint64_t* bar, uint32_t parity, int* error_flag, uint32_t limit) {
    const uint32_t addr = tc_smem_u32(bar);
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        // another role gave up? (the flag lives in host memory: look rarely, a read takes microseconds)
        if ((i & 0xFFFFu) == 0xFFFFu && *reinterpret_cast<volatile int*>(error_flag) != 0) return false;
    }
    *reinterpret_cast<volatile int*>(error_flag) = 1;
    return false;
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* error_flag) {
    return mbar_wait_limited(bar, parity, error_flag, TC_WAIT_LIMIT);
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(tc_smem_u32(smem_dst)), "l"(map), "r"(tc_smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile in the 128-byte swizzle: rows of 128 bytes, groups
// of 8 rows 1024 bytes apart (the stride byte offset); the leading byte offset is not used by this
// layout and carries its canonical value 1. Bits 46-47: descriptor version 1; bits 61-63: layout 2.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// Instruction descriptor of kind::f16: float32 accumulator, bfloat16 A and B, both K-major, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero) : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tc_smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld_16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// ---- thread-block clusters: rank, barrier, a float32 store into another block's shared memory ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

__device__ __forceinline__ void st_cluster_f32(uint32_t local_smem_addr, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(remote), "f"(v) : "memory");
}

// The driver's cuTensorMapEncodeTiled, looked up once through the runtime (nullptr when the driver has none).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn llmp_tensor_map_encoder();

// Tensor map over bfloat16 pages [num_pages, 2, nkv, page_size, 128], cached per tensor: boxes of box_tokens
// tokens of one page and key/value head and 64 elements, 128-byte swizzle; box_kv = 2 takes keys and values in one
// box; box_pages > 1 takes box_pages pages of consecutive page ids in one box (attention_prefill_tc.cu).
int llmp_pages_tensor_map(const void* pages, int nkv, int page_size, int num_pages, int box_tokens, int box_kv, int box_pages,
                          CUtensorMap* out);

// Five-dimensional box of the pages into shared memory: x = first element (0 or 64), token within the page,
// key/value head, 0 = keys or 1 = values, page. A page index out of range arrives as zeros.
__device__ __forceinline__ void tma_load_page_box(void* smem_dst, const CUtensorMap* map, int x, int token, int kvh, int kv,
                                                  int page, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n"
        ::"r"(tc_smem_u32(smem_dst)), "l"(map), "r"(tc_smem_u32(bar)), "r"(x), "r"(token), "r"(kvh), "r"(kv), "r"(page)
        : "memory");
}

// Tensor map over a [rows, K] bfloat16 row-major matrix with row pitch ld, seen as {64 elements, rows, K / 64
// blocks} and read in boxes of {64, box_rows, box_kb}: in shared memory box_kb planes of box_rows lines of 128 bytes
// in the 128-byte swizzle; cached per matrix (gemm_stream.cu).
int llmp_stream_tensor_map(const void* ptr, long rows, long k, long ld, int box_rows, int box_kb, CUtensorMap* out);

// Number of SMs of the current device (gemm_stream.cu).
int llmp_sm_count();

// Three-dimensional box into shared memory.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
        ::"r"(tc_smem_u32(smem_dst)), "l"(map), "r"(tc_smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
