// What the two streaming decode kernels for head size 128 share (attention_decode_tma.cu: a cluster of blocks per
// row group; attention_decode_list.cu: one list of key ranges dealt out evenly): the shape of a stage of the ring
// and a warp's work on one stage.
#pragma once
#include <cuda.h>

#include "attention_decode.cuh"
#include "common.cuh"
#include "tcgen05.cuh"

#define DT_D 128
#define DT_CWARPS 4                                  // compute warps: one key range of a wave each
#define DT_STAGE_KEYS 32
#define DT_ITEM_STAGES (DEC_SPLIT / DT_STAGE_KEYS)   // 4
#define DT_HALF_BYTES (DT_STAGE_KEYS * 128)          // 32 rows of 128 bytes: 64 elements of the head
#define DT_STAGE_BYTES (4 * DT_HALF_BYTES)           // K halves, then V halves: 16 KB
#define DT_STAGES 12
#define DT_THREADS ((DT_CWARPS + 1) * 32)
#define DT_MAX_HEADS 8                               // query heads per key/value head
#define DT_QSTRIDE (DT_D + 8)                        // padded query row, in elements

__device__ __forceinline__ void dt_ldmatrix_x4(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void dt_ldmatrix_x4_trans(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// D (16x8, float32) += A (16x16 bf16, row) * B (16x8 bf16, col)
__device__ __forceinline__ void dt_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned dt_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

// A stage holds 32 keys as [half of the head][box of box_tokens tokens][keys | values][token][64 elements]: one
// TMA box brings the keys and the values of a box's tokens for one half of the head. Address of 8 elements
// (16 bytes) of key row `key` (kv = 0) or value row (kv = 1) starting at element `elem` (a multiple of 8): rows of
// 128 bytes, 16-byte chunks swizzled with the row index.
__device__ __forceinline__ const unsigned char* dt_tile_at(const unsigned char* stage, int kv, int key, int elem, int box_shift) {
    const int b = key >> box_shift, i = key & ((1 << box_shift) - 1);
    return stage + (elem >> 6) * (2 * DT_HALF_BYTES) + ((b * 2 + kv) << (box_shift + 7)) + i * 128 + ((((elem & 63) >> 3) ^ (i & 7)) << 4);
}

__device__ __forceinline__ float dt_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Which of the 32 keys of the stage that starts at key0 lie in lo .. hi - 1, as a bit mask.
__device__ __forceinline__ unsigned dt_valid_keys(bool real, int lo, int hi, int key0) {
    int first = lo - key0, last = hi - key0;
    if (first < 0) first = 0;
    if (last > DT_STAGE_KEYS) last = DT_STAGE_KEYS;
    if (!real || last <= first) return 0u;
    return (last == 32 ? 0xffffffffu : ((1u << last) - 1u)) & ~((1u << first) - 1u);
}

// A warp's work on one stage with at least one valid key: S = Q K^T for the 8 query rows of the group (rows 8..15 of
// the tile are zero), the running maximum and sum of each row, O = O * alpha + P V. q_row is the lane's row of the
// query tile for ldmatrix; o, m_run (in units of log2) and l_run (the lane's share of the row sums) are the warp's
// running state for rows lane / 4 and lane / 4 + 8.
__device__ __forceinline__ void dt_stage_update(const unsigned char* stage, unsigned valid, const bf16* q_row, int lane,
                                                float scale_log2, int box_shift, float (&o)[DT_D / 8][4],
                                                float (&m_run)[2], float (&l_run)[2]) {
    const int t4 = lane & 3;
    float s[4][4];
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < DT_D / 16; ++ks) {
        unsigned a[4];
        dt_ldmatrix_x4(a, q_row + ks * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int nb = 0; nb < 4; nb += 2) {
            // four 8x8 blocks of K at once: keys nb*8.. and (nb+1)*8.., each with dims ks*16.. and ks*16+8..
            unsigned kf[4];
            dt_ldmatrix_x4(kf, dt_tile_at(stage, 0, (nb + (lane >> 4)) * 8 + (lane & 7), ks * 16 + ((lane >> 3) & 1) * 8, box_shift));
            dt_mma(s[nb], a, kf[0], kf[1]);
            dt_mma(s[nb + 1], a, kf[2], kf[3]);
        }
    }
    // mask keys outside the range; key of s[nb][c2] is nb*8 + 2 t4 + (c2 & 1), row g + 8*(c2 >> 1)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
        for (int c2 = 0; c2 < 4; ++c2) {
            if (valid != 0xffffffffu && !((valid >> (nb * 8 + 2 * t4 + (c2 & 1))) & 1u)) s[nb][c2] = -INFINITY;
            mx[c2 >> 1] = fmaxf(mx[c2 >> 1], s[nb][c2]);
        }
    }
    // running maximum and sum; at least one key of the stage is valid, so the new maximum is finite
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_run[h], mx[h] * scale_log2);
        alpha[h] = dt_ex2(m_run[h] - m_new);     // 0 while nothing was summed yet (2^-inf)
        m_run[h] = m_new;
        l_run[h] *= alpha[h];
    }
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
        for (int c2 = 0; c2 < 4; ++c2) {
            const float pr = dt_ex2(fmaf(s[nb][c2], scale_log2, -m_run[c2 >> 1]));
            s[nb][c2] = pr;
            l_run[c2 >> 1] += pr;
        }
    }
#pragma unroll
    for (int i = 0; i < DT_D / 8; ++i) {
        o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
        unsigned pa[4];
        pa[0] = dt_pack(s[2 * kk][0], s[2 * kk][1]);         // row g,     keys 16kk + 2 t4, +1
        pa[1] = dt_pack(s[2 * kk][2], s[2 * kk][3]);         // row g + 8
        pa[2] = dt_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]); // row g,     keys 16kk + 8 + 2 t4, +1
        pa[3] = dt_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]); // row g + 8
#pragma unroll
        for (int nb2 = 0; nb2 < DT_D / 16; ++nb2) {
            unsigned vv[4];
            dt_ldmatrix_x4_trans(vv, dt_tile_at(stage, 1, kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, nb2 * 16 + (lane >> 4) * 8, box_shift));
            dt_mma(o[nb2 * 2], pa, vv[0], vv[1]);
            dt_mma(o[nb2 * 2 + 1], pa, vv[2], vv[3]);
        }
    }
}
