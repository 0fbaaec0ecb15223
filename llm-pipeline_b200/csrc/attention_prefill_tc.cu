// Causal attention of prompt portions over bfloat16 pages on the fifth-generation tensor cores, head size 128,
// with the contract of llmp_paged_attention.
//
// A block takes 128 query rows of one request and one key/value head, a row being (token, query head of the
// group) with the head running fastest, so that the K and V tiles it streams serve every query head that
// shares the key/value head. Keys are walked in tiles of 128 aligned to key 0 (the same operations for a row
// however the prompt was cut). Per key tile:
//   S = Q K^T    one tcgen05.mma chain, Q and K in shared memory (128-byte swizzle, K-major), S in tensor memory
//   softmax      thread r owns row r: it reads the 128 scores of its row from tensor memory, keeps the running
//                maximum and sum in float32 and writes the probabilities back as bfloat16 over the first 64
//                columns of S
//   O += P V     one tcgen05.mma chain, P read from tensor memory as the A operand, V from shared memory as an
//                MN-major B operand (the head dimension is contiguous in a page), O in tensor memory
// The running maximum is only raised when a tile's maximum exceeds it by more than 8 (in log2 units): P then
// stays below 2^8 and O needs rescaling in the first tiles only; the result is the same softmax. The softmax
// reads its row twice from tensor memory, 32 columns at a time with the next 32 in flight (once for the
// maximum, once for the probabilities), which keeps it within 168 registers. K and V pages arrive by TMA, one
// box per page and half of the head (64 elements = one 128-byte swizzle span); a table entry that is missing
// or released is read at an out-of-range page coordinate, which the TMA unit fills with zeros.
// Roles: warps 0-3 softmax, warp 4 issues the loads (K of the next tile as soon as S is done, V as soon as
// P V is done), one thread of warp 5 issues the MMAs. Two blocks share an SM (96 KB of shared memory and 256
// tensor-memory columns each): while one is in its softmax the tensor cores work for the other.
//
// Long contexts: a tile of the list may come as up to FA_MAX_SEGMENTS items, each with an equal share of the tile's
// key tiles (tile_seg: item s of n; tile_slot: where the tile's items keep their sums), so that few query rows over
// many keys still fill the SMs and items are small against the whole. An item of a shared tile leaves its sums
// (O, the maximum they are scaled by, the row sum; float32) in global memory and counts itself with an atomic add;
// the item that counts last adds the sums in item order, normalises, stores and zeroes the counter. Nobody waits.
//
// Every wait on an mbarrier is bounded: when one runs out the kernel records 1 in *error_flag and goes on
// without waiting (its output is then wrong; the host reads the flag), so no thread is left behind at a
// barrier and the tensor memory is always freed.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

#define FA_ROWS 128
#define FA_KEYS 128
#define FA_D 128
#define FA_THREADS 192                           // four softmax warps, one load warp, one MMA warp
#define FA_HALF_BYTES (FA_ROWS * 128)            // 128 rows of 128 bytes
#define FA_TMEM_COLS 256                         // S (128 columns, P over its first 64) and O (128 columns)
#define FA_RESCALE_STEP 8.0f
#define FA_STAGGER_NS 1000
#define FA_MAX_SEGMENTS 8                        // items that may share the key tiles of one tile
#define FA_PART (FA_ROWS * FA_D + 2 * FA_ROWS)   // floats of an item's sums: O column by column, the rows' maxima, their sums

struct FaParams {
    const bf16* q;
    bf16* out;
    const int* block_tables;
    const int* q_start;
    const int* ctx_len;
    const int* tile_req;
    const int* tile_tok0;
    const int* tile_seg;     // null, or per item: its place among the items of its tile | their number << 8
    const int* tile_slot;    // per item of a shared tile: the first of the tile's places in `partials`
    float* partials;         // [places][nkv][FA_PART]
    unsigned* counters;      // [places][nkv], zero between launches
    long q_stride, out_stride;
    int table_stride;
    int nq, nkv, page_size, num_pages, window, tokens_per_cta, num_sms, num_tiles;
    int max_box_pages;       // the most pages a box may take (tensor maps exist up to this extent)
    float scale;
    int* error_flag;
};

__device__ __forceinline__ void fa_tma_load_page(void* smem_dst, const CUtensorMap* map, int x, int kvh, int kv, int page,
                                                 uint64_t* bar) {
    const int zero = 0;
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n"
        ::"r"(tc_smem_u32(smem_dst)), "l"(map), "r"(tc_smem_u32(bar)), "r"(x), "r"(zero), "r"(kvh), "r"(kv), "r"(page)
        : "memory");
}

// Shared-memory descriptor of an MN-major operand in the 128-byte swizzle: rows of 64 contiguous elements of
// the MN dimension, one row per K index, groups of 8 K indices 1024 bytes apart (stride byte offset), the
// next 64 elements of the MN dimension 16 KB further (leading byte offset).
__device__ __forceinline__ uint64_t fa_desc_mn_major(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(FA_HALF_BYTES >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from tensor memory (bfloat16 pairs per 32-bit column).
__device__ __forceinline__ void fa_umma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero) : "memory");
}

// 32 consecutive 32-bit columns of this thread's tensor-memory lane into r[OFF .. OFF + 31] (no wait).
#define FA_TMEM_LD32(taddr, r, OFF)                                                                                     \
    asm volatile(                                                                                                       \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, " \
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"                      \
        : "=r"(r[OFF + 0]), "=r"(r[OFF + 1]), "=r"(r[OFF + 2]), "=r"(r[OFF + 3]), "=r"(r[OFF + 4]), "=r"(r[OFF + 5]),   \
          "=r"(r[OFF + 6]), "=r"(r[OFF + 7]), "=r"(r[OFF + 8]), "=r"(r[OFF + 9]), "=r"(r[OFF + 10]), "=r"(r[OFF + 11]), \
          "=r"(r[OFF + 12]), "=r"(r[OFF + 13]), "=r"(r[OFF + 14]), "=r"(r[OFF + 15]), "=r"(r[OFF + 16]),                \
          "=r"(r[OFF + 17]), "=r"(r[OFF + 18]), "=r"(r[OFF + 19]), "=r"(r[OFF + 20]), "=r"(r[OFF + 21]),                \
          "=r"(r[OFF + 22]), "=r"(r[OFF + 23]), "=r"(r[OFF + 24]), "=r"(r[OFF + 25]), "=r"(r[OFF + 26]),                \
          "=r"(r[OFF + 27]), "=r"(r[OFF + 28]), "=r"(r[OFF + 29]), "=r"(r[OFF + 30]), "=r"(r[OFF + 31])                 \
        : "r"(taddr))

// r[OFF .. OFF + 31] into 32 consecutive 32-bit columns of this thread's tensor-memory lane (no wait).
#define FA_TMEM_ST32(taddr, r, OFF)                                                                                     \
    asm volatile(                                                                                                       \
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, " \
        "%15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};\n"                        \
        ::"r"(r[OFF + 0]), "r"(r[OFF + 1]), "r"(r[OFF + 2]), "r"(r[OFF + 3]), "r"(r[OFF + 4]), "r"(r[OFF + 5]),          \
          "r"(r[OFF + 6]), "r"(r[OFF + 7]), "r"(r[OFF + 8]), "r"(r[OFF + 9]), "r"(r[OFF + 10]), "r"(r[OFF + 11]),        \
          "r"(r[OFF + 12]), "r"(r[OFF + 13]), "r"(r[OFF + 14]), "r"(r[OFF + 15]), "r"(r[OFF + 16]), "r"(r[OFF + 17]),    \
          "r"(r[OFF + 18]), "r"(r[OFF + 19]), "r"(r[OFF + 20]), "r"(r[OFF + 21]), "r"(r[OFF + 22]), "r"(r[OFF + 23]),    \
          "r"(r[OFF + 24]), "r"(r[OFF + 25]), "r"(r[OFF + 26]), "r"(r[OFF + 27]), "r"(r[OFF + 28]), "r"(r[OFF + 29]),    \
          "r"(r[OFF + 30]), "r"(r[OFF + 31]), "r"(taddr)                                                                \
        : "memory")

__device__ __forceinline__ void fa_tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void fa_tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void fa_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fa_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// 2^x by the special-function unit (relative error about 2^-22; the probabilities are rounded to bfloat16 anyway)
__device__ __forceinline__ float fa_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t fa_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Applies the causal and window mask of one row to 32 scores that start at key `key0`.
__device__ __forceinline__ void fa_mask32(uint32_t (&v)[32], int key0, int last_ok, int first_ok) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const int key = key0 + i;
        if (key > last_ok || key < first_ok) v[i] = 0xff800000u;           // -inf
    }
}

__device__ __forceinline__ float fa_max32(const uint32_t (&v)[32], float mx) {
    float m0 = mx, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;          // four chains: no serial dependency
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        m0 = fmaxf(m0, __uint_as_float(v[i]));
        m1 = fmaxf(m1, __uint_as_float(v[i + 1]));
        m2 = fmaxf(m2, __uint_as_float(v[i + 2]));
        m3 = fmaxf(m3, __uint_as_float(v[i + 3]));
    }
    return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// 32 scores -> 16 packed bfloat16 pairs of 2^(s * scale - m); returns their float32 sum.
__device__ __forceinline__ float fa_exp32(const uint32_t (&v)[32], uint32_t (&pk)[16], float scale_log2, float m_eff) {
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        const float p0 = fa_ex2(fmaf(__uint_as_float(v[i]), scale_log2, -m_eff));
        const float p1 = fa_ex2(fmaf(__uint_as_float(v[i + 1]), scale_log2, -m_eff));
        s0 += p0;
        s1 += p1;
        pk[i >> 1] = fa_pack(p0, p1);
    }
    return s0 + s1;
}

#define FA_TMEM_ST16(taddr, r)                                                                                          \
    asm volatile(                                                                                                       \
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, " \
        "%15};\n"                                                                                                        \
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),  \
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)                            \
        : "memory")

// Warps 0-3: softmax (thread r owns row r and tensor-memory lane r). Warp 4: TMA loads. Warp 5: MMA issue.
__global__ void __launch_bounds__(FA_THREADS, 2)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_pages, const __grid_constant__ CUtensorMap map_pages2,
                            const __grid_constant__ CUtensorMap map_pages4, const __grid_constant__ CUtensorMap map_pages8, const FaParams p) {
    extern __shared__ unsigned char fa_raw[];
    __shared__ __align__(8) uint64_t k_full, v_full, s_done, o_done, p_ready;
    __shared__ uint32_t tmem_slot;
    __shared__ unsigned arrived_before;
    // the swizzled tiles want 1024-byte alignment
    const uint32_t raw_addr = tc_smem_u32(fa_raw);
    unsigned char* Qs = fa_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);   // [2 halves][128 rows][128 bytes]
    unsigned char* Ks = Qs + 2 * FA_HALF_BYTES;
    unsigned char* Vs = Ks + 2 * FA_HALF_BYTES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Later tiles of a prompt see more keys. Blocks start in the order of their index: the key/value heads of the
    // last tile first, then those of the tile before, so that the long blocks do not form the tail.
    const int tile = p.num_tiles - 1 - (int)(blockIdx.x / (unsigned)p.nkv);
    const int kvh = (int)(blockIdx.x % (unsigned)p.nkv);
    const int r = p.tile_req[tile];
    const int tok0 = p.tile_tok0[tile];
    const int G = p.nq / p.nkv;
    const int q_begin = p.q_start[r];
    const int q_len = p.q_start[r + 1] - q_begin;
    const int ctx = p.ctx_len[r];
    const int pos0 = ctx - q_len;
    int ntok = q_len - tok0;
    if (ntok > p.tokens_per_cta) ntok = p.tokens_per_cta;
    const int* table = p.block_tables + (size_t)r * p.table_stride;

    // keys this block needs: from the window start of its first token to the position of its last
    const int hi = pos0 + tok0 + ntok - 1;                             // last key (inclusive)
    int lo = 0;
    if (p.window > 0) {
        lo = pos0 + tok0 - p.window + 1;
        if (lo < 0) lo = 0;
    }
    const int first_tile_lo = (lo / FA_KEYS) * FA_KEYS;
    const int all_key_tiles = (hi - first_tile_lo) / FA_KEYS + 1;
    // this item's share of the tile's key tiles
    int seg = 0, nseg = 1, slot0 = 0;
    if (p.tile_seg != nullptr) {
        const int packed = p.tile_seg[tile];
        seg = packed & 0xff;
        nseg = (packed >> 8) & 0xff;
        slot0 = p.tile_slot[tile];
    }
    const int seg_begin = (int)((long)all_key_tiles * seg / nseg);
    const int tile_lo = first_tile_lo + seg_begin * FA_KEYS;
    const int num_key_tiles = (int)((long)all_key_tiles * (seg + 1) / nseg) - seg_begin;      // 0: more items than key tiles
    const int pages_per_tile = FA_KEYS / p.page_size;

    // warp 4: the boxes of the K and V tile j, one lane per (page, half of the head). Pages whose ids follow one another
    // come in one box: an aligned group of 2, 4 or 8 pages of the tile (the layout in shared memory is the same, page
    // after page). Pages of 16 tokens are 32 boxes of 2 KB a tile page by page; with a request's pages in ascending
    // order (what the page pool hands out, also after reuse) they are 4 boxes of 16 KB: 74.7 -> 71.7 us at 2,048 tokens.
    auto load_tile = [&](int j) {
        const int j0 = tile_lo + j * FA_KEYS;
        const int pg = lane >> 1;                                      // this lane's page of the tile (page sizes from 8 on: 32 boxes at most)
        const bool mine = lane < pages_per_tile * 2;
        int page = -1;                                                 // -1: read at an out-of-range page, which arrives as zeros
        {
            const int key = j0 + pg * p.page_size;
            if (mine && key <= hi) page = table[key / p.page_size];
        }
        // the group of this lane's page: 8, 4 or 2 pages whose ids follow one another, else the page alone
        const int delta = page >= 0 ? page - pg : -(1 << 28) - pg;     // equal over a run of consecutive ids; unique where a page is missing
        // (every lane takes part in every shuffle: none of them may sit behind a short-circuit)
        const int delta2 = __shfl_xor_sync(0xffffffffu, delta, 2), delta4 = __shfl_xor_sync(0xffffffffu, delta, 4);
        const int delta8 = __shfl_xor_sync(0xffffffffu, delta, 8);
        const bool eq2 = delta == delta2;
        const int other2 = __shfl_xor_sync(0xffffffffu, (int)eq2, 4);
        const bool eq4 = eq2 && other2 != 0 && delta == delta4;
        const int other4 = __shfl_xor_sync(0xffffffffu, (int)eq4, 8);
        const bool eq8 = eq4 && other4 != 0 && delta == delta8;
        int group = 1;
        if (eq8 && pages_per_tile >= 8 && p.max_box_pages >= 8) group = 8;
        else if (eq4 && pages_per_tile >= 4 && p.max_box_pages >= 4) group = 4;
        else if (eq2 && pages_per_tile >= 2 && p.max_box_pages >= 2) group = 2;
        const CUtensorMap* map = group == 8 ? &map_pages8 : (group == 4 ? &map_pages4 : (group == 2 ? &map_pages2 : &map_pages));
        const bool leads = mine && (pg & (group - 1)) == 0;
#pragma unroll
        for (int kv = 0; kv < 2; ++kv) {
            // K is free when S of the tile before is done, V when its P V is done
            if (j > 0) mbar_wait(kv == 0 ? &s_done : &o_done, (uint32_t)((j - 1) & 1), p.error_flag);
            uint64_t* bar = kv == 0 ? &k_full : &v_full;
            unsigned char* dst = kv == 0 ? Ks : Vs;
            if (lane == 0) mbar_expect_tx(bar, 2 * FA_HALF_BYTES);
            __syncwarp();
            if (leads)
                fa_tma_load_page(dst + (lane & 1) * FA_HALF_BYTES + pg * p.page_size * 128, map, (lane & 1) * 64, kvh, kv,
                                 page >= 0 ? page : p.num_pages, bar);
        }
    };

    if (warp == 4) {
        // the barriers, and at once the first K and V tiles: they need nothing but the block table
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_pages) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_pages8) : "memory");
            mbar_init(&k_full, 1);
            mbar_init(&v_full, 1);
            mbar_init(&s_done, 1);
            mbar_init(&o_done, 1);
            mbar_init(&p_ready, FA_ROWS);
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        }
        __syncwarp();
        if (num_key_tiles > 0) load_tile(0);
    } else if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem_u32(&tmem_slot)), "r"(FA_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    } else {
        // Query rows into shared memory in the layout of a K-major operand: row = token * G + head, 16-byte chunk
        // c of a row at chunk position (c % 8) ^ (row % 8) of the row's 128-byte line in half c / 8. All loads of
        // a thread are in flight before its first store.
        constexpr int PER_THREAD = FA_ROWS * 16 / 128;
        uint4 v[PER_THREAD];
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int e = tid + i * 128;
            const int row = e >> 4, c = e & 15;
            const int tl = row / G, h = row - tl * G;
            v[i] = make_uint4(0u, 0u, 0u, 0u);
            if (tl < ntok)
                v[i] = *reinterpret_cast<const uint4*>(p.q + (size_t)(q_begin + tok0 + tl) * p.q_stride + (size_t)(kvh * G + h) * FA_D + c * 8);
        }
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int e = tid + i * 128;
            const int row = e >> 4, c = e & 15;
            *reinterpret_cast<uint4*>(Qs + (c >> 3) * FA_HALF_BYTES + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = v[i];
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    fa_fence_before();
    __syncthreads();
    fa_fence_after();
    const uint32_t tmem_base = tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + FA_KEYS;

    if (warp == 4) {
        // ---- loads of the later tiles ----
        for (int j = 1; j < num_key_tiles; ++j) load_tile(j);
    } else if (warp == 5) {
        // ---- MMA issue ----
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc(FA_ROWS, FA_KEYS);
            constexpr uint32_t idesc_o = umma_idesc(FA_ROWS, FA_D) | (1u << 16);     // B is MN-major
            const uint32_t q_addr = tc_smem_u32(Qs), k_addr = tc_smem_u32(Ks), v_addr = tc_smem_u32(Vs);
            // The two blocks of an SM start together and would stay in step: both on the tensor cores, then both in
            // their softmax. The second block of each SM starts half a tile later, so that one's MMAs run under the
            // other's softmax.
            if ((blockIdx.x / p.num_sms) & 1) __nanosleep(FA_STAGGER_NS);
            for (int j = 0; j < num_key_tiles; ++j) {
                const uint32_t parity = (uint32_t)(j & 1);
                if (j == 0) mbar_wait(&k_full, 0, p.error_flag);       // later tiles: waited for below, ahead of time
                fa_fence_after();
#pragma unroll
                for (int k = 0; k < FA_D / 16; ++k) {
                    const uint32_t off = (uint32_t)(k >> 2) * FA_HALF_BYTES + (uint32_t)(k & 3) * 32;
                    umma_f16(tmem_s, umma_desc(q_addr + off), umma_desc(k_addr + off), idesc_s, k != 0 ? 1u : 0u);
                }
                umma_commit(&s_done);
                // V of this tile and K of the next have long been asked for: take these waits while the softmax works
                mbar_wait(&v_full, parity, p.error_flag);
                if (j + 1 < num_key_tiles) mbar_wait(&k_full, parity ^ 1u, p.error_flag);
                mbar_wait(&p_ready, parity, p.error_flag);
                fa_fence_after();
#pragma unroll
                for (int k = 0; k < FA_KEYS / 16; ++k)                  // 16 keys per MMA: 8 columns of P, 2 KB of V
                    fa_umma_a_tmem(tmem_o, tmem_s + (uint32_t)k * 8, fa_desc_mn_major(v_addr + (uint32_t)k * 2048), idesc_o,
                                   (j | k) != 0 ? 1u : 0u);
                umma_commit(&o_done);
            }
        }
    } else {
        // ---- softmax: this thread's row ----
        const uint32_t lane_field = (uint32_t)(warp * 32) << 16;      // this warp's quarter of the lanes
        const int my_tl = tid / G;
        const int my_head = tid - my_tl * G;
        const int my_pos = my_tl < ntok ? pos0 + tok0 + my_tl : -1;   // -1: the row does not exist
        const int first_ok = p.window > 0 ? my_pos - p.window + 1 : 0;
        const int first_pos = pos0 + tok0;                             // lowest position among the block's rows
        const float scale_log2 = p.scale * 1.4426950408889634f;
        float m_used = -INFINITY, l_run = 0.f;
        uint32_t a[32], b[32];
        for (int j = 0; j < num_key_tiles; ++j) {
            const int j0 = tile_lo + j * FA_KEYS;
            const bool need_mask = (j0 + FA_KEYS - 1 > first_pos) || (p.window > 0 && j0 < hi - p.window + 1);
            mbar_wait(&s_done, (uint32_t)(j & 1), p.error_flag);      // also: P V of the tile before is done
            fa_fence_after();
            // pass 1: the row's maximum; the load of the next 32 columns is in flight while 32 are reduced
            float mx = -INFINITY;
            FA_TMEM_LD32(tmem_s + lane_field + 0, a, 0);
            fa_tmem_wait_ld();
            FA_TMEM_LD32(tmem_s + lane_field + 32, b, 0);
            if (need_mask) fa_mask32(a, j0, my_pos, first_ok);
            mx = fa_max32(a, mx);
            fa_tmem_wait_ld();
            FA_TMEM_LD32(tmem_s + lane_field + 64, a, 0);
            if (need_mask) fa_mask32(b, j0 + 32, my_pos, first_ok);
            mx = fa_max32(b, mx);
            fa_tmem_wait_ld();
            FA_TMEM_LD32(tmem_s + lane_field + 96, b, 0);
            if (need_mask) fa_mask32(a, j0 + 64, my_pos, first_ok);
            mx = fa_max32(a, mx);
            fa_tmem_wait_ld();
            FA_TMEM_LD32(tmem_s + lane_field + 0, a, 0);               // first columns again, for pass 2
            if (need_mask) fa_mask32(b, j0 + 96, my_pos, first_ok);
            mx = fa_max32(b, mx);

            const float m_tile = mx * scale_log2;
            const bool raise = m_tile > m_used + FA_RESCALE_STEP;
            float alpha = 1.f;
            if (raise) {
                alpha = fa_ex2(m_used - m_tile);
                m_used = m_tile;
                l_run *= alpha;
            }
            fa_tmem_wait_ld();
            if (j > 0 && __any_sync(0xffffffffu, raise)) {             // O holds the sum of the tiles before
#pragma unroll
                for (int c = 0; c < FA_D; c += 32) {
                    FA_TMEM_LD32(tmem_o + lane_field + c, b, 0);
                    fa_tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) b[i] = __float_as_uint(__uint_as_float(b[i]) * alpha);
                    FA_TMEM_ST32(tmem_o + lane_field + c, b, 0);
                }
            }
            // pass 2: probabilities as bfloat16 pairs over the first 64 columns of S (16 columns per 32 scores:
            // always columns that were read before)
            const float m_eff = m_used > -INFINITY ? m_used : 0.f;    // a row without any key keeps p = 2^(-inf) = 0
            uint32_t pk[16];
            float sum = 0.f;
            FA_TMEM_LD32(tmem_s + lane_field + 32, b, 0);
            if (need_mask) fa_mask32(a, j0, my_pos, first_ok);
            sum += fa_exp32(a, pk, scale_log2, m_eff);
            fa_tmem_wait_ld();
            FA_TMEM_LD32(tmem_s + lane_field + 64, a, 0);
            FA_TMEM_ST16(tmem_s + lane_field + 0, pk);
            if (need_mask) fa_mask32(b, j0 + 32, my_pos, first_ok);
            sum += fa_exp32(b, pk, scale_log2, m_eff);
            fa_tmem_wait_ld();
            FA_TMEM_LD32(tmem_s + lane_field + 96, b, 0);
            FA_TMEM_ST16(tmem_s + lane_field + 16, pk);
            if (need_mask) fa_mask32(a, j0 + 64, my_pos, first_ok);
            sum += fa_exp32(a, pk, scale_log2, m_eff);
            fa_tmem_wait_ld();
            FA_TMEM_ST16(tmem_s + lane_field + 32, pk);
            if (need_mask) fa_mask32(b, j0 + 96, my_pos, first_ok);
            sum += fa_exp32(b, pk, scale_log2, m_eff);
            FA_TMEM_ST16(tmem_s + lane_field + 48, pk);
            l_run += sum;
            fa_tmem_wait_st();
            fa_fence_before();
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem_u32(&p_ready)) : "memory");
        }

        // O is complete when the last P V is done
        if (num_key_tiles > 0) mbar_wait(&o_done, (uint32_t)((num_key_tiles - 1) & 1), p.error_flag);
        fa_fence_after();
        bf16* dst = p.out + (size_t)(q_begin + tok0 + (my_pos >= 0 ? my_tl : 0)) * p.out_stride + (size_t)(kvh * G + my_head) * FA_D;
        if (nseg == 1) {
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
            for (int c = 0; c < FA_D; c += 32) {
                FA_TMEM_LD32(tmem_o + lane_field + c, a, 0);
                fa_tmem_wait_ld();
                if (my_pos >= 0) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 pack;
                        pack.x = fa_pack(__uint_as_float(a[i]) * inv, __uint_as_float(a[i + 1]) * inv);
                        pack.y = fa_pack(__uint_as_float(a[i + 2]) * inv, __uint_as_float(a[i + 3]) * inv);
                        pack.z = fa_pack(__uint_as_float(a[i + 4]) * inv, __uint_as_float(a[i + 5]) * inv);
                        pack.w = fa_pack(__uint_as_float(a[i + 6]) * inv, __uint_as_float(a[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c + i) = pack;
                    }
                }
            }
        } else {
            // ---- an item of a shared tile: its sums to global memory; the item that counts last adds them up ----
            float* part = p.partials + ((size_t)(slot0 + seg) * p.nkv + kvh) * FA_PART;
            if (num_key_tiles > 0) {
#pragma unroll
                for (int c = 0; c < FA_D; c += 32) {
                    FA_TMEM_LD32(tmem_o + lane_field + c, a, 0);
                    fa_tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) part[(size_t)(c + i) * FA_ROWS + tid] = __uint_as_float(a[i]);   // column by column: the lanes of a warp write one line
                }
            }
            part[FA_ROWS * FA_D + tid] = num_key_tiles > 0 ? m_used : -INFINITY;
            part[FA_ROWS * FA_D + FA_ROWS + tid] = num_key_tiles > 0 ? l_run : 0.f;
            __threadfence();                                         // the sums are visible before the count is
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            if (tid == 0) arrived_before = atomicAdd(&p.counters[(size_t)slot0 * p.nkv + kvh], 1u);
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            if (arrived_before == (unsigned)(nseg - 1)) {
                __threadfence();
                const float* first = p.partials + ((size_t)slot0 * p.nkv + kvh) * FA_PART;
                // weights of the items' sums for this row: 2^(m_s - m) with m the largest maximum
                float wgt[FA_MAX_SEGMENTS];
                float m = -INFINITY, l = 0.f;
#pragma unroll
                for (int x = 0; x < FA_MAX_SEGMENTS; ++x) {
                    wgt[x] = x < nseg ? __ldcg(first + (size_t)x * p.nkv * FA_PART + FA_ROWS * FA_D + tid) : -INFINITY;
                    m = fmaxf(m, wgt[x]);
                }
#pragma unroll
                for (int x = 0; x < FA_MAX_SEGMENTS; ++x) {
                    wgt[x] = wgt[x] > -INFINITY ? fa_ex2(wgt[x] - m) : 0.f;
                    if (x < nseg && wgt[x] != 0.f) l = fmaf(__ldcg(first + (size_t)x * p.nkv * FA_PART + FA_ROWS * FA_D + FA_ROWS + tid), wgt[x], l);
                }
                const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
                for (int c = 0; c < FA_D; c += 32) {
                    float acc[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
#pragma unroll
                    for (int x = 0; x < FA_MAX_SEGMENTS; ++x) {
                        if (x < nseg && wgt[x] != 0.f) {              // an item without keys for this row left no sums
                            const float* src = first + (size_t)x * p.nkv * FA_PART + (size_t)c * FA_ROWS + tid;
                            float v[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = __ldcg(src + (size_t)i * FA_ROWS);
#pragma unroll
                            for (int i = 0; i < 32; ++i) acc[i] = fmaf(v[i], wgt[x], acc[i]);
                        }
                    }
                    if (my_pos >= 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 pack;
                            pack.x = fa_pack(acc[i] * inv, acc[i + 1] * inv);
                            pack.y = fa_pack(acc[i + 2] * inv, acc[i + 3] * inv);
                            pack.z = fa_pack(acc[i + 4] * inv, acc[i + 5] * inv);
                            pack.w = fa_pack(acc[i + 6] * inv, acc[i + 7] * inv);
                            *reinterpret_cast<uint4*>(dst + c + i) = pack;
                        }
                    }
                }
                if (tid == 0) p.counters[(size_t)slot0 * p.nkv + kvh] = 0u;      // for the next launch
            }
        }
    }
    fa_fence_before();
    __syncthreads();
    if (warp == 5) {
        fa_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(FA_TMEM_COLS) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------------------
struct PagesKey {
    const void* ptr;
    int nkv, page_size, num_pages, box_tokens, box_kv, box_pages;
    bool operator==(const PagesKey& o) const {
        return ptr == o.ptr && nkv == o.nkv && page_size == o.page_size && num_pages == o.num_pages && box_tokens == o.box_tokens &&
               box_kv == o.box_kv && box_pages == o.box_pages;
    }
};
struct PagesKeyHash {
    size_t operator()(const PagesKey& k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ (size_t)k.nkv;
        h = h * 1000003u ^ (size_t)k.page_size;
        h = h * 1000003u ^ (size_t)k.num_pages;
        h = h * 1000003u ^ (size_t)k.box_tokens;
        h = h * 1000003u ^ (size_t)k.box_pages;
        return h * 1000003u ^ (size_t)k.box_kv;
    }
};

// Pages [num_pages, 2, nkv, page_size, 128] of bfloat16, read in boxes of box_tokens tokens of one page and head
// and 64 elements (128-byte swizzle); box_kv = 2 takes the keys and the values of these tokens in one box (keys first);
// box_pages > 1 takes that of box_pages pages with consecutive page ids in one box (page after page).
int llmp_pages_tensor_map(const void* pages, int nkv, int page_size, int num_pages, int box_tokens, int box_kv, int box_pages,
                          CUtensorMap* out) {
    static std::unordered_map<PagesKey, CUtensorMap, PagesKeyHash> cache;
    static std::mutex lock;
    const PagesKey key{pages, nkv, page_size, num_pages, box_tokens, box_kv, box_pages};
    std::lock_guard<std::mutex> guard(lock);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return 0;
    }
    EncodeTiledFn fn = llmp_tensor_map_encoder();
    LLMP_REQUIRE(fn != nullptr, "attention: the driver does not provide cuTensorMapEncodeTiled");
    const cuuint64_t row = FA_D * sizeof(bf16);
    const cuuint64_t dims[5] = {FA_D, (cuuint64_t)page_size, (cuuint64_t)nkv, 2, (cuuint64_t)num_pages};
    const cuuint64_t strides[4] = {row, row * page_size, row * page_size * nkv, row * page_size * nkv * 2};
    const cuuint32_t box[5] = {64, (cuuint32_t)box_tokens, 1, (cuuint32_t)box_kv, (cuuint32_t)box_pages};
    const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    const CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(pages), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    LLMP_REQUIRE(rc == CUDA_SUCCESS, "attention: cuTensorMapEncodeTiled failed with code %d", (int)rc);
    if (cache.size() > 1024) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

// Sizes this kernel takes: head size 128, pages of 8, 16, 32, 64 or 128 tokens, groups of up to 128 query heads.
bool llmp_prefill_tc_supports(int nq, int nkv, int d, int page_size) {
    if (d != FA_D || nkv <= 0 || nq % nkv != 0 || nq / nkv > FA_ROWS) return false;
    return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
}

// Query tokens per block for a group size: 128 rows of (token, head).
int llmp_prefill_tc_tokens_per_tile(int nq, int nkv) { return FA_ROWS / (nq / nkv); }

// Items that may share a tile's keys, and the floats of one place (one item and key/value head) for their sums.
int llmp_prefill_tc_max_segments() { return FA_MAX_SEGMENTS; }
long llmp_prefill_tc_place_floats() { return FA_PART; }

int llmp_launch_prefill_tc(const void* q, long q_stride, void* out, long out_stride, const void* pages, int num_pages,
                           const int* block_tables, int table_stride, const int* q_start, const int* ctx_len,
                           const int* tile_req, const int* tile_tok0, const int* tile_seg, const int* tile_slot,
                           float* partials, unsigned* counters, int num_tiles, int nq, int nkv, int page_size,
                           int window, float scale, int* error_flag, cudaStream_t stream) {
    LLMP_REQUIRE(error_flag != nullptr, "attention: an error flag in device memory is required");
    LLMP_REQUIRE(tile_seg == nullptr || (tile_slot != nullptr && partials != nullptr && counters != nullptr),
                 "attention: tiles whose keys are shared need places for their sums and counters");
    LLMP_REQUIRE((q_stride % 8) == 0 && (out_stride % 8) == 0 && ((size_t)q % 16) == 0 && ((size_t)out % 16) == 0 &&
                 ((size_t)pages % 16) == 0, "attention: rows must be 16-byte aligned");
    CUtensorMap map, map2, map4, map8;
    if (llmp_pages_tensor_map(pages, nkv, page_size, num_pages, page_size, 1, 1, &map)) return 1;
    // boxes of 2, 4 and 8 pages with consecutive ids, as far as a key tile has that many pages and the pool too
    const int pages_per_tile = FA_KEYS / page_size;
    int max_box_pages = 1;
    map2 = map4 = map8 = map;
    if (pages_per_tile >= 2 && num_pages >= 2) { if (llmp_pages_tensor_map(pages, nkv, page_size, num_pages, page_size, 1, 2, &map2)) return 1; max_box_pages = 2; }
    if (pages_per_tile >= 4 && num_pages >= 4) { if (llmp_pages_tensor_map(pages, nkv, page_size, num_pages, page_size, 1, 4, &map4)) return 1; max_box_pages = 4; }
    if (pages_per_tile >= 8 && num_pages >= 8) { if (llmp_pages_tensor_map(pages, nkv, page_size, num_pages, page_size, 1, 8, &map8)) return 1; max_box_pages = 8; }
    FaParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.block_tables = block_tables; p.q_start = q_start; p.ctx_len = ctx_len;
    p.tile_req = tile_req; p.tile_tok0 = tile_tok0; p.tile_seg = tile_seg; p.tile_slot = tile_slot; p.partials = partials;
    p.counters = counters; p.q_stride = q_stride; p.out_stride = out_stride;
    p.table_stride = table_stride; p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.num_pages = num_pages;
    p.window = window; p.tokens_per_cta = llmp_prefill_tc_tokens_per_tile(nq, nkv); p.scale = scale;
    p.error_flag = error_flag;
    p.max_box_pages = max_box_pages;
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    p.num_sms = sms;
    p.num_tiles = num_tiles;
    const size_t smem = 6 * (size_t)FA_HALF_BYTES + 1024;
    LLMP_ALLOW_SMEM(prefill_attention_tc_kernel, smem);
    LLMP_REQUIRE((long)num_tiles * nkv < (1L << 31), "attention: too many tiles");
    prefill_attention_tc_kernel<<<(unsigned)(num_tiles * nkv), FA_THREADS, smem, stream>>>(map, map2, map4, map8, p);
    return llmp_check_launch("prefill_attention_tc");
}
