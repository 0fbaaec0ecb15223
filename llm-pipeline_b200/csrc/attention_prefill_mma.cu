// Causal attention of prompt portions (and of any mixed batch) over bfloat16 pages on the tensor cores
// (mma.sync m16n8k16, float32 accumulate), with the contract of llmp_paged_attention.
//
// A block takes one tile of query rows of one request and one key/value head: PF_ROWS = 64 rows, a row
// being (token, query head of the group) with the head running fastest, so the K and V tiles it
// streams serve all query heads that share the key/value head. Each of the four warps owns 16 rows
// and keeps their online softmax and output in registers. Keys are walked in tiles of 64 aligned to
// key 0 (the same operations for a row however the prompt was cut), copied from the pages with
// 16-byte cp.async into one shared-memory tile per block (four blocks share an SM and cover each
// other's copies); tiles entirely above the causal diagonal or below the window are skipped.
#include "common.cuh"

#define PF_ROWS 64
#define PF_KEYS 64
#define PF_THREADS 128

struct PrefillParams {
    const bf16* q;
    bf16* out;
    const bf16* pages;
    const int* block_tables;
    const int* q_start;
    const int* ctx_len;
    const int* tile_req;
    const int* tile_tok0;
    long q_stride, out_stride;
    int table_stride;
    int nq, nkv, d, page_size, window;
    int heads_per_cta, tokens_per_cta, head_chunks, num_tiles;
    float scale;
};

__device__ __forceinline__ void pf_cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void pf_ldmatrix_x4(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void pf_ldmatrix_x4_trans(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void pf_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x by the special-function unit (relative error about 2^-22; the probabilities are rounded to bfloat16 anyway)
__device__ __forceinline__ float pf_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ unsigned pf_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

// D16: head size / 16 (the K steps of Q K^T; the output has 2 * D16 blocks of 8 columns).
template <int D16>
__global__ void __launch_bounds__(PF_THREADS, 4) prefill_attention_mma_kernel(const PrefillParams p) {
    extern __shared__ __align__(16) unsigned char pf_smem[];
    constexpr int D = D16 * 16;
    constexpr int STRIDE = D + 8;                                // padded rows: conflict-free ldmatrix
    constexpr int VEC_PER_ROW = D / 8;
    bf16* Qs = reinterpret_cast<bf16*>(pf_smem);                 // [PF_ROWS][STRIDE]
    bf16* ring = Qs + PF_ROWS * STRIDE;                          // [K tile | V tile], each [PF_KEYS][STRIDE]
    constexpr int STAGE_ELEMS = 2 * PF_KEYS * STRIDE;
    __shared__ long long key_off[1][PF_KEYS];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    // Later tiles of a prompt see more keys. Blocks start in the order of their index: every head of the last tile
    // first, then those of the tile before, so that the long blocks do not form the tail.
    const int per_tile = p.nkv * p.head_chunks;
    const int tile = p.num_tiles - 1 - (int)(blockIdx.x / (unsigned)per_tile);
    const int in_tile = (int)(blockIdx.x % (unsigned)per_tile);
    const int r = p.tile_req[tile];
    const int tok0 = p.tile_tok0[tile];
    const int kvh = in_tile / p.head_chunks, chunk = in_tile % p.head_chunks;
    const int G = p.nq / p.nkv;
    const int hpc = p.heads_per_cta;
    const int head0 = chunk * hpc;
    int heads = G - head0;
    if (heads > hpc) heads = hpc;
    const int q_begin = p.q_start[r];
    const int q_len = p.q_start[r + 1] - q_begin;
    const int ctx = p.ctx_len[r];
    const int pos0 = ctx - q_len;
    int ntok = q_len - tok0;
    if (ntok > p.tokens_per_cta) ntok = p.tokens_per_cta;
    const int* table = p.block_tables + (size_t)r * p.table_stride;
    const size_t plane = (size_t)p.nkv * p.page_size * D;

    // query rows: row = token * hpc + head
    for (int e = tid; e < PF_ROWS * VEC_PER_ROW; e += PF_THREADS) {
        const int row = e / VEC_PER_ROW, c = (e % VEC_PER_ROW) * 8;
        const int tl = row / hpc, h = row % hpc;
        const bool ok = tl < ntok && h < heads;
        const bf16* src = ok ? p.q + (size_t)(q_begin + tok0 + tl) * p.q_stride + (size_t)(kvh * G + head0 + h) * D + c : p.q;
        pf_cp_async_16(Qs + row * STRIDE + c, src, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");

    // keys this block needs: from the window start of its first token to the position of its last
    const int hi = pos0 + tok0 + ntok - 1;                       // last key (inclusive)
    int lo = 0;
    if (p.window > 0) {
        lo = pos0 + tok0 - p.window + 1;
        if (lo < 0) lo = 0;
    }
    auto issue_tile = [&](int j0, int buf) {
        if (tid < PF_KEYS) {
            const int j = j0 + tid;
            long long off = -1;
            if (j <= hi) {
                const int page = table[j / p.page_size];
                if (page >= 0)
                    off = (long long)((((size_t)page * 2) * p.nkv + kvh) * p.page_size + (j % p.page_size)) * D;
            }
            key_off[buf][tid] = off;
        }
        __syncthreads();
        bf16* Ks = ring + (size_t)buf * STAGE_ELEMS;
        bf16* Vs = Ks + PF_KEYS * STRIDE;
        for (int e = tid; e < PF_KEYS * VEC_PER_ROW; e += PF_THREADS) {
            const int key = e / VEC_PER_ROW, c = (e % VEC_PER_ROW) * 8;
            const long long off = key_off[buf][key];
            const bool ok = off >= 0;
            const bf16* src = ok ? p.pages + off + c : p.pages;
            pf_cp_async_16(Ks + key * STRIDE + c, src, ok);
            pf_cp_async_16(Vs + key * STRIDE + c, ok ? src + plane : p.pages, ok);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    // positions of this lane's two rows (row g and row g + 8 of the warp's 16); -1 for a row that does not exist
    int row_pos[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int row = warp * 16 + g + 8 * h2;
        const int tl = row / hpc, h = row % hpc;
        row_pos[h2] = (tl < ntok && h < heads) ? pos0 + tok0 + tl : -1;
    }

    float o[2 * D16][4];
#pragma unroll
    for (int i = 0; i < 2 * D16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};

    const float scale_log2 = p.scale * 1.4426950408889634f;
    const int warp_last_tok = (warp * 16 + 15) / hpc;
    const int warp_hi_pos = pos0 + tok0 + (warp_last_tok < ntok ? warp_last_tok : ntok - 1);
    // lowest position among this warp's rows: keys up to it need no causal mask (rows that do not exist have
    // zero queries and are never stored, so they need none either)
    const int warp_first_tok = (warp * 16) / hpc;
    const int warp_lo_pos = pos0 + tok0 + (warp_first_tok < ntok ? warp_first_tok : ntok - 1);
    const bf16* Ks = ring;
    const bf16* Vs = ring + PF_KEYS * STRIDE;
    const bf16* Qw = Qs + (size_t)(warp * 16 + (lane & 15)) * STRIDE + (lane >> 4) * 8;   // this lane's ldmatrix row of Q
    const int tile_lo = (lo / PF_KEYS) * PF_KEYS;
    for (int j0 = tile_lo; j0 <= hi; j0 += PF_KEYS) {
        issue_tile(j0, 0);
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();
        // two halves of 32 keys, so that a half's scores fit 16 registers
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int jh = j0 + half * 32;
            if (jh > warp_hi_pos) continue;          // every row of this warp lies before these keys
            float s[4][4];
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < D16; ++ks) {
                unsigned qa[4];
                pf_ldmatrix_x4(qa, Qw + ks * 16);
#pragma unroll
                for (int nb = 0; nb < 4; nb += 2) {
                    // four 8x8 blocks of K at once: keys nb*8.. and (nb+1)*8.., each with dims ks*16.. and ks*16+8..
                    unsigned kf[4];
                    pf_ldmatrix_x4(kf, Ks + (size_t)(half * 32 + (nb + (lane >> 4)) * 8 + (lane & 7)) * STRIDE + ks * 16 + ((lane >> 3) & 1) * 8);
                    pf_mma(s[nb], qa, kf[0], kf[1]);
                    pf_mma(s[nb + 1], qa, kf[2], kf[3]);
                }
            }
            // mask (only where the causal diagonal or the window edge crosses these keys), running max of raw scores
            const bool need_mask = (jh + 31 > warp_lo_pos) || (p.window > 0 && jh < warp_hi_pos - p.window + 1);
            float mx[2] = {-INFINITY, -INFINITY};
            if (need_mask) {
#pragma unroll
                for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int j = jh + nb * 8 + 2 * t + (c & 1);
                        const int pos = row_pos[c >> 1];
                        bool ok = j <= pos;
                        if (p.window > 0 && j < pos - p.window + 1) ok = false;
                        if (!ok) s[nb][c] = -INFINITY;
                    }
                }
            }
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
                for (int c = 0; c < 4; ++c) mx[c >> 1] = fmaxf(mx[c >> 1], s[nb][c]);
            }
            // running max and sum live in units of log2 (exp(x * scale) = 2^(x * scale * log2 e))
            float alpha[2], m_scaled[2];
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 1));
                mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 2));
                const float m_new = fmaxf(m_run[h2], mx[h2] * scale_log2);
                alpha[h2] = (m_new > -INFINITY) ? pf_ex2(m_run[h2] - m_new) : 1.f;
                m_run[h2] = m_new;
                m_scaled[h2] = (m_new > -INFINITY) ? m_new : 0.f;     // a row without any key keeps p = 2^(-inf) = 0
            }
            float sum[2] = {0.f, 0.f};
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float pr = pf_ex2(fmaf(s[nb][c], scale_log2, -m_scaled[c >> 1]));
                    s[nb][c] = pr;
                    sum[c >> 1] += pr;
                }
            }
            l_run[0] = l_run[0] * alpha[0] + sum[0];
            l_run[1] = l_run[1] * alpha[1] + sum[1];
            if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                for (int i = 0; i < 2 * D16; ++i) {
                    o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
                }
            }
            // O += P V, 16 keys per step
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                unsigned pa[4];
                pa[0] = pf_pack(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = pf_pack(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = pf_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = pf_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int nb2 = 0; nb2 < D16; ++nb2) {
                    unsigned v[4];
                    pf_ldmatrix_x4_trans(v, Vs + (size_t)(half * 32 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + nb2 * 16 + (lane >> 4) * 8);
                    pf_mma(o[nb2 * 2], pa, v[0], v[1]);
                    pf_mma(o[nb2 * 2 + 1], pa, v[2], v[3]);
                }
            }
        }
        __syncthreads();                                         // the tile's buffer may be overwritten now
    }

    // normalise and store
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 1);
        l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 2);
    }
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        if (row_pos[h2] < 0) continue;
        const int row = warp * 16 + g + 8 * h2;
        const int tl = row / hpc, h = row % hpc;
        const float inv = l_run[h2] > 0.f ? 1.f / l_run[h2] : 0.f;
        bf16* dst = p.out + (size_t)(q_begin + tok0 + tl) * p.out_stride + (size_t)(kvh * G + head0 + h) * D + 2 * t;
#pragma unroll
        for (int nb = 0; nb < 2 * D16; ++nb)
            *reinterpret_cast<unsigned*>(dst + nb * 8) = pf_pack(o[nb][2 * h2] * inv, o[nb][2 * h2 + 1] * inv);
    }
}

// Query tokens per block for a group size: 64 rows of (token, head).
int llmp_prefill_mma_tokens_per_tile(int nq, int nkv) {
    const int G = nq / nkv;
    const int hpc = G < 16 ? G : 16;
    return PF_ROWS / hpc;
}

// Head sizes this kernel is instantiated for.
bool llmp_prefill_mma_supports(int d) { return d >= 16 && d <= 128 && d % 16 == 0; }

int llmp_launch_prefill_mma(const void* q, long q_stride, void* out, long out_stride, const void* pages,
                            const int* block_tables, int table_stride, const int* q_start, const int* ctx_len,
                            const int* tile_req, const int* tile_tok0, int num_tiles, int nq, int nkv, int d,
                            int page_size, int window, float scale, cudaStream_t stream) {
    PrefillParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.pages = (const bf16*)pages; p.block_tables = block_tables;
    p.q_start = q_start; p.ctx_len = ctx_len; p.tile_req = tile_req; p.tile_tok0 = tile_tok0; p.q_stride = q_stride;
    p.out_stride = out_stride; p.table_stride = table_stride; p.nq = nq; p.nkv = nkv; p.d = d; p.page_size = page_size;
    p.window = window; p.scale = scale;
    const int G = nq / nkv;
    p.heads_per_cta = G < 16 ? G : 16;
    p.tokens_per_cta = PF_ROWS / p.heads_per_cta;
    p.head_chunks = (G + p.heads_per_cta - 1) / p.heads_per_cta;
    p.num_tiles = num_tiles;
    LLMP_REQUIRE((long)num_tiles * nkv * p.head_chunks < (1L << 31), "attention: too many tiles");
    LLMP_REQUIRE((q_stride % 8) == 0 && (out_stride % 2) == 0, "attention: query rows must be 16-byte aligned");
    const size_t smem = sizeof(bf16) * ((size_t)PF_ROWS * (d + 8) + (size_t)2 * PF_KEYS * (d + 8));
    const unsigned grid = (unsigned)(num_tiles * nkv * p.head_chunks);
#define PF_CASE(N)                                                               \
    case N:                                                                      \
        LLMP_ALLOW_SMEM(prefill_attention_mma_kernel<N>, smem);                   \
        prefill_attention_mma_kernel<N><<<grid, PF_THREADS, smem, stream>>>(p);  \
        break;
    switch (d / 16) {
        PF_CASE(1) PF_CASE(2) PF_CASE(3) PF_CASE(4) PF_CASE(5) PF_CASE(6) PF_CASE(7) PF_CASE(8)
        default:
            llmp_set_error("attention: head size %d has no tensor-core prefill kernel", d);
            return 1;
    }
#undef PF_CASE
    return llmp_check_launch("prefill_attention_mma");
}
