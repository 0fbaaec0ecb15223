// Decode attention for bfloat16 pages on the tensor cores (mma.sync m16n8k16, float32 accumulate).
//
// Same contract and the same split of the keys as the CUDA-core kernel in attention_decode.cu: one
// query row per request, fixed key ranges of DEC_SPLIT keys aligned to key 0, one block per
// (range, kv head x chunk of up to 16 query heads, request), unnormalised partials to scratch,
// merged by decode_merge_kernel. Inside a block the 16 rows of the MMA tile are the query heads
// that share the key/value head. Each of the four warps owns DEC_SPLIT / 4 consecutive keys of the
// range: it issues all of its K and V rows as 16-byte cp.async copies into its own shared-memory
// tile at once (so a block has its whole range in flight), then works through them in groups of 16
// keys with its own running softmax; the four warps are combined in shared memory at the end. There
// is no block-wide barrier inside the key loop.
#include "attention_decode.cuh"
#include "common.cuh"

#define DM_THREADS 128
#define DM_WARPS 4
#define DM_ROWS 16
#define DM_WARP_KEYS (DEC_SPLIT / DM_WARPS)     // 32 keys per warp
#define DM_GROUPS (DM_WARP_KEYS / 16)           // groups of 16 keys

struct DecodeMmaParams {
    const bf16* q;
    const bf16* pages;
    const int* block_tables;
    const int* ctx_len;
    float* part_o;           // [R, nq, max_splits, d]
    float* part_ml;          // [R, nq, max_splits, 2]
    long q_stride;
    int table_stride;
    int nq, nkv, d, page_size, window;
    int heads_per_cta, head_chunks, max_splits;
    float scale;
};

__device__ __forceinline__ void dm_cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;       // 0: nothing is read, the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// D (16x8, float32) += A (16x16 bf16, row) * B (16x8 bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

// MAXD8: head size / 8 rounded up to the template's step, the 8-column output blocks a warp accumulates.
template <int MAXD8>
__global__ void __launch_bounds__(DM_THREADS) decode_attention_mma_kernel(const DecodeMmaParams p) {
    extern __shared__ __align__(16) unsigned char dm_smem[];
    const int d = p.d;
    const int stride = d + 8;                                    // padded row of K, V and Q tiles, in elements
    const int warp_elems = 2 * DM_WARP_KEYS * stride;            // a warp's K rows, then its V rows
    bf16* tiles = reinterpret_cast<bf16*>(dm_smem);              // [warps][K rows | V rows]
    bf16* Qs = tiles + (size_t)DM_WARPS * warp_elems;            // [16][stride], rows beyond the heads are zero

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x;
    const int kvh = blockIdx.y / p.head_chunks, chunk = blockIdx.y % p.head_chunks;
    const int r = blockIdx.z;
    const int G = p.nq / p.nkv;
    const int head0 = chunk * p.heads_per_cta;
    int heads = G - head0;
    if (heads > p.heads_per_cta) heads = p.heads_per_cta;
    const int ctx = p.ctx_len[r];
    const int nsplits = (ctx + DEC_SPLIT - 1) / DEC_SPLIT;
    if (split >= nsplits) return;
    const int pos = ctx - 1;
    int lo = split * DEC_SPLIT, hi = lo + DEC_SPLIT;
    if (hi > ctx) hi = ctx;
    if (p.window > 0 && lo < pos - p.window + 1) lo = pos - p.window + 1;
    const bf16* q = p.q + (size_t)r * p.q_stride + (size_t)(kvh * G + head0) * d;
    const int* table = p.block_tables + (size_t)r * p.table_stride;
    const size_t plane = (size_t)p.nkv * p.page_size * d;
    const int vec_per_row = d / 8;

    // This warp's keys: lane l looks up key j0 + l; all K and V rows are requested at once.
    const int j0 = split * DEC_SPLIT + warp * DM_WARP_KEYS;
    long long my_off = -1;
    {
        const int j = j0 + lane;
        if (j >= lo && j < hi) {
            const int page = table[j / p.page_size];
            if (page >= 0)
                my_off = (long long)((((size_t)page * 2) * p.nkv + kvh) * p.page_size + (j % p.page_size)) * d;
        }
    }
    const unsigned valid = __ballot_sync(0xffffffffu, my_off >= 0);
    bf16* Ks = tiles + (size_t)warp * warp_elems;
    bf16* Vs = Ks + DM_WARP_KEYS * stride;
    // Copies, all asynchronous and 16 bytes wide: first the query rows (rows beyond the heads are
    // zero-filled), then the warp's key groups. With a power-of-two row (d = 16 << k) a warp
    // instruction covers 32 / vec_per_row whole rows and the indices are shifts and adds; other head
    // sizes take the general loops.
    // The kernel before this one wrote the query rows and the newest key and value (position ctx - 1); all
    // other keys are older. A block whose range holds the newest key waits for that kernel first; the others
    // ask for their keys and values, then wait, then fetch the query rows.
    const bool newest_here = hi == ctx;
    if (newest_here) pdl_wait();
    const bool pow2 = (vec_per_row & (vec_per_row - 1)) == 0;
    if (pow2) {
        const int sub = lane / vec_per_row, c = (lane % vec_per_row) * 8;
        const int rows_per_pass = DM_THREADS / vec_per_row;
        const int rows_per_instr = 32 / vec_per_row;
#pragma unroll
        for (int grp = 0; grp < DM_GROUPS; ++grp) {
            for (int k0 = 0; k0 < 16; k0 += rows_per_instr) {
                const int key = grp * 16 + k0 + sub;
                const long long off = __shfl_sync(0xffffffffu, my_off, key);
                const bool ok = off >= 0;
                const bf16* src = ok ? p.pages + off + c : p.pages;
                dm_cp_async_16(Ks + key * stride + c, src, ok);
                dm_cp_async_16(Vs + key * stride + c, ok ? src + plane : p.pages, ok);
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
        }
        if (!newest_here) pdl_wait();
        for (int row = tid / vec_per_row; row < DM_ROWS; row += rows_per_pass)
            dm_cp_async_16(Qs + row * stride + c, row < heads ? q + (size_t)row * d + c : q, row < heads);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    } else {
#pragma unroll
        for (int grp = 0; grp < DM_GROUPS; ++grp) {
            for (int e = lane; e < 16 * vec_per_row; e += 32) {
                const int key = grp * 16 + e / vec_per_row, c = (e % vec_per_row) * 8;
                const long long off = __shfl_sync(0xffffffffu, my_off, key);
                const bool ok = off >= 0;
                const bf16* src = ok ? p.pages + off + c : p.pages;
                dm_cp_async_16(Ks + key * stride + c, src, ok);
                dm_cp_async_16(Vs + key * stride + c, ok ? src + plane : p.pages, ok);
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
        }
        if (!newest_here) pdl_wait();
        for (int e = tid; e < DM_ROWS * vec_per_row; e += DM_THREADS) {
            const int row = e / vec_per_row, c = (e % vec_per_row) * 8;
            dm_cp_async_16(Qs + row * stride + c, row < heads ? q + (size_t)row * d + c : q, row < heads);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    pdl_trigger();                                               // the merge kernel may take its places
    // Everything this warp asked for has landed after wait_group 0; the query rows were written by all
    // warps, hence the block-wide barrier.
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();

    // A warp sees its DM_WARP_KEYS (32) keys at once: scores S[16 heads x 32 keys] as four 16x8 blocks, one
    // softmax over them, then O = P V. No running rescale is needed inside a warp.
    float o[MAXD8][4];
#pragma unroll
    for (int i = 0; i < MAXD8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};      // rows g and g + 8, in units of log2
    float l_run[2] = {0.f, 0.f};                  // this lane's share of the row sums
    const int d8 = d / 8, d16 = d / 16;
    const float scale_log2 = p.scale * 1.4426950408889634f;

    if (valid != 0u) {
        float s[4][4];
#pragma unroll
        for (int nb = 0; nb < 4; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
        for (int ks = 0; ks < d16; ++ks) {
            unsigned a[4];
            ldmatrix_x4(a, Qs + (size_t)(lane & 15) * stride + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int nb = 0; nb < 4; nb += 2) {
                // four 8x8 blocks of K at once: keys nb*8.. and (nb+1)*8.., each with dims ks*16.. and ks*16+8..
                unsigned kf[4];
                ldmatrix_x4(kf, Ks + (size_t)((nb + (lane >> 4)) * 8 + (lane & 7)) * stride + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16_16816(s[nb], a, kf[0], kf[1]);
                mma_bf16_16816(s[nb + 1], a, kf[2], kf[3]);
            }
        }
        // mask keys outside the range; key of s[nb][c] is nb*8 + 2t + (c & 1), row g + 8*(c >> 1)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (valid != 0xffffffffu && !((valid >> (nb * 8 + 2 * t + (c & 1))) & 1u)) s[nb][c] = -INFINITY;
                mx[c >> 1] = fmaxf(mx[c >> 1], s[nb][c]);
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            m_run[h] = mx[h] * scale_log2;         // at least one key is valid, so the maximum is finite
        }
#pragma unroll
        for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float pr;
                asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(pr) : "f"(fmaf(s[nb][c], scale_log2, -m_run[c >> 1])));
                s[nb][c] = pr;
                l_run[c >> 1] += pr;
            }
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            unsigned pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);         // row g,     keys 16kk + 2t, +1
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);         // row g + 8
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]); // row g,     keys 16kk + 8 + 2t, +1
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]); // row g + 8
#pragma unroll
            for (int nb2 = 0; nb2 < MAXD8 / 2; ++nb2) {
                if (nb2 * 2 < d8) {
                    unsigned v[4];
                    ldmatrix_x4_trans(v, Vs + (size_t)(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * stride + nb2 * 16 + (lane >> 4) * 8);
                    mma_bf16_16816(o[nb2 * 2], pa, v[0], v[1]);
                    mma_bf16_16816(o[nb2 * 2 + 1], pa, v[2], v[3]);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();                                             // every warp is done with its tile

    // combine the four warps' partials in shared memory (the tiles are free now)
    float* Ow = reinterpret_cast<float*>(dm_smem);               // [4][16][d + 8]
    __shared__ float mw[DM_WARPS][DM_ROWS], lw[DM_WARPS][DM_ROWS];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    if (t == 0) {
        mw[warp][g] = m_run[0];
        mw[warp][g + 8] = m_run[1];
        lw[warp][g] = l_run[0];
        lw[warp][g + 8] = l_run[1];
    }
    // rows of d + 8 floats: the 8-byte stores of a half-warp (4 rows x 4 column pairs) then fall into
    // distinct banks
    const int ostride = d + 8;
#pragma unroll
    for (int nb = 0; nb < MAXD8; ++nb) {
        if (nb < d8) {
            float* dst = Ow + ((size_t)warp * DM_ROWS + g) * ostride + nb * 8 + 2 * t;
            *reinterpret_cast<float2*>(dst) = make_float2(o[nb][0], o[nb][1]);
            if (heads > 8) *reinterpret_cast<float2*>(dst + (size_t)8 * ostride) = make_float2(o[nb][2], o[nb][3]);
        }
    }
    __syncthreads();
    // warp w combines rows w, w + 4, ...; a lane takes four columns at a time
    for (int row = warp; row < heads; row += DM_WARPS) {
        const float m = fmaxf(fmaxf(mw[0][row], mw[1][row]), fmaxf(mw[2][row], mw[3][row]));
        float wgt[DM_WARPS];
#pragma unroll
        for (int w = 0; w < DM_WARPS; ++w) wgt[w] = (mw[w][row] > -INFINITY) ? exp2f(mw[w][row] - m) : 0.f;
        float* dst = p.part_o + (((size_t)r * p.nq + kvh * G + head0 + row) * p.max_splits + split) * d;
        for (int c = lane * 4; c < d; c += 128) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < DM_WARPS; ++w) {
                const float4 v = *reinterpret_cast<const float4*>(Ow + ((size_t)w * DM_ROWS + row) * ostride + c);
                acc.x = fmaf(v.x, wgt[w], acc.x);
                acc.y = fmaf(v.y, wgt[w], acc.y);
                acc.z = fmaf(v.z, wgt[w], acc.z);
                acc.w = fmaf(v.w, wgt[w], acc.w);
            }
            *reinterpret_cast<float4*>(dst + c) = acc;
        }
    }
    if (tid < heads) {
        const int row = tid;
        const float m = fmaxf(fmaxf(mw[0][row], mw[1][row]), fmaxf(mw[2][row], mw[3][row]));
        float l = 0.f;
#pragma unroll
        for (int w = 0; w < DM_WARPS; ++w)
            if (mw[w][row] > -INFINITY) l += lw[w][row] * exp2f(mw[w][row] - m);
        float* ml = p.part_ml + (((size_t)r * p.nq + kvh * G + head0 + row) * p.max_splits + split) * 2;
        ml[0] = m * 0.6931471805599453f;             // the merge kernel works in natural-log units
        ml[1] = l;
    }
}

// Launches the tensor-core decode kernel; the caller (llmp_decode_attention) has checked the sizes and
// runs the merge kernel afterwards. Returns 0 on success.
int llmp_launch_decode_mma(const void* q, long q_stride, const void* pages, const int* block_tables, int table_stride,
                           const int* ctx_len, int R, int max_splits, int nq, int nkv, int d, int page_size,
                           int window, float scale, float* part_o, float* part_ml, cudaStream_t stream) {
    DecodeMmaParams p;
    const int G = nq / nkv;
    p.heads_per_cta = G < DM_ROWS ? G : DM_ROWS;
    p.head_chunks = (G + p.heads_per_cta - 1) / p.heads_per_cta;
    p.max_splits = max_splits;
    LLMP_REQUIRE((long)nkv * p.head_chunks <= 65535, "decode attention: too many heads");
    p.q = (const bf16*)q; p.pages = (const bf16*)pages; p.block_tables = block_tables; p.ctx_len = ctx_len;
    p.q_stride = q_stride; p.table_stride = table_stride; p.nq = nq; p.nkv = nkv; p.d = d; p.page_size = page_size;
    p.window = window; p.scale = scale; p.part_o = part_o; p.part_ml = part_ml;
    const size_t tiles = (size_t)DM_WARPS * 2 * DM_WARP_KEYS * (d + 8) * sizeof(bf16);
    const size_t qbytes = (size_t)DM_ROWS * (d + 8) * sizeof(bf16);
    const size_t merge = (size_t)DM_WARPS * DM_ROWS * (d + 8) * sizeof(float);
    size_t smem = tiles + qbytes;
    if (smem < merge) smem = merge;
    dim3 grid(max_splits, nkv * p.head_chunks, R);
    cudaError_t launched = cudaSuccess;
    if (d <= 64) {
        LLMP_ALLOW_SMEM(decode_attention_mma_kernel<8>, smem);
        launched = llmp_launch_dependent(decode_attention_mma_kernel<8>, grid, dim3(DM_THREADS), smem, stream, p);
    } else if (d <= 128) {
        LLMP_ALLOW_SMEM(decode_attention_mma_kernel<16>, smem);
        launched = llmp_launch_dependent(decode_attention_mma_kernel<16>, grid, dim3(DM_THREADS), smem, stream, p);
    } else {
        LLMP_ALLOW_SMEM(decode_attention_mma_kernel<32>, smem);
        launched = llmp_launch_dependent(decode_attention_mma_kernel<32>, grid, dim3(DM_THREADS), smem, stream, p);
    }
    if (launched != cudaSuccess) {
        llmp_set_error("decode_attention_mma: launch failed: %s", cudaGetErrorString(launched));
        return 2;
    }
    return llmp_check_launch("decode_attention_mma");
}
