// Causal attention over paged keys and values.
//
// Pages are [num_pages, 2 (K,V), nkv, page_size, d]. A request's block table maps its logical
// page i (tokens i*page_size ..) to a physical page, or -1 for a page that was given back.
// The query rows of a step are [N, q_stride]; request r owns rows q_start[r] .. q_start[r+1]-1,
// which are its newest tokens: row i of the request sits at position ctx_len[r] - q_len[r] + i
// and attends to keys max(0, pos - window + 1) .. pos (window <= 0: all earlier keys).
//
// llmp_paged_attention is the general kernel (any number of query rows per request, every
// head size that is a multiple of 16 up to 256, float32 or bfloat16 storage, float32 math):
// online softmax over key tiles of 32 that are aligned to key 0, so the operations applied to
// one query row are the same however the tokens were cut into steps or batched.
#include "common.cuh"

#define ATT_ROWS 16      // query rows (token x head of the group) per block
#define ATT_KEYS 32      // keys per tile
#define ATT_THREADS 128

struct AttnParams {
    const void* q;
    void* out;
    const void* pages;
    const int* block_tables;
    const int* q_start;
    const int* ctx_len;
    const int* tile_req;
    const int* tile_tok0;
    long q_stride, out_stride;
    int table_stride;
    int nq, nkv, d, page_size, window;
    int heads_per_cta, tokens_per_cta, head_chunks;
    float scale;
};

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS) paged_attention_kernel(const AttnParams p) {
    extern __shared__ float smem[];
    const int d = p.d;
    float* Qs = smem;                              // [ATT_ROWS][d]
    float* Os = Qs + ATT_ROWS * d;                 // [ATT_ROWS][d]
    float* Ks = Os + ATT_ROWS * d;                 // [ATT_KEYS][d + 1]
    float* Vs = Ks + ATT_KEYS * (d + 1);           // [ATT_KEYS][d]
    float* Ss = Vs + ATT_KEYS * d;                 // [ATT_ROWS][ATT_KEYS + 1]
    float* row_m = Ss + ATT_ROWS * (ATT_KEYS + 1); // [ATT_ROWS]
    float* row_l = row_m + ATT_ROWS;
    float* row_a = row_l + ATT_ROWS;
    __shared__ long long key_off[ATT_KEYS];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = p.tile_req[blockIdx.x];
    const int tok0 = p.tile_tok0[blockIdx.x];
    const int kvh = blockIdx.y / p.head_chunks;
    const int chunk = blockIdx.y % p.head_chunks;
    const int G = p.nq / p.nkv;
    const int head0 = chunk * p.heads_per_cta;     // first head of the group handled here
    const int q_begin = p.q_start[r];
    const int q_len = p.q_start[r + 1] - q_begin;
    const int ctx = p.ctx_len[r];
    const int pos0 = ctx - q_len;                  // position of the request's first row
    const int* table = p.block_tables + (size_t)r * p.table_stride;
    const T* q = reinterpret_cast<const T*>(p.q);
    const T* pages = reinterpret_cast<const T*>(p.pages);
    T* out = reinterpret_cast<T*>(p.out);
    const int rows = p.heads_per_cta * p.tokens_per_cta;

    // Stage the query rows; row rr = token (rr / heads_per_cta), head (rr % heads_per_cta).
    for (int e = tid; e < ATT_ROWS * d; e += ATT_THREADS) {
        const int rr = e / d, c = e % d;
        const int tl = tok0 + rr / p.heads_per_cta, hh = head0 + rr % p.heads_per_cta;
        float v = 0.f;
        if (rr < rows && tl < q_len && hh < G)
            v = to_float(q[(size_t)(q_begin + tl) * p.q_stride + (size_t)(kvh * G + hh) * d + c]);
        Qs[e] = v;
        Os[e] = 0.f;
    }
    if (tid < ATT_ROWS) {
        row_m[tid] = -INFINITY;
        row_l[tid] = 0.f;
    }
    // Keys needed by this block: from the window start of its first row to the position of its last row.
    int last_tok = tok0 + p.tokens_per_cta - 1;
    if (last_tok > q_len - 1) last_tok = q_len - 1;
    const int hi = pos0 + last_tok;
    int lo = 0;
    if (p.window > 0) {
        lo = pos0 + tok0 - p.window + 1;
        if (lo < 0) lo = 0;
    }
    const size_t plane = (size_t)p.nkv * p.page_size * d;      // K plane -> V plane of one page
    __syncthreads();

    for (int j0 = (lo / ATT_KEYS) * ATT_KEYS; j0 <= hi; j0 += ATT_KEYS) {
        if (tid < ATT_KEYS) {
            const int j = j0 + tid;
            long long off = -1;
            if (j <= hi && j < ctx) {
                const int page = table[j / p.page_size];
                if (page >= 0)
                    off = (long long)((((size_t)page * 2) * p.nkv + kvh) * p.page_size + (j % p.page_size)) * d;
            }
            key_off[tid] = off;
        }
        __syncthreads();
        for (int e = tid; e < ATT_KEYS * d; e += ATT_THREADS) {
            const int key = e / d, c = e % d;
            const long long off = key_off[key];
            float kv = 0.f, vv = 0.f;
            if (off >= 0) {
                kv = to_float(pages[off + c]);
                vv = to_float(pages[off + plane + c]);
            }
            Ks[key * (d + 1) + c] = kv;
            Vs[key * d + c] = vv;
        }
        __syncthreads();
        // Scores: thread -> key (lane), rows 4*warp .. 4*warp+3.
        {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const float* krow = Ks + lane * (d + 1);
            const float* qrow = Qs + (warp * 4) * d;
            for (int c = 0; c < d; ++c) {
                const float kv = krow[c];
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[i] = fmaf(qrow[i * d + c], kv, acc[i]);
            }
            const int j = j0 + lane;
            const bool key_ok = key_off[lane] >= 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int rr = warp * 4 + i;
                const int tl = tok0 + rr / p.heads_per_cta;
                const int pos = pos0 + tl;
                bool ok = key_ok && rr < rows && tl < q_len && j <= pos;
                if (p.window > 0 && j < pos - p.window + 1) ok = false;
                Ss[rr * (ATT_KEYS + 1) + lane] = ok ? acc[i] * p.scale : -INFINITY;
            }
        }
        __syncthreads();
        // Online softmax, one warp per four rows.
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int rr = warp * 4 + i;
            const float s = Ss[rr * (ATT_KEYS + 1) + lane];
            const float m_old = row_m[rr];
            const float m_new = fmaxf(m_old, warp_max(s));
            float pr = 0.f, alpha = 1.f;
            if (m_new > -INFINITY) {
                pr = expf(s - m_new);          // exp(-inf) = 0 for masked keys
                alpha = expf(m_old - m_new);   // 0 when nothing was seen before
            }
            const float sum = warp_sum(pr);
            Ss[rr * (ATT_KEYS + 1) + lane] = pr;
            __syncwarp();
            if (lane == 0) {
                row_m[rr] = m_new;
                row_l[rr] = row_l[rr] * alpha + sum;
                row_a[rr] = alpha;
            }
        }
        __syncthreads();
        // Output update: thread -> row tid/8, columns (tid%8) + 8k.
        {
            const int rr = tid >> 3;
            const float alpha = row_a[rr];
            const float* prow = Ss + rr * (ATT_KEYS + 1);
            for (int c = tid & 7; c < d; c += 8) {
                float o = Os[rr * d + c] * alpha;
#pragma unroll 8
                for (int j = 0; j < ATT_KEYS; ++j) o = fmaf(prow[j], Vs[j * d + c], o);
                Os[rr * d + c] = o;
            }
        }
        __syncthreads();
    }
    for (int e = tid; e < ATT_ROWS * d; e += ATT_THREADS) {
        const int rr = e / d, c = e % d;
        const int tl = tok0 + rr / p.heads_per_cta, hh = head0 + rr % p.heads_per_cta;
        if (rr < rows && tl < q_len && hh < G) {
            const float l = row_l[rr];
            const float v = l > 0.f ? Os[e] / l : 0.f;
            out[(size_t)(q_begin + tl) * p.out_stride + (size_t)(kvh * G + hh) * d + c] = from_float<T>(v);
        }
    }
}

// Number of query tokens one block covers for a given group size; the caller builds the tile
// list (tile_req, tile_tok0) with this step.
LLMP_API int llmp_attention_tokens_per_tile(int nq, int nkv) {
    if (nq <= 0 || nkv <= 0 || nq % nkv) return 0;
    const int G = nq / nkv;
    const int heads = G < ATT_ROWS ? G : ATT_ROWS;
    return ATT_ROWS / heads;
}

LLMP_API int llmp_paged_attention(const void* q, long q_stride, void* out, long out_stride, const void* pages,
                                  int dtype, const int* block_tables, int table_stride, const int* q_start,
                                  const int* ctx_len, const int* tile_req, const int* tile_tok0, int num_tiles,
                                  int nq, int nkv, int d, int page_size, int window, float scale,
                                  cudaStream_t stream) {
    if (num_tiles <= 0) return 0;
    LLMP_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads cannot share %d key/value heads", nq, nkv);
    LLMP_REQUIRE(d >= 16 && d <= 256 && d % 16 == 0, "attention: head size %d is not a multiple of 16 in 16..256", d);
    LLMP_REQUIRE(page_size > 0, "attention: bad page size %d", page_size);
    AttnParams p;
    p.q = q; p.out = out; p.pages = pages; p.block_tables = block_tables; p.q_start = q_start; p.ctx_len = ctx_len;
    p.tile_req = tile_req; p.tile_tok0 = tile_tok0; p.q_stride = q_stride; p.out_stride = out_stride;
    p.table_stride = table_stride; p.nq = nq; p.nkv = nkv; p.d = d; p.page_size = page_size; p.window = window;
    const int G = nq / nkv;
    p.heads_per_cta = G < ATT_ROWS ? G : ATT_ROWS;
    p.tokens_per_cta = ATT_ROWS / p.heads_per_cta;
    p.head_chunks = (G + p.heads_per_cta - 1) / p.heads_per_cta;
    p.scale = scale;
    LLMP_REQUIRE((long)nkv * p.head_chunks <= 65535, "attention: too many heads");
    const size_t smem = sizeof(float) * ((size_t)2 * ATT_ROWS * d + (size_t)ATT_KEYS * (d + 1) + (size_t)ATT_KEYS * d +
                                         (size_t)ATT_ROWS * (ATT_KEYS + 1) + 3 * ATT_ROWS);
    dim3 grid(num_tiles, nkv * p.head_chunks);
    if (dtype == LLMP_F32) {
        cudaFuncSetAttribute(paged_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        paged_attention_kernel<float><<<grid, ATT_THREADS, smem, stream>>>(p);
    } else {
        cudaFuncSetAttribute(paged_attention_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        paged_attention_kernel<bf16><<<grid, ATT_THREADS, smem, stream>>>(p);
    }
    return llmp_check_launch("paged_attention");
}

// ------------------------------------------------------------------------------------------
// Decode attention: one query row per request (row r of q belongs to request r, at position
// ctx_len[r] - 1), keys split into fixed ranges of DEC_SPLIT keys that are aligned to key 0, so
// where a range starts and ends depends on the key's index alone. Block (split, kv head x head
// chunk, request) computes the softmax-weighted sum over its range for the query heads of one
// key/value head and writes an unnormalised partial (max, sum, vector) to scratch memory;
// llmp_decode_merge combines the partials of a row in ascending range order.
// K and V tiles of DEC_TILE keys are staged in shared memory with 16-byte loads.
// ------------------------------------------------------------------------------------------
#define DEC_SPLIT 256
#define DEC_TILE 64
#define DEC_THREADS 128
#define DEC_MAX_HEADS 8      // query heads per block
#define DEC_MAX_ACC 8        // column pairs per thread: heads * d / 2 / DEC_THREADS <= 8

struct DecodeParams {
    const void* q;
    const void* pages;
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

template <typename T>
__global__ void __launch_bounds__(DEC_THREADS) decode_attention_kernel(const DecodeParams p) {
    extern __shared__ __align__(16) unsigned char dec_smem[];
    const int d = p.d;
    const int kstride = d + 16 / (int)sizeof(T);                 // padded key row, in elements
    T* Ks = reinterpret_cast<T*>(dec_smem);                      // [DEC_TILE][kstride]
    T* Vs = Ks + DEC_TILE * kstride;                             // [DEC_TILE][d]
    float* Qs = reinterpret_cast<float*>(Vs + DEC_TILE * d);     // [heads][d]
    float* Ss = Qs + DEC_MAX_HEADS * d;                          // [heads][DEC_TILE]
    float* row_m = Ss + DEC_MAX_HEADS * DEC_TILE;                // [heads]
    float* row_l = row_m + DEC_MAX_HEADS;
    float* row_a = row_l + DEC_MAX_HEADS;
    __shared__ long long key_off[DEC_TILE];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
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
    int lo = split * DEC_SPLIT, hi = lo + DEC_SPLIT;             // keys [lo, hi)
    if (hi > ctx) hi = ctx;
    if (p.window > 0 && lo < pos - p.window + 1) lo = pos - p.window + 1;   // may pass hi: empty range
    const T* q = reinterpret_cast<const T*>(p.q) + (size_t)r * p.q_stride + (size_t)(kvh * G + head0) * d;
    const T* pages = reinterpret_cast<const T*>(p.pages);
    const int* table = p.block_tables + (size_t)r * p.table_stride;
    const size_t plane = (size_t)p.nkv * p.page_size * d;
    constexpr int VEC = 16 / (int)sizeof(T);                     // elements per 16-byte load

    for (int e = tid; e < heads * d; e += DEC_THREADS) Qs[e] = to_float(q[e]);
    if (tid < DEC_MAX_HEADS) {
        row_m[tid] = -INFINITY;
        row_l[tid] = 0.f;
    }
    float acc[DEC_MAX_ACC][2];
#pragma unroll
    for (int i = 0; i < DEC_MAX_ACC; ++i) acc[i][0] = acc[i][1] = 0.f;
    const int pairs = heads * d / 2;                              // (head, column pair) outputs of this block
    __syncthreads();

    const int tile_lo = (lo / DEC_TILE) * DEC_TILE;
    for (int j0 = tile_lo; j0 < hi; j0 += DEC_TILE) {
        if (tid < DEC_TILE) {
            const int j = j0 + tid;
            long long off = -1;
            if (j >= lo && j < hi) {
                const int page = table[j / p.page_size];
                if (page >= 0)
                    off = (long long)((((size_t)page * 2) * p.nkv + kvh) * p.page_size + (j % p.page_size)) * d;
            }
            key_off[tid] = off;
        }
        __syncthreads();
        // stage K and V rows with 16-byte loads; rows without a key are zero
        const int vec_per_row = d / VEC;
        for (int e = tid; e < DEC_TILE * vec_per_row; e += DEC_THREADS) {
            const int key = e / vec_per_row, c = (e % vec_per_row) * VEC;
            const long long off = key_off[key];
            uint4 kv = make_uint4(0u, 0u, 0u, 0u), vv = kv;
            if (off >= 0) {
                kv = *reinterpret_cast<const uint4*>(pages + off + c);
                vv = *reinterpret_cast<const uint4*>(pages + off + plane + c);
            }
            *reinterpret_cast<uint4*>(Ks + key * kstride + c) = kv;
            *reinterpret_cast<uint4*>(Vs + key * d + c) = vv;
        }
        __syncthreads();
        // scores: thread -> key tid % DEC_TILE, heads (tid / DEC_TILE), +2, ...
        {
            const int key = tid % DEC_TILE;
            const bool key_ok = key_off[key] >= 0;
            for (int h = tid / DEC_TILE; h < heads; h += DEC_THREADS / DEC_TILE) {
                const T* krow = Ks + key * kstride;
                const float* qrow = Qs + h * d;
                float s = 0.f;
                for (int c = 0; c < d; c += VEC) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(krow + c);
                    const T* kk = reinterpret_cast<const T*>(&raw);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) s = fmaf(qrow[c + i], to_float(kk[i]), s);
                }
                Ss[h * DEC_TILE + key] = key_ok ? s * p.scale : -INFINITY;
            }
        }
        __syncthreads();
        // online softmax: warp w handles heads w, w + 4, ...; lane covers keys lane and lane + 32
        for (int h = warp; h < heads; h += DEC_THREADS / 32) {
            const float s0 = Ss[h * DEC_TILE + lane], s1 = Ss[h * DEC_TILE + lane + 32];
            const float m_old = row_m[h];
            const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
            float p0 = 0.f, p1 = 0.f, alpha = 1.f;
            if (m_new > -INFINITY) {
                p0 = expf(s0 - m_new);
                p1 = expf(s1 - m_new);
                alpha = expf(m_old - m_new);
            }
            const float sum = warp_sum(p0 + p1);
            Ss[h * DEC_TILE + lane] = p0;
            Ss[h * DEC_TILE + lane + 32] = p1;
            if (lane == 0) {
                row_m[h] = m_new;
                row_l[h] = row_l[h] * alpha + sum;
                row_a[h] = alpha;
            }
        }
        __syncthreads();
        // weighted sum: thread owns (head, column pair) outputs idx = tid, tid + 128, ...
#pragma unroll
        for (int i = 0; i < DEC_MAX_ACC; ++i) {
            const int idx = tid + i * DEC_THREADS;
            if (idx < pairs) {
                const int h = idx / (d / 2), c = (idx % (d / 2)) * 2;
                const float alpha = row_a[h];
                float a0 = acc[i][0] * alpha, a1 = acc[i][1] * alpha;
                const float* prow = Ss + h * DEC_TILE;
                for (int key = 0; key < DEC_TILE; ++key) {
                    const float pr = prow[key];
                    a0 = fmaf(pr, to_float(Vs[key * d + c]), a0);
                    a1 = fmaf(pr, to_float(Vs[key * d + c + 1]), a1);
                }
                acc[i][0] = a0;
                acc[i][1] = a1;
            }
        }
        __syncthreads();
    }
    // partials: unnormalised vector, running max and sum
#pragma unroll
    for (int i = 0; i < DEC_MAX_ACC; ++i) {
        const int idx = tid + i * DEC_THREADS;
        if (idx < pairs) {
            const int h = idx / (d / 2), c = (idx % (d / 2)) * 2;
            float* dst = p.part_o + (((size_t)r * p.nq + kvh * G + head0 + h) * p.max_splits + split) * d + c;
            dst[0] = acc[i][0];
            dst[1] = acc[i][1];
        }
    }
    if (tid < heads) {
        float* ml = p.part_ml + (((size_t)r * p.nq + kvh * G + head0 + tid) * p.max_splits + split) * 2;
        ml[0] = row_m[tid];
        ml[1] = row_l[tid];
    }
}

template <typename T>
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int* __restrict__ ctx_len, T* __restrict__ out, long out_stride, int nq, int d,
                                    int max_splits) {
    const int r = blockIdx.y, h = blockIdx.x;
    const int ctx = ctx_len[r];
    const int nsplits = (ctx + DEC_SPLIT - 1) / DEC_SPLIT;
    const float* ml = part_ml + ((size_t)r * nq + h) * max_splits * 2;
    const float* po = part_o + ((size_t)r * nq + h) * max_splits * d;
    float m = -INFINITY;
    for (int s = 0; s < nsplits; ++s) m = fmaxf(m, ml[2 * s]);
    float l = 0.f;
    for (int s = 0; s < nsplits; ++s) l += (ml[2 * s] > -INFINITY) ? ml[2 * s + 1] * expf(ml[2 * s] - m) : 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < nsplits; ++s)
            if (ml[2 * s] > -INFINITY) o = fmaf(po[(size_t)s * d + c], expf(ml[2 * s] - m), o);
        out[(size_t)r * out_stride + (size_t)h * d + c] = from_float<T>(l > 0.f ? o / l : 0.f);
    }
}

// Scratch floats the decode kernel needs for R rows whose longest context is max_ctx keys.
LLMP_API long llmp_decode_scratch_floats(int R, int nq, int d, int max_ctx) {
    const long splits = (max_ctx + DEC_SPLIT - 1) / DEC_SPLIT;
    return (long)R * nq * (splits > 0 ? splits : 1) * (d + 2);
}

LLMP_API int llmp_decode_attention(const void* q, long q_stride, void* out, long out_stride, const void* pages,
                                   int dtype, const int* block_tables, int table_stride, const int* ctx_len, int R,
                                   int max_ctx, int nq, int nkv, int d, int page_size, int window, float scale,
                                   float* scratch, long scratch_floats, cudaStream_t stream) {
    if (R <= 0) return 0;
    LLMP_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads cannot share %d key/value heads", nq, nkv);
    LLMP_REQUIRE(d >= 16 && d <= 256 && d % 16 == 0, "attention: head size %d is not a multiple of 16 in 16..256", d);
    LLMP_REQUIRE(page_size > 0 && max_ctx > 0, "decode attention: bad page size %d or context %d", page_size, max_ctx);
    LLMP_REQUIRE(R <= 65535, "decode attention: too many rows %d", R);
    const int esize = dtype == LLMP_F32 ? 4 : 2;
    LLMP_REQUIRE((q_stride * esize) % 16 == 0, "decode attention: query rows must be 16-byte aligned");
    DecodeParams p;
    const int G = nq / nkv;
    int hpc = G < DEC_MAX_HEADS ? G : DEC_MAX_HEADS;
    while (hpc > 1 && hpc * d / 2 > DEC_MAX_ACC * DEC_THREADS) --hpc;
    p.heads_per_cta = hpc;
    p.head_chunks = (G + hpc - 1) / hpc;
    p.max_splits = (max_ctx + DEC_SPLIT - 1) / DEC_SPLIT;
    LLMP_REQUIRE(llmp_decode_scratch_floats(R, nq, d, max_ctx) <= scratch_floats,
                 "decode attention: scratch of %ld floats is too small, %ld needed", scratch_floats,
                 llmp_decode_scratch_floats(R, nq, d, max_ctx));
    LLMP_REQUIRE((long)nkv * p.head_chunks <= 65535, "decode attention: too many heads");
    p.q = q; p.pages = pages; p.block_tables = block_tables; p.ctx_len = ctx_len; p.q_stride = q_stride;
    p.table_stride = table_stride; p.nq = nq; p.nkv = nkv; p.d = d; p.page_size = page_size; p.window = window;
    p.scale = scale;
    p.part_o = scratch;
    p.part_ml = scratch + (size_t)R * nq * p.max_splits * d;
    const size_t smem = (size_t)esize * (DEC_TILE * (d + 16 / esize) + DEC_TILE * d) +
                        sizeof(float) * ((size_t)DEC_MAX_HEADS * d + DEC_MAX_HEADS * DEC_TILE + 3 * DEC_MAX_HEADS);
    dim3 grid(p.max_splits, nkv * p.head_chunks, R);
    dim3 mgrid(nq, R);
    if (dtype == LLMP_F32) {
        cudaFuncSetAttribute(decode_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        decode_attention_kernel<float><<<grid, DEC_THREADS, smem, stream>>>(p);
        decode_merge_kernel<float><<<mgrid, 64, 0, stream>>>(p.part_o, p.part_ml, ctx_len, (float*)out, out_stride, nq, d,
                                                             p.max_splits);
    } else {
        cudaFuncSetAttribute(decode_attention_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        decode_attention_kernel<bf16><<<grid, DEC_THREADS, smem, stream>>>(p);
        decode_merge_kernel<bf16><<<mgrid, 64, 0, stream>>>(p.part_o, p.part_ml, ctx_len, (bf16*)out, out_stride, nq, d,
                                                            p.max_splits);
    }
    return llmp_check_launch("decode_attention");
}
