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

// The tensor-core kernel for bfloat16 pages (attention_prefill_mma.cu).
int llmp_prefill_mma_tokens_per_tile(int nq, int nkv);
bool llmp_prefill_mma_supports(int d);
int llmp_launch_prefill_mma(const void* q, long q_stride, void* out, long out_stride, const void* pages,
                            const int* block_tables, int table_stride, const int* q_start, const int* ctx_len,
                            const int* tile_req, const int* tile_tok0, int num_tiles, int nq, int nkv, int d,
                            int page_size, int window, float scale, cudaStream_t stream);

// The tcgen05 kernel for bfloat16 pages and head size 128 (attention_prefill_tc.cu).
bool llmp_prefill_tc_supports(int nq, int nkv, int d, int page_size);
int llmp_prefill_tc_tokens_per_tile(int nq, int nkv);
int llmp_prefill_tc_max_segments();
long llmp_prefill_tc_place_floats();
int llmp_launch_prefill_tc(const void* q, long q_stride, void* out, long out_stride, const void* pages, int num_pages,
                           const int* block_tables, int table_stride, const int* q_start, const int* ctx_len,
                           const int* tile_req, const int* tile_tok0, const int* tile_seg, const int* tile_slot,
                           float* partials, unsigned* counters, int num_tiles, int nq, int nkv, int page_size,
                           int window, float scale, int* error_flag, cudaStream_t stream);

// Number of query tokens one block covers for a given group size, element type, head size and page size (0:
// not known, which rules out the kernels that depend on it); the caller builds the tile list (tile_req,
// tile_tok0) with this step.
LLMP_API int llmp_attention_tokens_per_tile(int nq, int nkv, int dtype, int d, int page_size) {
    if (nq <= 0 || nkv <= 0 || nq % nkv) return 0;
    if (dtype == LLMP_BF16 && llmp_prefill_tc_supports(nq, nkv, d, page_size)) return llmp_prefill_tc_tokens_per_tile(nq, nkv);
    if (dtype == LLMP_BF16 && llmp_prefill_mma_supports(d)) return llmp_prefill_mma_tokens_per_tile(nq, nkv);
    const int G = nq / nkv;
    const int heads = G < ATT_ROWS ? G : ATT_ROWS;
    return ATT_ROWS / heads;
}

// How many items may share the keys of one tile of the list (1: the kernel for these sizes takes whole tiles only),
// and the floats that one place for an item's sums takes per key/value head.
LLMP_API int llmp_attention_max_segments(int nq, int nkv, int dtype, int d, int page_size) {
    if (nq <= 0 || nkv <= 0 || nq % nkv) return 1;
    return dtype == LLMP_BF16 && llmp_prefill_tc_supports(nq, nkv, d, page_size) ? llmp_prefill_tc_max_segments() : 1;
}
LLMP_API long llmp_attention_place_floats() { return llmp_prefill_tc_place_floats(); }

// pages: [num_pages, 2, nkv, page_size, d]. error_flag: one int in device-visible memory that a kernel with
// bounded waits sets to 1 when a wait ran out (the host checks it after synchronising).
// tile_seg (may be null): the list holds items that share the keys of a tile; item i is number tile_seg[i] & 255 of
// tile_seg[i] >> 8 items of its tile, which follow one another in the list, and tile_slot[i] is the first of the
// tile's places (one per item) in partials ([places][nkv][llmp_attention_place_floats()]) and in counters
// ([places][nkv] unsigned values, zero before the first launch; every launch leaves them zero).
LLMP_API int llmp_paged_attention(const void* q, long q_stride, void* out, long out_stride, const void* pages,
                                  int num_pages, int dtype, const int* block_tables, int table_stride,
                                  const int* q_start, const int* ctx_len, const int* tile_req, const int* tile_tok0,
                                  const int* tile_seg, const int* tile_slot, float* partials, unsigned* counters,
                                  int num_tiles, int nq, int nkv, int d, int page_size, int window, float scale,
                                  int tokens_per_tile, int* error_flag, cudaStream_t stream) {
    if (num_tiles <= 0) return 0;
    LLMP_REQUIRE(tile_seg == nullptr || llmp_attention_max_segments(nq, nkv, dtype, d, page_size) > 1,
                 "attention: the kernel for these sizes takes whole tiles only");
    LLMP_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads cannot share %d key/value heads", nq, nkv);
    LLMP_REQUIRE(d >= 16 && d <= 256 && d % 16 == 0, "attention: head size %d is not a multiple of 16 in 16..256", d);
    LLMP_REQUIRE(page_size > 0 && num_pages > 0, "attention: bad page size %d or page count %d", page_size, num_pages);
    LLMP_REQUIRE(tokens_per_tile == llmp_attention_tokens_per_tile(nq, nkv, dtype, d, page_size),
                 "attention: the tile list was built for %d tokens per tile, the kernel takes %d", tokens_per_tile,
                 llmp_attention_tokens_per_tile(nq, nkv, dtype, d, page_size));
    if (dtype == LLMP_BF16 && llmp_prefill_tc_supports(nq, nkv, d, page_size))
        return llmp_launch_prefill_tc(q, q_stride, out, out_stride, pages, num_pages, block_tables, table_stride, q_start,
                                      ctx_len, tile_req, tile_tok0, tile_seg, tile_slot, partials, counters, num_tiles, nq,
                                      nkv, page_size, window, scale, error_flag, stream);
    if (dtype == LLMP_BF16 && llmp_prefill_mma_supports(d))
        return llmp_launch_prefill_mma(q, q_stride, out, out_stride, pages, block_tables, table_stride, q_start, ctx_len,
                                       tile_req, tile_tok0, num_tiles, nq, nkv, d, page_size, window, scale, stream);
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
        LLMP_ALLOW_SMEM(paged_attention_kernel<float>, smem);
        paged_attention_kernel<float><<<grid, ATT_THREADS, smem, stream>>>(p);
    } else {
        LLMP_ALLOW_SMEM(paged_attention_kernel<bf16>, smem);
        paged_attention_kernel<bf16><<<grid, ATT_THREADS, smem, stream>>>(p);
    }
    return llmp_check_launch("paged_attention");
}
