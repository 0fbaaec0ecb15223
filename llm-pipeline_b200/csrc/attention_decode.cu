// Decode attention over paged keys and values: one query row per request (row r of q belongs
// to request r, at position ctx_len[r] - 1).
//
// Keys are split into fixed ranges of DEC_SPLIT keys that are aligned to key 0, so where a range
// starts and ends depends on the key's index alone, not on the batch. Block (range, kv head x head
// chunk, request) computes the softmax-weighted sum over its range for the query heads that share
// one key/value head and writes an unnormalised partial (running max, running sum, vector) to
// scratch memory; decode_merge_kernel combines the partials of a row in ascending range order.
// K and V tiles of DEC_TILE keys go from the pages to shared memory with 16-byte cp.async copies,
// two tiles in flight (one when two do not fit), so the next tile streams in while this one is used.
#include "attention_decode.cuh"
#include "common.cuh"

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
    int heads_per_cta, head_chunks, max_splits, stages;
    float scale;
};

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;       // 0: nothing is read, the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(DEC_THREADS) decode_attention_kernel(const DecodeParams p) {
    extern __shared__ __align__(16) unsigned char dec_smem[];
    const int d = p.d;
    constexpr int VEC = 16 / (int)sizeof(T);                     // elements per 16-byte copy
    const int kstride = d + VEC;                                 // padded key row, in elements
    const int stage_elems = DEC_TILE * kstride + DEC_TILE * d;   // one K tile and one V tile
    T* tiles = reinterpret_cast<T*>(dec_smem);                   // [stages][K tile | V tile]
    float* Qs = reinterpret_cast<float*>(tiles + (size_t)p.stages * stage_elems);   // [heads][d]
    float* Ss = Qs + DEC_MAX_HEADS * d;                          // [heads][DEC_TILE]
    float* row_m = Ss + DEC_MAX_HEADS * DEC_TILE;                // [heads]
    float* row_l = row_m + DEC_MAX_HEADS;
    float* row_a = row_l + DEC_MAX_HEADS;
    __shared__ long long key_off[2][DEC_TILE];

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
    const int vec_per_row = d / VEC;

    // Address of each key of a tile (or -1), then its K and V rows as asynchronous 16-byte copies.
    auto issue_tile = [&](int j0, int buf) {
        if (tid < DEC_TILE) {
            const int j = j0 + tid;
            long long off = -1;
            if (j >= lo && j < hi) {
                const int page = table[j / p.page_size];
                if (page >= 0)
                    off = (long long)((((size_t)page * 2) * p.nkv + kvh) * p.page_size + (j % p.page_size)) * d;
            }
            key_off[buf][tid] = off;
        }
        __syncthreads();
        T* Ks = tiles + (size_t)buf * stage_elems;
        T* Vs = Ks + DEC_TILE * kstride;
        for (int e = tid; e < DEC_TILE * vec_per_row; e += DEC_THREADS) {
            const int key = e / vec_per_row, c = (e % vec_per_row) * VEC;
            const long long off = key_off[buf][key];
            const bool ok = off >= 0;
            const T* src = ok ? pages + off + c : pages;
            cp_async_16(Ks + key * kstride + c, src, ok);
            cp_async_16(Vs + key * d + c, ok ? src + plane : pages, ok);
        }
        cp_async_commit();
    };

    for (int e = tid; e < heads * d; e += DEC_THREADS) Qs[e] = to_float(q[e]);
    if (tid < DEC_MAX_HEADS) {
        row_m[tid] = -INFINITY;
        row_l[tid] = 0.f;
    }
    float acc[DEC_MAX_ACC][2];
#pragma unroll
    for (int i = 0; i < DEC_MAX_ACC; ++i) acc[i][0] = acc[i][1] = 0.f;
    const int pairs = heads * d / 2;                              // (head, column pair) outputs of this block

    const int tile_lo = (lo / DEC_TILE) * DEC_TILE;
    const bool two = p.stages > 1;
    if (tile_lo < hi) issue_tile(tile_lo, 0);
    int buf = 0;
    for (int j0 = tile_lo; j0 < hi; j0 += DEC_TILE) {
        const bool more = j0 + DEC_TILE < hi;
        if (two && more) {
            issue_tile(j0 + DEC_TILE, buf ^ 1);      // streams in while this tile is used
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const T* Ks = tiles + (size_t)buf * stage_elems;
        const T* Vs = Ks + DEC_TILE * kstride;
        // scores: thread -> key tid % DEC_TILE, heads (tid / DEC_TILE), +2, ...
        {
            const int key = tid % DEC_TILE;
            const bool key_ok = key_off[buf][key] >= 0;
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
#pragma unroll 8
                for (int key = 0; key < DEC_TILE; ++key) {
                    const float pr = prow[key];
                    a0 = fmaf(pr, to_float(Vs[key * d + c]), a0);
                    a1 = fmaf(pr, to_float(Vs[key * d + c + 1]), a1);
                }
                acc[i][0] = a0;
                acc[i][1] = a1;
            }
        }
        __syncthreads();                              // this tile's buffer and Ss may be overwritten now
        if (two) {
            buf ^= 1;
        } else if (more) {
            issue_tile(j0 + DEC_TILE, 0);
        }
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

// One block per (query head, request): weights exp(m_s - m) of the ranges once, then each thread sums
// its columns over the ranges in ascending order.
#define MERGE_THREADS 128
#define MERGE_MAX_SPLITS 1024
template <typename T>
__global__ void __launch_bounds__(MERGE_THREADS)
decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                    const int* __restrict__ ctx_len, T* __restrict__ out, long out_stride, int nq, int d,
                    int max_splits) {
    __shared__ float wgt[MERGE_MAX_SPLITS];
    __shared__ float scratch[32];
    pdl_trigger();                                 // the product that follows may start fetching its weights
    pdl_wait();                                    // the partials are complete
    const int r = blockIdx.y, h = blockIdx.x;
    const int ctx = ctx_len[r];
    const int nsplits = (ctx + DEC_SPLIT - 1) / DEC_SPLIT;
    const float* ml = part_ml + ((size_t)r * nq + h) * max_splits * 2;
    const float* po = part_o + ((size_t)r * nq + h) * max_splits * d;
    float m = -INFINITY;
    for (int s = threadIdx.x; s < nsplits; s += MERGE_THREADS) m = fmaxf(m, ml[2 * s]);
    m = block_max(m, scratch);
    float l = 0.f;
    for (int s = threadIdx.x; s < nsplits; s += MERGE_THREADS) {
        const float ms = ml[2 * s];
        const float w = (ms > -INFINITY) ? expf(ms - m) : 0.f;
        wgt[s] = w;
        l += ml[2 * s + 1] * w;
    }
    l = block_sum(l, scratch);
    __syncthreads();
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int c = threadIdx.x; c < d; c += MERGE_THREADS) {
        float o = 0.f;
        for (int s = 0; s < nsplits; ++s) o = fmaf(po[(size_t)s * d + c], wgt[s], o);
        out[(size_t)r * out_stride + (size_t)h * d + c] = from_float<T>(o * inv);
    }
}

// The tensor-core variant for bfloat16 pages (attention_decode_mma.cu).
int llmp_launch_decode_mma(const void* q, long q_stride, const void* pages, const int* block_tables, int table_stride,
                           const int* ctx_len, int R, int max_splits, int nq, int nkv, int d, int page_size,
                           int window, float scale, float* part_o, float* part_ml, cudaStream_t stream);

// The streaming kernel for head size 128 (attention_decode_tma.cu).
bool llmp_decode_tma_supports(int nq, int nkv, int d, int page_size);
int llmp_launch_decode_tma(const void* q, long q_stride, void* out, long out_stride, const void* pages, int num_pages,
                           const int* block_tables, int table_stride, const int* ctx_len, int R, int max_splits, int nq,
                           int nkv, int page_size, int window, float scale, int* error_flag, cudaStream_t stream);

// The streaming kernel that deals the key ranges of all requests out evenly (attention_decode_list.cu).
int llmp_decode_list_max_rows();
long llmp_decode_list_scratch_floats();
int llmp_decode_list_counters();
int llmp_launch_decode_list(const void* q, long q_stride, void* out, long out_stride, const void* pages, int num_pages,
                            const int* block_tables, int table_stride, const int* ctx_len, int R, int nq, int nkv,
                            int page_size, int window, float scale, float* scratch, unsigned* counters, int* error_flag,
                            cudaStream_t stream);

// Scratch floats the decode kernel needs for R rows whose longest context is max_ctx keys.
LLMP_API long llmp_decode_scratch_floats(int R, int nq, int d, int max_ctx) {
    const long splits = (max_ctx + DEC_SPLIT - 1) / DEC_SPLIT;
    const long ranges = (long)R * nq * (splits > 0 ? splits : 1) * (d + 2);
    const long stream = llmp_decode_list_scratch_floats();
    return ranges > stream ? ranges : stream;
}

// Counters (unsigned, zero before the first launch; every launch leaves them zero) that the streaming kernel needs.
// Launches that may run at the same time need counters and scratch of their own.
LLMP_API int llmp_decode_counters() { return llmp_decode_list_counters(); }

// pages: [num_pages, 2, nkv, page_size, d]. error_flag: one int in device-visible memory that a kernel with bounded
// waits sets to 1 when a wait ran out (may be null: the kernels that need it are then not used).
// counters: llmp_decode_counters() zeroed unsigned values for the kernel that deals key ranges out evenly (may be
// null in the same way). uneven: the caller's word that the requests' contexts differ much or are too many for one
// block each, which is when that kernel is the faster one; the result does not depend on it beyond rounding.
LLMP_API int llmp_decode_attention(const void* q, long q_stride, void* out, long out_stride, const void* pages,
                                   int num_pages, int dtype, const int* block_tables, int table_stride,
                                   const int* ctx_len, int R, int max_ctx, int nq, int nkv, int d, int page_size,
                                   int window, float scale, float* scratch, long scratch_floats, unsigned* counters,
                                   int uneven, int* error_flag, cudaStream_t stream) {
    if (R <= 0) return 0;
    LLMP_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads cannot share %d key/value heads", nq, nkv);
    LLMP_REQUIRE(d >= 16 && d <= 256 && d % 16 == 0, "attention: head size %d is not a multiple of 16 in 16..256", d);
    LLMP_REQUIRE(page_size > 0 && max_ctx > 0, "decode attention: bad page size %d or context %d", page_size, max_ctx);
    LLMP_REQUIRE(R <= 65535, "decode attention: too many rows %d", R);
    LLMP_REQUIRE((max_ctx + DEC_SPLIT - 1) / DEC_SPLIT <= MERGE_MAX_SPLITS, "decode attention: a context of %d keys is beyond %d", max_ctx, MERGE_MAX_SPLITS * DEC_SPLIT);
    const int esize = dtype == LLMP_F32 ? 4 : 2;
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
    const size_t stage = (size_t)esize * (DEC_TILE * (d + 16 / esize) + DEC_TILE * d);
    const size_t rest = sizeof(float) * ((size_t)DEC_MAX_HEADS * d + DEC_MAX_HEADS * DEC_TILE + 3 * DEC_MAX_HEADS);
    p.stages = (2 * stage + rest <= 100 * 1024) ? 2 : 1;       // two tiles in flight while two blocks still fit an SM
    const size_t smem = p.stages * stage + rest;
    dim3 grid(p.max_splits, nkv * p.head_chunks, R);
    dim3 mgrid(nq, R);
    if (dtype == LLMP_F32) {
        LLMP_ALLOW_SMEM(decode_attention_kernel<float>, smem);
        decode_attention_kernel<float><<<grid, DEC_THREADS, smem, stream>>>(p);
        decode_merge_kernel<float><<<mgrid, MERGE_THREADS, 0, stream>>>(p.part_o, p.part_ml, ctx_len, (float*)out, out_stride, nq, d,
                                                             p.max_splits);
    } else {
        if (error_flag != nullptr && num_pages > 0 && llmp_decode_tma_supports(nq, nkv, d, page_size)) {
            // the streaming kernels write the finished output themselves: no merge kernel
            if (uneven && counters != nullptr && R <= llmp_decode_list_max_rows())
                return llmp_launch_decode_list(q, q_stride, out, out_stride, pages, num_pages, block_tables, table_stride,
                                               ctx_len, R, nq, nkv, page_size, window, scale, scratch, counters, error_flag,
                                               stream);
            return llmp_launch_decode_tma(q, q_stride, out, out_stride, pages, num_pages, block_tables, table_stride, ctx_len, R,
                                          p.max_splits, nq, nkv, page_size, window, scale, error_flag, stream);
        } else if (llmp_launch_decode_mma(q, q_stride, pages, block_tables, table_stride, ctx_len, R, p.max_splits, nq, nkv, d,
                                          page_size, window, scale, p.part_o, p.part_ml, stream))
            return 1;
        const cudaError_t launched = llmp_launch_dependent(decode_merge_kernel<bf16>, mgrid, dim3(MERGE_THREADS), 0, stream,
                                                           p.part_o, p.part_ml, ctx_len, (bf16*)out, out_stride, nq, d, p.max_splits);
        if (launched != cudaSuccess) {
            llmp_set_error("decode_merge: launch failed: %s", cudaGetErrorString(launched));
            return 2;
        }
    }
    return llmp_check_launch("decode_attention");
}
