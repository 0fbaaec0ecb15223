// Decode attention for bfloat16 pages with head size 128 as one stream per SM: a block whose load warp keeps a
// ring of TMA boxes in flight while four other warps work through what has landed, and which writes the finished
// attention output itself (no partial results in global memory, no merge kernel).
//
// The unit of work is a row group: one request and one key/value head, that is the G query heads that share it
// and all keys of the request. Keys are cut as in attention_decode_mma.cu into ranges of DEC_SPLIT (128) keys
// aligned to key 0, a range into four stages of 32 keys (K and V of a stage: 16 KB, as boxes of one page and half
// a head with keys and values together, 128-byte swizzle). A row group is worked on by C blocks (C = 1 when there
// are row groups enough for all SMs, else a thread-block cluster of 2, 4 or 8): in round j the warp w of block
// `rank` takes the range (j C + rank) 4 + w, walks its four stages with mma.sync and keeps one running softmax in
// registers over all its ranges. The load warp walks the same list, one stage of each of its block's four warps at
// a time, as soon as ring slots are free (a slot belongs to one warp and is handed back when read), so up to
// eight stages of later keys are in flight while four are being read. A table entry that is missing, and keys
// beyond the context, are read at an out-of-range page coordinate (zeros, no traffic); a range beyond the context
// passes its slots on unread.
// At the end of a row group the four warps' sums are added in warp order in shared memory; with C = 1 the block
// normalises and stores the output rows, else every block writes its sums into the shared memory of the cluster's
// first block (distributed shared memory, between two cluster barriers: the ring is used for it once all blocks
// have read their last stage), which adds them in block order, normalises and stores. With C = 1 a block takes
// the row groups b, b + grid, ... one after the other and its loads run ahead across them.
//
// As a dependent launch: the kernel before this one wrote the query rows and the newest key and value
// (position ctx - 1). The load warp waits for it before the first stage that can hold a newest key; the
// compute warps wait before they read their first query rows.
//
// Every wait on an mbarrier is bounded: when one runs out the kernel records 1 in *error_flag and goes on
// without waiting (its output is then wrong; the host reads the flag).
#include "attention_decode_tma.cuh"
#define DT_MAX_CLUSTER 8
#define DT_XROW (DT_D + 4)                           // a row of sums handed to the first block: 128 values, maximum, sum, padding

struct DecodeTmaParams {
    const bf16* q;
    bf16* out;
    const int* block_tables;
    const int* ctx_len;
    long q_stride, out_stride;
    int table_stride;
    int R, nq, nkv, page_size, num_pages, box_tokens, window, max_splits;
    int cluster;             // blocks per row group
    int group_begin, group_count;   // the row groups of this launch: group_begin .. group_begin + group_count - 1
    int rounds;              // rounds of 4 * cluster key ranges that cover max_splits
    float scale;
    int* error_flag;
};

__global__ void __launch_bounds__(DT_THREADS, 1)
decode_attention_tma_kernel(const __grid_constant__ CUtensorMap map_pages, const DecodeTmaParams p) {
    extern __shared__ unsigned char dt_raw[];
    __shared__ __align__(8) uint64_t full_bar[DT_STAGES], empty_bar[DT_STAGES];
    __shared__ float mw[DT_CWARPS][DT_MAX_HEADS], lw[DT_CWARPS][DT_MAX_HEADS];
    // the swizzled tiles want 1024-byte alignment
    const uint32_t raw_addr = tc_smem_u32(dt_raw);
    unsigned char* ring = dt_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
    bf16* Qall = reinterpret_cast<bf16*>(ring + (size_t)DT_STAGES * DT_STAGE_BYTES);   // [warps][8][DT_QSTRIDE]
    bf16* Qzero = Qall + (size_t)DT_CWARPS * DT_MAX_HEADS * DT_QSTRIDE;                // [8][DT_QSTRIDE]: rows 8..15 of every warp's tile
    float* Ow = reinterpret_cast<float*>(Qzero + (size_t)DT_MAX_HEADS * DT_QSTRIDE);   // [warps][8][DT_D]
    float* xch = reinterpret_cast<float*>(ring);         // [cluster][8][DT_XROW], in the first block, once the rings are idle

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = p.nq / p.nkv;
    const int C = p.cluster;
    const int rank = C > 1 ? (int)cluster_ctarank() : 0;
    const int num_groups = p.group_count;                        // groups are numbered from 0 within the launch
    // row groups of this block: with a cluster its own one, else blockIdx.x, blockIdx.x + grid, ...
    const int first_group = C > 1 ? (int)(blockIdx.x / (unsigned)C) : (int)blockIdx.x;
    const int group_step = C > 1 ? num_groups : (int)gridDim.x;      // a cluster has one row group only

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < DT_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_pages) : "memory");
    }
    // query rows beyond the heads of a group, and the common rows 8..15, stay zero
    for (int e = tid; e < (DT_CWARPS + 1) * DT_MAX_HEADS * DT_QSTRIDE / 2; e += DT_THREADS) reinterpret_cast<unsigned*>(Qall)[e] = 0u;
    __syncthreads();
    pdl_trigger();                                               // the kernel after this one may take its places

    // Wave v = t * rounds + j of this block: round j of its t-th row group. Warp w's key range in it is
    // (j C + rank) 4 + w, and stage k of that range is ring stage v * 16 + k * 4 + w, whether or not it has keys.
    if (warp == DT_CWARPS) {
        // ---- loads: lanes 8 wi .. 8 wi + 7 serve the range of compute warp wi ----
        const int wi = lane >> 3, op = lane & 7;
        const int ops = (DT_STAGE_KEYS / p.box_tokens) * 2;      // boxes per stage: tokens x (two halves): 2, 4 or 8
        bool waited = false;
        int ctx_next = 0, entry_next[DT_ITEM_STAGES];
        // context length and page entries of the lane's boxes, read one wave ahead
        auto fetch = [&](int t, int j) {
            const int group = first_group + t * group_step;
            ctx_next = 0;
            if (group >= num_groups) return;
            const int r = (p.group_begin + group) / p.nkv;
            const int c = (j * C + rank) * DT_CWARPS + wi;
            ctx_next = p.ctx_len[r];
            const int* table = p.block_tables + (size_t)r * p.table_stride;
#pragma unroll
            for (int k = 0; k < DT_ITEM_STAGES; ++k) {
                int index = (c * DEC_SPLIT + k * DT_STAGE_KEYS + (op >> 1) * p.box_tokens) / p.page_size;
                if (index >= p.table_stride) index = p.table_stride - 1;          // beyond the context: not used
                entry_next[k] = op < ops ? table[index] : -1;
            }
        };
        fetch(0, 0);
        unsigned v = 0;
        for (int t = 0; first_group + t * group_step < num_groups; ++t) {
            const int group = first_group + t * group_step;
            const int kvh = (p.group_begin + group) % p.nkv;
            for (int j = 0; j < p.rounds; ++j, ++v) {
                const int c = (j * C + rank) * DT_CWARPS + wi;
                const int ctx = ctx_next;
                int entry[DT_ITEM_STAGES];
#pragma unroll
                for (int k = 0; k < DT_ITEM_STAGES; ++k) entry[k] = entry_next[k];
                if (j + 1 < p.rounds) fetch(t, j + 1); else fetch(t + 1, 0);
                const bool real = c * DEC_SPLIT < ctx;
                int hi = (c + 1) * DEC_SPLIT;
                if (hi > ctx) hi = ctx;
#pragma unroll
                for (int k = 0; k < DT_ITEM_STAGES; ++k) {
                    const unsigned n = v * (DT_CWARPS * DT_ITEM_STAGES) + k * DT_CWARPS + wi;
                    const unsigned slot = n % DT_STAGES;
                    if (n >= DT_STAGES) mbar_wait(&empty_bar[slot], ((n / DT_STAGES) - 1) & 1, p.error_flag);
                    const int key0 = c * DEC_SPLIT + k * DT_STAGE_KEYS;
                    const bool newest = real && !waited && key0 + DT_STAGE_KEYS >= ctx;   // holds position ctx - 1, or lies beyond
                    if (__any_sync(0xffffffffu, newest)) {
                        pdl_wait();
                        waited = true;
                    }
                    if (op == 0) {
                        if (real) mbar_expect_tx(&full_bar[slot], DT_STAGE_BYTES);
                        else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem_u32(&full_bar[slot])) : "memory");
                    }
                    __syncwarp();
                    if (real && op < ops) {
                        unsigned char* stage = ring + (size_t)slot * DT_STAGE_BYTES;
                        const int b = op >> 1, half = op & 1;
                        const int key = key0 + b * p.box_tokens;
                        int page = p.num_pages;                  // out of range: the box arrives as zeros
                        if (key < hi && entry[k] >= 0) page = entry[k];
                        tma_load_page_box(stage + half * (2 * DT_HALF_BYTES) + b * (2 * p.box_tokens * 128), &map_pages, half * 64,
                                          key % p.page_size, kvh, 0, page, &full_bar[slot]);
                    }
                }
            }
        }
        if (C > 1) {                                             // the exchange of the sums: every thread of the cluster takes part
            cluster_sync_all();
            cluster_sync_all();
        }
    } else {
        // ---- compute: warp w walks the four stages of its key range of every round ----
        const int w = warp;
        const int g = lane >> 2, t4 = lane & 3;
        bf16* Qs = Qall + (size_t)w * DT_MAX_HEADS * DT_QSTRIDE;
        const float scale_log2 = p.scale * 1.4426950408889634f;
        const int box_shift = 31 - __clz(p.box_tokens);          // box_tokens is 8, 16 or 32
        const int pieces = G * (DT_D / 8);                       // 16-byte pieces of the group's query rows: at most 128
        // this lane's row of the query tile for ldmatrix: rows 0..7 are the warp's own, rows 8..15 the common zero rows
        const bf16* q_row = (lane & 15) < DT_MAX_HEADS ? Qs + (size_t)(lane & 15) * DT_QSTRIDE
                                                        : Qzero + (size_t)((lane & 15) - DT_MAX_HEADS) * DT_QSTRIDE;
        pdl_wait();                                              // the query rows are complete
        // the context length and the query rows of a row group are read one group ahead
        int ctx_next = 0;
        uint4 q_next[4];
        auto fetch = [&](int t) {
            const int group = first_group + t * group_step;
            ctx_next = 0;
            if (group >= num_groups) return;
            const int r = (p.group_begin + group) / p.nkv, kvh = (p.group_begin + group) % p.nkv;
            ctx_next = p.ctx_len[r];
            const bf16* q = p.q + (size_t)r * p.q_stride + (size_t)(kvh * G) * DT_D;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (lane + 32 * i < pieces) q_next[i] = *reinterpret_cast<const uint4*>(q + (size_t)(lane + 32 * i) * 8);
        };
        fetch(0);
        unsigned v = 0;
        for (int t = 0; first_group + t * group_step < num_groups; ++t) {
            const int group = first_group + t * group_step;
            const int r = (p.group_begin + group) / p.nkv, kvh = (p.group_begin + group) % p.nkv;
            const int ctx = ctx_next;
            // the query rows of the group: rows of 128 elements, piece i of the group at row i / 16
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int piece = lane + 32 * i;
                if (piece < pieces) *reinterpret_cast<uint4*>(Qs + (piece >> 4) * DT_QSTRIDE + (piece & 15) * 8) = q_next[i];
            }
            fetch(t + 1);
            __syncwarp();
            const int pos = ctx - 1;

            float o[DT_D / 8][4];
#pragma unroll
            for (int i = 0; i < DT_D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
            float m_run[2] = {-INFINITY, -INFINITY};             // rows g and g + 8, in units of log2
            float l_run[2] = {0.f, 0.f};                         // this lane's share of the row sums
            for (int j = 0; j < p.rounds; ++j, ++v) {
                const int c = (j * C + rank) * DT_CWARPS + w;
                const bool real = c * DEC_SPLIT < ctx;
                int lo = c * DEC_SPLIT, hi = lo + DEC_SPLIT;
                if (hi > ctx) hi = ctx;
                if (p.window > 0 && lo < pos - p.window + 1) lo = pos - p.window + 1;
#pragma unroll 1
                for (int k = 0; k < DT_ITEM_STAGES; ++k) {
                    const unsigned n = v * (DT_CWARPS * DT_ITEM_STAGES) + k * DT_CWARPS + w;
                    const unsigned slot = n % DT_STAGES;
                    mbar_wait(&full_bar[slot], (n / DT_STAGES) & 1, p.error_flag);
                    const unsigned char* stage = ring + (size_t)slot * DT_STAGE_BYTES;
                    const unsigned valid = dt_valid_keys(real, lo, hi, c * DEC_SPLIT + k * DT_STAGE_KEYS);
                    if (valid != 0u) dt_stage_update(stage, valid, q_row, lane, scale_log2, box_shift, o, m_run, l_run);
                    // this warp has read the stage: the slot may be filled again
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem_u32(&empty_bar[slot])) : "memory");
                }
            }

            // ---- the row group is read: the four warps' sums in warp order (rows g < 8; rows g + 8 are padding) ----
            l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
            l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
            if (t4 == 0) {
                mw[w][g] = m_run[0];
                lw[w][g] = l_run[0];
            }
#pragma unroll
            for (int nb = 0; nb < DT_D / 8; ++nb)
                *reinterpret_cast<float2*>(Ow + ((size_t)w * DT_MAX_HEADS + g) * DT_D + nb * 8 + 2 * t4) = make_float2(o[nb][0], o[nb][1]);
            asm volatile("bar.sync 1, %0;\n" ::"n"(DT_CWARPS * 32) : "memory");
            if (C > 1) cluster_sync_all();                       // every block of the cluster has read its last stage
            // thread `tid` takes column `tid` of every row
            for (int row = 0; row < G; ++row) {
                float m = mw[0][row];
#pragma unroll
                for (int x = 1; x < DT_CWARPS; ++x) m = fmaxf(m, mw[x][row]);
                float acc = 0.f, l = 0.f;
#pragma unroll
                for (int x = 0; x < DT_CWARPS; ++x) {
                    const float wgt = mw[x][row] > -INFINITY ? exp2f(mw[x][row] - m) : 0.f;
                    acc = fmaf(Ow[((size_t)x * DT_MAX_HEADS + row) * DT_D + tid], wgt, acc);
                    l = fmaf(lw[x][row], wgt, l);
                }
                if (C == 1) {
                    const float inv = l > 0.f ? 1.f / l : 0.f;
                    p.out[(size_t)r * p.out_stride + (size_t)(kvh * G + row) * DT_D + tid] = __float2bfloat16_rn(acc * inv);
                } else {
                    // to the first block of the cluster: [rank][row][128 values | maximum | sum]
                    const uint32_t at = tc_smem_u32(xch + ((size_t)rank * DT_MAX_HEADS + row) * DT_XROW);
                    st_cluster_f32(at + 4u * (uint32_t)tid, 0, acc);
                    if (tid == 0) {
                        st_cluster_f32(at + 4u * DT_D, 0, m);
                        st_cluster_f32(at + 4u * (DT_D + 1), 0, l);
                    }
                }
            }
            if (C > 1) {
                cluster_sync_all();                              // the sums of every block have arrived
                if (rank == 0) {
                    for (int row = 0; row < G; ++row) {
                        float m = -INFINITY;
                        for (int k = 0; k < C; ++k) m = fmaxf(m, xch[((size_t)k * DT_MAX_HEADS + row) * DT_XROW + DT_D]);
                        float acc = 0.f, l = 0.f;
                        for (int k = 0; k < C; ++k) {
                            const float* src = xch + ((size_t)k * DT_MAX_HEADS + row) * DT_XROW;
                            const float wgt = src[DT_D] > -INFINITY ? exp2f(src[DT_D] - m) : 0.f;
                            acc = fmaf(src[tid], wgt, acc);
                            l = fmaf(src[DT_D + 1], wgt, l);
                        }
                        const float inv = l > 0.f ? 1.f / l : 0.f;
                        p.out[(size_t)r * p.out_stride + (size_t)(kvh * G + row) * DT_D + tid] = __float2bfloat16_rn(acc * inv);
                    }
                }
            }
            asm volatile("bar.sync 1, %0;\n" ::"n"(DT_CWARPS * 32) : "memory");      // the sums are read: the next group may write its own
        }
    }
}

// Sizes this kernel takes: head size 128, at most 8 query heads per key/value head, pages of 8 to 128 tokens.
bool llmp_decode_tma_supports(int nq, int nkv, int d, int page_size) {
    if (d != DT_D || nkv <= 0 || nq % nkv != 0 || nq / nkv > DT_MAX_HEADS) return false;
    return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
}

int llmp_launch_decode_tma(const void* q, long q_stride, void* out, long out_stride, const void* pages, int num_pages,
                           const int* block_tables, int table_stride, const int* ctx_len, int R, int max_splits, int nq,
                           int nkv, int page_size, int window, float scale, int* error_flag, cudaStream_t stream) {
    LLMP_REQUIRE(error_flag != nullptr, "decode attention: an error flag in device memory is required");
    LLMP_REQUIRE((q_stride % 8) == 0 && ((size_t)q % 16) == 0 && ((size_t)pages % 16) == 0,
                 "decode attention: rows must be 16-byte aligned");
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const long groups = (long)R * nkv;
    LLMP_REQUIRE(groups * DT_MAX_CLUSTER < (1L << 31), "decode attention: too many rows");
    DecodeTmaParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.block_tables = block_tables; p.ctx_len = ctx_len;
    p.q_stride = q_stride; p.out_stride = out_stride; p.table_stride = table_stride; p.R = R; p.nq = nq; p.nkv = nkv;
    p.page_size = page_size; p.num_pages = num_pages; p.box_tokens = page_size < DT_STAGE_KEYS ? page_size : DT_STAGE_KEYS;
    p.window = window; p.max_splits = max_splits; p.scale = scale; p.error_flag = error_flag;
    CUtensorMap map;
    if (llmp_pages_tensor_map(pages, nkv, page_size, num_pages, p.box_tokens, 2, 1, &map)) return 1;
    const size_t smem = (size_t)DT_STAGES * DT_STAGE_BYTES + (size_t)(DT_CWARPS + 1) * DT_MAX_HEADS * DT_QSTRIDE * sizeof(bf16) +
                        (size_t)DT_CWARPS * DT_MAX_HEADS * DT_D * sizeof(float) + 1024;
    LLMP_ALLOW_SMEM(decode_attention_tma_kernel, smem);
    // One launch takes `count` row groups from `begin`: with blocks enough for all SMs one block per SM walks its
    // groups one after the other, else a cluster of 2, 4 or 8 blocks (as many as keep the grid within the SMs and
    // give every block at least one round of four key ranges) shares each group.
    auto launch = [&](long begin, long count) -> int {
        int cluster = 1;
        while (cluster < DT_MAX_CLUSTER && count * cluster * 2 <= sms && cluster * 2 * DT_CWARPS <= max_splits + DT_CWARPS - 1) cluster *= 2;
        p.cluster = cluster;
        p.rounds = (max_splits + cluster * DT_CWARPS - 1) / (cluster * DT_CWARPS);
        p.group_begin = (int)begin;
        p.group_count = (int)count;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3((unsigned)(cluster > 1 ? count * cluster : (count < sms ? count : sms)));
        config.blockDim = dim3(DT_THREADS);
        config.dynamicSmemBytes = smem;
        config.stream = stream;
        cudaLaunchAttribute attr[2];
        int n = 0;
        if (llmp_pdl_enabled()) {
            attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // see pdl_wait() in the kernel
            attr[n].val.programmaticStreamSerializationAllowed = 1;
            ++n;
        }
        if (cluster > 1) {
            attr[n].id = cudaLaunchAttributeClusterDimension;
            attr[n].val.clusterDim.x = (unsigned)cluster;
            attr[n].val.clusterDim.y = 1;
            attr[n].val.clusterDim.z = 1;
            ++n;
        }
        config.attrs = attr;
        config.numAttrs = n;
        const cudaError_t launched = cudaLaunchKernelEx(&config, decode_attention_tma_kernel, map, p);
        if (launched != cudaSuccess) {
            llmp_set_error("decode_attention_tma: launch failed: %s", cudaGetErrorString(launched));
            return 2;
        }
        return 0;
    };
    // Row groups all take the same time, so a count that is no multiple of the SMs leaves SMs idle for up to a whole
    // group (512 groups on 148 SMs: 4 rounds for 3.46 rounds of work). The groups beyond the last full multiple go
    // to a second launch, where clusters share them: 3 rounds and half a round.
    const long rest = groups % sms;
    if (groups > sms && rest != 0 && rest * 2 <= sms) {
        if (int rc = launch(0, groups - rest)) return rc;
        if (int rc = launch(groups - rest, rest)) return rc;
    } else if (int rc = launch(0, groups)) {
        return rc;
    }
    return llmp_check_launch("decode_attention_tma");
}
