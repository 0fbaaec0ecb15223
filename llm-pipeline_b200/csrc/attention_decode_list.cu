// Decode attention for bfloat16 pages with head size 128 as one stream per SM: a block whose load warp keeps a
// ring of TMA boxes in flight while four other warps work through what has landed, and which writes the finished
// attention output itself (no merge kernel).
//
// A row group is one request and one key/value head: the G query heads that share it and the keys of the request
// (with a window, those that the newest position still sees). Keys are cut as in attention_decode_mma.cu into ranges
// of DEC_SPLIT (128) keys aligned to key 0, a range into four stages of 32 keys (K and V of a stage: 16 KB, as boxes
// of one page and half a head with keys and values together, 128-byte swizzle). All ranges of all row groups of the
// launch form one list (request by request, head by head, key 0 first), and block b of B takes the places
// b N / B .. (b + 1) N / B - 1 of its N entries: every block streams the same number of bytes whatever the lengths
// of the requests are, and a request far longer than the others is shared by many blocks. A block's share falls into
// segments, the ranges of one row group each; it walks a segment four ranges at a time, one per compute warp, with
// mma.sync and one running softmax in registers per warp. The load warp walks the same list, one stage of each of
// the four warps at a time, as soon as ring slots are free (a slot belongs to one warp and is handed back when
// read), so up to eight stages of later keys are in flight while four are being read. A table entry that is
// missing, and keys beyond the context, are read at an out-of-range page coordinate (zeros, no traffic).
//
// At the end of a segment the four warps' sums are added in warp order in shared memory. A segment that is a whole
// row group is normalised and stored. Of a row group that several blocks share, every block leaves its sums in
// global memory (a block has at most two such segments: one that began in an earlier block, one that goes on in a
// later one), counts itself on the counter of the block where the group began, and the block that counts last adds
// the sums in block order, normalises, stores and sets the counter back to zero. Nobody waits for anybody.
//
// As a dependent launch: the kernel before this one wrote the query rows and the newest key and value
// (position ctx - 1). The load warp waits for it before the first stage that can hold a newest key; the
// compute warps wait before they read their first query rows. Context lengths are inputs of the step.
//
// Every wait on an mbarrier is bounded: when one runs out the kernel records 1 in *error_flag and goes on
// without waiting (its output is then wrong; the host reads the flag).
#include "attention_decode_tma.cuh"
#define DT_MAX_ROWS 512                              // requests of a launch: their range counts live in shared memory
#define DT_MAX_BLOCKS 256
#define DT_GROUP_COST 2                              // places of a row group in the list besides its ranges
#define DT_MIN_SHARE 6                               // places of a block's share at least
#define DT_PART (DT_MAX_HEADS * DT_D + 2 * DT_MAX_HEADS)   // floats of a segment's sums: 8 rows, their maxima, their weights

struct DecodeListParams {
    const bf16* q;
    bf16* out;
    const int* block_tables;
    const int* ctx_len;
    long q_stride, out_stride;
    int table_stride;
    int R, nq, nkv, page_size, num_pages, box_tokens, window;
    float scale;
    float* partials;         // [blocks][2][DT_PART]: a block's segment that began earlier, its segment that goes on later
    unsigned* arrivals;      // [blocks]: zero between launches
    int* error_flag;
};

// Ranges i0 .. i1 - 1 of the n ranges of row group (r, h). The group's range i covers the keys of range first + i
// of the request. In the launch's list a row group holds n + DT_GROUP_COST places, its ranges first: the places
// after them stand for the time a block spends on a group besides reading its keys (its query rows, the sums at the
// end), so that a block with many short groups gets fewer of them. x is the place of range i0, x_end the place
// after the segment's last one (which may be one of the group's places without a range).
struct DtSegment {
    int r, h, i0, i1, n, first, ctx;
    long x, x_end;
    bool ok;
};

// ranges of a request of ctx keys: first range that the newest position sees, and how many (at least one, so that
// every row group is somebody's and gets its output written)
__device__ __forceinline__ int dt_first_range(int ctx, int window) {
    return (window > 0 && ctx > window) ? (ctx - window) / DEC_SPLIT : 0;
}
__device__ __forceinline__ int dt_num_ranges(int ctx, int window) {
    const int n = (ctx + DEC_SPLIT - 1) / DEC_SPLIT - dt_first_range(ctx, window);
    return n > 0 ? n : 1;
}

__device__ __forceinline__ void dt_enter_request(DtSegment& s, const int* pre, const int* ctxs, int window) {
    s.ctx = ctxs[s.r];
    s.n = pre[s.r + 1] - pre[s.r] - DT_GROUP_COST;
    s.first = dt_first_range(s.ctx, window);
}

// the segment at the start of the next row group, in a share that ends at place x1 (x < x1)
__device__ __forceinline__ void dt_enter_group(DtSegment& s, long x, long x1) {
    s.x = x;
    s.i0 = 0;
    const long left = x1 - x;
    s.i1 = (long)s.n <= left ? s.n : (int)left;
    s.x_end = (long)(s.n + DT_GROUP_COST) <= left ? x + s.n + DT_GROUP_COST : x1;
}

// the segment after s in a share that ends at place x1
__device__ __forceinline__ void dt_next(DtSegment& s, long x1, const int* pre, const int* ctxs, int nkv, int window) {
    if (s.x_end >= x1) {
        s.ok = false;
        return;
    }
    if (++s.h == nkv) {                                          // s ended with its row group: the next group starts
        s.h = 0;
        ++s.r;
        dt_enter_request(s, pre, ctxs, window);
    }
    dt_enter_group(s, s.x_end, x1);
}

// the first segment with a range in the places x .. x1 - 1 of the list
__device__ __forceinline__ DtSegment dt_open(long x, long x1, const int* pre, const int* ctxs, int R, int nkv, int window) {
    DtSegment s;
    s.ok = x < x1;
    s.x = s.x_end = x;
    s.r = s.h = s.i0 = s.i1 = s.first = s.ctx = 0;
    s.n = 1;
    if (!s.ok) return s;
    int lo = 0, hi = R - 1;                                      // the last request whose places start at or before x
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if ((long)nkv * pre[mid] <= x) lo = mid; else hi = mid - 1;
    }
    s.r = lo;
    dt_enter_request(s, pre, ctxs, window);
    const int places = s.n + DT_GROUP_COST;
    const int rel = (int)(x - (long)nkv * pre[lo]);
    s.h = rel / places;
    const int at = rel - s.h * places;                           // the group's place that x is
    const long left = x1 - x;
    s.x_end = (long)(places - at) <= left ? x + (places - at) : x1;
    s.i0 = at;
    s.i1 = (long)(s.n - at) <= left ? s.n : at + (int)left;
    if (s.i0 >= s.i1) dt_next(s, x1, pre, ctxs, nkv, window);     // only places without a range: on to the next group
    return s;
}

__global__ void __launch_bounds__(DT_THREADS, 1)
decode_attention_list_kernel(const __grid_constant__ CUtensorMap map_pages, const DecodeListParams p) {
    extern __shared__ unsigned char dt_raw[];
    __shared__ __align__(8) uint64_t full_bar[DT_STAGES], empty_bar[DT_STAGES];
    __shared__ float mw[DT_CWARPS][DT_MAX_HEADS], lw[DT_CWARPS][DT_MAX_HEADS];
    __shared__ int pre[DT_MAX_ROWS + 1], ctxs[DT_MAX_ROWS];      // ranges of the requests before r; context lengths
    __shared__ unsigned arrived_before;
    // the swizzled tiles want 1024-byte alignment
    const uint32_t raw_addr = tc_smem_u32(dt_raw);
    unsigned char* ring = dt_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
    bf16* Qall = reinterpret_cast<bf16*>(ring + (size_t)DT_STAGES * DT_STAGE_BYTES);   // [warps][8][DT_QSTRIDE]
    bf16* Qzero = Qall + (size_t)DT_CWARPS * DT_MAX_HEADS * DT_QSTRIDE;                // [8][DT_QSTRIDE]: rows 8..15 of every warp's tile
    float* Ow = reinterpret_cast<float*>(Qzero + (size_t)DT_MAX_HEADS * DT_QSTRIDE);   // [warps][8][DT_D]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = p.nq / p.nkv;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < DT_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_pages) : "memory");
        pre[0] = 0;
    }
    for (int r = tid; r < p.R; r += DT_THREADS) {
        const int ctx = p.ctx_len[r];
        ctxs[r] = ctx;
        pre[r + 1] = dt_num_ranges(ctx, p.window) + DT_GROUP_COST;
    }
    // query rows beyond the heads of a group, and the common rows 8..15, stay zero
    for (int e = tid; e < (DT_CWARPS + 1) * DT_MAX_HEADS * DT_QSTRIDE / 2; e += DT_THREADS) reinterpret_cast<unsigned*>(Qall)[e] = 0u;
    __syncthreads();
    if (warp == 0) {                                             // running sums of the range counts
        int carry = 0;
        for (int base = 0; base < p.R; base += 32) {
            int val = base + lane < p.R ? pre[base + lane + 1] : 0;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, val, off);
                if (lane >= off) val += up;
            }
            if (base + lane < p.R) pre[base + lane + 1] = val + carry;
            carry += __shfl_sync(0xffffffffu, val, 31);
        }
    }
    __syncthreads();
    pdl_trigger();                                               // the kernel after this one may take its places

    // this block's share of the list
    const long N = (long)p.nkv * pre[p.R];
    // a share is at least DT_MIN_SHARE places (a wave of four ranges and a group's cost): with fewer places than that
    // for every block the last blocks have none
    const long most = N / DT_MIN_SHARE > 0 ? N / DT_MIN_SHARE : 1;
    const long blocks = (long)gridDim.x < most ? (long)gridDim.x : most;
    if ((long)blockIdx.x >= blocks) return;
    const long x0 = (long)blockIdx.x * N / blocks, x1 = ((long)blockIdx.x + 1) * N / blocks;

    // Wave v of this block: four consecutive ranges of a segment, one per compute warp. Stage k of warp w's range
    // is ring stage v * 16 + k * 4 + w, whether or not it has keys.
    if (warp == DT_CWARPS) {
        // ---- loads: lanes 8 wi .. 8 wi + 7 serve the range of compute warp wi ----
        const int wi = lane >> 3, op = lane & 7;
        const int ops = (DT_STAGE_KEYS / p.box_tokens) * 2;      // boxes per stage: tokens x (two halves): 2, 4 or 8
        bool waited = false;
        DtSegment seg = dt_open(x0, x1, pre, ctxs, p.R, p.nkv, p.window);
        int j = 0;                                               // wave of the segment
        // the lane's range of the coming wave and the page entries of its boxes, read one wave ahead
        int ctx_next = 0, kvh_next = 0, c_next = 0, entry_next[DT_ITEM_STAGES];
        bool real_next = false;
        auto fetch = [&]() {
            real_next = false;
            if (!seg.ok) return;
            const int i = seg.i0 + j * DT_CWARPS + wi;
            c_next = seg.first + i;
            ctx_next = seg.ctx;
            kvh_next = seg.h;
            real_next = i < seg.i1 && c_next * DEC_SPLIT < ctx_next;
            const int* table = p.block_tables + (size_t)seg.r * p.table_stride;
#pragma unroll
            for (int k = 0; k < DT_ITEM_STAGES; ++k) {
                int index = (c_next * DEC_SPLIT + k * DT_STAGE_KEYS + (op >> 1) * p.box_tokens) / p.page_size;
                if (index >= p.table_stride) index = p.table_stride - 1;          // beyond the context: not used
                entry_next[k] = (real_next && op < ops) ? table[index] : -1;
            }
        };
        fetch();
        bool have = seg.ok;
        for (unsigned v = 0; have; ++v) {
            const int ctx = ctx_next, kvh = kvh_next, c = c_next;
            const bool real = real_next;
            int entry[DT_ITEM_STAGES];
#pragma unroll
            for (int k = 0; k < DT_ITEM_STAGES; ++k) entry[k] = entry_next[k];
            // the wave after this one
            if ((j + 1) * DT_CWARPS < seg.i1 - seg.i0) {
                ++j;
            } else {
                dt_next(seg, x1, pre, ctxs, p.nkv, p.window);
                j = 0;
            }
            fetch();
            have = seg.ok;
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
                    int page = p.num_pages;                      // out of range: the box arrives as zeros
                    if (key < hi && entry[k] >= 0) page = entry[k];
                    tma_load_page_box(stage + half * (2 * DT_HALF_BYTES) + b * (2 * p.box_tokens * 128), &map_pages, half * 64,
                                      key % p.page_size, kvh, 0, page, &full_bar[slot]);
                }
            }
        }
    } else {
        // ---- compute: warp w walks the four stages of its key range of every wave ----
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
        // the query rows of a row group are read one segment ahead
        uint4 q_next[4];
        auto fetch = [&](const DtSegment& of) {
            if (!of.ok) return;
            const bf16* q = p.q + (size_t)of.r * p.q_stride + (size_t)(of.h * G) * DT_D;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (lane + 32 * i < pieces) q_next[i] = *reinterpret_cast<const uint4*>(q + (size_t)(lane + 32 * i) * 8);
        };
        DtSegment seg = dt_open(x0, x1, pre, ctxs, p.R, p.nkv, p.window);
        fetch(seg);
        unsigned v = 0;
        while (seg.ok) {
            const int r = seg.r, kvh = seg.h, ctx = seg.ctx;
            // the query rows of the group: rows of 128 elements, piece i of the group at row i / 16
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int piece = lane + 32 * i;
                if (piece < pieces) *reinterpret_cast<uint4*>(Qs + (piece >> 4) * DT_QSTRIDE + (piece & 15) * 8) = q_next[i];
            }
            DtSegment after = seg;
            dt_next(after, x1, pre, ctxs, p.nkv, p.window);
            fetch(after);
            __syncwarp();
            const int pos = ctx - 1;

            float o[DT_D / 8][4];
#pragma unroll
            for (int i = 0; i < DT_D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
            float m_run[2] = {-INFINITY, -INFINITY};             // rows g and g + 8, in units of log2
            float l_run[2] = {0.f, 0.f};                         // this lane's share of the row sums
            const int waves = (seg.i1 - seg.i0 + DT_CWARPS - 1) / DT_CWARPS;
            for (int j = 0; j < waves; ++j, ++v) {
                const int i = seg.i0 + j * DT_CWARPS + w;
                const int c = seg.first + i;
                const bool real = i < seg.i1 && c * DEC_SPLIT < ctx;
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

            // ---- the segment is read: the four warps' sums in warp order (rows g < 8; rows g + 8 are padding) ----
            l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
            l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
            if (t4 == 0) {
                mw[w][g] = m_run[0];
                lw[w][g] = l_run[0];
            }
#pragma unroll
            for (int col8 = 0; col8 < DT_D / 8; ++col8)
                *reinterpret_cast<float2*>(Ow + ((size_t)w * DT_MAX_HEADS + g) * DT_D + col8 * 8 + 2 * t4) = make_float2(o[col8][0], o[col8][1]);
            asm volatile("bar.sync 1, %0;\n" ::"n"(DT_CWARPS * 32) : "memory");
            // A row group that is not wholly this block's: the blocks first .. first + shared_by - 1 hold its segments.
            const bool whole = seg.i0 == 0 && seg.i1 == seg.n;
            int first_block = 0, shared_by = 1;
            float* part = nullptr;
            if (!whole) {
                const long xg = seg.x - seg.i0;                      // the group's first place in the list
                first_block = (int)(((xg + 1) * blocks - 1) / N);    // the last block whose share starts at or before a place
                shared_by = (int)(((xg + seg.n) * blocks - 1) / N) - first_block + 1;
                part = p.partials + ((size_t)blockIdx.x * 2 + (seg.i0 > 0 ? 0 : 1)) * DT_PART;
            }
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
                if (whole) {
                    const float inv = l > 0.f ? 1.f / l : 0.f;
                    p.out[(size_t)r * p.out_stride + (size_t)(kvh * G + row) * DT_D + tid] = __float2bfloat16_rn(acc * inv);
                } else {
                    part[row * DT_D + tid] = acc;
                    if (tid == 0) {
                        part[DT_MAX_HEADS * DT_D + row] = m;
                        part[DT_MAX_HEADS * DT_D + DT_MAX_HEADS + row] = l;
                    }
                }
            }
            if (!whole) {
                __threadfence();                                 // the sums are visible before the count is
                asm volatile("bar.sync 1, %0;\n" ::"n"(DT_CWARPS * 32) : "memory");
                if (tid == 0) arrived_before = atomicAdd(&p.arrivals[first_block], 1u);
                asm volatile("bar.sync 1, %0;\n" ::"n"(DT_CWARPS * 32) : "memory");
                if (arrived_before == (unsigned)(shared_by - 1)) {
                    // Every block of the group has left its sums: add them in block order (the first block's segment
                    // goes on later, the others' began earlier). Loads that do not depend on one another are issued
                    // together: the maxima and weights of all segments first (into the place of the warps' sums,
                    // which are read), then the sums of four segments at a time.
                    __threadfence();
                    float* ml = Ow;                              // [shared_by][maxima of 8 rows | weights of 8 rows]
                    for (int e = tid; e < shared_by * 2 * DT_MAX_HEADS; e += DT_CWARPS * 32) {
                        const int k = e / (2 * DT_MAX_HEADS);
                        ml[e] = __ldcg(p.partials + ((size_t)(first_block + k) * 2 + (k == 0 ? 1 : 0)) * DT_PART + DT_MAX_HEADS * DT_D +
                                       (e - k * 2 * DT_MAX_HEADS));
                    }
                    asm volatile("bar.sync 1, %0;\n" ::"n"(DT_CWARPS * 32) : "memory");
                    float m[DT_MAX_HEADS], acc[DT_MAX_HEADS], l[DT_MAX_HEADS];
#pragma unroll
                    for (int row = 0; row < DT_MAX_HEADS; ++row) {
                        m[row] = -INFINITY;
                        acc[row] = l[row] = 0.f;
                    }
                    for (int k = 0; k < shared_by; ++k) {
#pragma unroll
                        for (int row = 0; row < DT_MAX_HEADS; ++row) m[row] = fmaxf(m[row], ml[k * 2 * DT_MAX_HEADS + row]);
                    }
                    for (int k0 = 0; k0 < shared_by; k0 += 4) {
                        float val[4][DT_MAX_HEADS];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int k = k0 + u;
                            const float* src = p.partials + ((size_t)(first_block + k) * 2 + (k == 0 ? 1 : 0)) * DT_PART;
#pragma unroll
                            for (int row = 0; row < DT_MAX_HEADS; ++row)
                                val[u][row] = (k < shared_by && row < G) ? __ldcg(src + row * DT_D + tid) : 0.f;
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int k = k0 + u;
                            if (k < shared_by) {
#pragma unroll
                                for (int row = 0; row < DT_MAX_HEADS; ++row) {
                                    const float mk = ml[k * 2 * DT_MAX_HEADS + row];
                                    const float wgt = mk > -INFINITY ? exp2f(mk - m[row]) : 0.f;
                                    acc[row] = fmaf(val[u][row], wgt, acc[row]);
                                    l[row] = fmaf(ml[k * 2 * DT_MAX_HEADS + DT_MAX_HEADS + row], wgt, l[row]);
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int row = 0; row < DT_MAX_HEADS; ++row) {
                        if (row < G) {
                            const float inv = l[row] > 0.f ? 1.f / l[row] : 0.f;
                            p.out[(size_t)r * p.out_stride + (size_t)(kvh * G + row) * DT_D + tid] = __float2bfloat16_rn(acc[row] * inv);
                        }
                    }
                    if (tid == 0) p.arrivals[first_block] = 0u;  // for the next launch
                }
            }
            asm volatile("bar.sync 1, %0;\n" ::"n"(DT_CWARPS * 32) : "memory");      // the sums are read: the next segment may write its own
            seg = after;
        }
    }
}

// Requests a launch takes, floats of scratch it needs for the sums of shared row groups, and counters (zero
// between launches) it needs.
int llmp_decode_list_max_rows() { return DT_MAX_ROWS; }
long llmp_decode_list_scratch_floats() { return (long)DT_MAX_BLOCKS * 2 * DT_PART; }
int llmp_decode_list_counters() { return DT_MAX_BLOCKS; }

int llmp_launch_decode_list(const void* q, long q_stride, void* out, long out_stride, const void* pages, int num_pages,
                           const int* block_tables, int table_stride, const int* ctx_len, int R, int nq, int nkv,
                           int page_size, int window, float scale, float* scratch, unsigned* counters, int* error_flag,
                           cudaStream_t stream) {
    LLMP_REQUIRE(error_flag != nullptr && scratch != nullptr && counters != nullptr,
                 "decode attention: an error flag, scratch and counters in device memory are required");
    LLMP_REQUIRE(R <= DT_MAX_ROWS, "decode attention: %d rows are more than the streaming kernel's %d", R, DT_MAX_ROWS);
    LLMP_REQUIRE((q_stride % 8) == 0 && ((size_t)q % 16) == 0 && ((size_t)pages % 16) == 0,
                 "decode attention: rows must be 16-byte aligned");
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        if (sms > DT_MAX_BLOCKS) sms = DT_MAX_BLOCKS;
    }
    DecodeListParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.block_tables = block_tables; p.ctx_len = ctx_len;
    p.q_stride = q_stride; p.out_stride = out_stride; p.table_stride = table_stride; p.R = R; p.nq = nq; p.nkv = nkv;
    p.page_size = page_size; p.num_pages = num_pages; p.box_tokens = page_size < DT_STAGE_KEYS ? page_size : DT_STAGE_KEYS;
    p.window = window; p.scale = scale; p.partials = scratch; p.arrivals = counters; p.error_flag = error_flag;
    CUtensorMap map;
    if (llmp_pages_tensor_map(pages, nkv, page_size, num_pages, p.box_tokens, 2, 1, &map)) return 1;
    const size_t smem = (size_t)DT_STAGES * DT_STAGE_BYTES + (size_t)(DT_CWARPS + 1) * DT_MAX_HEADS * DT_QSTRIDE * sizeof(bf16) +
                        (size_t)DT_CWARPS * DT_MAX_HEADS * DT_D * sizeof(float) + 1024;
    LLMP_ALLOW_SMEM(decode_attention_list_kernel, smem);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)sms);                        // one block per SM; blocks without a share leave at once
    config.blockDim = dim3(DT_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    int n = 0;
    if (llmp_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;         // see pdl_wait() in the kernel
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    config.attrs = attr;
    config.numAttrs = n;
    const cudaError_t launched = cudaLaunchKernelEx(&config, decode_attention_list_kernel, map, p);
    if (launched != cudaSuccess) {
        llmp_set_error("decode_attention_list: launch failed: %s", cudaGetErrorString(launched));
        return 2;
    }
    return llmp_check_launch("decode_attention_list");
}
