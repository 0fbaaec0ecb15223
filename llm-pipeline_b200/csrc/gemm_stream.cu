// Y[M, N] = X[M, K] * W[N, K]^T for the few rows of a decode step (M <= 64), bound by reading W once from HBM:
// one persistent block per SM streams its share of W through a ring of TMA boxes.
//
// The rows of W are dealt out evenly: block b owns the contiguous rows [b * per, (b + 1) * per) and walks them
// in chunks of RB <= 128 rows; for each chunk it walks K in steps of KB blocks of 64 elements. A ring stage
// holds one step: a box of W (RB rows x KB x 64 elements, as KB planes of rows of 128 bytes in the 128-byte
// swizzle) and the matching box of X (8, 16, 32 or 64 rows). A load warp fills the ring as slots come free and runs
// ahead across chunks; four compute warps take the stages of a chunk in turn (warp w the steps w, w + 4, ...
// of K), multiply with mma.sync m16n8k16 (the rows of W on the 16-row side, the rows of X on the
// 8-column side, float32 accumulators in registers) and hand the slot back. At the end of a chunk the four
// warps' sums are added in warp order in shared memory and stored. A ring slot belongs to one compute warp (warp
// w owns the slots w, w + 4, ...), so a warp sees every phase of its barriers in turn. The order of the additions
// depends on N and K alone, so a row of X gives the same result whatever else is in X.
//
// With glu_rows = I the matrix holds the I gate rows and then the I up rows of a SwiGLU feed-forward: a block owns
// the same rows of both halves, walks its gate chunks, then its up chunks, keeps the gate sums in shared memory
// and stores silu(gate) * up (float32 inside): the activation never goes through global memory as two halves.
//
// As a dependent launch: W is constant, X may still be in the making by the kernel before this one. The load
// warp fills the whole ring with boxes of W, then waits for that kernel, then adds the boxes of X.
//
// Every wait on an mbarrier is bounded: when one runs out the kernel records 1 in *error_flag and goes on
// without waiting (its output is then wrong; the host reads the flag).
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "gemm_stream.cuh"

struct StreamParams {
    void* Y;
    long ldy;
    int M, N, K;
    int per;              // rows of W per block
    int RB;               // rows of W per chunk and box
    int KB;               // 64-element blocks of K per stage
    int MB;               // rows of the X box: 8 NT
    int part_rows;        // rows of W per warp in the buffer of partial sums: 16 MT
    int stages;
    int out_f32;
    int glu_rows;         // 0, or I: W is [gate rows; up rows] of I rows each and Y[m, i] = silu(gate_i . x_m) * (up_i . x_m)
    // Rows of X that still lack a factor (M <= 8): row m of the product is multiplied by
    // rsqrt(sum over in_parts of in_sumsq[part][m] * in_inv_width + in_eps) before anything else is done with it.
    const float* in_sumsq;
    int in_parts;
    float in_inv_width, in_eps;
    // The product as an addend of a float32 residual that a norm follows (M <= 8): r = residual + product is stored back,
    // r * norm_w goes to xw in bfloat16, and this block's sums of r^2 over its columns go to out_sumsq[block][m], from
    // which the next product takes the rows' factors. Y is not written.
    float* residual;
    long ldr;
    const void* norm_w;
    int norm_w_f32;
    bf16* xw;
    long ldxw;
    float* out_sumsq;
    int* error_flag;
};

// MT: 16-row tiles of W per chunk (RB <= 16 MT). NT: 8-row tiles of X (M <= 8 NT).
template <int MT, int NT>
__global__ void __launch_bounds__(GS_THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const StreamParams p) {
    extern __shared__ unsigned char gs_raw[];
    __shared__ __align__(8) uint64_t full_bar[GS_MAX_STAGES], empty_bar[GS_MAX_STAGES];
    __shared__ float row_factor[8];                              // in_sumsq: the rows' factors
    const uint32_t raw_addr = tc_smem_u32(gs_raw);
    unsigned char* ring = gs_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);      // 1024-byte aligned stages
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // a stage: KB planes of RB lines of W, then KB planes of MB lines of X, rounded up to 1024 bytes
    const uint32_t w_bytes = (uint32_t)p.RB * 128 * p.KB, x_bytes = (uint32_t)p.MB * 128 * p.KB;
    const uint32_t stage_bytes = (w_bytes + x_bytes + 1023u) & ~1023u;
    float* part = reinterpret_cast<float*>(ring + (size_t)p.stages * stage_bytes);   // [warps][16 MT][8 NT + 1]

    // the rows of this block: [row_begin, row_end) of W, or with glu_rows of each of its two halves
    const int row_limit = p.glu_rows ? p.glu_rows : p.N;
    const int row_begin = blockIdx.x * p.per;
    int row_end = row_begin + p.per;
    if (row_end > row_limit) row_end = row_limit;
    const int half_chunks = row_begin < row_end ? (row_end - row_begin + p.RB - 1) / p.RB : 0;
    const int chunks = p.glu_rows ? 2 * half_chunks : half_chunks;
    const int ksteps = p.K / (64 * p.KB);                       // stages per chunk
    const int total = chunks * ksteps;
    // first row of W of chunk c: the up chunks follow the gate chunks
    auto chunk_row = [&](int c) { return c < half_chunks ? row_begin + c * p.RB : p.glu_rows + row_begin + (c - half_chunks) * p.RB; };
    float* gate = part + (size_t)GS_CWARPS * p.part_rows * (8 * NT + 1);     // [rows of the block][8 NT]: the gate sums (glu_rows only)

    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_x) : "memory");
    }
    __syncthreads();
    pdl_trigger();                                              // the kernel after this one may take its places

    if (warp == GS_CWARPS) {
        if (lane == 0) {
            // Stage (chunk, ks) belongs to compute warp w = ks % 4 and is that warp's j-th stage; warp w owns the ring
            // slots w, w + 4, ... and the stage lives in the (j mod their number)-th of them. A slot is thus filled for
            // one warp only, which sees every phase of its barrier in turn.
            auto slot_of = [&](int chunk, int ks, int& round) {
                const int w = ks % GS_CWARPS;
                const int per_chunk = (ksteps - w + GS_CWARPS - 1) / GS_CWARPS;     // stages of warp w in a chunk
                const int mine = (p.stages - w + GS_CWARPS - 1) / GS_CWARPS;        // ring slots of warp w: w, w + 4, ...
                const int j = chunk * per_chunk + ks / GS_CWARPS;
                round = j / mine;
                return GS_CWARPS * (j % mine) + w;
            };
            // the first round of every slot is filled with boxes of W at once; the boxes of X follow after pdl_wait()
            int first_later = total;                             // first stage (in issue order) of a later round
            for (int i = 0; i < total; ++i) {
                const int chunk = i / ksteps, ks = i - chunk * ksteps;
                int round;
                const int slot = slot_of(chunk, ks, round);
                if (round > 0) {
                    first_later = i;
                    break;
                }
                mbar_expect_tx(&full_bar[slot], w_bytes + x_bytes);
                gs_tma_load_3d(ring + (size_t)slot * stage_bytes, &map_w, 0, chunk_row(chunk), ks * p.KB, &full_bar[slot]);
            }
            pdl_wait();
            for (int i = 0; i < first_later; ++i) {
                const int chunk = i / ksteps, ks = i - chunk * ksteps;
                int round;
                const int slot = slot_of(chunk, ks, round);
                gs_tma_load_3d(ring + (size_t)slot * stage_bytes + w_bytes, &map_x, 0, 0, ks * p.KB, &full_bar[slot]);
            }
            for (int i = first_later; i < total; ++i) {
                const int chunk = i / ksteps, ks = i - chunk * ksteps;
                int round;
                const int slot = slot_of(chunk, ks, round);
                if (round > 0) mbar_wait(&empty_bar[slot], (uint32_t)((round - 1) & 1), p.error_flag);
                mbar_expect_tx(&full_bar[slot], w_bytes + x_bytes);
                unsigned char* stage = ring + (size_t)slot * stage_bytes;
                gs_tma_load_3d(stage, &map_w, 0, chunk_row(chunk), ks * p.KB, &full_bar[slot]);
                gs_tma_load_3d(stage + w_bytes, &map_x, 0, 0, ks * p.KB, &full_bar[slot]);
            }
        }
    } else {
        const int g = lane >> 2, t = lane & 3;
        float acc[MT][NT][4];
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
        // 16 threads per row of X: thread `part16` of row `row16`
        const int row16 = tid >> 4, part16 = tid & 15;
        float block_squares = 0.f;                               // residual: this block's sum of r^2 of row row16 (in part16 == 0)
        if (p.in_sumsq != nullptr) {
            // The rows' factors, while the boxes of X are on their way: the sums of squares that the blocks of the
            // product before left, added in a fixed order (16 threads a row, each its parts in turn, then a tree).
            pdl_wait();
            // (every part's sum is asked for before the first is added: ten dependent trips to L2 one after the other
            // would cost some 3 us right where the product waits for its rows' factors; the order of the additions stays)
            float sum = 0.f;
            for (int b0 = part16; b0 < p.in_parts; b0 += 16 * 12) {
                float part_sum[12];
#pragma unroll
                for (int i = 0; i < 12; ++i) {
                    const int b = b0 + 16 * i;
                    part_sum[i] = (row16 < p.M && b < p.in_parts) ? __ldcg(p.in_sumsq + (size_t)b * 8 + row16) : 0.f;
                }
#pragma unroll
                for (int i = 0; i < 12; ++i) sum += part_sum[i];
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            if (part16 == 0 && row16 < p.M) row_factor[row16] = rsqrtf(sum * p.in_inv_width + p.in_eps);
        }
        const int steps16 = 4 * p.KB;                            // 16-element K steps per stage
        const int mine = (p.stages - warp + GS_CWARPS - 1) / GS_CWARPS;      // ring slots of this warp: warp, warp + 4, ...
        int j = 0;                                               // stages this warp has taken
        if (p.residual != nullptr && p.in_sumsq == nullptr) pdl_wait();      // the residual is read below
        for (int chunk = 0; chunk < chunks; ++chunk) {
            // residual: this thread's entries of the residual and of the norm weight for the chunk's columns, asked for
            // now so that they are there when the sums are (thread part16 of row row16: columns part16, part16 + 16, ...)
            float r_before[GS_MAX_RB / 16], w_norm[GS_MAX_RB / 16];
            if (p.residual != nullptr) {
                const int n0 = row_begin + chunk * p.RB;
                int rows = row_end - n0;
                if (rows > p.RB) rows = p.RB;
#pragma unroll
                for (int i = 0; i < GS_MAX_RB / 16; ++i) {
                    const int c = part16 + 16 * i;
                    r_before[i] = w_norm[i] = 0.f;
                    if (row16 < p.M && c < rows) {
                        r_before[i] = p.residual[(size_t)row16 * p.ldr + n0 + c];
                        w_norm[i] = p.norm_w_f32 ? reinterpret_cast<const float*>(p.norm_w)[n0 + c]
                                                 : __bfloat162float(reinterpret_cast<const bf16*>(p.norm_w)[n0 + c]);
                    }
                }
            }
            // warp w takes the chunk's stages w, w + 4, ... whole: a wait and a hand-back per stage and warp
            for (int ks = warp; ks < ksteps; ks += GS_CWARPS, ++j) {
                const int slot = GS_CWARPS * (j % mine) + warp;  // this warp's j-th stage: see the load warp
                mbar_wait(&full_bar[slot], (uint32_t)((j / mine) & 1), p.error_flag);
                const unsigned char* stage = ring + (size_t)slot * stage_bytes;
                for (int s = 0; s < steps16; ++s) {
                    const int w_line = (s >> 2) * p.RB;                              // first line of this 64-element block of W
                    const int x_line = p.KB * p.RB + (s >> 2) * p.MB;                //                                    and of X
                    const int chunk16 = (s & 3) * 2;                                // first 16-byte chunk of the K step
                    unsigned b[NT][2];
#pragma unroll
                    for (int j = 0; j < NT; ++j)
                        gs_ldmatrix_x2(b[j], gs_at(stage, x_line + j * 8 + (lane & 7), chunk16 + ((lane >> 3) & 1)));
                    // All fragments of W of this K step are asked for before the first product needs one: a warp issues in
                    // order, so a load directly followed by the product that reads it costs the load's whole latency per tile.
                    // Rows beyond RB in the last tile read the lines that follow (finite data of the stage or of the next
                    // one); their sums are never stored.
                    unsigned a[MT][4];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
                        if (mt * 16 < p.RB) gs_ldmatrix_x4(a[mt], gs_at(stage, w_line + mt * 16 + (lane & 15), chunk16 + (lane >> 4)));
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        if (mt * 16 < p.RB) {
#pragma unroll
                            for (int j = 0; j < NT; ++j) gs_mma(acc[mt][j], a[mt], b[j][0], b[j][1]);
                        }
                    }
                }
                // this warp has read the stage
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem_u32(&empty_bar[slot])) : "memory");
            }
            // the chunk is complete: the four warps' sums, added in warp order
            // acc[mt][j] holds W rows mt*16 + g (+8) and X rows j*8 + 2t (+1)
            asm volatile("bar.sync 1, %0;\n" ::"n"(GS_CWARPS * 32) : "memory");      // the sums of the chunk before are read
            const int pstride = 8 * NT + 1;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    float* base = part + ((size_t)warp * p.part_rows + mt * 16 + g) * pstride + j * 8 + 2 * t;
                    base[0] = acc[mt][j][0];
                    base[1] = acc[mt][j][1];
                    base[8 * pstride] = acc[mt][j][2];
                    base[8 * pstride + 1] = acc[mt][j][3];
                    acc[mt][j][0] = acc[mt][j][1] = acc[mt][j][2] = acc[mt][j][3] = 0.f;
                }
            }
            asm volatile("bar.sync 1, %0;\n" ::"n"(GS_CWARPS * 32) : "memory");
            const int sub = chunk < half_chunks ? chunk : chunk - half_chunks;
            const int n0 = row_begin + sub * p.RB;               // first column of Y of this chunk
            int rows = row_end - n0;
            if (rows > p.RB) rows = p.RB;
            if (p.residual != nullptr) {
                // Thread part16 of row row16 takes the columns part16, part16 + 16, ... of its row: r = residual + product,
                // r * norm weight for the next product, and r^2 added in a fixed order (its columns in turn, then a tree).
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < GS_MAX_RB / 16; ++i) {
                    const int c = part16 + 16 * i;
                    if (row16 < p.M && c < rows) {
                        float v = 0.f;
#pragma unroll
                        for (int w = 0; w < GS_CWARPS; ++w) v += part[((size_t)w * p.part_rows + c) * pstride + row16];
                        if (p.in_sumsq != nullptr) v *= row_factor[row16];
                        const float r = r_before[i] + v;
                        p.residual[(size_t)row16 * p.ldr + n0 + c] = r;
                        p.xw[(size_t)row16 * p.ldxw + n0 + c] = __float2bfloat16_rn(r * w_norm[i]);
                        sum = fmaf(r, r, sum);
                    }
                }
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                block_squares += sum;
                continue;
            }
            for (int e = tid; e < rows * p.M; e += GS_CWARPS * 32) {
                const int m = e / rows, row = e - m * rows;     // consecutive threads store consecutive columns of Y
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < GS_CWARPS; ++w) v += part[((size_t)w * p.part_rows + row) * pstride + m];
                if (p.in_sumsq != nullptr) v *= row_factor[m];
                if (p.glu_rows) {
                    float* kept = gate + (size_t)(sub * p.RB + row) * (8 * NT) + m;
                    if (chunk < half_chunks) {                   // a gate chunk: kept for the up chunk of the same rows
                        *kept = v;
                        continue;
                    }
                    const float z = *kept;
                    v = (z / (1.f + expf(-z))) * v;
                }
                if (p.out_f32) reinterpret_cast<float*>(p.Y)[(size_t)m * p.ldy + n0 + row] = v;
                else reinterpret_cast<bf16*>(p.Y)[(size_t)m * p.ldy + n0 + row] = __float2bfloat16_rn(v);
            }
        }
        if (p.residual != nullptr && part16 == 0) p.out_sumsq[(size_t)blockIdx.x * 8 + row16] = row16 < p.M ? block_squares : 0.f;
    }
}

// ---- host side ---------------------------------------------------------------------------------------------
struct StreamMapKey {
    const void* ptr;
    long rows, k, ld;
    int box_rows, box_kb;
    bool operator==(const StreamMapKey& o) const {
        return ptr == o.ptr && rows == o.rows && k == o.k && ld == o.ld && box_rows == o.box_rows && box_kb == o.box_kb;
    }
};
struct StreamMapKeyHash {
    size_t operator()(const StreamMapKey& m) const {
        size_t h = (size_t)m.ptr;
        h = h * 1000003u ^ (size_t)m.rows;
        h = h * 1000003u ^ (size_t)m.k;
        h = h * 1000003u ^ (size_t)m.ld;
        h = h * 1000003u ^ (size_t)m.box_rows;
        return h * 1000003u ^ (size_t)m.box_kb;
    }
};

// A [rows, K] bfloat16 row-major matrix with row pitch ld, seen as {64 elements, rows, K / 64 blocks} and read in
// boxes of {64, box_rows, box_kb}: in shared memory box_kb planes of box_rows lines of 128 bytes.
int llmp_stream_tensor_map(const void* ptr, long rows, long k, long ld, int box_rows, int box_kb, CUtensorMap* out) {
    static std::unordered_map<StreamMapKey, CUtensorMap, StreamMapKeyHash> cache;
    static std::mutex lock;
    const StreamMapKey key{ptr, rows, k, ld, box_rows, box_kb};
    std::lock_guard<std::mutex> guard(lock);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return 0;
    }
    EncodeTiledFn fn = llmp_tensor_map_encoder();
    LLMP_REQUIRE(fn != nullptr, "gemm_stream: the driver does not provide cuTensorMapEncodeTiled");
    const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(k / 64)};
    const cuuint64_t strides[2] = {(cuuint64_t)ld * sizeof(bf16), 128};
    const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)box_kb};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    LLMP_REQUIRE(rc == CUDA_SUCCESS, "gemm_stream: cuTensorMapEncodeTiled failed with code %d", (int)rc);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

int llmp_sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    return sms;
}

bool llmp_stream_plan(int M, int N, int K, long ldx, long ldw, int glu_rows, StreamPlan* out) {
    if (!(M > 0 && M <= 64 && N > 0 && K >= 64 && K % 64 == 0 && ldx % 8 == 0 && ldw % 8 == 0)) return false;
    if (glu_rows && (N != 2 * glu_rows || M > 16)) return false;
    const int sms = llmp_sm_count();
    StreamPlan q;
    // rows per block: an even share (of each half with glu_rows)
    const int share = glu_rows ? glu_rows : N;
    q.per = (share + sms - 1) / sms;
    if (q.per < 8) q.per = 8;
    q.grid = (share + q.per - 1) / q.per;
    const int chunks = (q.per + GS_MAX_RB - 1) / GS_MAX_RB;
    q.rb = (q.per + chunks - 1) / chunks;
    q.nt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
    q.mt = (q.rb + 15) / 16 <= 2 ? 2 : ((q.rb + 15) / 16 <= 4 ? 4 : 8);       // the kernel's template steps
    if (q.mt * q.nt > 16) return false;      // more than 128 accumulator registers a thread are not built
    // blocks of K per stage: as many as leave at least four stages (longer pieces of a weight row per box read
    // DRAM better: the head product went from 5.7 to 6.3 TB/s with two blocks instead of one), KB a power of two
    // that divides K / 64. KB decides which warp
    // adds which part of K, so it is chosen from N and K alone: the result of a row of X must not depend on M.
    q.kb = 1;
    while (q.kb < 8 && (long)(q.rb + 16) * 128 * q.kb * 2 <= GS_STAGE_LIMIT && (K / 64) % (q.kb * 2) == 0) q.kb *= 2;
    q.stage_bytes = ((size_t)(q.rb + 8 * q.nt) * 128 * q.kb + 1023) / 1024 * 1024;
    q.part_bytes = (size_t)GS_CWARPS * q.mt * 16 * (8 * q.nt + 1) * sizeof(float);
    if (glu_rows) q.part_bytes += (size_t)chunks * q.rb * 8 * q.nt * sizeof(float);        // the gate sums of the block's rows
    int stages = (int)((GS_SMEM_BUDGET - q.part_bytes) / q.stage_bytes);
    if (stages > GS_MAX_STAGES) stages = GS_MAX_STAGES;
    q.stages = stages;
    if (q.stages < GS_CWARPS) return false;                      // every compute warp has slots of its own
    q.smem = (size_t)q.stages * q.stage_bytes + q.part_bytes + 2048;   // 1024 for the alignment, 1024 for reads past the last stage
    *out = q;
    return true;
}

// Shapes this kernel takes: M <= 64 rows of X (more than 16 only for narrow outputs), K a multiple of 64, rows of 16
// bytes' alignment.
LLMP_API int llmp_gemm_stream_supports(int M, int N, int K, long ldx, long ldw) {
    StreamPlan q;
    return llmp_stream_plan(M, N, K, ldx, ldw, 0, &q) ? 1 : 0;
}

// X and W bfloat16, rows 16-byte aligned; out_dtype bfloat16 or float32; shapes as llmp_gemm_stream_supports says.
struct StreamExtras {                                           // see StreamParams
    const float* in_sumsq = nullptr;
    int in_parts = 0;
    float in_inv_width = 0.f, in_eps = 0.f;
    float* residual = nullptr;
    long ldr = 0;
    const void* norm_w = nullptr;
    int norm_w_f32 = 0;
    void* xw = nullptr;
    long ldxw = 0;
    float* out_sumsq = nullptr;
};
static int gemm_stream_launch(const void* X, const void* W, void* Y, int out_dtype, int M, int N, int K, long ldx, long ldw,
                              long ldy, int glu_rows, const StreamExtras& extras, int* error_flag, cudaStream_t stream);

LLMP_API int llmp_gemm_stream(const void* X, const void* W, void* Y, int out_dtype, int M, int N, int K, long ldx, long ldw,
                              long ldy, int* error_flag, cudaStream_t stream) {
    return gemm_stream_launch(X, W, Y, out_dtype, M, N, K, ldx, ldw, ldy, 0, StreamExtras(), error_flag, stream);
}

// W holds the I gate rows and then the I up rows of a SwiGLU feed-forward (N = 2 I rows of K):
// Y[m, i] = silu(W[i] . X[m]) * (W[I + i] . X[m]), Y being [M, I]. M <= 16.
LLMP_API int llmp_gemm_stream_swiglu_supports(int M, int I, int K, long ldx, long ldw) {
    StreamPlan q;
    return llmp_stream_plan(M, 2 * I, K, ldx, ldw, I, &q) ? 1 : 0;
}

LLMP_API int llmp_gemm_stream_swiglu(const void* X, const void* W, void* Y, int out_dtype, int M, int I, int K, long ldx,
                                     long ldw, long ldy, int* error_flag, cudaStream_t stream) {
    return gemm_stream_launch(X, W, Y, out_dtype, M, 2 * I, K, ldx, ldw, ldy, I, StreamExtras(), error_flag, stream);
}

// Blocks that a product of these sizes is dealt out to (each leaves one row of out_sumsq); 0: the sizes are not taken.
LLMP_API int llmp_gemm_stream_blocks(int M, int N, int K, long ldx, long ldw) {
    StreamPlan q;
    return llmp_stream_plan(M, N, K, ldx, ldw, 0, &q) ? q.grid : 0;
}

// The streaming product between a norm and the residual sum, for at most 8 rows of X. Either part may be left out.
//  - in_sumsq != null: the rows of X lack the factor rsqrt(sum of in_sumsq[0 .. in_parts)[m] * in_inv_width + in_eps); the
//    product is multiplied by it (before SwiGLU when glu_rows = N / 2 > 0: W is then [gate rows; up rows], Y is [M, N / 2]).
//  - residual != null (glu_rows = 0, N the width of the residual): residual[m, n] += product, xw[m, n] =
//    bfloat16(residual[m, n] * norm_w[n]) and out_sumsq[block][m] = this block's sum of residual[m, n]^2 (8 floats a block,
//    llmp_gemm_stream_blocks(...) blocks); Y is not written. xw and out_sumsq are what the next product takes as X and in_sumsq.
LLMP_API int llmp_gemm_stream_fused(const void* X, const void* W, void* Y, int out_dtype, int M, int N, int K, long ldx, long ldw,
                                    long ldy, int glu_rows, const float* in_sumsq, int in_parts, float in_inv_width,
                                    float in_eps, float* residual, long ldr, const void* norm_w, int norm_w_dtype, void* xw,
                                    long ldxw, float* out_sumsq, int* error_flag, cudaStream_t stream) {
    LLMP_REQUIRE(M <= 8, "gemm_stream: the fused forms take at most 8 rows, not %d", M);
    LLMP_REQUIRE(glu_rows == 0 || glu_rows * 2 == N, "gemm_stream: %d gate rows do not make %d rows of W", glu_rows, N);
    StreamExtras e;
    if (in_sumsq != nullptr) {
        LLMP_REQUIRE(in_parts > 0, "gemm_stream: sums of squares need their number");
        e.in_sumsq = in_sumsq; e.in_parts = in_parts; e.in_inv_width = in_inv_width; e.in_eps = in_eps;
    }
    if (residual != nullptr) {
        LLMP_REQUIRE(glu_rows == 0 && norm_w != nullptr && xw != nullptr && out_sumsq != nullptr,
                     "gemm_stream: the residual form needs a norm weight and places for its results, and no SwiGLU");
        LLMP_REQUIRE(norm_w_dtype == LLMP_F32 || norm_w_dtype == LLMP_BF16, "gemm_stream: norm weights are float32 or bfloat16");
        e.residual = residual; e.ldr = ldr; e.norm_w = norm_w; e.norm_w_f32 = norm_w_dtype == LLMP_F32; e.xw = xw; e.ldxw = ldxw;
        e.out_sumsq = out_sumsq;
    }
    return gemm_stream_launch(X, W, Y, out_dtype, M, N, K, ldx, ldw, ldy, glu_rows, e, error_flag, stream);
}

static int gemm_stream_launch(const void* X, const void* W, void* Y, int out_dtype, int M, int N, int K, long ldx, long ldw,
                              long ldy, int glu_rows, const StreamExtras& extras, int* error_flag, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    StreamPlan q;
    LLMP_REQUIRE(llmp_stream_plan(M, N, K, ldx, ldw, glu_rows, &q), "gemm_stream: M=%d, N=%d, K=%d (a multiple of 64) or the row strides are not taken", M, N, K);
    LLMP_REQUIRE(((size_t)X % 16) == 0 && ((size_t)W % 16) == 0, "gemm_stream: operands must be 16-byte aligned");
    LLMP_REQUIRE(error_flag != nullptr, "gemm_stream: an error flag in device memory is required");
    StreamParams p;
    p.Y = Y; p.ldy = ldy; p.M = M; p.N = N; p.K = K; p.out_f32 = out_dtype == LLMP_F32; p.error_flag = error_flag;
    p.glu_rows = glu_rows;
    p.in_sumsq = extras.in_sumsq; p.in_parts = extras.in_parts; p.in_inv_width = extras.in_inv_width; p.in_eps = extras.in_eps;
    p.residual = extras.residual; p.ldr = extras.ldr; p.norm_w = extras.norm_w; p.norm_w_f32 = extras.norm_w_f32;
    p.xw = (bf16*)extras.xw; p.ldxw = extras.ldxw; p.out_sumsq = extras.out_sumsq;
    p.per = q.per; p.RB = q.rb; p.MB = 8 * q.nt; p.KB = q.kb; p.part_rows = q.mt * 16; p.stages = q.stages;
    const int grid = q.grid, rb = q.rb, kb = q.kb, nt = q.nt, mt = q.mt;
    const size_t smem = q.smem;
    CUtensorMap map_w, map_x;
    if (llmp_stream_tensor_map(W, N, K, ldw, rb, kb, &map_w) || llmp_stream_tensor_map(X, M, K, ldx, p.MB, kb, &map_x)) return 1;
    cudaError_t launched = cudaSuccess;
#define GS_LAUNCH(MT, NT)                                                                                     \
    do {                                                                                                      \
        LLMP_ALLOW_SMEM((gemm_stream_kernel<MT, NT>), smem);                                                  \
        launched = llmp_launch_dependent(gemm_stream_kernel<MT, NT>, dim3(grid), dim3(GS_THREADS), smem, stream, \
                                         map_w, map_x, p);                                                    \
    } while (0)
    if (mt == 2) {
        if (nt == 1) GS_LAUNCH(2, 1); else if (nt == 2) GS_LAUNCH(2, 2); else if (nt == 4) GS_LAUNCH(2, 4); else GS_LAUNCH(2, 8);
    } else if (mt == 4) {
        if (nt == 1) GS_LAUNCH(4, 1); else if (nt == 2) GS_LAUNCH(4, 2); else GS_LAUNCH(4, 4);
    } else {
        if (nt == 1) GS_LAUNCH(8, 1); else GS_LAUNCH(8, 2);
    }
#undef GS_LAUNCH
    if (launched != cudaSuccess) {
        llmp_set_error("gemm_stream: launch failed: %s", cudaGetErrorString(launched));
        return 2;
    }
    return llmp_check_launch("gemm_stream");
}
