// Several weight-streaming products of a decode step in one persistent launch (at most 8 rows of X).
//
// A decode step is a chain of skinny products, each of which needs the whole result of the one before:
// output projection -> (residual, norm) -> gate/up with SwiGLU -> down projection -> (residual, norm) -> the next
// layer's q/k/v projection. As separate launches (gemm_stream.cu) every product drains its ring of weight boxes at its
// end and the next one fills its ring again before it computes: the memory system idles at each boundary. Here the
// phases share one ring. The load warp walks straight from the last weight box of a phase to the first of the next
// and keeps the ring full; only the boxes of X of the next phase (the result of the phase before, a few KB) wait
// until every block has finished that phase, which the blocks tell each other through a counter in global memory.
// While blocks wait there, their rings already hold the next phase's weights.
//
// A phase is exactly one product of gemm_stream.cu: the same rows per block, rows per chunk and blocks of K per
// stage (they follow from N and K alone), the same order of additions, the same three epilogues (plain rows of Y;
// SwiGLU of [gate rows; up rows]; residual += product with the next norm's weight applied and the sums of squares
// left for the phase after, whose rows then carry the norm's factor). A chain therefore gives the same bits as its
// products launched one by one.
//
// Measured on a B200 (Qwen3-8B shapes, 8 rows, weights from HBM): the chain of four takes 98 us alone where the four
// products launched one by one take 102 us alone but 75 us inside a replayed decode graph, where each is a dependent
// launch whose ring fills while the kernel before it ends and has six to eight stages of its own size (a chain's ring
// has slots of one size for all phases, four here); a decode step through chains took 4.55 ms against 3.63 ms. A phase
// boundary costs 2.6 us (5 to 6 us where the next phase first adds up the rows' sums of squares), a dependent launch
// about 3. So the engine does not take this path unless LLMP_B200_CHAIN=1 says so; the kernel stays as the tested
// record of that experiment.
//
// The blocks wait for each other, so the kernel is launched cooperatively (all blocks resident: one per SM). Every
// wait is bounded: on an mbarrier as in the other kernels, on the counters by a limit of polls; a wait that runs out
// records 1 in *error_flag and the kernel goes on without waiting (its output is then wrong; the host reads the flag).
#include <cuda.h>

#include "gemm_stream.cuh"

#define GC_MAX_PHASES 4
#define GC_POLL_LIMIT (1u << 22)

struct ChainPhase {
    void* Y;              // plain rows or SwiGLU rows; unused in the residual form
    long ldy;
    int N, K;
    int per, RB, KB;      // rows of W per block and per chunk, 64-element blocks of K per stage
    int mt;               // 16-row tiles of W per chunk as the compute loops are built: 2, 4 or 8
    int out_f32;
    int glu_rows;
    const float* in_sumsq;
    int in_parts;
    float in_inv_width, in_eps;
    float* residual;
    long ldr;
    const void* norm_w;
    int norm_w_f32;
    bf16* xw;
    long ldxw;
    float* out_sumsq;
};

struct ChainParams {
    int M, phases, stages;
    uint32_t stage_bytes;
    unsigned* counters;   // [GC_MAX_PHASES + 1], zero between launches: blocks that finished phase i, blocks that are done
    int* error_flag;
    ChainPhase ph[GC_MAX_PHASES];
};

struct ChainMaps {
    CUtensorMap w[GC_MAX_PHASES], x[GC_MAX_PHASES];
};

// Waits until `target` blocks have counted themselves at `counter`; false (and *error_flag = 1) when the polls run out.
__device__ __forceinline__ bool gc_wait_blocks(const unsigned* counter, unsigned target, int* error_flag) {
    for (uint32_t i = 0; i < GC_POLL_LIMIT; ++i) {
        unsigned seen;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(counter) : "memory");
        if (seen >= target) return true;
        __nanosleep(20);
    }
    *reinterpret_cast<volatile int*>(error_flag) = 1;
    return false;
}

// The rows of W that block `b` owns in a phase, as chunks.
struct PhaseShare {
    int row_begin, row_end, half_chunks, chunks, ksteps;
};

__device__ __forceinline__ PhaseShare gc_share(const ChainPhase& q, int block) {
    PhaseShare s;
    const int row_limit = q.glu_rows ? q.glu_rows : q.N;
    s.row_begin = block * q.per;
    s.row_end = s.row_begin + q.per;
    if (s.row_end > row_limit) s.row_end = row_limit;
    s.half_chunks = s.row_begin < s.row_end ? (s.row_end - s.row_begin + q.RB - 1) / q.RB : 0;
    s.chunks = q.glu_rows ? 2 * s.half_chunks : s.half_chunks;
    s.ksteps = q.K / (64 * q.KB);
    return s;
}

// One phase of one block's compute warps, with MT 16-row tiles of W per chunk (RB <= 16 MT): the inner loops of
// gemm_stream_kernel<MT, 1>. j counts the stages this warp has taken over all phases.
template <int MT>
__device__ __forceinline__ void gc_phase(const ChainParams& p, const int ph, unsigned char* ring, float* part_any, float* gate,
                                         uint64_t* full_bar, uint64_t* empty_bar, float* row_factor, int& j) {
    constexpr int NT = 1;
    constexpr int part_rows = 128;                               // the buffer of partial sums is laid out for the largest MT
    constexpr int pstride = 8 * NT + 1;
    float* part = part_any;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t stage_bytes = p.stage_bytes;
    const unsigned blocks = gridDim.x;
    const int g = lane >> 2, t = lane & 3;
    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i][0][0] = acc[i][0][1] = acc[i][0][2] = acc[i][0][3] = 0.f;
    const int row16 = tid >> 4, part16 = tid & 15;               // 16 threads per row of X
    const int mine = (p.stages - warp + GS_CWARPS - 1) / GS_CWARPS;
    {
            const ChainPhase& q = p.ph[ph];
            const PhaseShare sh = gc_share(q, blockIdx.x);
            // the phase's geometry in registers: q is indexed by the phase, and a field read in the inner loop would be a
            // load from the parameter bank with a computed address every time
            const int RB = q.RB, KB = q.KB, glu_rows = q.glu_rows, out_f32 = q.out_f32, norm_w_f32 = q.norm_w_f32;
            float* const residual = q.residual;
            bf16* const xw = q.xw;
            const void* const norm_w = q.norm_w;
            void* const Y = q.Y;
            const long ldr = q.ldr, ldxw = q.ldxw, ldy = q.ldy;
            const bool factors = q.in_sumsq != nullptr;
            const uint32_t w_lines = (uint32_t)RB * KB;          // lines of W in a stage; the lines of X follow
            // what this phase reads of the phase before through plain loads (sums of squares, the residual)
            if (ph == 0) {
                if (q.in_sumsq != nullptr || q.residual != nullptr) pdl_wait();
            } else {
                if (tid == 0) gc_wait_blocks(&p.counters[ph - 1], blocks, p.error_flag);
                asm volatile("bar.sync 1, %0;\n" ::"n"(GS_CWARPS * 32) : "memory");
            }
            float block_squares = 0.f;
            if (q.in_sumsq != nullptr) {
                float sum = 0.f;
                const int in_parts = q.in_parts;
                const float* const in_sumsq = q.in_sumsq;
                for (int b0 = part16; b0 < in_parts; b0 += 16 * 12) {          // (all loads first: see gemm_stream.cu)
                    float part_sum[12];
#pragma unroll
                    for (int i = 0; i < 12; ++i) {
                        const int b = b0 + 16 * i;
                        part_sum[i] = (row16 < p.M && b < in_parts) ? __ldcg(in_sumsq + (size_t)b * 8 + row16) : 0.f;
                    }
#pragma unroll
                    for (int i = 0; i < 12; ++i) sum += part_sum[i];
                }
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                if (part16 == 0 && row16 < p.M) row_factor[row16] = rsqrtf(sum * q.in_inv_width + q.in_eps);
            }
            const int steps16 = 4 * KB;
            for (int chunk = 0; chunk < sh.chunks; ++chunk) {
                float r_before[GS_MAX_RB / 16], w_norm[GS_MAX_RB / 16];
                if (residual != nullptr) {
                    const int n0 = sh.row_begin + chunk * RB;
                    int rows = sh.row_end - n0;
                    if (rows > RB) rows = RB;
#pragma unroll
                    for (int i = 0; i < GS_MAX_RB / 16; ++i) {
                        const int c = part16 + 16 * i;
                        r_before[i] = w_norm[i] = 0.f;
                        if (row16 < p.M && c < rows) {
                            r_before[i] = __ldcg(residual + (size_t)row16 * ldr + n0 + c);
                            w_norm[i] = norm_w_f32 ? reinterpret_cast<const float*>(norm_w)[n0 + c]
                                                     : __bfloat162float(reinterpret_cast<const bf16*>(norm_w)[n0 + c]);
                        }
                    }
                }
                for (int ks = warp; ks < sh.ksteps; ks += GS_CWARPS, ++j) {
                    const int slot = GS_CWARPS * (j % mine) + warp;
                    mbar_wait(&full_bar[slot], (uint32_t)((j / mine) & 1), p.error_flag);
                    const unsigned char* stage = ring + (size_t)slot * stage_bytes;
                    for (int s = 0; s < steps16; ++s) {
                        const int w_line = (s >> 2) * RB;
                        const int x_line = (int)w_lines + (s >> 2) * 8;
                        const int chunk16 = (s & 3) * 2;
                        unsigned b[2];
                        gs_ldmatrix_x2(b, gs_at(stage, x_line + (lane & 7), chunk16 + ((lane >> 3) & 1)));
                        // (all loads of the K step before its first product: see gemm_stream.cu)
                        unsigned a[MT][4];
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
                            if (mt * 16 < RB) gs_ldmatrix_x4(a[mt], gs_at(stage, w_line + mt * 16 + (lane & 15), chunk16 + (lane >> 4)));
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
                            if (mt * 16 < RB) gs_mma(acc[mt][0], a[mt], b[0], b[1]);
                    }
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem_u32(&empty_bar[slot])) : "memory");
                }
                asm volatile("bar.sync 1, %0;\n" ::"n"(GS_CWARPS * 32) : "memory");
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    float* base = part + ((size_t)warp * part_rows + mt * 16 + g) * pstride + 2 * t;
                    base[0] = acc[mt][0][0];
                    base[1] = acc[mt][0][1];
                    base[8 * pstride] = acc[mt][0][2];
                    base[8 * pstride + 1] = acc[mt][0][3];
                    acc[mt][0][0] = acc[mt][0][1] = acc[mt][0][2] = acc[mt][0][3] = 0.f;
                }
                asm volatile("bar.sync 1, %0;\n" ::"n"(GS_CWARPS * 32) : "memory");
                const int sub = chunk < sh.half_chunks ? chunk : chunk - sh.half_chunks;
                const int n0 = sh.row_begin + sub * RB;
                int rows = sh.row_end - n0;
                if (rows > RB) rows = RB;
                if (residual != nullptr) {
                    float sum = 0.f;
#pragma unroll
                    for (int i = 0; i < GS_MAX_RB / 16; ++i) {
                        const int c = part16 + 16 * i;
                        if (row16 < p.M && c < rows) {
                            float v = 0.f;
#pragma unroll
                            for (int w = 0; w < GS_CWARPS; ++w) v += part[((size_t)w * part_rows + c) * pstride + row16];
                            if (factors) v *= row_factor[row16];
                            const float r = r_before[i] + v;
                            residual[(size_t)row16 * ldr + n0 + c] = r;
                            xw[(size_t)row16 * ldxw + n0 + c] = __float2bfloat16_rn(r * w_norm[i]);
                            sum = fmaf(r, r, sum);
                        }
                    }
#pragma unroll
                    for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                    block_squares += sum;
                    continue;
                }
                for (int e = tid; e < rows * p.M; e += GS_CWARPS * 32) {
                    const int m = e / rows, row = e - m * rows;
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < GS_CWARPS; ++w) v += part[((size_t)w * part_rows + row) * pstride + m];
                    if (factors) v *= row_factor[m];
                    if (glu_rows) {
                        float* kept = gate + (size_t)(sub * RB + row) * 8 + m;
                        if (chunk < sh.half_chunks) {
                            *kept = v;
                            continue;
                        }
                        const float z = *kept;
                        v = (z / (1.f + expf(-z))) * v;
                    }
                    if (out_f32) reinterpret_cast<float*>(Y)[(size_t)m * ldy + n0 + row] = v;
                    else reinterpret_cast<bf16*>(Y)[(size_t)m * ldy + n0 + row] = __float2bfloat16_rn(v);
                }
            }
            if (q.residual != nullptr && part16 == 0 && sh.chunks > 0)         // (a block without rows here has no place in out_sumsq)
                q.out_sumsq[(size_t)blockIdx.x * 8 + row16] = row16 < p.M ? block_squares : 0.f;
            if (ph + 1 < p.phases) {
                // this block's results of the phase are out: visible to every block (and to their TMA units) before it counts
                __threadfence();
                asm volatile("fence.proxy.async;\n" ::: "memory");
                asm volatile("bar.sync 1, %0;\n" ::"n"(GS_CWARPS * 32) : "memory");
                if (tid == 0) {
                    unsigned one = 1u, old;
                    asm volatile("atom.release.gpu.global.add.u32 %0, [%1], %2;\n" : "=r"(old) : "l"(&p.counters[ph]), "r"(one) : "memory");
                }
            }
    }
}

__global__ void __launch_bounds__(GS_THREADS, 1)
gemm_stream_chain_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainParams p) {
    extern __shared__ unsigned char gc_raw[];
    __shared__ __align__(8) uint64_t full_bar[GS_MAX_STAGES], empty_bar[GS_MAX_STAGES];
    __shared__ float row_factor[8];
    const uint32_t raw_addr = tc_smem_u32(gc_raw);
    unsigned char* ring = gc_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t stage_bytes = p.stage_bytes;
    float* part = reinterpret_cast<float*>(ring + (size_t)p.stages * stage_bytes);   // [warps][128][9]
    float* gate = part + (size_t)GS_CWARPS * 128 * 9;                   // [rows of the block][8]
    const unsigned blocks = gridDim.x;

    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        for (int i = 0; i < p.phases; ++i) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&maps.w[i]) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&maps.x[i]) : "memory");
        }
    }
    __syncthreads();
    pdl_trigger();

    if (warp == GS_CWARPS) {
        if (lane == 0) {
            // Stage (phase, chunk, ks) belongs to compute warp w = ks % 4 and is that warp's j-th stage over all phases;
            // warp w owns the ring slots w, w + 4, ... and the stage lives in the (j mod their number)-th of them.
            int taken[GS_CWARPS] = {0, 0, 0, 0};
            int x_ready = -1;                                    // boxes of X may be asked for up to this phase
            int waiting_slot[GS_MAX_STAGES], waiting_ks[GS_MAX_STAGES], waiting = 0;      // stages that hold W and lack X
            for (int ph = 0; ph < p.phases; ++ph) {
                const ChainPhase& q = p.ph[ph];
                const PhaseShare sh = gc_share(q, blockIdx.x);
                const int RB = q.RB, KB = q.KB, glu_rows = q.glu_rows;
                const uint32_t w_bytes = (uint32_t)RB * 128 * KB, x_bytes = 8u * 128 * KB;
                // the boxes of X of this phase: after the kernel before this one (phase 0), after every block's phase before
                auto release_x = [&]() {
                    if (ph == 0) pdl_wait();
                    else gc_wait_blocks(&p.counters[ph - 1], blocks, p.error_flag);
                    asm volatile("fence.proxy.async;\n" ::: "memory");             // other blocks' stores, then TMA reads
                    for (int i = 0; i < waiting; ++i)
                        gs_tma_load_3d(ring + (size_t)waiting_slot[i] * stage_bytes + w_bytes, &maps.x[ph], 0, 0,
                                       waiting_ks[i] * KB, &full_bar[waiting_slot[i]]);
                    waiting = 0;
                    x_ready = ph;
                };
                for (int chunk = 0; chunk < sh.chunks; ++chunk) {
                    const int row = chunk < sh.half_chunks ? sh.row_begin + chunk * RB
                                                           : glu_rows + sh.row_begin + (chunk - sh.half_chunks) * RB;
                    for (int ks = 0; ks < sh.ksteps; ++ks) {
                        const int w = ks % GS_CWARPS;
                        const int mine = (p.stages - w + GS_CWARPS - 1) / GS_CWARPS;
                        const int j = taken[w]++;
                        const int slot = GS_CWARPS * (j % mine) + w, round = j / mine;
                        if (round > 0) {
                            // a slot whose stage lacks X cannot come free: hand the boxes of X out first
                            if (x_ready < ph && waiting > 0) {
                                bool held = false;
                                for (int i = 0; i < waiting; ++i) held |= waiting_slot[i] == slot;
                                if (held) release_x();
                            }
                            mbar_wait(&empty_bar[slot], (uint32_t)((round - 1) & 1), p.error_flag);
                        }
                        mbar_expect_tx(&full_bar[slot], w_bytes + x_bytes);
                        unsigned char* stage = ring + (size_t)slot * stage_bytes;
                        gs_tma_load_3d(stage, &maps.w[ph], 0, row, ks * KB, &full_bar[slot]);
                        if (x_ready >= ph) {
                            gs_tma_load_3d(stage + w_bytes, &maps.x[ph], 0, 0, ks * KB, &full_bar[slot]);
                        } else {
                            waiting_slot[waiting] = slot;
                            waiting_ks[waiting] = ks;
                            ++waiting;
                            if (waiting == p.stages) release_x();            // the ring is full of this phase's weights
                        }
                    }
                }
                if (x_ready < ph) release_x();                   // (also a block without rows in this phase passes the wait)
            }
        }
    } else {
        int j = 0;                                               // stages this warp has taken, over all phases
        for (int ph = 0; ph < p.phases; ++ph) {
            switch (p.ph[ph].mt) {
                case 2: gc_phase<2>(p, ph, ring, part, gate, full_bar, empty_bar, row_factor, j); break;
                case 4: gc_phase<4>(p, ph, ring, part, gate, full_bar, empty_bar, row_factor, j); break;
                default: gc_phase<8>(p, ph, ring, part, gate, full_bar, empty_bar, row_factor, j); break;
            }
        }
    }
    // the block that leaves last zeroes the counters for the next launch: every block has passed all its waits by then
    __syncthreads();
    if (tid == 0) {
        const unsigned before = atomicAdd(&p.counters[GC_MAX_PHASES], 1u);
        if (before == blocks - 1) {
            for (int i = 0; i <= GC_MAX_PHASES; ++i) p.counters[i] = 0u;
            __threadfence();
        }
    }
}

// ---- host side ---------------------------------------------------------------------------------------------
// One phase as the caller describes it (the layout is shared with the Python binding).
struct LlmpChainPhase {
    const void* X;        // [M, K] bfloat16
    const void* W;        // [N, K] bfloat16
    void* Y;              // [M, N] (or [M, N / 2] with glu_rows), or null in the residual form
    long ldx, ldw, ldy;
    int N, K, out_dtype, glu_rows;
    const float* in_sumsq;
    int in_parts;
    float in_inv_width, in_eps;
    float* residual;
    long ldr;
    const void* norm_w;
    int norm_w_dtype;
    void* xw;
    long ldxw;
    float* out_sumsq;
};

LLMP_API int llmp_gemm_stream_chain_counters() { return GC_MAX_PHASES + 1; }
LLMP_API int llmp_gemm_stream_chain_max_phases() { return GC_MAX_PHASES; }

// 1 when these phases can run as one chain on this device: each a product that gemm_stream takes at M rows, with
// plans that fit one ring together.
static bool chain_plan(const LlmpChainPhase* phases, int count, int M, ChainParams* out_params, StreamPlan* plans, size_t* out_smem) {
    if (count < 1 || count > GC_MAX_PHASES || M < 1 || M > 8) return false;
    size_t stage_bytes = 0, gate_bytes = 0;
    const int sms = llmp_sm_count();
    for (int i = 0; i < count; ++i) {
        const LlmpChainPhase& c = phases[i];
        if (!llmp_stream_plan(M, c.N, c.K, c.ldx, c.ldw, c.glu_rows, &plans[i])) return false;
        if (plans[i].nt != 1 || plans[i].mt > 8 || plans[i].grid > sms) return false;
        if (plans[i].stage_bytes > stage_bytes) stage_bytes = plans[i].stage_bytes;
        if (c.glu_rows) {
            const int chunks = (plans[i].per + GS_MAX_RB - 1) / GS_MAX_RB;
            const size_t bytes = (size_t)chunks * plans[i].rb * 8 * sizeof(float);
            if (bytes > gate_bytes) gate_bytes = bytes;
        }
    }
    const size_t part_bytes = (size_t)GS_CWARPS * 128 * 9 * sizeof(float) + gate_bytes;
    int stages = (int)((GS_SMEM_BUDGET - part_bytes) / stage_bytes);
    if (stages > GS_MAX_STAGES) stages = GS_MAX_STAGES;
    if (stages < GS_CWARPS) return false;
    out_params->stages = stages;
    out_params->stage_bytes = (uint32_t)stage_bytes;
    *out_smem = (size_t)stages * stage_bytes + part_bytes + 2048;
    return true;
}

LLMP_API int llmp_gemm_stream_chain_supports(const LlmpChainPhase* phases, int count, int M) {
    ChainParams p;
    StreamPlan plans[GC_MAX_PHASES];
    size_t smem;
    return chain_plan(phases, count, M, &p, plans, &smem) ? 1 : 0;
}

// Runs the phases as one launch. Phase i + 1 reads as its X what phase i wrote (its Y, or its xw in the residual form);
// the caller says so by passing those pointers. counters: llmp_gemm_stream_chain_counters() zeroed uint32 that
// launches on one device share (launches must follow one another in one stream, as they do in a decode step).
LLMP_API int llmp_gemm_stream_chain(const LlmpChainPhase* phases, int count, int M, unsigned* counters, int* error_flag,
                                    cudaStream_t stream) {
    LLMP_REQUIRE(counters != nullptr && error_flag != nullptr, "gemm_stream_chain: counters and an error flag are required");
    ChainParams p;
    StreamPlan plans[GC_MAX_PHASES];
    size_t smem = 0;
    LLMP_REQUIRE(chain_plan(phases, count, M, &p, plans, &smem), "gemm_stream_chain: these %d products of %d rows do not form a chain", count, M);
    ChainMaps maps;
    p.M = M; p.phases = count; p.counters = counters; p.error_flag = error_flag;
    for (int i = 0; i < count; ++i) {
        const LlmpChainPhase& c = phases[i];
        LLMP_REQUIRE(((size_t)c.X % 16) == 0 && ((size_t)c.W % 16) == 0, "gemm_stream_chain: operands must be 16-byte aligned");
        LLMP_REQUIRE(c.glu_rows == 0 || c.glu_rows * 2 == c.N, "gemm_stream_chain: %d gate rows do not make %d rows of W", c.glu_rows, c.N);
        ChainPhase& q = p.ph[i];
        q.Y = c.Y; q.ldy = c.ldy; q.N = c.N; q.K = c.K; q.per = plans[i].per; q.RB = plans[i].rb; q.KB = plans[i].kb; q.mt = plans[i].mt;
        q.out_f32 = c.out_dtype == LLMP_F32; q.glu_rows = c.glu_rows;
        q.in_sumsq = c.in_sumsq; q.in_parts = c.in_parts; q.in_inv_width = c.in_inv_width; q.in_eps = c.in_eps;
        q.residual = c.residual; q.ldr = c.ldr; q.norm_w = c.norm_w; q.norm_w_f32 = c.norm_w_dtype == LLMP_F32;
        q.xw = (bf16*)c.xw; q.ldxw = c.ldxw; q.out_sumsq = c.out_sumsq;
        if (c.residual != nullptr)
            LLMP_REQUIRE(c.glu_rows == 0 && c.norm_w != nullptr && c.xw != nullptr && c.out_sumsq != nullptr,
                         "gemm_stream_chain: the residual form needs a norm weight and places for its results, and no SwiGLU");
        else
            LLMP_REQUIRE(c.Y != nullptr, "gemm_stream_chain: a phase that is no residual addend needs an output");
        if (llmp_stream_tensor_map(c.W, c.N, c.K, c.ldw, q.RB, q.KB, &maps.w[i]) ||
            llmp_stream_tensor_map(c.X, M, c.K, c.ldx, 8, q.KB, &maps.x[i]))
            return 1;
    }
    const int grid = llmp_sm_count();
    LLMP_ALLOW_SMEM((gemm_stream_chain_kernel), smem);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(GS_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    const cudaError_t launched = cudaLaunchKernelEx(&config, gemm_stream_chain_kernel, maps, p);
    if (launched != cudaSuccess) {
        llmp_set_error("gemm_stream_chain: launch failed: %s", cudaGetErrorString(launched));
        return 2;
    }
    return llmp_check_launch("gemm_stream_chain");
}
