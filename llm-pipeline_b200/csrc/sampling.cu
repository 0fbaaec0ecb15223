// Token selection on float32 logits: argmax, and temperature sampling with the filters of the
// reference sampler in its order (temperature, top-k, top-p, min-p, typical-p, softmax, draw).
// One block per row. No sort: every filter is a threshold in value space found by bisection
// over the order-preserving integer image of the floats, with fixed-order block reductions,
// so a row's result does not depend on the other rows of the call.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned ordered_key(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"), first output word.
__device__ __host__ inline unsigned philox_first(unsigned long long seed, unsigned long long counter) {
    unsigned c0 = (unsigned)counter, c1 = (unsigned)(counter >> 32), c2 = 0u, c3 = 0u;
    unsigned k0 = (unsigned)seed, k1 = (unsigned)(seed >> 32);
    for (int round = 0; round < 10; ++round) {
        const unsigned long long p0 = (unsigned long long)0xD2511F53u * c0;
        const unsigned long long p1 = (unsigned long long)0xCD9E8D57u * c2;
        const unsigned n0 = (unsigned)(p1 >> 32) ^ c1 ^ k0;
        const unsigned n1 = (unsigned)p1;
        const unsigned n2 = (unsigned)(p0 >> 32) ^ c3 ^ k1;
        const unsigned n3 = (unsigned)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c0;
}

LLMP_API unsigned llmp_philox_first(unsigned long long seed, unsigned long long counter) {
    return philox_first(seed, counter);
}

struct ArgBest {
    float v;
    int i;
};

__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
    if (b.i >= 0 && (a.i < 0 || b.v > a.v || (b.v == a.v && b.i < a.i))) return b;
    return a;
}

// Largest value of the row, lowest index among equals; every thread gets the result.
__device__ ArgBest block_argmax(const float* row, int V, float inv_div, ArgBest* scratch) {
    ArgBest best = {-INFINITY, -1};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i] / inv_div;
        if (!(v != v)) best = better(best, ArgBest{v, i});
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other;
        other.v = __shfl_xor_sync(0xffffffffu, best.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, best.i, o);
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = best;
    __syncthreads();
    ArgBest r = lane < nwarps ? scratch[lane] : ArgBest{-INFINITY, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other;
        other.v = __shfl_xor_sync(0xffffffffu, r.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, r.i, o);
        r = better(r, other);
    }
    return r;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) argmax_kernel(const float* __restrict__ logits, long stride, int V,
                                                                int* __restrict__ out) {
    __shared__ ArgBest scratch[32];
    const ArgBest r = block_argmax(logits + (size_t)blockIdx.x * stride, V, 1.f, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = r.i < 0 ? 0 : r.i;
}

// Long rows and few of them: ARG_CHUNKS blocks per row find the best of their slice, a second pass
// takes the best of the slices (lowest index among equals in both).
#define ARG_CHUNKS 32
__global__ void __launch_bounds__(256) argmax_partial_kernel(const float* __restrict__ logits, long stride, int V,
                                                             float* __restrict__ part_v, int* __restrict__ part_i) {
    __shared__ ArgBest scratch[32];
    const int m = blockIdx.y, chunk = blockIdx.x;
    const int per = (V + ARG_CHUNKS - 1) / ARG_CHUNKS;
    const int begin = chunk * per;
    const int count = begin >= V ? 0 : (begin + per <= V ? per : V - begin);
    ArgBest r = block_argmax(logits + (size_t)m * stride + begin, count, 1.f, scratch);
    if (threadIdx.x == 0) {
        part_v[m * ARG_CHUNKS + chunk] = r.v;
        part_i[m * ARG_CHUNKS + chunk] = r.i < 0 ? -1 : r.i + begin;
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i, int* __restrict__ out) {
    const int m = blockIdx.x, lane = threadIdx.x;
    ArgBest best = {part_v[m * ARG_CHUNKS + lane], part_i[m * ARG_CHUNKS + lane]};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other;
        other.v = __shfl_xor_sync(0xffffffffu, best.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, best.i, o);
        best = better(best, other);
    }
    if (lane == 0) out[m] = best.i < 0 ? 0 : best.i;
}

// scratch: M * ARG_CHUNKS floats followed by M * ARG_CHUNKS ints, or null (then one block per row).
LLMP_API int llmp_argmax(const float* logits, long stride, int M, int V, int* out, void* scratch, cudaStream_t stream) {
    if (M <= 0) return 0;
    LLMP_REQUIRE(V > 0, "argmax: bad vocabulary size %d", V);
    static_assert(ARG_CHUNKS == 32, "the final pass is one warp per row");
    if (scratch && V >= 8192 && M <= 1024) {
        float* part_v = (float*)scratch;
        int* part_i = (int*)(part_v + (size_t)M * ARG_CHUNKS);
        argmax_partial_kernel<<<dim3(ARG_CHUNKS, M), 256, 0, stream>>>(logits, stride, V, part_v, part_i);
        argmax_final_kernel<<<M, 32, 0, stream>>>(part_v, part_i, out);
    } else {
        argmax_kernel<<<M, SAMPLE_THREADS, 0, stream>>>(logits, stride, V, out);
    }
    return llmp_check_launch("argmax");
}

// CTRL-style repetition penalty in place: for each listed token id of a row, a positive logit is
// divided by the penalty, another multiplied. token ids of row m are tokens[offsets[m] .. offsets[m+1]);
// the caller lists each id once.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, long stride, int V, const int* __restrict__ tokens,
                                          const int* __restrict__ offsets, const float* __restrict__ penalty) {
    const int m = blockIdx.x;
    const float pen = penalty[m];
    if (pen == 1.f) return;
    float* row = logits + (size_t)m * stride;
    for (int e = offsets[m] + threadIdx.x; e < offsets[m + 1]; e += blockDim.x) {
        const int t = tokens[e];
        if (t >= 0 && t < V) {
            const float v = row[t];
            row[t] = v > 0.f ? v / pen : v * pen;
        }
    }
}

LLMP_API int llmp_repetition_penalty(float* logits, long stride, int M, int V, const int* tokens, const int* offsets,
                                     const float* penalty, cudaStream_t stream) {
    if (M <= 0) return 0;
    repetition_penalty_kernel<<<M, 256, 0, stream>>>(logits, stride, V, tokens, offsets, penalty);
    return llmp_check_launch("repetition_penalty");
}

struct SampleRow {
    float temperature;
    int top_k;
    float top_p;
    float min_p;
    float typical_p;
    unsigned seed_lo, seed_hi;
    unsigned step;
};

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long stride, int V, const SampleRow* __restrict__ params,
              int* __restrict__ out, float* __restrict__ out_u) {
    __shared__ ArgBest arg_scratch[32];
    __shared__ float scratch[32];
    __shared__ float chunk_sum[SAMPLE_THREADS];
    __shared__ int found;
    const int m = blockIdx.x;
    const float* row = logits + (size_t)m * stride;
    const SampleRow sp = params[m];
    const int tid = threadIdx.x;

    if (!(sp.temperature > 0.f)) {          // greedy
        const ArgBest r = block_argmax(row, V, 1.f, arg_scratch);
        if (tid == 0) {
            out[m] = r.i < 0 ? 0 : r.i;
            if (out_u) out_u[m] = 0.f;
        }
        return;
    }
    const float T = sp.temperature;
    const ArgBest top = block_argmax(row, V, T, arg_scratch);
    const float mx = top.v;                 // largest scaled logit; it survives every filter

    // top-k: the largest key t with count(key >= t) >= k.
    unsigned lower = 0u;
    if (sp.top_k > 0 && sp.top_k < V) {
        unsigned t = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = t | (1u << bit);
            float cnt = 0.f;
            for (int i = tid; i < V; i += SAMPLE_THREADS) cnt += ordered_key(row[i] / T) >= cand ? 1.f : 0.f;
            cnt = block_sum(cnt, scratch);
            if (cnt >= (float)sp.top_k) t = cand;
        }
        lower = t;
    }
    // top-p: a value is kept when the mass of the strictly larger kept values is <= p.
    if (sp.top_p < 1.f) {
        float z = 0.f;
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
            const float x = row[i] / T;
            if (ordered_key(x) >= lower) z += expf(x - mx);
        }
        z = block_sum(z, scratch);
        const float limit = sp.top_p * z;
        unsigned t = 0u;                    // largest key whose mass above it still exceeds the limit
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = t | (1u << bit);
            float s = 0.f;
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const float x = row[i] / T;
                const unsigned k = ordered_key(x);
                if (k >= lower && k > cand) s += expf(x - mx);
            }
            s = block_sum(s, scratch);
            if (s > limit) t = cand;
        }
        if (t + 1u > lower) lower = t + 1u;
    }
    // min-p: prob < min_p * max prob  <=>  exp(x - max) < min_p (the maximum is always kept).
    const float min_e = sp.min_p > 0.f ? sp.min_p : 0.f;
    // typical-p: keep -log p <= exp(entropy) * typical_p over what is kept so far.
    float info_limit = INFINITY, log_z = 0.f;
    bool only_top = false;
    if (sp.typical_p < 1.f) {
        float z = 0.f;
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
            const float x = row[i] / T;
            const float e = expf(x - mx);
            if (ordered_key(x) >= lower && e >= min_e) z += e;
        }
        z = block_sum(z, scratch);
        log_z = logf(z);
        float h = 0.f;
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
            const float x = row[i] / T;
            const float e = expf(x - mx);
            if (ordered_key(x) >= lower && e >= min_e) {
                const float lp = x - mx - log_z;
                h -= (e / z) * lp;
            }
        }
        h = block_sum(h, scratch);
        info_limit = expf(h) * sp.typical_p;
        if (log_z > info_limit) only_top = true;     // even the most likely token fails: keep it alone
    }
    if (only_top) {
        if (tid == 0) {
            out[m] = top.i;
            if (out_u) out_u[m] = 0.f;
        }
        return;
    }
    // Draw: first index whose running sum of kept weights exceeds u * total. Thread t owns the
    // contiguous indices [t*per, (t+1)*per).
    const int per = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = tid * per;
    const int end = begin + per < V ? begin + per : V;
    float mine = 0.f;
    int last_kept = -1;
    for (int i = begin; i < end; ++i) {
        const float x = row[i] / T;
        const float e = expf(x - mx);
        if (ordered_key(x) >= lower && e >= min_e && -(x - mx - log_z) <= info_limit) {
            mine += e;
            last_kept = i;
        }
    }
    chunk_sum[tid] = mine;
    if (tid == 0) found = -1;
    __syncthreads();
    // Exclusive prefix over the chunks, in chunk order, by one warp (32 chunks per lane).
    __shared__ float chunk_base[SAMPLE_THREADS];
    __shared__ float total_s;
    if (tid < 32) {
        float acc = 0.f;
        const int c0 = tid * (SAMPLE_THREADS / 32);
        for (int c = 0; c < SAMPLE_THREADS / 32; ++c) acc += chunk_sum[c0 + c];
        float incl = acc;
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, incl, o);
            if (tid >= o) incl += up;
        }
        float run = incl - acc;
        for (int c = 0; c < SAMPLE_THREADS / 32; ++c) {
            chunk_base[c0 + c] = run;
            run += chunk_sum[c0 + c];
        }
        if (tid == 31) total_s = incl;
    }
    __syncthreads();
    const unsigned long long seed = ((unsigned long long)sp.seed_hi << 32) | sp.seed_lo;
    const float u = (float)(philox_first(seed, sp.step) >> 8) * (1.0f / 16777216.0f);
    const float target = u * total_s;
    const float base = chunk_base[tid];
    if (mine > 0.f && base <= target && target < base + mine) {
        float run = base;
        int pick = last_kept;
        for (int i = begin; i < end; ++i) {
            const float x = row[i] / T;
            const float e = expf(x - mx);
            if (ordered_key(x) >= lower && e >= min_e && -(x - mx - log_z) <= info_limit) {
                run += e;
                if (run > target) {
                    pick = i;
                    break;
                }
            }
        }
        atomicMax(&found, pick);
    }
    __syncthreads();
    if (tid == 0) {
        out[m] = found >= 0 ? found : top.i;    // rounding left the target past every chunk: most likely token
        if (out_u) out_u[m] = u;
    }
}

// params: M rows of 8 32-bit words {temperature f32, top_k i32, top_p f32, min_p f32, typical_p f32,
// seed low u32, seed high u32, step u32}.  out_u (optional) receives the uniform number of each row.
LLMP_API int llmp_sample(const float* logits, long stride, int M, int V, const void* params, int* out, float* out_u,
                         cudaStream_t stream) {
    if (M <= 0) return 0;
    LLMP_REQUIRE(V > 0, "sample: bad vocabulary size %d", V);
    sample_kernel<<<M, SAMPLE_THREADS, 0, stream>>>(logits, stride, V, (const SampleRow*)params, out, out_u);
    return llmp_check_launch("sample");
}

// ------------------------------------------------------------------------------------------
// Entropy of softmax(logits / temperature) per row, in nats, float32 (what Mirostat v2 steers by):
//   H = log Z - (sum_i e_i z_i) / Z   with z_i = x_i / T - max, e_i = exp(z_i), Z = sum_i e_i.
// One block per row; fixed-order block sums. temperature <= 0: the logits as they are.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(SAMPLE_THREADS) entropy_kernel(const float* __restrict__ logits, long stride, int V,
                                                                 float temperature, float* __restrict__ out) {
    __shared__ float scratch[32];
    const float* row = logits + (size_t)blockIdx.x * stride;
    const float inv = temperature > 0.f ? 1.f / temperature : 1.f;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i] * inv);
    mx = block_max(mx, scratch);
    float z = 0.f, ez = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float d = row[i] * inv - mx;
        if (d > -INFINITY) {                                       // a removed token (-inf) adds nothing
            const float e = expf(d);
            z += e;
            ez = fmaf(e, d, ez);
        }
    }
    z = block_sum(z, scratch);
    ez = block_sum(ez, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = logf(z) - ez / z;
}

LLMP_API int llmp_entropy(const float* logits, long stride, int M, int V, float temperature, float* out, cudaStream_t stream) {
    if (M <= 0) return 0;
    LLMP_REQUIRE(V > 0, "entropy: bad vocabulary size %d", V);
    entropy_kernel<<<M, SAMPLE_THREADS, 0, stream>>>(logits, stride, V, temperature, out);
    return llmp_check_launch("entropy");
}
