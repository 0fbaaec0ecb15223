// Memory-bound kernels of the forward pass: embedding gather, rotary tables, fused
// residual-add + RMSNorm, fused per-head q/k RMSNorm + rotary + paged K/V write, SwiGLU.
// All statistics (mean square, rsqrt, angles, sigmoid) are computed in float32.
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// Embedding: residual[n, :] = float(table[ids[n], :]).  The residual stream is float32.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int H, int V) {
    const int n = blockIdx.x;
    const int id = ids[n];
    const bool ok = id >= 0 && id < V;
    const T* row = table + (size_t)(ok ? id : 0) * H;
    float* dst = out + (size_t)n * H;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < H; c += gridDim.y * blockDim.x)
        dst[c] = ok ? to_float(row[c]) : 0.f;
}

LLMP_API int llmp_embedding(const int* ids, const void* table, int dtype, float* out, int N, int H, int V,
                            cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(H > 0 && V > 0, "embedding: bad sizes H=%d V=%d", H, V);
    const int threads = H >= 1024 ? 256 : 128;
    int col_blocks = (H + threads - 1) / threads;              // few tokens: spread a row over several blocks
    if ((long)N * col_blocks > 4096) col_blocks = 1;
    dim3 grid(N, col_blocks);
    if (dtype == LLMP_F32)
        embedding_kernel<float><<<grid, threads, 0, stream>>>(ids, (const float*)table, out, H, V);
    else
        embedding_kernel<bf16><<<grid, threads, 0, stream>>>(ids, (const bf16*)table, out, H, V);
    return llmp_check_launch("embedding");
}

// ------------------------------------------------------------------------------------------
// Rotary tables: cos/sin[n, j] = cos/sin(float(pos[n]) * inv_freq[j]) * scaling, float32.
// ------------------------------------------------------------------------------------------
__global__ void rope_tables_kernel(const int* __restrict__ pos, const float* __restrict__ inv_freq, float scaling,
                                   float* __restrict__ cos_out, float* __restrict__ sin_out, int N, int half) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)N * half) return;
    const int n = (int)(i / half), j = (int)(i % half);
    const float angle = (float)pos[n] * inv_freq[j];
    float s, c;
    sincosf(angle, &s, &c);
    cos_out[i] = c * scaling;
    sin_out[i] = s * scaling;
}

LLMP_API int llmp_rope_tables(const int* pos, const float* inv_freq, float scaling, float* cos_out, float* sin_out,
                              int N, int half, cudaStream_t stream) {
    if (N <= 0 || half <= 0) return 0;
    const size_t total = (size_t)N * half;
    rope_tables_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(pos, inv_freq, scaling, cos_out, sin_out,
                                                                           N, half);
    return llmp_check_launch("rope_tables");
}

// ------------------------------------------------------------------------------------------
// Fused residual add + RMSNorm.  For output row m (input row r = rows ? rows[m] : m):
//   x = residual[r] + delta[r] + delta_bias          (delta, delta_bias optional)
//   if (!rows) residual[r] = x
//   out[m] = weight * (x * rsqrt(mean(x^2) + eps))   rounded once to the output type
// One block per row; the row is staged in shared memory between the two passes.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const void* __restrict__ delta_bias, int bias_bf16,
                                   const void* __restrict__ weight, int weight_bf16, float eps,
                                   T* __restrict__ out, const int* __restrict__ rows, int H) {
    extern __shared__ float row_smem[];
    __shared__ float scratch[32];
    const int m = blockIdx.x;
    const int r = rows ? rows[m] : m;
    float* res = residual + (size_t)r * H;
    const T* del = delta ? delta + (size_t)r * H : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float x = res[c];
        if (del) x += to_float(del[c]);
        if (delta_bias) x += load_as_float(delta_bias, bias_bf16, c);
        row_smem[c] = x;
        ss += x * x;
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)H + eps);
    T* dst = out + (size_t)m * H;
    const bool write_back = (rows == nullptr) && (del != nullptr || delta_bias != nullptr);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float x = row_smem[c];
        if (write_back) res[c] = x;
        dst[c] = from_float<T>(load_as_float(weight, weight_bf16, c) * (x * rstd));
    }
}

// The same operation for rows of at most 16384 entries whose width is a multiple of 4: one, two or four 4-entry
// pieces per thread, held in registers from the first load to the store, so the row makes one trip.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[4]) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[4]) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 raw;
        raw.x = *reinterpret_cast<const unsigned*>(&a);
        raw.y = *reinterpret_cast<const unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

// PIECES 4-entry pieces per thread (piece p of thread t at column 4 (t + p * blockDim)): rows of at most 4096 PIECES entries.
// The launcher starts up to 1024 threads (the widest rows of each PIECES); the bound keeps the registers within that.
template <typename T, int PIECES>
__global__ void __launch_bounds__(1024) add_rmsnorm_row4_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                        const void* __restrict__ delta_bias, int bias_bf16,
                                        const void* __restrict__ weight, int weight_bf16, float eps,
                                        T* __restrict__ out, const int* __restrict__ rows, int H) {
    __shared__ float scratch[32];
    const int m = blockIdx.x;
    const int r = rows ? rows[m] : m;
    float x[PIECES][4], w[PIECES][4];
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
        const int c = (threadIdx.x + p * blockDim.x) * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[p][i] = 0.f;
            w[p][i] = c < H ? load_as_float(weight, weight_bf16, c + i) : 0.f;
        }
    }
    pdl_wait();                                    // the addend (and the residual of the kernel before) is complete
    pdl_trigger();
    float ss = 0.f;
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
        const int c = (threadIdx.x + p * blockDim.x) * 4;
        if (c < H) {
            Vec4<float>::load(residual + (size_t)r * H + c, x[p]);
            if (delta) {
                float dl[4];
                Vec4<T>::load(delta + (size_t)r * H + c, dl);
#pragma unroll
                for (int i = 0; i < 4; ++i) x[p][i] += dl[i];
            }
            if (delta_bias) {
#pragma unroll
                for (int i = 0; i < 4; ++i) x[p][i] += load_as_float(delta_bias, bias_bf16, c + i);
            }
        }
        ss += x[p][0] * x[p][0] + x[p][1] * x[p][1] + x[p][2] * x[p][2] + x[p][3] * x[p][3];
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
        const int c = (threadIdx.x + p * blockDim.x) * 4;
        if (c < H) {
            if (rows == nullptr && (delta != nullptr || delta_bias != nullptr)) Vec4<float>::store(residual + (size_t)r * H + c, x[p]);
            float y[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) y[i] = w[p][i] * (x[p][i] * rstd);
            Vec4<T>::store(out + (size_t)m * H + c, y);
        }
    }
}

template <typename T, int PIECES>
static cudaError_t launch_add_rmsnorm_row4(float* residual, const void* delta, const void* delta_bias, int bias_dtype,
                                           const void* weight, int weight_dtype, float eps, void* out, const int* rows, int M,
                                           int H, cudaStream_t stream) {
    const int per_thread = 4 * PIECES;
    const int threads = (((H + per_thread - 1) / per_thread + 31) / 32) * 32;
    return llmp_launch_dependent(add_rmsnorm_row4_kernel<T, PIECES>, dim3(M), dim3(threads), 0, stream, residual, (const T*)delta,
                                 delta_bias, (int)(bias_dtype == LLMP_BF16), weight, (int)(weight_dtype == LLMP_BF16), eps, (T*)out,
                                 rows, H);
}

LLMP_API int llmp_add_rmsnorm(float* residual, const void* delta, const void* delta_bias, int bias_dtype,
                              const void* weight, int weight_dtype, float eps, void* out, int dtype,
                              const int* rows, int M, int H, cudaStream_t stream) {
    if (M <= 0) return 0;
    LLMP_REQUIRE(H > 0, "add_rmsnorm: bad width %d", H);
    if (H % 4 == 0 && H <= 16384) {
        // the register-resident kernel: one, two or four 4-entry pieces per thread
        cudaError_t launched;
        // Pieces per thread follow from the width alone (never from the number of rows: a row's sum of squares must be
        // added in one order however many rows the step has). From 2,048 entries on a thread holds four pieces: a
        // prompt portion's rows fill the GPU by themselves and more loads in flight per thread read faster (2,048 rows
        // of 4,096: 24.6 us with one piece per thread), and the few rows of a decode step lose nothing measurable.
#define NORM_LAUNCH(T)                                                                                                          \
    (H < 1024 ? launch_add_rmsnorm_row4<T, 1>(residual, delta, delta_bias, bias_dtype, weight, weight_dtype, eps, out, rows, M, H, stream) \
     : H < 2048 ? launch_add_rmsnorm_row4<T, 2>(residual, delta, delta_bias, bias_dtype, weight, weight_dtype, eps, out, rows, M, H, stream) \
                : launch_add_rmsnorm_row4<T, 4>(residual, delta, delta_bias, bias_dtype, weight, weight_dtype, eps, out, rows, M, H, stream))
        launched = dtype == LLMP_F32 ? NORM_LAUNCH(float) : NORM_LAUNCH(bf16);
#undef NORM_LAUNCH
        if (launched != cudaSuccess) {
            llmp_set_error("add_rmsnorm: launch failed: %s", cudaGetErrorString(launched));
            return 2;
        }
        return llmp_check_launch("add_rmsnorm");
    }
    const size_t smem = (size_t)H * sizeof(float);
    LLMP_REQUIRE(smem <= 200 * 1024, "add_rmsnorm: width %d needs %zu bytes of shared memory (limit 204800)", H, smem);
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (dtype == LLMP_F32) {
        LLMP_ALLOW_SMEM(add_rmsnorm_kernel<float>, smem);
        add_rmsnorm_kernel<float><<<M, threads, smem, stream>>>(residual, (const float*)delta, delta_bias,
                                                                bias_dtype == LLMP_BF16, weight,
                                                                weight_dtype == LLMP_BF16, eps, (float*)out, rows, H);
    } else {
        LLMP_ALLOW_SMEM(add_rmsnorm_kernel<bf16>, smem);
        add_rmsnorm_kernel<bf16><<<M, threads, smem, stream>>>(residual, (const bf16*)delta, delta_bias,
                                                               bias_dtype == LLMP_BF16, weight,
                                                               weight_dtype == LLMP_BF16, eps, (bf16*)out, rows, H);
    }
    return llmp_check_launch("add_rmsnorm");
}

// ------------------------------------------------------------------------------------------
// Fused projection bias + per-head RMSNorm + rotary + paged K/V write.
// qkv is [N, (nq + 2*nkv) * d] with columns [q heads | k heads | v heads].  For token n:
//   q head: (+bias) -> RMSNorm over d (optional) -> rotate the first rotary_dim entries -> written in place
//   k head: same, then stored to the page slot of the token
//   v head: (+bias) -> stored to the page slot
// Rotation pairs entry j with j + rotary_dim/2:  y[j] = x[j]*cos - x[j+h]*sin,  y[j+h] = x[j+h]*cos + x[j]*sin.
// Pages are [num_pages, 2 (K,V), nkv, page_size, d];  slot = page * page_size + offset, or -1 to skip.
// One warp per (token, head); 4 warps per block.
// ------------------------------------------------------------------------------------------
// Contiguous pieces of VEC elements as one load or store (VEC = 1, 2 or 4; the address must be aligned to the piece).
template <typename T, int VEC> struct Piece;
template <int VEC> struct Piece<float, VEC> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[VEC]) {
        if (VEC == 4) { const float4 x = *reinterpret_cast<const float4*>(p); v[0] = x.x; v[1 % VEC] = x.y; v[2 % VEC] = x.z; v[3 % VEC] = x.w; }
        else if (VEC == 2) { const float2 x = *reinterpret_cast<const float2*>(p); v[0] = x.x; v[1 % VEC] = x.y; }
        else v[0] = p[0];
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[VEC]) {
        if (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1 % VEC], v[2 % VEC], v[3 % VEC]);
        else if (VEC == 2) *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1 % VEC]);
        else p[0] = v[0];
    }
};
template <int VEC> struct Piece<bf16, VEC> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[VEC]) {
        if (VEC == 4) {
            const uint2 raw = *reinterpret_cast<const uint2*>(p);
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
            v[0] = __low2float(a); v[1 % VEC] = __high2float(a); v[2 % VEC] = __low2float(b); v[3 % VEC] = __high2float(b);
        } else if (VEC == 2) {
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(p);
            v[0] = __low2float(a); v[1 % VEC] = __high2float(a);
        } else v[0] = __bfloat162float(p[0]);
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[VEC]) {
        if (VEC == 4) {
            const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1 % VEC]), b = __floats2bfloat162_rn(v[2 % VEC], v[3 % VEC]);
            uint2 raw;
            raw.x = *reinterpret_cast<const unsigned*>(&a);
            raw.y = *reinterpret_cast<const unsigned*>(&b);
            *reinterpret_cast<uint2*>(p) = raw;
        } else if (VEC == 2) {
            *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1 % VEC]);
        } else p[0] = __float2bfloat16_rn(v[0]);
    }
};

#define QKV_WARPS 4
template <typename T, int VEC>
__global__ void qkv_post_kernel(T* __restrict__ qkv, const void* __restrict__ bias, int bias_bf16,
                                const void* __restrict__ q_w, const void* __restrict__ k_w, int w_bf16,
                                float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                int rotary_dim, const int* __restrict__ slots, T* __restrict__ pages,
                                int nq, int nkv, int d, int page_size) {
    extern __shared__ float head_smem[];           // [QKV_WARPS][d]
    pdl_trigger();                                 // the attention kernel may start fetching keys of earlier steps
    pdl_wait();                                    // the projection is complete
    const int n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* x = head_smem + (size_t)warp * d;
    const int heads = nq + 2 * nkv;
    const size_t row_width = (size_t)heads * d;
    T* row = qkv + (size_t)n * row_width;
    const int half = rotary_dim / 2;
    const int slot = slots ? slots[n] : -1;
    for (int h = blockIdx.y * QKV_WARPS + warp; h < heads; h += gridDim.y * QKV_WARPS) {
        const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
        T* src = row + (size_t)h * d;
        float ss = 0.f;
        for (int i = lane * VEC; i < d; i += 32 * VEC) {
            float v[VEC];
            Piece<T, VEC>::load(src + i, v);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                if (bias) v[e] += load_as_float(bias, bias_bf16, (size_t)h * d + i + e);
                x[i + e] = v[e];
                ss += v[e] * v[e];
            }
        }
        __syncwarp();
        const void* w = is_q ? q_w : k_w;
        if ((is_q || is_k) && w) {
            ss = warp_sum(ss);
            const float rstd = rsqrtf(ss / (float)d + eps);
            for (int i = lane; i < d; i += 32) x[i] = load_as_float(w, w_bf16, i) * (x[i] * rstd);
            __syncwarp();
        }
        if ((is_q || is_k) && half > 0) {
            const float* c = cos_t + (size_t)n * half;
            const float* s = sin_t + (size_t)n * half;
            for (int j = lane; j < half; j += 32) {
                const float a = x[j], b = x[j + half];
                x[j] = a * c[j] - b * s[j];
                x[j + half] = b * c[j] + a * s[j];
            }
            __syncwarp();
        }
        T* dst = nullptr;
        if (is_q) {
            dst = src;
        } else if (pages && slot >= 0) {
            const int kvh = is_k ? h - nq : h - nq - nkv;
            const size_t page = (size_t)(slot / page_size), off = (size_t)(slot % page_size);
            dst = pages + (((page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + off) * d;
        }
        if (dst) {
            for (int i = lane * VEC; i < d; i += 32 * VEC) {
                float v[VEC];
#pragma unroll
                for (int e = 0; e < VEC; ++e) v[e] = x[i + e];
                Piece<T, VEC>::store(dst + i, v);
            }
        }
        __syncwarp();
    }
}

// Head size 128 with the whole head rotated: a half-warp per head, 8 elements per lane held in registers.
// Element j pairs with j + 64, which lane (l ^ 8) of the half-warp holds at the same register index.
template <typename T> struct Piece8;
template <> struct Piece8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
};
template <> struct Piece8<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            v[2 * e] = __uint_as_float(w[e] << 16);
            v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[8]) {
        unsigned w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
            w[e] = *reinterpret_cast<const unsigned*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

#define QKV_UNROLL 3
template <typename T>
__global__ void __launch_bounds__(QKV_WARPS * 32)
qkv_post_d128_kernel(T* __restrict__ qkv, const void* __restrict__ bias, int bias_bf16,
                     const void* __restrict__ q_w, const void* __restrict__ k_w, int w_bf16, float eps,
                     const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int* __restrict__ slots,
                     T* __restrict__ pages, int nq, int nkv, int page_size) {
    constexpr int D = 128;
    pdl_trigger();                                 // the attention kernel may start fetching keys of earlier steps
    const int n = blockIdx.x;
    const int hl = threadIdx.x & 15;                               // lane within the half-warp
    const int half_warp = threadIdx.x >> 4;
    const int heads = nq + 2 * nkv;
    T* row = qkv + (size_t)n * heads * D;
    const int slot = slots ? slots[n] : -1;
    const int e0 = hl * 8;                                         // first element of this lane
    float c[8], s[8], wq[8], wk[8];
    {
        const float* cp = cos_t + (size_t)n * (D / 2) + (e0 & 63);
        const float* sp = sin_t + (size_t)n * (D / 2) + (e0 & 63);
        Piece8<float>::load(cp, c);
        Piece8<float>::load(sp, s);
        if (hl < 8) {                                              // y[j] = x[j] cos - x[j + 64] sin
#pragma unroll
            for (int e = 0; e < 8; ++e) s[e] = -s[e];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) wq[e] = wk[e] = 1.f;
        if (q_w) { if (w_bf16) Piece8<bf16>::load((const bf16*)q_w + e0, wq); else Piece8<float>::load((const float*)q_w + e0, wq); }
        if (k_w) { if (w_bf16) Piece8<bf16>::load((const bf16*)k_w + e0, wk); else Piece8<float>::load((const float*)k_w + e0, wk); }
    }
    pdl_wait();                                    // the projection is complete (tables and weights were read before)
    // Heads in rounds of QKV_UNROLL per half-warp: the loads of a round are issued before any of its stores.
    const int step = gridDim.y * (QKV_WARPS * 2);
    for (int h0 = blockIdx.y * (QKV_WARPS * 2); h0 < heads; h0 += step * QKV_UNROLL) {  // uniform over the warp
        float v[QKV_UNROLL][8];
#pragma unroll
        for (int u = 0; u < QKV_UNROLL; ++u) {
            const int h = h0 + u * step + half_warp;
            const size_t at = (size_t)(h < heads ? h : 0) * D + e0;
            Piece8<T>::load(row + at, v[u]);
            if (bias) {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[u][e] += load_as_float(bias, bias_bf16, at + e);
            }
        }
#pragma unroll
        for (int u = 0; u < QKV_UNROLL; ++u) {
            if (h0 + u * step >= heads) break;                     // uniform over the warp
            const int h = h0 + u * step + half_warp;
            const bool live = h < heads;
            const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
            {                                                      // every lane takes part in the shuffles
                const void* w = is_q ? q_w : (is_k ? k_w : nullptr);
                float ss = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) ss += v[u][e] * v[u][e];
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (w) {
                    const float rstd = rsqrtf(ss / (float)D + eps);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[u][e] = (is_q ? wq[e] : wk[e]) * (v[u][e] * rstd);
                }
            }
            float other[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) other[e] = __shfl_xor_sync(0xffffffffu, v[u][e], 8);
            if (is_q || is_k) {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[u][e] = v[u][e] * c[e] + other[e] * s[e];
            }
            T* dst = nullptr;
            if (is_q) {
                dst = row + (size_t)h * D + e0;
            } else if (live && pages && slot >= 0) {
                const int kvh = is_k ? h - nq : h - nq - nkv;
                const size_t page = (size_t)(slot / page_size), off = (size_t)(slot % page_size);
                dst = pages + (((page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + off) * D + e0;
            }
            if (dst) Piece8<T>::store(dst, v[u]);
        }
    }
}

LLMP_API int llmp_qkv_post(void* qkv, int dtype, const void* bias, int bias_dtype, const void* q_w, const void* k_w,
                           int w_dtype, float eps, const float* cos_t, const float* sin_t, int rotary_dim,
                           const int* slots, void* pages, int N, int nq, int nkv, int d, int page_size,
                           cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(nq > 0 && nkv >= 0 && d > 0, "qkv_post: bad sizes nq=%d nkv=%d d=%d", nq, nkv, d);
    LLMP_REQUIRE(rotary_dim >= 0 && rotary_dim <= d && rotary_dim % 2 == 0,
                 "qkv_post: rotary_dim %d must be even and at most head_dim %d", rotary_dim, d);
    LLMP_REQUIRE(rotary_dim == 0 || (cos_t && sin_t), "qkv_post: rotary tables missing");
    LLMP_REQUIRE(!pages || page_size > 0, "qkv_post: bad page size %d", page_size);
    const size_t smem = (size_t)QKV_WARPS * d * sizeof(float);
    LLMP_REQUIRE(smem <= 48 * 1024, "qkv_post: head_dim %d too large", d);
    // Few tokens: one warp per head so that the heads run side by side; many tokens: a block walks the heads.
    const int heads = nq + 2 * nkv;
    int head_blocks = (heads + QKV_WARPS - 1) / QKV_WARPS;
    if ((long)N * head_blocks > (1L << 18)) head_blocks = 1;
    const bool aligned16 = (((uintptr_t)qkv | (uintptr_t)pages | (uintptr_t)q_w | (uintptr_t)k_w | (uintptr_t)cos_t |
                             (uintptr_t)sin_t) & 15) == 0;
    if (d == 128 && rotary_dim == 128 && aligned16) {
        // Few tokens: the heads of a token spread over blocks; many: one block walks all heads of its token, so
        // that the tables and norm weights are read once per token.
        const int blocks_y = N >= 512 ? 1 : (heads + 2 * QKV_WARPS - 1) / (2 * QKV_WARPS);
        dim3 grid128(N, blocks_y);
        if (dtype == LLMP_F32)
            qkv_post_d128_kernel<float><<<grid128, QKV_WARPS * 32, 0, stream>>>(
                (float*)qkv, bias, bias_dtype == LLMP_BF16, q_w, k_w, w_dtype == LLMP_BF16, eps, cos_t, sin_t, slots,
                (float*)pages, nq, nkv, page_size);
        else
            llmp_launch_dependent(qkv_post_d128_kernel<bf16>, grid128, dim3(QKV_WARPS * 32), 0, stream,
                                  (bf16*)qkv, bias, bias_dtype == LLMP_BF16, q_w, k_w, w_dtype == LLMP_BF16, eps, cos_t, sin_t,
                                  slots, (bf16*)pages, nq, nkv, page_size);
        return llmp_check_launch("qkv_post");
    }
    dim3 grid(N, head_blocks);
    // pieces of 4 elements when every head starts on such a piece in the qkv rows and in the pages, else 2, else 1
    const int vec = d % 4 == 0 ? 4 : (d % 2 == 0 ? 2 : 1);
#define QKV_LAUNCH(T, V)                                                                                              \
    qkv_post_kernel<T, V><<<grid, QKV_WARPS * 32, smem, stream>>>(                                                    \
        (T*)qkv, bias, bias_dtype == LLMP_BF16, q_w, k_w, w_dtype == LLMP_BF16, eps, cos_t, sin_t, rotary_dim, slots, \
        (T*)pages, nq, nkv, d, page_size)
    if (dtype == LLMP_F32) {
        if (vec == 4) QKV_LAUNCH(float, 4); else if (vec == 2) QKV_LAUNCH(float, 2); else QKV_LAUNCH(float, 1);
    } else {
        if (vec == 4) QKV_LAUNCH(bf16, 4); else if (vec == 2) QKV_LAUNCH(bf16, 2); else QKV_LAUNCH(bf16, 1);
    }
#undef QKV_LAUNCH
    return llmp_check_launch("qkv_post");
}

// ------------------------------------------------------------------------------------------
// SwiGLU: out[n, i] = silu(gu[n, i]) * gu[n, I + i],  silu(z) = z / (1 + exp(-z)), float32 inside.
// ------------------------------------------------------------------------------------------
// The float32 path divides and exponentiates exactly; the bfloat16 path uses the fast float32 intrinsics, whose
// error (about 2 ulp of float32) is far below the rounding of the bfloat16 result.
template <typename T> __device__ __forceinline__ float silu(float z);
template <> __device__ __forceinline__ float silu<float>(float z) { return z / (1.f + expf(-z)); }
template <> __device__ __forceinline__ float silu<bf16>(float z) { return __fdividef(z, 1.f + __expf(-z)); }

template <typename T, int VEC>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I) {
    pdl_trigger();                                 // the product that follows may start fetching its weights
    pdl_wait();                                    // the gate and up projections are complete
    const int n = blockIdx.y;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (i >= I) return;
    const T* row = gu + (size_t)n * 2 * I;
    float g[VEC], u[VEC], y[VEC];
    Piece<T, VEC>::load(row + i, g);
    Piece<T, VEC>::load(row + (size_t)I + i, u);
#pragma unroll
    for (int e = 0; e < VEC; ++e) y[e] = silu<T>(g[e]) * u[e];
    Piece<T, VEC>::store(out + (size_t)n * I + i, y);
}

// bfloat16 rows whose width is a multiple of 8: 16-byte pieces.
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I) {
    pdl_trigger();                                 // the product that follows may start fetching its weights
    pdl_wait();                                    // the gate and up projections are complete
    const int n = blockIdx.y;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= I) return;
    const bf16* row = gu + (size_t)n * 2 * I;
    float g[8], u[8], y[8];
    Piece8<bf16>::load(row + i, g);
    Piece8<bf16>::load(row + (size_t)I + i, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = silu<bf16>(g[e]) * u[e];
    Piece8<bf16>::store(out + (size_t)n * I + i, y);
}

LLMP_API int llmp_swiglu(const void* gu, void* out, int dtype, int N, int I, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(I > 0, "swiglu: bad width %d", I);
    LLMP_REQUIRE(N <= 65535 * 1024, "swiglu: too many rows %d", N);
    // gridDim.y is limited to 65535: fold larger row counts into several launches.
    const int max_rows = 65535;
    for (int n0 = 0; n0 < N; n0 += max_rows) {
        const int rows = N - n0 < max_rows ? N - n0 : max_rows;
        const int vec = I % 4 == 0 ? 4 : 1;
        dim3 grid((I / vec + 255) / 256, rows);
        if (dtype == LLMP_F32) {
            const float* src = (const float*)gu + (size_t)n0 * 2 * I;
            float* dst = (float*)out + (size_t)n0 * I;
            if (vec == 4) swiglu_kernel<float, 4><<<grid, 256, 0, stream>>>(src, dst, I);
            else swiglu_kernel<float, 1><<<grid, 256, 0, stream>>>(src, dst, I);
        } else {
            const bf16* src = (const bf16*)gu + (size_t)n0 * 2 * I;
            bf16* dst = (bf16*)out + (size_t)n0 * I;
            if (I % 8 == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0)
                llmp_launch_dependent(swiglu_bf16x8_kernel, dim3((I / 8 + 255) / 256, rows), dim3(256), 0, stream, src, dst, I);
            else if (vec == 4) swiglu_kernel<bf16, 4><<<grid, 256, 0, stream>>>(src, dst, I);
            else swiglu_kernel<bf16, 1><<<grid, 256, 0, stream>>>(src, dst, I);
        }
    }
    return llmp_check_launch("swiglu");
}
