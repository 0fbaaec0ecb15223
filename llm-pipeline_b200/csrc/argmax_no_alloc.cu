// llmp_argmax_no_alloc: row-wise argmax whose scratch memory is part of the library image.
// See no_alloc.h for who this is for and for the rules of use.
#include "no_alloc.h"

#include <mutex>

#include "common.cuh"

#define NA_SLICES 32
#define NA_MAX_DEVICES 64

// Winners of the first pass: for row m and slice s, value at [m * 32 + s] and index at
// [MAX_ROWS * 32 + m * 32 + s] (stored as int bits). File scope, so it lives in every GPU that loads
// the library. In host code this name is only a handle for cudaGetSymbolAddress, never a pointer to
// hand to a kernel.
static __device__ __align__(256) float na_scratch[2 * LLMP_NO_ALLOC_MAX_ROWS * NA_SLICES];

struct NaBest {
    float v;
    int i;
};

__device__ __forceinline__ NaBest na_better(NaBest a, NaBest b) {
    if (b.i >= 0 && (a.i < 0 || b.v > a.v || (b.v == a.v && b.i < a.i))) return b;
    return a;
}

__device__ __forceinline__ NaBest na_warp_best(NaBest x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        NaBest other;
        other.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = na_better(x, other);
    }
    return x;
}

// Pass 1: block (slice, row) finds the best entry of its slice of the row.
__global__ void __launch_bounds__(256) na_partial_kernel(const float* __restrict__ logits, long stride, int V,
                                                         float* __restrict__ scratch) {
    __shared__ NaBest per_warp[8];
    const int m = blockIdx.y, slice = blockIdx.x;
    // in long: near V = 2^31 the last slices' bounds and the loop's increment would wrap an int
    const long per = ((long)V + NA_SLICES - 1) / NA_SLICES;
    const long begin = slice * per;
    const long end = begin + per < V ? begin + per : V;
    const float* row = logits + (size_t)m * stride;
    NaBest best = {-INFINITY, -1};
    for (long i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = row[i];
        if (!(v != v)) best = na_better(best, NaBest{v, (int)i});
    }
    best = na_warp_best(best);
    if ((threadIdx.x & 31) == 0) per_warp[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        NaBest r = threadIdx.x < 8 ? per_warp[threadIdx.x] : NaBest{-INFINITY, -1};
        r = na_warp_best(r);
        if (threadIdx.x == 0) {
            scratch[m * NA_SLICES + slice] = r.v;
            reinterpret_cast<int*>(scratch)[LLMP_NO_ALLOC_MAX_ROWS * NA_SLICES + m * NA_SLICES + slice] = r.i;
        }
    }
}

// Pass 2: one warp per row takes the best of the 32 slices.
__global__ void na_final_kernel(const float* __restrict__ scratch, int* __restrict__ out) {
    const int m = blockIdx.x, lane = threadIdx.x;
    NaBest best = {scratch[m * NA_SLICES + lane],
                   reinterpret_cast<const int*>(scratch)[LLMP_NO_ALLOC_MAX_ROWS * NA_SLICES + m * NA_SLICES + lane]};
    best = na_warp_best(best);
    if (lane == 0) out[m] = best.i < 0 ? 0 : best.i;
}

// Device address of na_scratch on the current device, looked up once per device.
static int na_scratch_address(float** out) {
    static float* address[NA_MAX_DEVICES] = {nullptr};
    static std::mutex lock;
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess || device < 0 || device >= NA_MAX_DEVICES) {
        llmp_set_error("argmax_no_alloc: cannot tell the current device (%s)", cudaGetErrorString(err));
        return 1;
    }
    std::lock_guard<std::mutex> guard(lock);
    if (address[device] == nullptr) {
        void* p = nullptr;
        err = cudaGetSymbolAddress(&p, na_scratch);
        if (err != cudaSuccess || p == nullptr) {
            llmp_set_error("argmax_no_alloc: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(err));
            return 1;
        }
        address[device] = static_cast<float*>(p);
    }
    *out = address[device];
    return 0;
}

int llmp_argmax_no_alloc(const float* logits, long row_stride, int M, int V, int* out, cudaStream_t stream) {
    LLMP_REQUIRE(M >= 1 && M <= LLMP_NO_ALLOC_MAX_ROWS,
                 "argmax_no_alloc: %d rows; the built-in scratch holds 1..%d rows", M, LLMP_NO_ALLOC_MAX_ROWS);
    LLMP_REQUIRE(V >= 1, "argmax_no_alloc: bad row length %d", V);
    LLMP_REQUIRE(logits != nullptr && out != nullptr, "argmax_no_alloc: null input or output");
    float* scratch = nullptr;
    if (na_scratch_address(&scratch)) return 1;
    na_partial_kernel<<<dim3(NA_SLICES, M), 256, 0, stream>>>(logits, row_stride, V, scratch);
    na_final_kernel<<<M, 32, 0, stream>>>(scratch, out);
    return llmp_check_launch("argmax_no_alloc");
}
