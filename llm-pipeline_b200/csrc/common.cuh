// Shared helpers of the sm_100a kernels: element types, conversions, reductions and the
// error reporting of the C entry points.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LLMP_API extern "C" __attribute__((visibility("default")))

// Element type codes used by the C entry points.
enum LlmpDtype : int { LLMP_F32 = 0, LLMP_BF16 = 1 };

// Every entry point returns 0 on success. A non-zero return means nothing useful was computed;
// llmp_last_error() then gives the reason as text.
void llmp_set_error(const char* fmt, ...);
int llmp_check_launch(const char* what);

#define LLMP_REQUIRE(cond, ...)            \
    do {                                   \
        if (!(cond)) {                     \
            llmp_set_error(__VA_ARGS__);   \
            return 1;                      \
        }                                  \
    } while (0)

// Raises a kernel's dynamic shared memory limit once per size (per call site), outside the launch path
// of later calls. The limit belongs to the current device's context; the library drives one device.
#define LLMP_ALLOW_SMEM(kernel, smem)                                                              \
    do {                                                                                           \
        static size_t allowed_ = 48 * 1024;                                                        \
        if ((size_t)(smem) > allowed_) {                                                           \
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(smem)); \
            allowed_ = (size_t)(smem);                                                             \
        }                                                                                          \
    } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

// Reads element i of a vector whose element type is chosen at run time (norm weights and
// biases keep the type they were stored in).
__device__ __forceinline__ float load_as_float(const void* p, int is_bf16, size_t i) {
    return is_bf16 ? __bfloat162float(reinterpret_cast<const bf16*>(p)[i])
                   : reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a thread block; every thread gets the result. scratch holds 32 floats.
// The order of the additions is fixed by the block size alone.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.f;
    r = warp_sum(r);
    return r;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

// ---- programmatic dependent launch --------------------------------------------------------------------
// A kernel launched with llmp_launch_dependent may start while the kernel before it in the stream still
// runs, once every block of that kernel has called pdl_trigger() or ended. Whatever it reads of that
// kernel's output, and whatever it writes, comes after pdl_wait(), which returns when the kernel before it
// has completed and its writes are visible; before it the kernel only fetches what no kernel of the step
// writes (weights, keys and values of earlier steps). Both calls do nothing in a launch without such a
// dependency.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// False when the environment variable LLMP_B200_PDL is "0": dependent launches then become plain ones.
bool llmp_pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t llmp_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                         Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = llmp_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, KArgs(args)...);
}
