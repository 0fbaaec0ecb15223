// A self-check of the bounded waits: one thread waits on a barrier that nothing will ever complete, with a small
// limit, through the same wait that every TMA and tcgen05 kernel of this library uses. The wait gives up, sets the
// error word that the host reads after its next synchronisation, and the kernel returns normally: nothing faults or
// hangs, and the next launch works. The engine never calls this; tests do, to see the whole path from a wait that ran
// out to the exception on the host.
#include "tcgen05.cuh"

__global__ void bounded_wait_check_kernel(int* error_flag, uint32_t limit, int* gave_up) {
    __shared__ __align__(8) uint64_t barrier;
    if (threadIdx.x == 0) {
        mbar_init(&barrier, 1);                                  // one arrival expected; nobody arrives
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        const bool completed = mbar_wait_limited(&barrier, 0, error_flag, limit);
        *gave_up = completed ? 0 : 1;
    }
}

// error_flag: the int32 in mapped host memory that the kernels' waits report to; limit: tries before the wait gives
// up (1 to 65,536); gave_up: one int32 on the device, set to 1 when the wait returned without completion.
LLMP_API int llmp_bounded_wait_check(int* error_flag, int limit, int* gave_up, cudaStream_t stream) {
    LLMP_REQUIRE(error_flag != nullptr && gave_up != nullptr, "bounded_wait_check needs the error word and an output");
    LLMP_REQUIRE(limit >= 1 && limit <= 65536, "bounded_wait_check takes a limit of 1 to 65,536 tries, got %d", limit);
    bounded_wait_check_kernel<<<1, 32, 0, stream>>>(error_flag, (uint32_t)limit, gave_up);
    return llmp_check_launch("bounded_wait_check");
}
