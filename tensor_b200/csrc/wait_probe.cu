// A kernel whose only job is to let a bounded wait run out (see launch_wait_probe in kernels.h): the way the host learns
// of a kernel that gave up (status word -> OTT_ERR_DEVICE_WAIT at the next ott_sync, word cleared) can then be tested without
// faulting, trapping or hanging anything.
#include "kernels.h"
#include "umma_primitives.cuh"

namespace ottk {

namespace {
__global__ void wait_probe_kernel(uint32_t* status, unsigned long long limit_ns) {
    __shared__ alignas(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        umma::mbar_init(umma::smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // phase 0 of a freshly initialised barrier with one pending arrival never completes: nobody arrives
    if (threadIdx.x == 0) (void)umma::mbar_wait(umma::smem_u32(&bar), 0, &abort_flag, status, 0x100u, limit_ns);
    __syncthreads();
}
}  // namespace

cudaError_t launch_wait_probe(cudaStream_t stream, uint32_t* status, unsigned long long limit_ns) {
    wait_probe_kernel<<<1, 32, 0, stream>>>(status, limit_ns);
    return cudaGetLastError();
}

}  // namespace ottk
