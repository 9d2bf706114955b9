// Programmatic dependent launch: a kernel launched through launch_overlapped may begin (barrier set-up, TMEM allocation,
// loads of constant data such as weights) while the previous kernel on the stream is still draining its last wave; it must
// execute pdl_wait() before it reads anything an earlier kernel wrote or writes anything an earlier kernel may still read.
// pdl_launch_dependents() tells the hardware that the next kernel may be scheduled as soon as there is room for it. Both
// instructions do nothing in a kernel that was launched the ordinary way or has no predecessor.
#pragma once

#include <cuda_runtime.h>

#include <utility>

namespace ottk {

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace ottk
