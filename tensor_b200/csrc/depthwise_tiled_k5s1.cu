// Instantiations of the tiled depthwise kernel for 5x5 filters, stride 1 (see depthwise_tiled.cuh).
#include "depthwise_tiled.cuh"

namespace ottk {

cudaError_t launch_depthwise_tiled_k5s1(cudaStream_t stream, const ConvShape& s, const void* x, const PlaneGather& G, int in_dtype, const uint32_t* wq,
                                        const float* in_scales, int n_in_scales, const EpilogueParams& ep, void* out, int out_dtype) {
    return dwt::launch_ks<5, 1>(stream, s, x, G, in_dtype, wq, in_scales, n_in_scales, ep, out, out_dtype);
}

}  // namespace ottk
