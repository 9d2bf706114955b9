// Host side of the tiled depthwise kernel: shape gate, filter packing, dispatch on (kernel size, stride).
#include "depthwise_tiled.cuh"

namespace ottk {

bool depthwise_tiled_supports(const ConvShape& s, int out_dtype) {
    const bool plain = s.dh == 1 && s.dw == 1 && s.kh == s.kw && s.sh == s.sw && (s.kh == 3 || s.kh == 5) && (s.sh == 1 || s.sh == 2);
    return plain && (out_dtype == DT_S8_NHWC || out_dtype == DT_F32_NCHW);
}

int depthwise_tiled_weight_words(int k) { return k * ((k + 3) / 4); }

void depthwise_tiled_pack_weights(const int8_t* w_oihw, int c, int c_pad, int k, uint32_t* dst) {
    // dst[c_pad][k rows][KK words]: byte j of word kk = tap kx = 4*kk + j of that filter row (0 beyond k)
    const int kk_n = (k + 3) / 4;
    for (long i = 0; i < (long)c_pad * k * kk_n; ++i) dst[i] = 0;
    for (int ch = 0; ch < c; ++ch)
        for (int ky = 0; ky < k; ++ky)
            for (int kx = 0; kx < k; ++kx) {
                const uint32_t byte = (uint8_t)w_oihw[((long)ch * k + ky) * k + kx];
                dst[((long)ch * k + ky) * kk_n + kx / 4] |= byte << (8 * (kx % 4));
            }
}

cudaError_t launch_depthwise_tiled(cudaStream_t stream, const ConvShape& s, const void* x, const PlaneGather* gather, int in_dtype, const uint32_t* wq,
                                   const float* in_scales, int n_in_scales, const EpilogueParams& ep, void* out, int out_dtype) {
    static const PlaneGather none{};
    PlaneGather ident;
    const PlaneGather* G = gather;
    if (!G) {
        if (in_dtype == DT_F32_NCHW) {
            if (s.cin > kGatherMaxChannels) return cudaErrorInvalidValue;
            gather_identity(&ident, static_cast<const float*>(x), s.cin, s.cin, (long)s.h * s.w);
            G = &ident;
        } else {
            G = &none;
        }
    }
    if (s.kh == 3 && s.sh == 1) return launch_depthwise_tiled_k3s1(stream, s, x, *G, in_dtype, wq, in_scales, n_in_scales, ep, out, out_dtype);
    if (s.kh == 3 && s.sh == 2) return launch_depthwise_tiled_k3s2(stream, s, x, *G, in_dtype, wq, in_scales, n_in_scales, ep, out, out_dtype);
    if (s.kh == 5 && s.sh == 1) return launch_depthwise_tiled_k5s1(stream, s, x, *G, in_dtype, wq, in_scales, n_in_scales, ep, out, out_dtype);
    if (s.kh == 5 && s.sh == 2) return launch_depthwise_tiled_k5s2(stream, s, x, *G, in_dtype, wq, in_scales, n_in_scales, ep, out, out_dtype);
    return cudaErrorInvalidValue;
}

}  // namespace ottk
