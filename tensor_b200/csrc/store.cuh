// Output stores shared by the CUDA-core convolution kernels: four consecutive output channels of one
// output pixel, after the fused epilogue, in one of the three boundary layouts.
#pragma once

#include "kernels.h"

namespace ottk {

// acc[0..3] are the s32 accumulators of channels c..c+3 (c % 4 == 0) at pixel (img, oy, ox).
__device__ __forceinline__ void epilogue_store4(const int acc[4], int c, int img, int oy, int ox, const ConvShape& s,
                                                const EpilogueParams& ep, void* out, int out_dtype) {
    const long pix = ((long)img * s.oh + oy) * s.ow + ox;
    if (out_dtype == DT_S32_NHWC) {
        int4 v = make_int4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<int4*>(reinterpret_cast<int32_t*>(out) + pix * s.cout_pad + c) = v;
        return;
    }
    const float4 si = __ldg(reinterpret_cast<const float4*>(ep.scale_in + c));
    const float4 bi = __ldg(reinterpret_cast<const float4*>(ep.bias + c));
    const float sia[4] = {si.x, si.y, si.z, si.w};
    const float bia[4] = {bi.x, bi.y, bi.z, bi.w};
    if (out_dtype == DT_S8_NHWC) {
        const float4 so = __ldg(reinterpret_cast<const float4*>(ep.scale_out + c));
        const float soa[4] = {so.x, so.y, so.z, so.w};
        int q[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) q[j] = requant(acc[j], sia[j], bia[j], soa[j], ep);
        *reinterpret_cast<uint32_t*>(reinterpret_cast<int8_t*>(out) + pix * s.cout_pad + c) = pack4(q[0], q[1], q[2], q[3]);
    } else {  // DT_F32_NCHW
        float* o = reinterpret_cast<float*>(out);
        const long plane = (long)s.oh * s.ow;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (c + j < s.cout) o[((long)img * s.cout + c + j) * plane + (long)oy * s.ow + ox] = dequant_act(acc[j], sia[j], bia[j], ep);
    }
}

__device__ __forceinline__ void unpack4(uint32_t wd, int v[4]) {
    v[0] = (int)(int8_t)(wd & 0xff);
    v[1] = (int)(int8_t)((wd >> 8) & 0xff);
    v[2] = (int)(int8_t)((wd >> 16) & 0xff);
    v[3] = (int)(wd) >> 24;
}

}  // namespace ottk
