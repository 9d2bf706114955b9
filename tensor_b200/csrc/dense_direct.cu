// Direct dense int8 convolution on CUDA cores (dp4a), NHWC activations.
//
// Serves the dense shapes the tensor-core kernel does not take: very few input channels (the 3->24
// stem: conv2d_3x3s2_int8_pack1to4, Tensor/ConvolutionMM2DInt8X86Pack.cpp:2569-2651), strided or dilated
// dense convolutions (Tensor/ConvolutionMM2D.cpp:553-649 is the plain statement of the sum).
// acc[o,y,x] = sum_{c,ky,kx} w[o,c,ky,kx] * x[c, y*s-p+ky*d, x*s-p+kx*d], exact s32, zero padding.
// One thread = one output pixel x 4 output channels; lanes run along output pixels so the weight words
// are warp-uniform and fp32 NCHW stores are coalesced.
#include "store.cuh"

namespace ottk {

__global__ void __launch_bounds__(128)
dense_direct_kernel(const int8_t* __restrict__ x, const int8_t* __restrict__ wt, EpilogueParams ep,
                    void* __restrict__ out, int out_dtype, ConvShape s, long pixels) {
    const long pix = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int co = blockIdx.y * 4;
    if (pix >= pixels) return;
    const int ox = (int)(pix % s.ow);
    long rest = pix / s.ow;
    const int oy = (int)(rest % s.oh);
    const int img = (int)(rest / s.oh);
    int acc[4] = {0, 0, 0, 0};
    const int cw = s.cin_pad / 16;
    const int taps = s.kh * s.kw;
    const int8_t* ximg = x + (long)img * s.h * s.w * s.cin_pad;
    for (int ky = 0; ky < s.kh; ++ky) {
        const int iy = oy * s.sh - s.ph + ky * s.dh;
        if (iy < 0 || iy >= s.h) continue;
        for (int kx = 0; kx < s.kw; ++kx) {
            const int ix = ox * s.sw - s.pw + kx * s.dw;
            if (ix < 0 || ix >= s.w) continue;
            const uint4* xp = reinterpret_cast<const uint4*>(ximg + ((long)iy * s.w + ix) * s.cin_pad);
            const int tap = ky * s.kw + kx;
            for (int i = 0; i < cw; ++i) {
                const uint4 xv = __ldg(xp + i);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wt + ((long)(co + j) * taps + tap) * s.cin_pad) + i);
                    acc[j] = __dp4a((int)xv.x, (int)wv.x, acc[j]);
                    acc[j] = __dp4a((int)xv.y, (int)wv.y, acc[j]);
                    acc[j] = __dp4a((int)xv.z, (int)wv.z, acc[j]);
                    acc[j] = __dp4a((int)xv.w, (int)wv.w, acc[j]);
                }
            }
        }
    }
    epilogue_store4(acc, co, img, oy, ox, s, ep, out, out_dtype);
}

cudaError_t launch_dense_direct(cudaStream_t stream, const ConvShape& s, const int8_t* x, const int8_t* w_okc,
                                const EpilogueParams& ep, void* out, int out_dtype) {
    const long pixels = (long)s.n * s.oh * s.ow;
    if (pixels == 0) return cudaSuccess;
    dim3 grid((unsigned)((pixels + 127) / 128), (unsigned)(s.cout_pad / 4));
    dense_direct_kernel<<<grid, 128, 0, stream>>>(x, w_okc, ep, out, out_dtype, s, pixels);
    return cudaGetLastError();
}

}  // namespace ottk
