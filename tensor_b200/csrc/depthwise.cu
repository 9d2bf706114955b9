// Depthwise int8 convolution on CUDA cores: depthwise_conv2d_int8_x86_pack8_out
// (Tensor/DepthwiseConvKernelInt8X86Pack.cpp:19-119) + the fused epilogue
// (Tensor/QuantizeX86.cpp:1723-1870 / :851-903), on NHWC int8 activations.
//
// acc[c,y,x] = sum_k w[c,k] * x[c, y*s - p + ky*d, x*s - p + kx*d], exact s32; zero padding.
// HBM-bound by design: each thread owns 4 channels (one 32-bit word) of a short strip of output pixels,
// so a warp reads 128 contiguous bytes per input pixel; input rows are reused from L1/L2.
#include "store.cuh"

namespace ottk {

template <int K, int S, int XT>
__global__ void __launch_bounds__(256)
depthwise_kernel(const int8_t* __restrict__ x, const int8_t* __restrict__ wt, EpilogueParams ep, void* __restrict__ out,
                 int out_dtype, ConvShape s, int cquads, int strips, long total) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int cq = (int)(idx % cquads);
    long rest = idx / cquads;
    const int xs = (int)(rest % strips);
    rest /= strips;
    const int oy = (int)(rest % s.oh);
    const int img = (int)(rest / s.oh);
    const int c = cq * 4;
    const int ox0 = xs * XT;
    constexpr int NC = (XT - 1) * S + K;

    int acc[XT][4];
#pragma unroll
    for (int t = 0; t < XT; ++t)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[t][j] = 0;

    const int8_t* ximg = x + (long)img * s.h * s.w * s.cin_pad + c;
#pragma unroll
    for (int ky = 0; ky < K; ++ky) {
        const int iy = oy * S - s.ph + ky;
        if (iy < 0 || iy >= s.h) continue;
        const int8_t* xrow = ximg + (long)iy * s.w * s.cin_pad;
        int v[NC][4];
#pragma unroll
        for (int col = 0; col < NC; ++col) {
            const int ix = ox0 * S - s.pw + col;
            uint32_t wd = 0;
            if (ix >= 0 && ix < s.w) wd = __ldg(reinterpret_cast<const uint32_t*>(xrow + (long)ix * s.cin_pad));
            unpack4(wd, v[col]);
        }
#pragma unroll
        for (int kx = 0; kx < K; ++kx) {
            int w4[4];
            unpack4(__ldg(reinterpret_cast<const uint32_t*>(wt + (long)(ky * K + kx) * s.cin_pad + c)), w4);
#pragma unroll
            for (int t = 0; t < XT; ++t)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[t][j] += v[t * S + kx][j] * w4[j];
        }
    }
#pragma unroll
    for (int t = 0; t < XT; ++t) {
        const int ox = ox0 + t;
        if (ox < s.ow) epilogue_store4(acc[t], c, img, oy, ox, s, ep, out, out_dtype);
    }
}

// Any kernel size, stride and dilation; one output pixel x 4 channels per thread.
__global__ void __launch_bounds__(256)
depthwise_generic_kernel(const int8_t* __restrict__ x, const int8_t* __restrict__ wt, EpilogueParams ep,
                         void* __restrict__ out, int out_dtype, ConvShape s, int cquads, long total) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int cq = (int)(idx % cquads);
    long rest = idx / cquads;
    const int ox = (int)(rest % s.ow);
    rest /= s.ow;
    const int oy = (int)(rest % s.oh);
    const int img = (int)(rest / s.oh);
    const int c = cq * 4;
    int acc[4] = {0, 0, 0, 0};
    const int8_t* ximg = x + (long)img * s.h * s.w * s.cin_pad + c;
    for (int ky = 0; ky < s.kh; ++ky) {
        const int iy = oy * s.sh - s.ph + ky * s.dh;
        if (iy < 0 || iy >= s.h) continue;
        for (int kx = 0; kx < s.kw; ++kx) {
            const int ix = ox * s.sw - s.pw + kx * s.dw;
            if (ix < 0 || ix >= s.w) continue;
            int v[4], w4[4];
            unpack4(__ldg(reinterpret_cast<const uint32_t*>(ximg + ((long)iy * s.w + ix) * s.cin_pad)), v);
            unpack4(__ldg(reinterpret_cast<const uint32_t*>(wt + (long)(ky * s.kw + kx) * s.cin_pad + c)), w4);
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] += v[j] * w4[j];
        }
    }
    epilogue_store4(acc, c, img, oy, ox, s, ep, out, out_dtype);
}

template <int K, int S, int XT>
static cudaError_t launch_dw_t(cudaStream_t stream, const ConvShape& s, const int8_t* x, const int8_t* wt,
                               const EpilogueParams& ep, void* out, int out_dtype) {
    const int cquads = s.cout_pad / 4;
    const int strips = (s.ow + XT - 1) / XT;
    const long total = (long)s.n * s.oh * strips * cquads;
    if (total == 0) return cudaSuccess;
    const long blocks = (total + 255) / 256;
    depthwise_kernel<K, S, XT><<<(unsigned)blocks, 256, 0, stream>>>(x, wt, ep, out, out_dtype, s, cquads, strips, total);
    return cudaGetLastError();
}

cudaError_t launch_depthwise(cudaStream_t stream, const ConvShape& s, const int8_t* x, const int8_t* w_taps,
                             const EpilogueParams& ep, void* out, int out_dtype) {
    const bool plain = s.dh == 1 && s.dw == 1 && s.kh == s.kw && s.sh == s.sw;
    if (plain && s.kh == 3 && s.sh == 1) return launch_dw_t<3, 1, 4>(stream, s, x, w_taps, ep, out, out_dtype);
    if (plain && s.kh == 3 && s.sh == 2) return launch_dw_t<3, 2, 2>(stream, s, x, w_taps, ep, out, out_dtype);
    if (plain && s.kh == 5 && s.sh == 1) return launch_dw_t<5, 1, 4>(stream, s, x, w_taps, ep, out, out_dtype);
    if (plain && s.kh == 5 && s.sh == 2) return launch_dw_t<5, 2, 2>(stream, s, x, w_taps, ep, out, out_dtype);
    const int cquads = s.cout_pad / 4;
    const long total = (long)s.n * s.oh * s.ow * cquads;
    if (total == 0) return cudaSuccess;
    depthwise_generic_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(x, w_taps, ep, out, out_dtype, s, cquads, total);
    return cudaGetLastError();
}

}  // namespace ottk
