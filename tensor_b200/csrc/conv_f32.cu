// The fp32 half of ConvolutionLayer (int8_scale_term == 0; Tensor/ConvolutionLayer.cpp:507-664), for the layers a "mixed"
// quantized model keeps in floating point (its first convolution: benchmark/nanodet-plus-m-1.5x_416_int8_mixed.otter:26).
// Direct convolution on fp32 NCHW tensors, dense (groups == 1) or depthwise, any kernel size / stride / padding / dilation,
// bias and activation fused:
//   y[n,o,y,x] = act(bias[o] + sum_{c,ky,kx} w[o,c,ky,kx] * x[n, c, y*s-p+ky*d, x*s-p+kx*d])
// The sum starts from the bias and runs over c, ky, kx in that order with one fused multiply-add per term. The reference
// computes the same sum with its build's own vector order and -ffast-math contractions, so the two agree to rounding, not to
// the bit: the tests bound the difference by a few units in the last place of sum |w*x| + |bias|.
// One thread = one output pixel x 8 output channels; lanes run along output pixels, so loads along a row and the NCHW stores
// are coalesced and the weight reads are warp-uniform.
#include "kernels.h"

namespace ottk {

namespace {
constexpr int F32_CO = 8;

template <int ACT>
__global__ void __launch_bounds__(128)
conv_f32_kernel(const float* __restrict__ x, const float* __restrict__ wt, const float* __restrict__ bias, float* __restrict__ out, ConvShape s,
                int depthwise, float act_p0, long pixels) {
    const long pix = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int co0 = blockIdx.y * F32_CO;
    if (pix >= pixels) return;
    const int ox = (int)(pix % s.ow);
    const long rest = pix / s.ow;
    const int oy = (int)(rest % s.oh);
    const int img = (int)(rest / s.oh);
    float acc[F32_CO];
#pragma unroll
    for (int j = 0; j < F32_CO; ++j) acc[j] = __ldg(bias + co0 + j);
    const long plane = (long)s.h * s.w;
    const int taps = s.kh * s.kw;
    if (depthwise) {
        // channel o reads channel o: wt is [tap][cout_pad]
        for (int ky = 0; ky < s.kh; ++ky) {
            const int iy = oy * s.sh - s.ph + ky * s.dh;
            if (iy < 0 || iy >= s.h) continue;
            for (int kx = 0; kx < s.kw; ++kx) {
                const int ix = ox * s.sw - s.pw + kx * s.dw;
                if (ix < 0 || ix >= s.w) continue;
                const float* wp = wt + (long)(ky * s.kw + kx) * s.cout_pad + co0;
#pragma unroll
                for (int j = 0; j < F32_CO; ++j)
                    if (co0 + j < s.cout)
                        acc[j] = __fmaf_rn(__ldg(wp + j), __ldg(x + ((long)img * s.cin + co0 + j) * plane + (long)iy * s.w + ix), acc[j]);
            }
        }
    } else {
        // wt is [cin][tap][cout_pad]: the 8 weights of a term are one 32-byte warp-uniform read
        const float* ximg = x + (long)img * s.cin * plane;
        for (int c = 0; c < s.cin; ++c) {
            for (int ky = 0; ky < s.kh; ++ky) {
                const int iy = oy * s.sh - s.ph + ky * s.dh;
                if (iy < 0 || iy >= s.h) continue;
                for (int kx = 0; kx < s.kw; ++kx) {
                    const int ix = ox * s.sw - s.pw + kx * s.dw;
                    if (ix < 0 || ix >= s.w) continue;
                    const float xv = __ldg(ximg + c * plane + (long)iy * s.w + ix);
                    const float4* wp = reinterpret_cast<const float4*>(wt + ((long)c * taps + ky * s.kw + kx) * s.cout_pad + co0);
                    const float4 w0 = __ldg(wp), w1 = __ldg(wp + 1);
                    acc[0] = __fmaf_rn(w0.x, xv, acc[0]); acc[1] = __fmaf_rn(w0.y, xv, acc[1]);
                    acc[2] = __fmaf_rn(w0.z, xv, acc[2]); acc[3] = __fmaf_rn(w0.w, xv, acc[3]);
                    acc[4] = __fmaf_rn(w1.x, xv, acc[4]); acc[5] = __fmaf_rn(w1.y, xv, acc[5]);
                    acc[6] = __fmaf_rn(w1.z, xv, acc[6]); acc[7] = __fmaf_rn(w1.w, xv, acc[7]);
                }
            }
        }
    }
    const long oplane = (long)s.oh * s.ow;
    float* o = out + ((long)img * s.cout + co0) * oplane + (long)oy * s.ow + ox;
#pragma unroll
    for (int j = 0; j < F32_CO; ++j)
        if (co0 + j < s.cout) o[j * oplane] = activate_t<ACT>(acc[j], act_p0);
}
}  // namespace

int conv_f32_channel_stride(int cout) { return (cout + F32_CO - 1) / F32_CO * F32_CO; }

void conv_f32_pack_weights(const float* w_oihw, int cin_per_group, int cout, int taps, bool depthwise, float* dst) {
    const int cp = conv_f32_channel_stride(cout);
    const long total = (long)(depthwise ? 1 : cin_per_group) * taps * cp;
    for (long i = 0; i < total; ++i) dst[i] = 0.f;
    for (int o = 0; o < cout; ++o)
        for (int c = 0; c < cin_per_group; ++c)
            for (int t = 0; t < taps; ++t) dst[((long)c * taps + t) * cp + o] = w_oihw[((long)o * cin_per_group + c) * taps + t];
}

cudaError_t launch_conv_f32(cudaStream_t stream, const ConvShape& s, int depthwise, const float* x, const float* w_packed, const float* bias_padded,
                            int act_type, float act_param0, float* out) {
    const long pixels = (long)s.n * s.oh * s.ow;
    if (pixels == 0) return cudaSuccess;
    ConvShape sp = s;
    sp.cout_pad = conv_f32_channel_stride(s.cout);
    dim3 grid((unsigned)((pixels + 127) / 128), (unsigned)(sp.cout_pad / F32_CO));
    switch (act_type) {
        case ACT_RELU: conv_f32_kernel<ACT_RELU><<<grid, 128, 0, stream>>>(x, w_packed, bias_padded, out, sp, depthwise, act_param0, pixels); break;
        case ACT_LRELU: conv_f32_kernel<ACT_LRELU><<<grid, 128, 0, stream>>>(x, w_packed, bias_padded, out, sp, depthwise, act_param0, pixels); break;
        case ACT_RELU6: conv_f32_kernel<ACT_RELU6><<<grid, 128, 0, stream>>>(x, w_packed, bias_padded, out, sp, depthwise, act_param0, pixels); break;
        default: conv_f32_kernel<ACT_NONE><<<grid, 128, 0, stream>>>(x, w_packed, bias_padded, out, sp, depthwise, act_param0, pixels); break;
    }
    return cudaGetLastError();
}

}  // namespace ottk
