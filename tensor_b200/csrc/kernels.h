// Launchers of the CUDA kernels, as seen by the host-side C-ABI (c_api.cu). Device pointers only.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "epilogue.cuh"

namespace ottk {

// channel stride of the NHWC layouts: a multiple of 16 bytes so that one pixel row can be a TMA box row
__host__ __device__ inline int nhwc_channels(int c) { return (c + 15) & ~15; }

enum : int { DT_F32_NCHW = 0, DT_S8_NHWC = 1, DT_S32_NHWC = 2 };

// Shape of one convolution call (all kernels).
struct ConvShape {
    int n, h, w, oh, ow;
    int cin, cout, cin_pad, cout_pad;  // *_pad = NHWC channel strides
    int kh, kw, sh, sw, ph, pw, dh, dw;
};

// Where the channel planes of an fp32 NCHW input live. The reference's Concat / Crop / ChannelShuffle only re-order or
// select channel planes (Tensor/ConcatLayer.cpp:55-70, Tensor/CropLayer.cpp:67-75, Tensor/ChannelShuffleLayer.cpp:37-41), so
// instead of copying planes around, a consumer kernel is told, per logical input channel, which buffer and which plane of
// that buffer to read. Passed by value in the kernel parameter bank.
constexpr int kGatherMaxBufs = 12, kGatherMaxChannels = 512;
struct PlaneGather {
    const float* base[kGatherMaxBufs];
    long long img_stride[kGatherMaxBufs];  // elements between consecutive images of that buffer
    uint32_t ref[kGatherMaxChannels];      // logical channel -> (buffer << 24) | plane index inside the buffer
    __host__ __device__ const float* plane(int c, int img, long hw) const {
        const uint32_t r = ref[c];
        const int b = (int)(r >> 24);
        return base[b] + (long long)img * img_stride[b] + (long long)(r & 0xFFFFFFu) * hw;
    }
};
// the table of a plain tensor: one buffer of c_total channels per image, logical channel i = plane c0 + i
void gather_identity(PlaneGather* g, const float* x, int c, int c_total, long hw);

cudaError_t launch_quantize_nchw_to_nhwc(cudaStream_t stream, const PlaneGather& src, int8_t* out, const float* scales_dev,
                                         int n_scales, int n, int c, int h, int w, int rounding);

// the same for a plain tensor (c of c_total channels per image, any channel count)
cudaError_t launch_quantize_dense(cudaStream_t stream, const float* x, int c_total, int8_t* out, const float* scales_dev, int n_scales,
                                  int n, int c, int h, int w, int rounding);

// dense fp32 NCHW copy of the gathered planes (for consumers that want one contiguous tensor)
cudaError_t launch_gather_planes(cudaStream_t stream, const PlaneGather& src, float* dst, int n, int c, long hw);

// dst = a + b, fp32 NCHW, both operands read through plane tables
cudaError_t launch_add_planes(cudaStream_t stream, const PlaneGather& a, const PlaneGather& b, float* dst, int n, int c, long hw);

// Depthwise: x int8 NHWC [n,h,w,c_pad]; weights int8 [kh*kw][c_pad] (tap-major, channel innermost).
cudaError_t launch_depthwise(cudaStream_t stream, const ConvShape& s, const int8_t* x, const int8_t* w_taps,
                             const EpilogueParams& ep, void* out, int out_dtype);

// Shared-memory tiled depthwise (3x3 / 5x5, stride 1 / 2, no dilation) with the quantize prologue fused:
// x is fp32 NCHW (in_dtype DT_F32_NCHW) or int8 NHWC; weights packed by depthwise_tiled_pack_weights.
bool depthwise_tiled_supports(const ConvShape& s, int out_dtype);
int depthwise_tiled_weight_words(int k);  // 32-bit words per channel
void depthwise_tiled_pack_weights(const int8_t* w_oihw, int c, int c_pad, int k, uint32_t* dst);
cudaError_t launch_depthwise_tiled(cudaStream_t stream, const ConvShape& s, const void* x, const PlaneGather* gather, int in_dtype, const uint32_t* wq,
                                   const float* in_scales, int n_in_scales, const EpilogueParams& ep, void* out, int out_dtype);

// Direct dense convolution on CUDA cores: x int8 NHWC; weights int8 [cout_pad][kh*kw][cin_pad].
cudaError_t launch_dense_direct(cudaStream_t stream, const ConvShape& s, const int8_t* x, const int8_t* w_okc,
                                const EpilogueParams& ep, void* out, int out_dtype);

// First-layer kernel: 3 input channels, 3x3, stride 1/2, fp32 NCHW in (quantize fused), fp32 NCHW or int8 NHWC out.
// Filters (OIHW int8) and per-channel epilogue vectors are HOST pointers: they travel in the kernel parameter bank.
bool dense_stem_supports(const ConvShape& s, int in_dtype, int out_dtype);
cudaError_t launch_dense_stem(cudaStream_t stream, const ConvShape& s, const float* x, const int8_t* w_oihw_host, const float* scale_in_host,
                              const float* bias_host, const float* scale_out_host, float in_scale, const EpilogueParams& ep, void* out,
                              int out_dtype);

// The first layer (fp32 output) and the 3x3 stride-2 pad-1 max-pool that consumes it, in one kernel; out is the pooled
// fp32 NCHW tensor [n][cout][(oh-1)/2+1][(ow-1)/2+1], or (out_dtype DT_S8_NHWC) the same values quantized with scale_out_host per
// channel as an int8 NHWC tensor. Runs on the tensor cores; status: the word a timed-out wait is reported in.
cudaError_t launch_dense_stem_pool(cudaStream_t stream, const ConvShape& s, const float* x, const int8_t* w_oihw_host, const float* scale_in_host,
                                   const float* bias_host, const float* scale_out_host, float in_scale, const EpilogueParams& ep, void* out,
                                   int out_dtype, int pad_zero, uint32_t* status);

// fp32 convolution (the layers a mixed model keeps in floating point): x, out fp32 NCHW; weights packed by
// conv_f32_pack_weights into [cin/groups][tap][conv_f32_channel_stride(cout)] (depthwise: [tap][stride]); bias padded to the same stride.
int conv_f32_channel_stride(int cout);
void conv_f32_pack_weights(const float* w_oihw, int cin_per_group, int cout, int taps, bool depthwise, float* dst);
cudaError_t launch_conv_f32(cudaStream_t stream, const ConvShape& s, int depthwise, const float* x, const float* w_packed, const float* bias_padded,
                            int act_type, float act_param0, float* out);

// Test support for the bounded waits: one CTA waits on an mbarrier that nothing ever completes, with the given limit, and
// reports the expiry in *status exactly as the tensor-core kernels do (code 0x100). It loads nothing, issues no MMA and
// owns no TMEM, so giving up leaves nothing in flight.
cudaError_t launch_wait_probe(cudaStream_t stream, uint32_t* status, unsigned long long limit_ns);

}  // namespace ottk
