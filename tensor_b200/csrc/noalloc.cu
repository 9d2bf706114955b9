// ott_conv_int8_forward_noalloc: the forward for callers that must not allocate device memory.
//
// The ordinary forward, given fp32 input for a dense layer, takes a scratch block for the quantized
// activations from the context's caching allocator, and the first request of a new size there ends in
// cudaMalloc. Some hosts cannot tolerate that: a serving process whose device memory has been handed out
// up front to fixed pools and which must not grow at run time, or a control loop with a hard latency
// budget in which the implicit device-wide synchronisation of a cudaMalloc/cudaFree is not acceptable.
// For them this file keeps one fixed scratch array in the library's own device image and runs the same
// two kernels (quantize, then convolution) over it. Nothing here calls cudaMalloc, cudaFree or any
// allocating routine.
#include <mutex>

#include "conv_object.h"
#include "ctx.h"
#include "kernels.h"

using namespace ottk;

// The scratch itself: lives in every GPU that loads this library, for the life of the process.
static __device__ __align__(256) unsigned char g_noalloc_scratch[OTT_NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
unsigned char* g_scratch_addr[kMaxDevices] = {};  // device address of g_noalloc_scratch, per device

// In host code the name `g_noalloc_scratch` is only a handle for the runtime, not a device address: the
// address a kernel can use has to be asked for, once per device, with that device current.
int scratch_address(ott_ctx* ctx, unsigned char** out) {
    if (ctx->device < 0 || ctx->device >= kMaxDevices) return ctx->fail(OTT_ERR_INVALID, "device index %d out of range", ctx->device);
    std::lock_guard<std::mutex> g(g_setup_mu);
    if (!g_scratch_addr[ctx->device]) {
        OTT_CUDA_CHECK(ctx, cudaSetDevice(ctx->device));
        void* p = nullptr;
        OTT_CUDA_CHECK(ctx, cudaGetSymbolAddress(&p, g_noalloc_scratch));
        if (!p) return ctx->fail(OTT_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        g_scratch_addr[ctx->device] = static_cast<unsigned char*>(p);
    }
    *out = g_scratch_addr[ctx->device];
    return OTT_OK;
}

}  // namespace

extern "C" int ott_conv_int8_forward_noalloc(ott_ctx* ctx, const ott_conv* conv, const float* in_f32_nchw_dev, int n, int h, int w,
                                             void* out_dev, int out_dtype) {
    if (!ctx || !conv || !in_f32_nchw_dev || !out_dev || n < 0 || h <= 0 || w <= 0) return OTT_ERR_INVALID;
    const size_t need = (size_t)n * h * w * conv->cin_pad;  // int8 NHWC activations, padded channel stride
    if (need > (size_t)OTT_NOALLOC_SCRATCH_BYTES)
        return ctx->fail(OTT_ERR_INVALID,
                         "ott_conv_int8_forward_noalloc: %zu bytes of quantized activations (n=%d h=%d w=%d channel stride %d) exceed the "
                         "fixed scratch of %u bytes; split the batch or use ott_conv_int8_forward",
                         need, n, h, w, conv->cin_pad, (unsigned)OTT_NOALLOC_SCRATCH_BYTES);
    // Everything the convolution stage would refuse is refused here, before the quantize kernel has touched the shared array.
    if (!conv->src_channels.empty())
        return ctx->fail(OTT_ERR_INVALID, "ott_conv_int8_forward_noalloc: a layer created with gathered input reads its producers' int8 tensors, "
                                          "not an fp32 tensor; use ott_conv_int8_forward_io");
    const bool requant = conv->d.int8_scale_term > 100;
    if (out_dtype != OTT_S8_NHWC && out_dtype != OTT_F32_NCHW && out_dtype != OTT_S32_NHWC) return ctx->fail(OTT_ERR_INVALID, "bad output dtype");
    if (out_dtype == OTT_S8_NHWC && !requant) return ctx->fail(OTT_ERR_INVALID, "int8 output needs int8_scale_term > 100");
    if (out_dtype == OTT_F32_NCHW && requant) return ctx->fail(OTT_ERR_INVALID, "fp32 output needs int8_scale_term < 100");
    int oh = 0, ow = 0;
    ott_conv_int8_out_shape(conv, h, w, &oh, &ow);
    if (oh <= 0 || ow <= 0) return ctx->fail(OTT_ERR_INVALID, "empty output");
    if (n == 0) return OTT_OK;
    unsigned char* scratch = nullptr;
    int rc = scratch_address(ctx, &scratch);
    if (rc != OTT_OK) return rc;
    OTT_CUDA_CHECK(ctx, cudaSetDevice(ctx->device));
    // The quantize kernel writes every byte of the [n, h, w, channel stride] block, padding channels included,
    // so nothing left in the array by an earlier call can leak into this one and nothing needs clearing.
    OTT_CUDA_CHECK(ctx, launch_quantize_dense(ctx->stream, in_f32_nchw_dev, conv->d.cin, reinterpret_cast<int8_t*>(scratch), conv->in_scales_dev,
                                                      conv->n_in_scales, n, conv->d.cin, h, w, conv->d.rounding));
    ctx->launches += (uint64_t)((conv->cin_pad + kGatherMaxChannels - 1) / kGatherMaxChannels);  // one launch per 512-channel slice
    // int8 input: this path of the ordinary forward launches the convolution kernel and takes no scratch
    return ott_conv_int8_forward(ctx, conv, scratch, OTT_S8_NHWC, n, h, w, out_dev, out_dtype, nullptr);
}
