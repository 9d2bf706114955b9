/* otter_b200 — C-ABI of the B200 (sm_100a) int8 convolution path for Otter/Tensor.
 *
 * This is the whole boundary between host code (the C++17 Net / Layer / ConvolutionLayer mirror in
 * tensor_b200/host, a test, a benchmark, or the reference itself through a thin stub) and the CUDA
 * kernels. Plain pointers and sizes only. Every function returns an int status: 0 = success
 * (the reference's convention, Tensor/Layer.hpp:44), negative = failure; nothing throws or aborts.
 * There is no CPU path behind any entry point: without a CUDA device every compute call fails.
 *
 * Layouts
 *   OTT_F32_NCHW  fp32, the reference's boundary layout (Tensor/TensorPacking.cpp:126-139 elempack 1).
 *   OTT_S8_NHWC   int8, channels innermost, channel stride padded to ott_nhwc_channels(c)
 *                 (a multiple of 16 so a pixel row can be a TMA box row). Padding channels hold 0.
 *                 This replaces the reference's int8 elempack-8 blobs (Byte8) that flow between a
 *                 requantizing convolution and its consumer (Tensor/ConvolutionLayer.cpp:770-775).
 *   OTT_S32_NHWC  the exact s32 accumulators, same padding rule; for tests of the integer part alone.
 */
#ifndef OTTER_B200_H
#define OTTER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library is built with -fvisibility=hidden; these are its exports */
#endif

#define OTT_OK 0
#define OTT_ERR_UNSUPPORTED (-1) /* Layer.cpp:50-59 uses -1 for "not implemented" */
#define OTT_ERR_INVALID (-2)     /* bad argument */
#define OTT_ERR_CUDA (-3)        /* a CUDA runtime/driver call failed; see ott_last_error */
#define OTT_ERR_DEVICE_WAIT (-4) /* a kernel gave up a bounded wait and reported it in its status word */
#define OTT_ERR_ALLOC (-100)     /* Layer.cpp:50-59 uses -100 for allocation failure */

typedef struct ott_ctx ott_ctx;   /* one per GPU: device, stream, caching allocator */
typedef struct ott_conv ott_conv; /* one quantized ConvolutionLayer's device-side state */
typedef struct ott_event ott_event;

enum ott_dtype { OTT_F32_NCHW = 0, OTT_S8_NHWC = 1, OTT_S32_NHWC = 2 };

/* int8 rounding rule of the epilogue and of the fused quantization.
 * OTT_ROUND_ADD_HALF_TRUNC = float2int8_sse (Tensor/VecIntrinsic.hpp:71-161), the reference's default
 * packed path; OTT_ROUND_HALF_AWAY = scalar float2int8 (Tensor/QuantizeX86.cpp:18-23) of its unpacked
 * path and aarch64 (Tensor/QuantizeNeon.hpp:27-29). */
enum ott_rounding { OTT_ROUND_ADD_HALF_TRUNC = 0, OTT_ROUND_HALF_AWAY = 1 };

/* Which kernel family serves a layer; chosen at create time from the shape, reported for tests. */
enum ott_kernel_kind {
    OTT_KERNEL_DEPTHWISE = 1,   /* CUDA-core depthwise */
    OTT_KERNEL_DENSE_UMMA = 2,  /* tcgen05 implicit GEMM */
    OTT_KERNEL_DENSE_DIRECT = 3 /* CUDA-core direct convolution (few input channels, strided/dilated dense) */
};

/* The options of a quantized ConvolutionLayer (Tensor/ConvolutionLayer.hpp:41-62, option keys parsed at
 * Tensor/ConvolutionLayer.cpp:58-156). act_type: 0 none, 1 ReLU, 2 LeakyReLU(act_param0), 3 ReLU6.
 * int8_scale_term 1/2: fp32 output; 101/102: int8 output (ConvolutionLayer.cpp:834-844). */
typedef struct {
    int cin, cout, kh, kw, sh, sw, ph, pw, dh, dw, groups;
    int bias_term;
    int int8_scale_term;
    int act_type;
    float act_param0;
    int rounding; /* enum ott_rounding */
} ott_conv_desc;

/* ---- device context: replaces otter::GetAllocator(Device) + the implicit single CPU "stream"
 *      (Tensor/Allocator.hpp:125-144, Tensor/CPUCachingAllocator.hpp:18-72) ---- */
int ott_cuda_device_count(int* n);
int ott_ctx_create(int device, ott_ctx** out);
int ott_ctx_destroy(ott_ctx* ctx);
const char* ott_last_error(const ott_ctx* ctx); /* never NULL; valid until the next failing call on ctx */
void* ott_ctx_stream(ott_ctx* ctx);             /* the cudaStream_t every call on ctx is ordered on */
int ott_sync(ott_ctx* ctx);

/* Failure detection (no counterpart in the reference, whose CPU kernels cannot wait on anything). Every wait inside a kernel
 * (on an mbarrier that a TMA copy or an MMA completes) is bounded: when the limit passes the kernel gives up, frees what it
 * holds, and ORs a code into the context's status word; the next ott_sync (or *_host call) then returns OTT_ERR_DEVICE_WAIT,
 * names the word in ott_last_error, and clears it, and the context stays usable. The limit is 2000 ms per wait unless changed
 * here (calls enqueued afterwards use the new value). */
int ott_set_wait_limit_ms(ott_ctx* ctx, int ms);
/* Depthwise 3x3 layers (stride 1 / 2, pad 1) whose input is int8 NHWC can run on the tensor cores (each filter tap one
 * tcgen05.mma against a diagonal weight matrix, so the channel-innermost layout needs no byte transposes). mode 1 (default):
 * where that is faster (layers of at most 64 channels, and wider layers on input maps of 2048 pixels or more: every tap
 * costs one 128-row MMA per 32 channels, which small wide layers lose against the CUDA-core kernel); 0: none; 2: every layer
 * the kernel supports. Same bits in every mode. */
int ott_set_depthwise_tensor_cores(ott_ctx* ctx, int mode);
/* Test hooks for the failure paths; neither touches a GPU in a way that can fault it.
 * ott_debug_wait_probe enqueues a one-CTA kernel whose only wait can never complete (nobody arrives on its barrier), so
 * it runs out after the context's wait limit and reports through the status word like the real kernels.
 * ott_debug_fail_alloc_after makes the n-th allocation of the context's allocator from now on fail on the host
 * (cudaErrorMemoryAllocation without calling cudaMalloc); n <= 0 switches the injection off. */
int ott_debug_wait_probe(ott_ctx* ctx);
int ott_debug_fail_alloc_after(ott_ctx* ctx, int n);
/* Guard bands, the tests' stand-in for a device memory checker: after ott_debug_guard_bands(ctx, bytes) every block the
 * context's allocator obtains from the driver carries `bytes` (rounded up to 512) of a fill pattern on both sides;
 * ott_debug_check_guards synchronizes the stream, reads every band of every block (in use or cached) back and returns
 * OTT_ERR_CUDA with *bad_blocks > 0 if a kernel wrote outside a block. Call the first before anything is allocated; the
 * environment variable OTT_DEBUG_GUARD_BYTES=<bytes> does the same for every context created afterwards (the GPU tests set it). */
int ott_debug_guard_bands(ott_ctx* ctx, size_t bytes);
int ott_debug_check_guards(ott_ctx* ctx, long* bad_blocks);
/* Measurement hook: cycles one tcgen05.mma kind::i8 (M = 128, K = 32, N = n_cols) occupies an SM when issuing_warps x
 * issuing_lanes threads of each of ctas_per_sm CTAs per SM issue `reps` of them back to back (zero operands; the design notes
 * argue tile shapes from these numbers: 128 / 64 / 48 / 40 cycles at N = 256 / 128 / 64 / 32, one issuing thread alone 56). */
int ott_debug_mma_rate(ott_ctx* ctx, int n_cols, int issuing_warps, int issuing_lanes, int ctas_per_sm, int reps, float* cycles_per_mma);

/* Stream-ordered, size-keyed caching allocator: a freed block is handed back to the next request of the
 * same rounded size without touching cudaMalloc (the policy of CPUCachingAllocator::allocate/free,
 * Tensor/CPUCachingAllocator.hpp:62-70, moved to device memory). */
int ott_malloc(ott_ctx* ctx, size_t bytes, void** out);
int ott_free(ott_ctx* ctx, void* p);
int ott_alloc_stats(ott_ctx* ctx, uint64_t* n_device_mallocs, uint64_t* n_cache_hits, uint64_t* bytes_in_use,
                    uint64_t* bytes_cached);
int ott_alloc_release_cached(ott_ctx* ctx); /* CPUCachingAllocator::free_cached */
int ott_host_alloc(size_t bytes, void** out); /* pinned host staging memory */
int ott_host_free(void* p);
int ott_memcpy_h2d(ott_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes); /* async on the stream */
int ott_memcpy_d2h(ott_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes); /* async on the stream */
int ott_memset(ott_ctx* ctx, void* dst_dev, int value, size_t bytes);
/* Copies that overlap kernels: direction 0 = host->device on a side stream (compute work enqueued AFTER this call waits for
 * the copy), 1 = device->host on another side stream (the copy waits for compute work enqueued BEFORE this call). Host
 * memory should be pinned (ott_host_alloc). ott_sync waits for these copies too. The device source of a device->host copy
 * must stay allocated until ott_sync. */
int ott_memcpy_overlapped(ott_ctx* ctx, int direction, void* dst, const void* src, size_t bytes);

/* CUDA events on the context's stream, for timing the kernels where they are launched. */
int ott_event_create(ott_ctx* ctx, ott_event** out);
int ott_event_record(ott_ctx* ctx, ott_event* ev);
int ott_event_elapsed_ms(ott_event* start, ott_event* stop, float* ms); /* synchronizes on stop */
int ott_event_destroy(ott_event* ev);

/* channel stride (in elements) of the NHWC layouts for c logical channels */
int ott_nhwc_channels(int c);

/* ---- quantize: otter::quantize_to_int8 (Tensor/Quantize.cpp:52-58 -> Tensor/QuantizeX86.cpp:47-644)
 *      fp32 NCHW -> int8 NHWC, scale per tensor (n_scales==1) or per channel; scales on the HOST. ---- */
int ott_quantize_f32_nchw_to_s8_nhwc(ott_ctx* ctx, const float* x_dev, int n, int c, int h, int w,
                                     const float* scales_host, int n_scales, int rounding, int8_t* out_dev);

/* ---- the layer: ConvolutionLayer::create_pipeline_int8 / forward_int8
 *      (Tensor/ConvolutionLayer.cpp:666-752, :754-847) ---- */

/* All array arguments are HOST pointers, in the reference's own field layouts:
 *   w_oihw      weight_data, int8 [cout][cin/groups][kh][kw]
 *   bias        bias_data [cout] or NULL when bias_term == 0
 *   w_scales    weight_data_int8_scales [cout]
 *   in_scales   bottom_blob_int8_scales, n_in_scales = 1 (dense) or groups (depthwise)
 *   out_scales  top_blob_int8_scales, n_out_scales = 1 or cout; ignored when int8_scale_term < 100
 * Computes scale_in = 1/(in_scales[0]*w_scales[p]) (0 where w_scales[p]==0) in fp32 on the host exactly as
 * ConvolutionLayer.cpp:667-679, re-lays the weights for the chosen kernel and uploads everything once. */
int ott_conv_int8_create(ott_ctx* ctx, const ott_conv_desc* desc, const int8_t* w_oihw, const float* bias,
                         const float* w_scales, const float* in_scales, int n_in_scales,
                         const float* out_scales, int n_out_scales, ott_conv** out);
int ott_conv_int8_destroy(ott_ctx* ctx, ott_conv* conv);
int ott_conv_int8_kernel_kind(const ott_conv* conv); /* enum ott_kernel_kind */
int ott_conv_int8_out_shape(const ott_conv* conv, int h, int w, int* oh, int* ow);
/* name of the convolution kernel a plain (not gathered) forward of this layer launches for the given input / output types and
 * input size (the choice between the two depthwise kernels depends on them); for benchmark records */
const char* ott_conv_int8_kernel_name(const ott_ctx* ctx, const ott_conv* conv, int in_dtype, int out_dtype, int h, int w);

/* One forward on DEVICE buffers, asynchronous on the context's stream.
 *   in_dtype  OTT_F32_NCHW (quantized on the way in, as ConvolutionLayer.cpp:770-775) or OTT_S8_NHWC
 *   out_dtype OTT_F32_NCHW (int8_scale_term < 100), OTT_S8_NHWC (int8_scale_term > 100), or OTT_S32_NHWC
 *             (accumulators before the epilogue, any int8_scale_term)
 * A batch of n images gives, per image, exactly what the reference gives for that image alone (its int8
 * kernels are batch-1: Tensor/ConvolutionMM2DInt8X86Pack.cpp:159, Tensor/Padding.cpp:27-29).
 * status_word_dev: optional device uint32 the kernels OR an error code into if a bounded wait gives up. */
int ott_conv_int8_forward(ott_ctx* ctx, const ott_conv* conv, const void* in_dev, int in_dtype, int n, int h, int w,
                          void* out_dev, int out_dtype, uint32_t* status_word_dev);

/* The same forward when the fp32 NCHW input is a channel range of a wider tensor (what the reference's Crop layer hands
 * on: native::slice returns a view, Tensor/CropLayer.cpp:67-75): in_dev points at the first channel of the range and
 * in_channels_total is the channel count of the tensor it lives in (the per-image stride in planes). For int8 NHWC input
 * in_channels_total must equal cin. */
int ott_conv_int8_forward_ex(ott_ctx* ctx, const ott_conv* conv, const void* in_dev, int in_dtype, int in_channels_total, int n,
                             int h, int w, void* out_dev, int out_dtype, uint32_t* status_word_dev);

/* The same forward when the fp32 input is scattered over several device tensors: logical input channel i is plane
 * (plane_refs[i] & 0xFFFFFF) of buffers[plane_refs[i] >> 24], whose consecutive images are image_strides[b] floats apart.
 * This is how a consumer reads the result of the reference's Concat / Crop / ChannelShuffle layers, which only select and
 * re-order channel planes (Tensor/ConcatLayer.cpp:55-70, Tensor/CropLayer.cpp:67-75, Tensor/ChannelShuffleLayer.cpp:37-41),
 * without those planes ever being copied. At most 12 buffers and 512 channels; plane_refs has cin entries (host array). */
int ott_conv_int8_forward_gather(ott_ctx* ctx, const ott_conv* conv, const float* const* buffers, const int64_t* image_strides,
                                 int n_buffers, const uint32_t* plane_refs, int n, int h, int w, void* out_dev, int out_dtype,
                                 uint32_t* status_word_dev);

/* ---- int8 hand-over through Concat / Crop / ChannelShuffle ----
 * The reference quantizes a layer's fp32 input with float2int8(v * bottom_blob_int8_scale) (ConvolutionLayer.cpp:763-779,
 * Tensor/QuantizeX86.cpp:23-71) and the requantizing epilogue ends with float2int8(v * scale_out) on the same fp32 v
 * (Tensor/QuantizeX86.cpp:1723-1870). So when every reader of an output channel is known, the producer can store that channel
 * already quantized for its reader (per-channel out_scales) and the reader needs no quantize pass; the glue layers between the
 * two only select and re-order channels. Two pieces:
 *
 * ott_conv_int8_create_gathered: a 1x1, stride-1, unpadded dense layer whose logical input channel i is channel
 * channel_index[i] of int8 NHWC tensor channel_source[i] (n_sources tensors of source_channels[s] channels each, every one
 * written whole by one producer, at most 12). The kernel reads, per source, the aligned 32-channel blocks that cover the
 * channels it needs (at most 64 blocks) with weights laid out to match, zero for channels that belong to other readers.
 * The other arguments are those of ott_conv_int8_create (n_in_scales must be 1). Such a layer only runs through
 * ott_conv_int8_forward_io with `sources` set.
 * A depthwise layer (groups == cin == cout, 3x3 / 5x5, stride 1 / 2, int8 output, equal input scales) can be created the same
 * way. Its kernel reads whole 16-channel groups, so the layer runs on a permuted and padded channel order made of the sources'
 * aligned groups, and its OUTPUT tensor has that order as well: ott_conv_int8_gathered_layout gives the number of channels
 * stored (a multiple of 16) and, for every logical channel, its position; the other positions hold zeros. (The layer that
 * reads this output is in turn created with ott_conv_int8_create_gathered over one source.) For any other layer
 * stored_channels comes back 0. */
int ott_conv_int8_create_gathered(ott_ctx* ctx, const ott_conv_desc* desc, const int8_t* w_oihw, const float* bias,
                                  const float* w_scales, const float* in_scales, int n_in_scales, const float* out_scales,
                                  int n_out_scales, int n_sources, const int* source_channels, const int* channel_source,
                                  const int* channel_index, ott_conv** out);

int ott_conv_int8_gathered_layout(const ott_conv* conv, int* stored_channels, int* position, int n_position);

/* One forward described by a struct. Plain use (sources NULL, out_f32_dev NULL) equals ott_conv_int8_forward.
 *   sources / n_sources   the int8 NHWC inputs of a layer made by ott_conv_int8_create_gathered (in_dev is ignored)
 *   out_f32_dev, f32_channel_mask   only with out_dtype OTT_S8_NHWC on the tensor-core kernel, cout <= 1024: output channel c
 *       with bit (c & 31) of f32_channel_mask[c >> 5] set is ALSO stored as the fp32 NCHW plane c of the [n][cout][oh][ow]
 *       tensor out_f32_dev, holding activation(dequantize(acc)), i.e. what the same layer with fp32 output stores; the other
 *       planes of out_f32_dev are not touched. f32_channel_mask is a host array of (cout + 31) / 32 words. After
 *       ott_conv_int8_set_f32_plane_map(conv, plane_of_channel, planes_total) channel c is instead stored as plane
 *       plane_of_channel[c] of a tensor with planes_total channels (a layer whose output channels were re-ordered).
 *   chunk_dst, chunk_pitch, n_chunks   scattered int8 output (tensor-core kernel, out_dtype OTT_S8_NHWC; out_dev is ignored):
 *       output channels 16c..16c+15 of every pixel p are stored at chunk_dst[c] + p * chunk_pitch[c] (NULL: not stored), so that a
 *       layer whose channels were laid out reader by reader writes each reader's channels straight into that reader's input
 *       tensor. n_chunks = ott_nhwc_channels(cout) / 16, at most 64; addresses and pitches multiples of 16 bytes. Host arrays. */
typedef struct ott_conv_io {
    const void* in_dev;
    int in_dtype;
    const int8_t* const* sources;
    int n_sources;
    void* out_dev;
    int out_dtype;
    float* out_f32_dev;
    const uint32_t* f32_channel_mask;
    int8_t* const* chunk_dst;
    const uint32_t* chunk_pitch;
    int n_chunks;
} ott_conv_io;
int ott_conv_int8_forward_io(ott_ctx* ctx, const ott_conv* conv, const ott_conv_io* io, int n, int h, int w,
                             uint32_t* status_word_dev);
int ott_conv_int8_set_f32_plane_map(ott_ctx* ctx, ott_conv* conv, const int* plane_of_channel, int planes_total);

/* One ShuffleNetV2 unit branch as one launch: the chain 1x1 convolution -> depthwise 3x3 (stride 1, pad 1) -> 1x1 convolution,
 * i.e. three consecutive ConvolutionLayer::forward_int8 calls (Tensor/ConvolutionLayer.cpp:754-847) whose two intermediate int8
 * blobs stay in shared memory. Built from three existing layer objects (the last one must outlive the unit): pw1 and dw
 * requantizing (int8_scale_term > 100), pw1 plain or created with gathered input, pw2 with either output kind; all with a
 * bias, the 1x1 layers sharing one activation, the depthwise layer without one; at most 128 channels between the layers.
 * OTT_ERR_UNSUPPORTED otherwise (run the three layers one by one). The result equals theirs bit for bit.
 * ott_unit_int8_forward_io takes the first layer's input (io->sources for a gathered layer, else io->in_dev as int8 NHWC) and
 * delivers the last layer's output (out_dev / out_dtype / out_f32_dev / f32_channel_mask as for ott_conv_int8_forward_io). */
typedef struct ott_unit ott_unit;
int ott_unit_int8_create(ott_ctx* ctx, const ott_conv* pw1, const ott_conv* dw, const ott_conv* pw2, ott_unit** out);
int ott_unit_int8_forward_io(ott_ctx* ctx, const ott_unit* unit, const ott_conv_io* io, int n, int h, int w, uint32_t* status_word_dev);
int ott_unit_int8_destroy(ott_ctx* ctx, ott_unit* unit);

/* A depthwise 3x3 layer (pad 1, stride 1 or 2) and the 1x1 layer that reads its output, as one launch: two consecutive
 * ConvolutionLayer::forward_int8 calls (Tensor/ConvolutionLayer.cpp:754-847) whose intermediate int8 blob stays in shared
 * memory; unlike the whole unit above, nothing is computed twice (the depthwise layer's halo is input that already exists).
 * Built from two existing layer objects (both must outlive the pair): dw requantizing (int8_scale_term > 100), without
 * activation, plain or created with gathered input in 32-channel groups; pw plain, or created with gathered input whose one
 * source is dw's output tensor; both with a bias and the add-half-truncate rounding rule; at most 256 stored depthwise
 * channels and 256 output channels. OTT_ERR_UNSUPPORTED otherwise (run the two layers one by one). Same bits as the two layers.
 * ott_dwpw_int8_forward_io takes the depthwise layer's input (io->sources for a gathered layer, else io->in_dev as int8 NHWC;
 * h, w = its input size) and delivers the 1x1 layer's output (out_dev / out_dtype / out_f32_dev / f32_channel_mask as for
 * ott_conv_int8_forward_io). */
typedef struct ott_dwpw ott_dwpw;
int ott_dwpw_int8_create(ott_ctx* ctx, const ott_conv* dw, const ott_conv* pw, ott_dwpw** out);
int ott_dwpw_int8_forward_io(ott_ctx* ctx, const ott_dwpw* pair, const ott_conv_io* io, int n, int h, int w, uint32_t* status_word_dev);
int ott_dwpw_int8_destroy(ott_ctx* ctx, ott_dwpw* pair);

/* Dense fp32 NCHW copy [n][channels][hw] of planes described the same way (for consumers that need one tensor). */
int ott_gather_channels_f32(ott_ctx* ctx, const float* const* buffers, const int64_t* image_strides, int n_buffers,
                            const uint32_t* plane_refs, int channels, int n, int hw, float* dst_dev);

/* ShortCutLayer (Tensor/ShortCutLayer.cpp) with both operands described as plane tables (see ott_conv_int8_forward_gather):
 * dst[n][channels][hw] = a + b, so that the result of a Concat can be added without first being copied into one tensor. */
int ott_add_gather_f32(ott_ctx* ctx, const float* const* a_buffers, const int64_t* a_image_strides, int a_n_buffers,
                       const uint32_t* a_plane_refs, const float* const* b_buffers, const int64_t* b_image_strides, int b_n_buffers,
                       const uint32_t* b_plane_refs, int channels, int n, int hw, float* dst_dev);

/* First layer + the max-pool that consumes it, in one kernel: out = MaxPool3x3/stride2/pad1(forward(in)), fp32 NCHW
 * [n][cout][(oh-1)/2+1][(ow-1)/2+1]. Replaces the pair conv1 -> pool1 of the reference's graphs (Tensor/ConvolutionLayer.cpp:754-847
 * followed by Tensor/MaxPoolLayer.cpp:123-133) when nothing else reads conv1; the values pooled are exactly the ones the
 * separate layer would have stored. Only for the 3-input-channel 3x3 layer with fp32 output (else OTT_ERR_UNSUPPORTED).
 * pad_with_zero as in ott_maxpool_f32_nchw. */
int ott_conv_int8_forward_maxpool(ott_ctx* ctx, const ott_conv* conv, const float* in_dev, int n, int h, int w, int pad_with_zero,
                                  float* out_dev);
/* The same with the pooled values quantized on the way out: int8 NHWC [n][ph][pw][ott_nhwc_channels(cout)], channel c holding
 * float2int8(pooled * out_scales[c]): what the quantize pass of a layer reading the pooled blob computes (ConvolutionLayer.cpp:
 * 763-779). For a layer created with int8_scale_term > 100. */
int ott_conv_int8_forward_maxpool_s8(ott_ctx* ctx, const ott_conv* conv, const float* in_dev, int n, int h, int w, int pad_with_zero,
                                     int8_t* out_dev);

/* The same forward on HOST buffers: copies the input to the device, runs, copies the output back and
 * waits for it. This is the call a host-tensor Layer::forward maps to (Tensor/Net.cpp:442). */
int ott_conv_int8_forward_host(ott_ctx* ctx, const ott_conv* conv, const void* in_host, int in_dtype, int n, int h,
                               int w, void* out_host, int out_dtype);

/* ---- fp32 glue layers of the benchmark graphs (device fp32 NCHW tensors, asynchronous on the stream) ---- */

/* dst[b][dst_c0 + j*dst_cstride][:] = src[b][src_c0 + j*src_cstride][:] for j < count, b < n; hw = H*W.
 * One primitive for Concat along channels (Tensor/ConcatLayer.cpp:55-70), Crop along channels
 * (Tensor/CropLayer.cpp:67-75 -> native::slice) and ChannelShuffle (Tensor/ChannelShuffleLayer.cpp:37-41:
 * output channel i*g + k is input channel k*(C/g) + i, i.e. g strided copies). */
int ott_copy_channels_f32(ott_ctx* ctx, const float* src, int src_channels, int src_c0, int src_cstride, float* dst,
                          int dst_channels, int dst_c0, int dst_cstride, int count, int n, int hw);

/* MaxPoolLayer::forward (Tensor/MaxPoolLayer.cpp:123-133 -> otter::max_pool2d, Tensor/Pool.cpp:1166-1201), no
 * dilation, floor mode. pad_with_zero = 1 reproduces the reference's packed 3x3 stride-2 kernels, which pad the
 * input with zeros (Tensor/Pool.cpp:972-975, :807-810); 0 reproduces its plain kernel (padding never wins). */
int ott_maxpool_f32_nchw(ott_ctx* ctx, const float* in, int n, int c, int h, int w, int kh, int kw, int sh, int sw, int ph,
                         int pw, int pad_with_zero, float* out);

/* UpsampleLayer::forward, bilinear, align_corner = false (Tensor/UpsampleLayer.cpp:113-131 -> otter::Interpolate,
 * Tensor/TensorInterpolation.cpp:1444-1472). scale_h / scale_w are the layer's scale factors (0: derive from the sizes).
 * packed_rule = 1 reproduces what the reference computes on a packed blob (channels a multiple of 4 under
 * use_packing_layout: ncnn-style coefficients and operand order, TensorInterpolation.cpp:16-46,161-273), 0 what it
 * computes on a plain blob (Tensor/UpSampleKernel.cpp:74-140 with the coefficients of Tensor/UpSample.hpp:133-158). The two
 * differ in the last bit of about a third of the outputs and in how the far border is weighted. */
int ott_upsample_bilinear_f32_nchw(ott_ctx* ctx, const float* in, int n, int c, int h, int w, int oh, int ow, double scale_h,
                                   double scale_w, int packed_rule, float* out);

/* UpsampleLayer::forward, nearest (Tensor/UpsampleLayer.cpp:113-131 -> otter::Interpolate): every output pixel is a copy of
 * one source pixel. packed_rule = 1 picks it as the reference does on a packed blob (min((int)(d * (in / (float)out)),
 * in - 1), Tensor/TensorInterpolation.cpp:660-676), 0 as on a plain blob (Tensor/UpSampleKernel.cpp:41-60: the index itself
 * for equal sizes, d >> 1 for a doubled size, else min(floor(d * (float)(1 / scale)), in - 1)); the two differ only for
 * scale factors that are not integers. scale_h / scale_w as for the bilinear call. */
int ott_upsample_nearest_f32_nchw(ott_ctx* ctx, const float* in, int n, int c, int h, int w, int oh, int ow, double scale_h,
                                  double scale_w, int packed_rule, float* out);

/* ShortCutLayer: out = a + b (Tensor/ShortCutLayer.cpp) */
int ott_add_f32(ott_ctx* ctx, const float* a, const float* b, float* out, size_t count);

/* stand-alone ReluLayer / LReluLayer / Relu6Layer, in place (act_type as in ott_conv_desc) */
int ott_activation_f32(ott_ctx* ctx, float* x, size_t count, int act_type, float param0);

/* CUDA graphs. No counterpart in the reference (its CPU layers have no launch cost to amortise): everything enqueued on the
 * context's stream between capture_begin and capture_end is frozen into one launch. A small-layer network is dozens of
 * kernels of 10-30 us each; replaying them as a graph removes the gaps between them (7 % on the ShuffleNetV2 forward).
 * Rules: nothing in between may synchronise or copy to pageable host memory; device pointers baked into the graph must
 * stay valid - ott_graph_seal takes the allocator blocks that were handed out during the capture and have been returned
 * since (the temporaries) out of circulation until ott_graph_destroy; blocks still held by the caller stay the caller's.
 * ott_graph_capture_end with out = NULL abandons a capture. ott_net_capture (otter_b200_net.h) wraps all of this for a Net. */
typedef struct ott_graph ott_graph;
int ott_graph_capture_begin(ott_ctx* ctx);
int ott_graph_capture_end(ott_ctx* ctx, ott_graph** out);
int ott_graph_seal(ott_ctx* ctx, ott_graph* graph);
int ott_graph_launch(ott_ctx* ctx, ott_graph* graph);
int ott_graph_destroy(ott_ctx* ctx, ott_graph* graph);

/* NanodetPlusDetectionOutputLayer::forward (Tensor/NanodetPlusDetectionOutputLayer.cpp:65-260) for a batch: heads_dev[l] is the
 * fp32 NCHW output [n][num_class + 4*reg_bins][grid_h[l]][grid_w[l]] of pyramid level l on the device. Per image: best class
 * logit per cell, sigmoid >= prob_threshold, softmax over the reg_bins distance bins of each box side, box; then sort by
 * score and greedy NMS, one CTA per image, all on the GPU (an image with more than 4096 proposals is sorted and filtered on
 * the host); one copy brings every image's rows back. out_host receives, per image, up to max_det
 * rows {label + 1, score, x, y, width, height} at out_host + img*max_det*6; counts_host[img] the number of detections kept
 * (which may exceed max_det). The reference decodes image 0 only; scores agree with it to 1-2 ulp and boxes to ~1e-4 pixels
 * (its -Ofast build and the GPU round expf and the divisions differently). Synchronises the stream. */
int ott_nanodet_detect(ott_ctx* ctx, const float* const* heads_dev, const int* grid_h, const int* grid_w, const int* strides,
                       int n_levels, int n, int num_class, int reg_bins, float prob_threshold, float nms_threshold, float* out_host,
                       int* counts_host, int max_det);

/* ---- the fp32 layer: ConvolutionLayer with int8_scale_term == 0 (Tensor/ConvolutionLayer.cpp:507-664), which a "mixed"
 *      quantized model keeps for its first convolution (benchmark/nanodet-plus-m-1.5x_416_int8_mixed.otter:26). Dense or
 *      depthwise, bias and activation (none/ReLU/LeakyReLU/ReLU6) fused; fp32 NCHW device tensors in and out. w_oihw (fp32
 *      [cout][cin/groups][kh][kw]) and bias are HOST pointers. The result agrees with the reference's fp32 kernels to rounding
 *      (a few units in the last place of sum |w*x| + |bias|: its -ffast-math build sums in its own vector order), not to the bit. ---- */
typedef struct ott_conv_f32 ott_conv_f32;
int ott_conv_f32_create(ott_ctx* ctx, const ott_conv_desc* desc, const float* w_oihw, const float* bias, ott_conv_f32** out);
int ott_conv_f32_forward(ott_ctx* ctx, const ott_conv_f32* conv, const float* in_dev, int n, int h, int w, float* out_dev);
int ott_conv_f32_destroy(ott_ctx* ctx, ott_conv_f32* conv);

/* The forward for hosts that may not allocate device memory while running. No counterpart in the
 * reference (its CPU path simply calls otter::empty for every temporary).
 * Who needs it: a process whose device memory was divided into fixed pools at start-up and must not grow
 * afterwards, or a loop with a hard latency bound that cannot absorb the device-wide synchronisation a
 * cudaMalloc or cudaFree implies. ott_conv_int8_forward can end in cudaMalloc the first time it sees a new
 * size, because it takes the buffer for the quantized activations from the context's allocator. This
 * variant does the same work (quantize fp32 NCHW input, then the layer's convolution kernel) but keeps
 * that buffer in a fixed array of OTT_NOALLOC_SCRATCH_BYTES that is part of the library image on every GPU
 * that loads it, for the life of the process. It calls no cudaMalloc, cudaFree or allocating routine.
 *   - Input is fp32 NCHW on the device; output as for ott_conv_int8_forward; the caller owns both.
 *   - n*h*w*ott_nhwc_channels(cin) must fit OTT_NOALLOC_SCRATCH_BYTES; larger calls fail with
 *     OTT_ERR_INVALID and a message naming both sizes (split the batch, or use the ordinary forward).
 *   - The first call on each GPU looks up the array's device address (cudaGetSymbolAddress). With CUDA's
 *     default lazy module loading that look-up is also the moment the module holding the array is loaded
 *     onto that GPU, i.e. when its OTT_NOALLOC_SCRATCH_BYTES are reserved; it can synchronise the device and
 *     it can fail for lack of memory. So make one call per GPU during start-up: before the pools are
 *     carved, before the latency-bound loop begins, and before starting any stream capture.
 *   - A call that the layer would refuse (a layer created with gathered input, an output type the layer
 *     does not produce, an empty output) fails before anything is launched or the array is touched.
 *   - All calls on one GPU share the one array. It keeps whatever the last call left; this entry point
 *     overwrites every byte it later reads, so nothing has to be cleared. Two calls whose kernels can be
 *     in flight on the same GPU at once (different contexts or streams) race on it: serialise them. */
#define OTT_NOALLOC_SCRATCH_BYTES (32u << 20)
int ott_conv_int8_forward_noalloc(ott_ctx* ctx, const ott_conv* conv, const float* in_f32_nchw_dev, int n, int h, int w,
                                  void* out_dev, int out_dtype);

/* number of kernels this library launched on ctx since creation (for benchmark bookkeeping) */
uint64_t ott_launch_count(const ott_ctx* ctx);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* OTTER_B200_H */
