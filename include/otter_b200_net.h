/* otter_b200 — C-ABI over the host-side graph runtime (tensor_b200/host: the C++17 mirror of the reference's
 * Net / Layer / Extractor API). It exists so that hosts without a C++ toolchain — the Python tests and the
 * benchmark here — can build a Net from the reference's own LayerOption key/value pairs and run it.
 * C++ hosts use tensor_b200/host/otter_api.hpp directly. Status codes as in otter_b200.h.
 */
#ifndef OTTER_B200_NET_H
#define OTTER_B200_NET_H

#include "otter_b200.h"

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

typedef struct ott_net ott_net;

/* Net::Net + NetOption::device (Tensor/Net.hpp:22-27) */
int ott_net_create(int device, ott_net** out);
int ott_net_destroy(ott_net* net);
const char* ott_net_last_error(const ott_net* net);
ott_ctx* ott_net_context(ott_net* net); /* valid after ott_net_compile */

/* The public fields of Net::option (Tensor/NetOption.hpp:16-24), to be set before ott_net_compile. Keys: "lightmode",
 * "use_packing_layout", "int8_rounding" (OTT_ROUND_*), and the three switches this library adds, all on by default:
 * "fuse_first_layer_pool" (first convolution + 3x3 stride-2 max-pool as one kernel), "int8_handover" (a convolution
 * whose fp32 result is read only by another quantized convolution writes that layer's int8 input directly) and
 * "int8_routing" (the same through Concat / Crop / ChannelShuffle / Split: a producer stores each output channel already
 * quantized for the one 1x1 convolution that reads it, which then gathers its input from its producers' int8 tensors). All
 * three leave every extracted blob bit-identical. "fuse_depthwise_pointwise" (default 0): a depthwise 3x3 layer whose int8
 * output only the 1x1 layer behind it reads runs inside that layer's kernel (ott_dwpw_*; same bits; fewer launches, which pays
 * for small batches). "host_chunk" (default 64): images per chunk when ott_net_forward pipelines a host
 * batch (upload, kernels and download of different chunks overlap). Unknown key: OTT_ERR_INVALID. */
int ott_net_set_option(ott_net* net, const char* key, int value);

/* Net::addLayer (Tensor/Net.cpp:40-80). `options` is one LayerOption as "key=value;key=value;...", with the
 * keys of the .otter format (type, name, input, output, and the layer's own parameters: out_channels, kernel_h,
 * stride, int8_scale_term, activation, groups, axis, start, end, ...). */
int ott_net_add_layer(ott_net* net, const char* options);

/* Net::load_otter(path, CompileMode::Initial) (Tensor/Net.cpp:518-536): reads a `.otter` text graph (Tensor/Otter.cpp),
 * adds its layers and compiles. Use instead of ott_net_add_layer + ott_net_compile. */
int ott_net_load_otter(ott_net* net, const char* path);

/* A real model: Net::load_otter(otter_path, CompileMode::Inference) followed by Net::load_weight(weight_path, type)
 * (Tensor/Net.cpp:518-607). weight_type 1 = WeightType::Ncnn, the ncnn `.bin` of a quantized model (int8 weights tagged
 * 0x000D4B38, then bias, weight scales, input scale and - for requantizing layers - output scale per Convolution, in graph
 * order: Tensor/ConvolutionLayer.cpp:245-296, Tensor/Initializer.cpp:64-188); 0 = WeightType::Otter (plain fp32, which only
 * fp32 layers can use, so an int8 graph fails in create_pipeline). A file with bytes left over is an error, as in the
 * reference. */
int ott_net_load_model(ott_net* net, const char* otter_path, const char* weight_path, int weight_type);

/* The `.otter` reader alone (no GPU needed): parses `text` and writes one line per layer, "key=value;key=value;..." with
 * the layer type under key "type", into out (NUL-terminated, at most cap bytes). Returns the number of layers, or a
 * negative status (OTT_ERR_INVALID on a syntax error or when cap is too small). */
int ott_otter_parse_text(const char* text, char* out, int cap);

/* Net::compile(CompileMode::Initial) (Tensor/Net.cpp:174-280): builds the graph (automatic Split layers for
 * fan-out), creates the layers, infers shapes, gives every layer random parameters and builds its pipeline. */
int ott_net_compile(ott_net* net);

int ott_net_layer_count(const ott_net* net);
/* type and name of layer i; for Convolution layers geom = {cin, cout, kh, kw, sh, sw, ph, pw, groups, bias_term,
 * int8_scale_term, activation_type}, else zeros */
int ott_net_layer_info(const ott_net* net, int i, char* type, int type_cap, char* name, int name_cap, int geom[12]);
int ott_net_blob_shape(const ott_net* net, const char* blob, int shape[4]);
int ott_net_blob_element_size(const ott_net* net, const char* blob); /* 1: the int8 blob of a requantizing convolution; 4: fp32; 0: unknown blob */
/* How Convolution layer i takes part in the "int8_routing" hand-over (zeros for every other layer, or with the switch off):
 * info[0] = number of int8 tensors its input channels are gathered from (0: it reads its input blob as usual),
 * info[1] = output channels it stores quantized for their reader, info[2] = output channels it (also) stores as fp32 planes
 * because something else reads them. Plans the hand-over if that has not happened yet. */
int ott_net_layer_routing(ott_net* net, int i, int info[3]);

/* Replace a Convolution layer's parameters (the public fields weight_data, bias_data, weight_data_int8_scales,
 * bottom_blob_int8_scales, top_blob_int8_scales of Tensor/ConvolutionLayer.hpp:62-77) and rebuild its pipeline. */
int ott_net_set_conv_params(ott_net* net, const char* layer, const int8_t* w_oihw, const float* bias, const float* w_scales,
                            const float* in_scales, int n_in_scales, const float* out_scales, int n_out_scales);

/* The same for an fp32 Convolution layer (int8_scale_term == 0): weight_data fp32 [cout][cin/groups][kh][kw] and bias_data. */
int ott_net_set_conv_params_f32(ott_net* net, const char* layer, const float* w_oihw, const float* bias);

/* Extractor::input + Extractor::extract (Tensor/Net.cpp:686-736) for one input blob and n_out output blobs.
 * in: fp32 NCHW, on the host (in_on_device = 0; copied to the GPU) or already on the GPU (1).
 * out_host[i]: NULL = only compute the blob; else a host buffer that receives the blob in the reference's plain
 * layout (fp32 NCHW, or int8 NCHW for int8 blobs) after the stream has been synchronised.
 * With every out_host NULL the call is asynchronous on the Net's stream. */
int ott_net_forward(ott_net* net, const char* input_blob, const void* in, int in_on_device, int n, int c, int h, int w,
                    int n_out, const char* const* out_blobs, void* const* out_host);

/* A whole forward frozen into a CUDA graph (see ott_graph_* in otter_b200.h): Extractor::input(input_blob, the device
 * tensor [n,c,h,w] at in_dev) + Extractor::extract of every blob in out_blobs, captured once. ott_net_graph_launch replays
 * it on the Net's stream (asynchronous); the caller refills in_dev between launches and reads the outputs from the device
 * pointers ott_net_graph_output reports (dense fp32 NCHW, or int8 NHWC for a requantizing layer's blob; valid until
 * ott_net_graph_destroy). One warm-up forward runs first so that nothing has to be allocated inside the capture. Layers
 * that synchronise (NanodetPlusDetectionOutput) cannot be captured. Results are bit-identical to ott_net_forward. */
typedef struct ott_net_graph ott_net_graph;
int ott_net_capture(ott_net* net, const char* input_blob, const void* in_dev, int n, int c, int h, int w, int n_out,
                    const char* const* out_blobs, ott_net_graph** out);
int ott_net_graph_launch(ott_net_graph* graph);
int ott_net_graph_output(ott_net_graph* graph, int index, void** dev_ptr, int shape[4]);
int ott_net_graph_destroy(ott_net_graph* graph);

/* Extractor::input + Extractor::extract for a blob whose size is only known after the forward: the [count, 6] result of a
 * NanodetPlusDetectionOutput layer (Tensor/NanodetPlusDetectionOutputLayer.cpp:65-110; image 0 of the batch, as in the
 * reference). Up to capacity_rows rows are copied to out_host; *rows is the blob's row count, *cols its row length. */
int ott_net_forward_rows(ott_net* net, const char* input_blob, const void* in, int in_on_device, int n, int c, int h, int w,
                         const char* out_blob, float* out_host, int capacity_rows, int* rows, int* cols);

/* Extractor::benchmark_info (Tensor/Net.cpp:811-850, Tensor/Benchmark.cpp:45-102): the same forward with CUDA events
 * around every layer; ms_per_layer[i] (ott_net_layer_count entries) receives layer i's device time in milliseconds.
 * Layers run serialised while profiling. */
int ott_net_profile(ott_net* net, const char* input_blob, const void* in, int in_on_device, int n, int c, int h, int w,
                    const char* out_blob, float* ms_per_layer);

/* ---- several GPUs behind one call (no counterpart in the reference, which runs one image on the host cores) ----
 * A group holds one Net replica per listed device (a device may be listed more than once: each entry gets its own context
 * and stream). Configure every member the same way through the ott_net_* calls (ott_net_group_member), then:
 * ott_net_group_forward = Extractor::input + Extractor::extract (Tensor/Net.cpp:686-736) for a host batch of n images: the
 * batch is cut into contiguous slices (ott_net_group_partition: sizes differ by at most one, earlier slices take the extra
 * images), slice p runs on member p through ott_net_forward on its own host thread, and its outputs are copied to
 * out_host[i] + first_image_of_slice * bytes_per_image(out_blobs[i]). Returns when every slice is done. Images are
 * independent, so the result equals the unsharded forward bit for bit; no data moves between the GPUs. Host buffers
 * should be pinned (ott_host_alloc) for the copies to overlap the kernels. */
typedef struct ott_net_group ott_net_group;
int ott_net_group_create(const int* devices, int n_devices, ott_net_group** out);
int ott_net_group_destroy(ott_net_group* group);
int ott_net_group_size(const ott_net_group* group);
ott_net* ott_net_group_member(ott_net_group* group, int index); /* owned by the group */
const char* ott_net_group_last_error(const ott_net_group* group);
void ott_net_group_partition(int n, int parts, int index, int* first, int* count);
int ott_net_group_forward(ott_net_group* group, const char* input_blob, const float* in_host, int n, int c, int h, int w, int n_out,
                          const char* const* out_blobs, void* const* out_host);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* OTTER_B200_NET_H */
