// C-ABI driver over the compiled reference (otter) for the int8 convolution path.
//
// TEST INFRASTRUCTURE ONLY. This file is linked with the reference's own objects into
// oracle/_ref/libotter_ref.so by oracle/Makefile (`make ref`). It is the checker the parity
// tests and the bench's CPU-baseline leg call; nothing the GPU library ships may load it.
//
// It drives the reference exactly the way its Net drives a layer
// (Tensor/Net.cpp:196-273 compile, :380-411 convert_layout, :434-446 forward):
//   ConvolutionLayer: parse_param -> compute_output_shape -> load_param
//                     (Tensor/ConvolutionLayer.cpp:58-206), public weight/scale fields assigned,
//                     create_pipeline (:298-304, :666-752), forward (:507-511 -> forward_int8 :754-847).
// The reference's int8 kernels only index batch 0 (e.g. Tensor/ConvolutionMM2DInt8X86Pack.cpp:159,
// Tensor/DepthwiseConvKernelInt8X86Pack.cpp:75-76), so a batch is a loop of N=1 forwards here.

#include "ConvolutionLayer.hpp"
#include "Convolution.hpp"
#include "Quantize.hpp"
#include "TensorMaker.hpp"
#include "TensorFactory.hpp"
#include "TensorPacking.hpp"
#include "Parallel.hpp"
#include "NetOption.hpp"

#include <chrono>
#include <memory>
#include <cstring>
#include <string>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {

struct RefConvDesc {
    int cin, cout, kh, kw, sh, sw, ph, pw, dh, dw, groups;
    int bias_term;        // 0/1
    int int8_scale_term;  // 1,2 -> fp32 out ; 101,102 -> int8 out
    int act_type;         // 0 none 1 relu 2 lrelu 3 relu6
    float act_param0;     // lrelu slope
};

thread_local std::string g_err;

otter::Tensor vec_tensor(const float* p, int n) {
    otter::Tensor t = otter::empty({n}, otter::ScalarType::Float);
    std::memcpy(t.data_ptr<float>(), p, sizeof(float) * n);
    return t;
}

struct RefLayer {
    otter::ConvolutionLayer layer;
    otter::NetOption opt;
    RefConvDesc d;
};

int build_layer(RefLayer& L, const RefConvDesc& d, const int8_t* w_oihw, const float* bias,
                const float* w_scales, const float* in_scales, int n_in_scales,
                const float* out_scales, int n_out_scales, int h, int w, int packed) {
    L.d = d;
    L.opt.use_packing_layout = packed != 0;
    otter::LayerOption option;
    option["in_channels"] = std::to_string(d.cin);
    option["out_channels"] = std::to_string(d.cout);
    option["kernel_h"] = std::to_string(d.kh);
    option["kernel_w"] = std::to_string(d.kw);
    option["stride_h"] = std::to_string(d.sh);
    option["stride_w"] = std::to_string(d.sw);
    option["padding_h"] = std::to_string(d.ph);
    option["padding_w"] = std::to_string(d.pw);
    option["dilation_h"] = std::to_string(d.dh);
    option["dilation_w"] = std::to_string(d.dw);
    option["groups"] = std::to_string(d.groups);
    option["bias_term"] = d.bias_term ? "true" : "false";
    option["int8_scale_term"] = std::to_string(d.int8_scale_term);
    if (d.act_type == 1) option["activation"] = "Relu";
    if (d.act_type == 2) { option["activation"] = "LRelu"; option["activation_params"] = std::to_string(d.act_param0); }
    if (d.act_type == 3) option["activation"] = "Relu6";

    otter::ParamDict pd;
    L.layer.parse_param(option, pd);
    L.layer.bottom_shapes.clear();
    L.layer.bottom_shapes.push_back(otter::tensor({1, d.cin, h, w}, otter::ScalarType::Int).view({1, -1}));
    L.layer.compute_output_shape(pd);
    L.layer.load_param(pd);
    if (d.act_type == 2) {
        // std::to_string keeps 6 decimals only; hand the exact slope over.
        L.layer.activation_params = vec_tensor(&d.act_param0, 1);
    }

    const int wsize = d.cout * (d.cin / d.groups) * d.kh * d.kw;
    L.layer.weight_data = otter::empty({d.cout, d.cin / d.groups, d.kh, d.kw}, otter::ScalarType::Byte);
    std::memcpy(L.layer.weight_data.raw_data(), w_oihw, wsize);
    if (d.bias_term) L.layer.bias_data = vec_tensor(bias, d.cout);
    L.layer.weight_data_int8_scales = vec_tensor(w_scales, d.cout);
    L.layer.bottom_blob_int8_scales = vec_tensor(in_scales, n_in_scales);
    if (d.int8_scale_term > 100) L.layer.top_blob_int8_scales = vec_tensor(out_scales, n_out_scales);
    return L.layer.create_pipeline(L.opt);
}

// What Net::convert_layout does before handing a blob to a packing-capable layer
// (Tensor/Net.cpp:380-411).
otter::Tensor to_layer_layout(const otter::Tensor& t, bool packed, bool is_byte) {
    if (!packed) return t;
    int c = (int)t.size(1);
    if (is_byte) return (c % 8 == 0) ? t.packing(8) : t;
    if (c % 8 == 0) return t.packing(8);
    if (c % 4 == 0) return t.packing(4);
    return t;
}

}  // namespace

REF_API const char* ref_last_error() { return g_err.c_str(); }

REF_API int ref_max_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

REF_API void ref_set_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#endif
    otter::set_num_threads(n);
}

// One ConvolutionLayer int8 forward per image. Any output pointer may be NULL.
//   x_f32 : [n, cin, h, w] fp32 NCHW, or NULL when x_s8 ([n, cin, h, w] int8 NCHW) is given
//   xq_out: the int8 activations the layer convolved (NCHW)
//   acc   : exact s32 accumulators [n, cout, oh, ow] (what otter::convolution returns, bias not applied)
//   y_f32 : final output when int8_scale_term < 100 ; y_s8: final output when > 100  (NCHW)
REF_API int ref_conv_int8_forward(const RefConvDesc* d, const int8_t* w_oihw, const float* bias,
                                  const float* w_scales, const float* in_scales, int n_in_scales,
                                  const float* out_scales, int n_out_scales,
                                  const float* x_f32, const int8_t* x_s8, int n, int h, int w, int packed,
                                  int8_t* xq_out, int32_t* acc, float* y_f32, int8_t* y_s8) {
    try {
        RefLayer L;
        int rc = build_layer(L, *d, w_oihw, bias, w_scales, in_scales, n_in_scales, out_scales, n_out_scales, h, w, packed);
        if (rc != 0) { g_err = "create_pipeline failed"; return rc; }
        const int oh = (h + 2 * d->ph - d->dh * (d->kh - 1) - 1) / d->sh + 1;
        const int ow = (w + 2 * d->pw - d->dw * (d->kw - 1) - 1) / d->sw + 1;
        const size_t in_elems = (size_t)d->cin * h * w, out_elems = (size_t)d->cout * oh * ow;
        for (int i = 0; i < n; ++i) {
            otter::Tensor bottom;
            if (x_f32) {
                otter::Tensor x = otter::from_blob((void*)(x_f32 + i * in_elems), {1, d->cin, h, w}, otter::ScalarType::Float);
                bottom = to_layer_layout(x, packed != 0, false);
            } else {
                otter::Tensor x = otter::from_blob((void*)(x_s8 + i * in_elems), {1, d->cin, h, w}, otter::ScalarType::Byte);
                bottom = to_layer_layout(x, packed != 0, true);
            }
            if (xq_out || acc) {
                otter::Tensor q = x_f32 ? otter::quantize_to_int8(bottom, L.layer.bottom_blob_int8_scales, L.opt.use_packing_layout) : bottom;
                if (xq_out) {
                    otter::Tensor q1 = q.packing(1).contiguous();
                    std::memcpy(xq_out + i * in_elems, q1.raw_data(), in_elems);
                }
                if (acc) {
                    const bool depthwise = d->groups == d->cin && d->groups == d->cout;
                    otter::Tensor a = otter::convolution(q, L.layer.weight_data,
                        depthwise ? L.layer.weight_data_tf : L.layer.weight_sgemm_int8_data, L.layer.bias_data,
                        {d->sh, d->sw}, {d->ph, d->pw}, {d->dh, d->dw}, false, {0, 0}, d->groups,
                        L.opt.use_packing_layout, L.layer.bottom_blob_int8_scales, L.layer.weight_data_int8_scales);
                    otter::Tensor a1 = a.packing(1).contiguous();
                    std::memcpy(acc + i * out_elems, a1.raw_data(), out_elems * 4);
                }
            }
            if (y_f32 || y_s8) {
                otter::Tensor top;
                rc = L.layer.forward(bottom, top, L.opt);
                if (rc != 0) { g_err = "forward failed"; return rc; }
                otter::Tensor t1 = top.packing(1).contiguous();
                if (d->int8_scale_term > 100) {
                    if (y_s8) std::memcpy(y_s8 + i * out_elems, t1.raw_data(), out_elems);
                } else {
                    if (y_f32) std::memcpy(y_f32 + i * out_elems, t1.raw_data(), out_elems * 4);
                }
            }
        }
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -2;
    } catch (const char* s) {
        g_err = s;
        return -3;
    } catch (...) {
        g_err = "unknown exception";
        return -4;
    }
}

// The fp32 ConvolutionLayer (int8_scale_term == 0; Tensor/ConvolutionLayer.cpp:298-664): fp32 OIHW weights, one image at a time.
// Used to state how far the GPU's fp32 first layer may lie from the reference's -Ofast fp32 kernels.
REF_API int ref_conv_f32_forward(const RefConvDesc* d, const float* w_oihw, const float* bias, const float* x_f32, int n, int h, int w,
                                 int packed, float* y_f32) {
    try {
        RefLayer L;
        L.d = *d;
        L.opt.use_packing_layout = packed != 0;
        otter::LayerOption option;
        option["in_channels"] = std::to_string(d->cin);
        option["out_channels"] = std::to_string(d->cout);
        option["kernel_h"] = std::to_string(d->kh);
        option["kernel_w"] = std::to_string(d->kw);
        option["stride_h"] = std::to_string(d->sh);
        option["stride_w"] = std::to_string(d->sw);
        option["padding_h"] = std::to_string(d->ph);
        option["padding_w"] = std::to_string(d->pw);
        option["dilation_h"] = std::to_string(d->dh);
        option["dilation_w"] = std::to_string(d->dw);
        option["groups"] = std::to_string(d->groups);
        option["bias_term"] = d->bias_term ? "true" : "false";
        option["int8_scale_term"] = "0";
        if (d->act_type == 1) option["activation"] = "Relu";
        if (d->act_type == 2) { option["activation"] = "LRelu"; option["activation_params"] = std::to_string(d->act_param0); }
        if (d->act_type == 3) option["activation"] = "Relu6";
        otter::ParamDict pd;
        L.layer.parse_param(option, pd);
        L.layer.bottom_shapes.clear();
        L.layer.bottom_shapes.push_back(otter::tensor({1, d->cin, h, w}, otter::ScalarType::Int).view({1, -1}));
        L.layer.compute_output_shape(pd);
        L.layer.load_param(pd);
        if (d->act_type == 2) L.layer.activation_params = vec_tensor(&d->act_param0, 1);
        const int wsize = d->cout * (d->cin / d->groups) * d->kh * d->kw;
        L.layer.weight_data = otter::empty({d->cout, d->cin / d->groups, d->kh, d->kw}, otter::ScalarType::Float);
        std::memcpy(L.layer.weight_data.raw_data(), w_oihw, sizeof(float) * wsize);
        if (d->bias_term) L.layer.bias_data = vec_tensor(bias, d->cout);
        int rc = L.layer.create_pipeline(L.opt);
        if (rc != 0) { g_err = "create_pipeline failed"; return rc; }
        const int oh = (h + 2 * d->ph - d->dh * (d->kh - 1) - 1) / d->sh + 1;
        const int ow = (w + 2 * d->pw - d->dw * (d->kw - 1) - 1) / d->sw + 1;
        const size_t in_elems = (size_t)d->cin * h * w, out_elems = (size_t)d->cout * oh * ow;
        for (int i = 0; i < n; ++i) {
            otter::Tensor x = otter::from_blob((void*)(x_f32 + i * in_elems), {1, d->cin, h, w}, otter::ScalarType::Float);
            otter::Tensor bottom = to_layer_layout(x, packed != 0, false);
            otter::Tensor top;
            rc = L.layer.forward(bottom, top, L.opt);
            if (rc != 0) { g_err = "forward failed"; return rc; }
            otter::Tensor t1 = top.packing(1).contiguous();
            std::memcpy(y_f32 + i * out_elems, t1.raw_data(), out_elems * 4);
        }
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -2; } catch (const char* s) { g_err = s; return -3; } catch (...) { g_err = "unknown"; return -4; }
}

// Best-of-`iters` wall time (ms) of ONE N=1 ConvolutionLayer::forward on image 0, after `warmup` runs.
REF_API double ref_conv_int8_time_ms(const RefConvDesc* d, const int8_t* w_oihw, const float* bias,
                                     const float* w_scales, const float* in_scales, int n_in_scales,
                                     const float* out_scales, int n_out_scales,
                                     const float* x_f32, const int8_t* x_s8, int h, int w, int packed,
                                     int warmup, int iters, double* mean_ms) {
    try {
        RefLayer L;
        int rc = build_layer(L, *d, w_oihw, bias, w_scales, in_scales, n_in_scales, out_scales, n_out_scales, h, w, packed);
        if (rc != 0) { g_err = "create_pipeline failed"; return -1.0; }
        otter::Tensor bottom;
        if (x_f32) bottom = to_layer_layout(otter::from_blob((void*)x_f32, {1, d->cin, h, w}, otter::ScalarType::Float), packed != 0, false);
        else bottom = to_layer_layout(otter::from_blob((void*)x_s8, {1, d->cin, h, w}, otter::ScalarType::Byte), packed != 0, true);
        double best = 1e30, sum = 0;
        for (int i = 0; i < warmup + iters; ++i) {
            otter::Tensor top;
            auto t0 = std::chrono::steady_clock::now();
            rc = L.layer.forward(bottom, top, L.opt);
            auto t1 = std::chrono::steady_clock::now();
            if (rc != 0) { g_err = "forward failed"; return -1.0; }
            if (i >= warmup) {
                double ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
                best = ms < best ? ms : best;
                sum += ms;
            }
        }
        if (mean_ms) *mean_ms = sum / (iters > 0 ? iters : 1);
        return best;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1.0;
    } catch (...) {
        g_err = "unknown exception";
        return -1.0;
    }
}

// The three epilogue/prologue functions alone (Tensor/Quantize.hpp:15-19), on NCHW buffers.
REF_API int ref_quantize(const float* x, int c, int h, int w, const float* scales, int n_scales, int packed, int8_t* out) {
    try {
        otter::Tensor t = to_layer_layout(otter::from_blob((void*)x, {1, c, h, w}, otter::ScalarType::Float), packed != 0, false);
        otter::Tensor q = otter::quantize_to_int8(t, vec_tensor(scales, n_scales), packed != 0).packing(1).contiguous();
        std::memcpy(out, q.raw_data(), (size_t)c * h * w);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -2; } catch (...) { g_err = "unknown"; return -4; }
}

REF_API int ref_dequantize(const int32_t* acc, int c, int h, int w, const float* scale_in, int n_scale,
                           const float* bias, int n_bias, int packed, float* out) {
    try {
        otter::Tensor a = otter::from_blob((void*)acc, {1, c, h, w}, otter::ScalarType::Int);
        if (packed && c % 4 == 0) a = a.packing(4);
        otter::Tensor b = n_bias ? vec_tensor(bias, n_bias) : otter::Tensor();
        otter::Tensor y = otter::dequantize_from_int32(a, vec_tensor(scale_in, n_scale), b, packed != 0).packing(1).contiguous();
        std::memcpy(out, y.raw_data(), (size_t)c * h * w * 4);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -2; } catch (...) { g_err = "unknown"; return -4; }
}

REF_API int ref_requantize(const int32_t* acc, int c, int h, int w, const float* scale_in, int n_scale_in,
                           const float* scale_out, int n_scale_out, const float* bias, int n_bias,
                           int act_type, float act_param0, int packed, int8_t* out) {
    try {
        otter::Tensor a = otter::from_blob((void*)acc, {1, c, h, w}, otter::ScalarType::Int);
        if (packed && c % 4 == 0) a = a.packing(4);
        otter::Tensor b = n_bias ? vec_tensor(bias, n_bias) : otter::Tensor();
        otter::Tensor ap = act_type == 2 ? vec_tensor(&act_param0, 1) : otter::Tensor();
        otter::Tensor y = otter::requantize_from_int32_to_int8(a, vec_tensor(scale_in, n_scale_in), vec_tensor(scale_out, n_scale_out),
                                                               b, act_type, ap, packed != 0).packing(1).contiguous();
        std::memcpy(out, y.raw_data(), (size_t)c * h * w);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -2; } catch (...) { g_err = "unknown"; return -4; }
}

// Any fp32 layer of the reference by its registry name ("MaxPool", "Concat", "Crop", "ChannelShuffle", "ShortCut",
// "Relu", "LRelu", "Relu6", ...), driven the way Net::compile / do_forward_layer drive it (Tensor/Net.cpp:196-273,
// :413-505). options = "key=value;key=value". Inputs and the output are fp32 NCHW with batch 1.
// shapes: 4 ints per input. out_shape receives 4 ints. out may be NULL to query the shape only.
#include "LayerRegistry.hpp"
REF_API int ref_layer_forward(const char* type, const char* options, int n_in, const float* const* ins, const int* shapes,
                              int packed, float* out, int* out_shape) {
    try {
        otter::Layer* layer = otter::LayerRegistry::CreateLayer(type);
        std::unique_ptr<otter::Layer> guard(layer);
        otter::LayerOption option;
        std::string s(options ? options : "");
        size_t pos = 0;
        while (pos < s.size()) {
            size_t end = s.find(';', pos);
            if (end == std::string::npos) end = s.size();
            const std::string item = s.substr(pos, end - pos);
            const size_t eq = item.find('=');
            if (eq != std::string::npos) option[item.substr(0, eq)] = item.substr(eq + 1);
            pos = end + 1;
        }
        otter::NetOption opt;
        opt.use_packing_layout = packed != 0;
        otter::ParamDict pd;
        layer->parse_param(option, pd);
        layer->bottom_shapes.clear();
        for (int i = 0; i < n_in; ++i)
            layer->bottom_shapes.push_back(otter::tensor({shapes[4 * i], shapes[4 * i + 1], shapes[4 * i + 2], shapes[4 * i + 3]}, otter::ScalarType::Int).view({1, -1}));
        layer->compute_output_shape(pd);
        layer->load_param(pd);
        layer->create_pipeline(opt);
        std::vector<otter::Tensor> bottoms;
        for (int i = 0; i < n_in; ++i) {
            otter::Tensor t = otter::from_blob((void*)ins[i], {shapes[4 * i], shapes[4 * i + 1], shapes[4 * i + 2], shapes[4 * i + 3]}, otter::ScalarType::Float).clone();
            if (packed && layer->support_packing) t = to_layer_layout(t, true, false);
            bottoms.push_back(t);
        }
        otter::Tensor top;
        int rc;
        if (layer->one_blob_only) {
            if (layer->support_inplace) { top = bottoms[0]; rc = layer->forward_inplace(top, opt); }
            else rc = layer->forward(bottoms[0], top, opt);
        } else {
            std::vector<otter::Tensor> tops(1);
            rc = layer->forward(bottoms, tops, opt);
            top = tops[0];
        }
        if (rc != 0) { g_err = "layer forward failed"; return rc; }
        otter::Tensor t1 = top.packing(1).contiguous();
        for (int i = 0; i < 4; ++i) out_shape[i] = i < t1.dim() ? (int)t1.size(i) : 1;  // e.g. [count, 6] from the detection layer
        if (out && t1.numel() > 0) std::memcpy(out, t1.raw_data(), (size_t)t1.numel() * 4);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -2; } catch (const char* s) { g_err = s; return -3; } catch (...) { g_err = "unknown"; return -4; }
}

// ---- the reference's whole Net (Tensor/Net.cpp) on a .otter graph, with caller-supplied convolution parameters ----
// Net keeps its layers private; this test driver reaches them to replace the random parameters CompileMode::Initial
// gives (the reference's own way in is a weight file). Access specifiers do not change object layout.
#define private public
#include "Net.hpp"
#undef private

namespace {
std::unique_ptr<otter::Net> g_net;
}

REF_API int ref_net_open(const char* otter_path, int packed) {
    try {
        g_net.reset(new otter::Net());
        g_net->option.use_packing_layout = packed != 0;
        g_net->option.lightmode = true;
        return g_net->load_otter(otter_path, otter::CompileMode::Initial);
    } catch (const std::exception& e) { g_err = e.what(); g_net.reset(); return -2; } catch (const char* s) { g_err = s; g_net.reset(); return -3; } catch (...) { g_err = "unknown"; g_net.reset(); return -4; }
}

// The reference's own way in for real models: graph from the .otter text, parameters from an ncnn-format weight file
// (Net::load_otter with CompileMode::Inference, then Net::load_weight(path, WeightType::Ncnn): Tensor/Net.cpp:518-607).
REF_API int ref_net_open_weights(const char* otter_path, const char* ncnn_bin_path, int packed) {
    try {
        g_net.reset(new otter::Net());
        g_net->option.use_packing_layout = packed != 0;
        g_net->option.lightmode = true;
        int rc = g_net->load_otter(otter_path, otter::CompileMode::Inference);
        if (rc != 0) { g_err = "load_otter failed"; return rc; }
        rc = g_net->load_weight(ncnn_bin_path, otter::Net::WeightType::Ncnn);
        if (rc != 0) g_err = "load_weight failed (or bytes were left over in the file)";
        return rc;
    } catch (const std::exception& e) { g_err = e.what(); g_net.reset(); return -2; } catch (const char* s) { g_err = s; g_net.reset(); return -3; } catch (...) { g_err = "unknown"; g_net.reset(); return -4; }
}

REF_API void ref_net_close() { g_net.reset(); }

REF_API int ref_net_set_conv(const char* layer_name, const int8_t* w_oihw, const float* bias, const float* w_scales, const float* in_scales,
                             int n_in_scales, const float* out_scales, int n_out_scales) {
    try {
        if (!g_net) { g_err = "no net"; return -1; }
        for (otter::Layer* l : g_net->layers) {
            if (l->name != layer_name) continue;
            auto* c = dynamic_cast<otter::ConvolutionLayer*>(l);
            if (!c) { g_err = "not a convolution"; return -1; }
            const int wsize = c->out_channels * (c->in_channels / c->groups) * c->kernel_height * c->kernel_width;
            c->weight_data = otter::empty({c->out_channels, c->in_channels / c->groups, c->kernel_height, c->kernel_width}, otter::ScalarType::Byte);
            std::memcpy(c->weight_data.raw_data(), w_oihw, wsize);
            if (c->bias_term) c->bias_data = vec_tensor(bias, c->out_channels);
            c->weight_data_int8_scales = vec_tensor(w_scales, c->out_channels);
            c->bottom_blob_int8_scales = vec_tensor(in_scales, n_in_scales);
            if (c->int8_scale_term > 100) c->top_blob_int8_scales = vec_tensor(out_scales, n_out_scales);
            return c->create_pipeline(g_net->option);
        }
        g_err = std::string("no layer named ") + layer_name;
        return -1;
    } catch (const std::exception& e) { g_err = e.what(); return -2; } catch (...) { g_err = "unknown"; return -4; }
}

// one image (the reference's int8 path is batch-1): fp32 NCHW in, the named blob out as fp32 NCHW
REF_API int ref_net_forward(const char* input_blob, const float* x, int c, int h, int w, const char* out_blob, float* out, int* out_shape) {
    try {
        if (!g_net) { g_err = "no net"; return -1; }
        otter::Extractor ex = g_net->create_extractor();
        otter::Tensor in = otter::from_blob((void*)x, {1, c, h, w}, otter::ScalarType::Float).clone();
        ex.input(input_blob, in);
        otter::Tensor feat;
        int rc = ex.extract(out_blob, feat, 0);
        if (rc != 0) { g_err = "extract failed"; return rc; }
        otter::Tensor t1 = feat.packing(1).contiguous();
        for (int i = 0; i < 4; ++i) out_shape[i] = i < t1.dim() ? (int)t1.size(i) : 1;
        if (out) std::memcpy(out, t1.raw_data(), (size_t)t1.numel() * 4);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -2; } catch (const char* s) { g_err = s; return -3; } catch (...) { g_err = "unknown"; return -4; }
}
