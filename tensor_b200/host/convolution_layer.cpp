// ConvolutionLayer of the host-side API mirror: the quantized (int8_scale_term != 0) layer of
// Tensor/ConvolutionLayer.cpp, with create_pipeline_int8 (:666-752) and forward_int8 (:754-847) handed to the
// CUDA library through its C-ABI. Option keys, ParamDict ids, shape rule and field names follow the reference
// (:58-206). The fp32 half of the layer (int8_scale_term == 0, :507-664) runs as one direct fp32 kernel: it is what a
// "mixed" quantized model keeps for its first convolution.
#include <cstring>
#include <random>
#include <sstream>

#include "otter_api.hpp"

namespace otter {

ConvolutionLayer::ConvolutionLayer() {
    one_blob_only = true;
    support_inplace = false;
    support_packing = true;
    accepts_tables = true;  // the planes of a Concat / Crop / ChannelShuffle result are read where they lie
}

ConvolutionLayer::~ConvolutionLayer() { release_gpu(); }

// Tensor/ConvolutionLayer.cpp:58-156
int ConvolutionLayer::parse_param(LayerOption& option, ParamDict& pd) {
    pd.clear();
    auto pair = [&](const char* both, const char* h, const char* w, int def, int& oh, int& ow) {
        oh = opt_find_int(option, h, -1);
        ow = opt_find_int(option, w, -1);
        const int b = opt_find_int(option, both, def);
        if (oh < 0) oh = b;
        if (ow < 0) ow = b;
    };
    int kh, kw, sh, sw, ph, pw, dh, dw, oph, opw;
    pair("kernel", "kernel_h", "kernel_w", 3, kh, kw);
    pair("stride", "stride_h", "stride_w", 1, sh, sw);
    pair("padding", "padding_h", "padding_w", 0, ph, pw);
    pair("dilation", "dilation_h", "dilation_w", 1, dh, dw);
    pair("output_padding", "output_padding_h", "output_padding_w", 0, oph, opw);
    int bias = opt_find(option, "batchnorm") ? 0 : 1;
    if (opt_find(option, "bias_term")) bias = option["bias_term"] == "false" ? 0 : 1;
    const std::string act = opt_find_string(option, "activation", "");
    int act_type = act == "Relu" ? 1 : act == "LRelu" ? 2 : act == "Relu6" ? 3 : act == "Sigmoid" ? 4 : 0;
    if (opt_find(option, "batchnorm")) act_type = 0;
    Tensor act_params;
    if (opt_check_string(option, "activation_params")) {
        const std::string& s = option["activation_params"];
        const int n = (int)std::count(s.begin(), s.end(), ',') + 1;
        act_params = empty({n}, ScalarType::Float);
        std::stringstream ss(s);
        for (int i = 0; i < n; ++i) {
            float v = 0;
            char comma;
            ss >> v >> comma;
            act_params.data_ptr<float>()[i] = v;
        }
    }
    pd.set((int)ConvParam::In_channels, opt_find_int(option, "in_channels", 1));
    pd.set((int)ConvParam::Out_channels, opt_find_int(option, "out_channels", 1));
    pd.set((int)ConvParam::Kernel_height, kh);
    pd.set((int)ConvParam::Kernel_width, kw);
    pd.set((int)ConvParam::Stride_height, sh);
    pd.set((int)ConvParam::Stride_width, sw);
    pd.set((int)ConvParam::Padding_height, ph);
    pd.set((int)ConvParam::Padding_width, pw);
    pd.set((int)ConvParam::Dilation_height, dh);
    pd.set((int)ConvParam::Dilation_width, dw);
    pd.set((int)ConvParam::Output_padding_height, oph);
    pd.set((int)ConvParam::Output_padding_width, opw);
    pd.set((int)ConvParam::Group, opt_find_int(option, "groups", 1));
    pd.set((int)ConvParam::Bias_term, bias);
    pd.set((int)ConvParam::Int8_scale_term, opt_find_int(option, "int8_scale_term", 0));
    pd.set((int)ConvParam::Activation_type, act_type);
    if (act_params.defined()) pd.set((int)ConvParam::Activation_params, act_params);
    return 0;
}

// Tensor/ConvolutionLayer.cpp:158-183
int ConvolutionLayer::compute_output_shape(ParamDict& pd) {
    if (bottom_shapes.empty() || !bottom_shapes[0].defined()) return -1;
    int n, c, h, w;
    read_shape(bottom_shapes[0], n, c, h, w);
    const int oc = pd.get((int)ConvParam::Out_channels, 1);
    const int kh = pd.get((int)ConvParam::Kernel_height, 3), kw = pd.get((int)ConvParam::Kernel_width, 3);
    const int sh = pd.get((int)ConvParam::Stride_height, 1), sw = pd.get((int)ConvParam::Stride_width, 1);
    const int ph = pd.get((int)ConvParam::Padding_height, 0), pw = pd.get((int)ConvParam::Padding_width, 0);
    const int dh = pd.get((int)ConvParam::Dilation_height, 1), dw = pd.get((int)ConvParam::Dilation_width, 1);
    const int g = pd.get((int)ConvParam::Group, 1);
    const int ow = (w + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
    const int oh = (h + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
    pd.set((int)ConvParam::In_channels, c);
    pd.set((int)ConvParam::Weight_data_size, c / g * kh * kw * oc);
    pd.set(OUTPUT_SHAPE_HINT, shape_tensor(n, oc, oh, ow));
    return 0;
}

// Tensor/ConvolutionLayer.cpp:185-206
int ConvolutionLayer::load_param(const ParamDict& pd) {
    in_channels = pd.get((int)ConvParam::In_channels, 1);
    out_channels = pd.get((int)ConvParam::Out_channels, 1);
    kernel_height = pd.get((int)ConvParam::Kernel_height, 3);
    kernel_width = pd.get((int)ConvParam::Kernel_width, 3);
    stride_height = pd.get((int)ConvParam::Stride_height, 1);
    stride_width = pd.get((int)ConvParam::Stride_width, 1);
    padding_height = pd.get((int)ConvParam::Padding_height, 0);
    padding_width = pd.get((int)ConvParam::Padding_width, 0);
    dilation_height = pd.get((int)ConvParam::Dilation_height, 1);
    dilation_width = pd.get((int)ConvParam::Dilation_width, 1);
    output_padding_height = pd.get((int)ConvParam::Output_padding_height, 0);
    output_padding_width = pd.get((int)ConvParam::Output_padding_width, 0);
    groups = pd.get((int)ConvParam::Group, 1);
    bias_term = pd.get((int)ConvParam::Bias_term, 0);
    weight_data_size = pd.get((int)ConvParam::Weight_data_size, 0);
    int8_scale_term = pd.get((int)ConvParam::Int8_scale_term, 0);
    activation_type = pd.get((int)ConvParam::Activation_type, 0);
    activation_params = pd.get((int)ConvParam::Activation_params, Tensor());
    return 0;
}

// Random parameters of the right shapes, as CompileMode::Initial gives in the reference
// (Tensor/ConvolutionLayer.cpp:208-243: int8 weights, [groups] or [1] activation scales, [Cout] weight scales).
// Deterministic here: the generator is seeded from the layer name.
int ConvolutionLayer::init_model() {
    std::mt19937 rng((unsigned)std::hash<std::string>{}(name) ^ 0x0771E5u);
    if (!int8_scale_term) {  // the fp32 layer: fp32 weights of the right shape
        std::normal_distribution<float> nd(0.f, 0.05f);
        weight_data = empty({out_channels, in_channels / groups, kernel_height, kernel_width}, ScalarType::Float);
        for (int64_t i = 0; i < weight_data.numel(); ++i) weight_data.data_ptr<float>()[i] = nd(rng);
        if (bias_term) {
            bias_data = empty({out_channels}, ScalarType::Float);
            for (int i = 0; i < out_channels; ++i) bias_data.data_ptr<float>()[i] = 0.1f * nd(rng);
        }
        return 0;
    }
    std::uniform_int_distribution<int> wd(-127, 127);
    std::uniform_real_distribution<float> u(0.f, 1.f);
    const bool depthwise = in_channels == groups && groups == out_channels && groups > 1;
    weight_data = empty({out_channels, in_channels / groups, kernel_height, kernel_width}, ScalarType::Byte);
    for (int64_t i = 0; i < weight_data.numel(); ++i) weight_data.data_ptr<int8_t>()[i] = (int8_t)wd(rng);
    if (bias_term) {
        bias_data = empty({out_channels}, ScalarType::Float);
        for (int i = 0; i < out_channels; ++i) bias_data.data_ptr<float>()[i] = u(rng) - 0.5f;
    }
    weight_data_int8_scales = empty({out_channels}, ScalarType::Float);
    for (int i = 0; i < out_channels; ++i) weight_data_int8_scales.data_ptr<float>()[i] = 50.f + 200.f * u(rng);
    const float s_in = 20.f + 100.f * u(rng);
    bottom_blob_int8_scales = full({depthwise ? groups : 1}, s_in, ScalarType::Float);
    if (int8_scale_term > 100) top_blob_int8_scales = full({depthwise ? groups : 1}, 5.f + 20.f * u(rng), ScalarType::Float);
    return 0;
}

// Tensor/ConvolutionLayer.cpp:245-296. Order of the values in an ncnn file: weights (tagged), bias, weight scales, the
// input scale, and for a requantizing layer the output scale. Depthwise layers replicate the scalar scales to [groups];
// int8_scale_term 2 / 102 on a depthwise layer means one weight scale for all channels.
int ConvolutionLayer::load_model(const Initializer& initializer) {
    const bool ncnn = initializer.type == InitializerType::Ncnn;
    if (!ncnn && bias_term) bias_data = initializer.load({out_channels}, 1);
    weight_data = initializer.load({out_channels, in_channels / groups, kernel_height, kernel_width}, 0);
    if (!weight_data.defined()) return -1;
    if (!ncnn) return 0;
    if (bias_term) {
        bias_data = initializer.load({out_channels}, 1);
        if (!bias_data.defined()) return -1;
    }
    auto scalar_to = [&](int n) {
        Tensor one = initializer.load({1}, 1);
        return one.defined() ? full({n}, one.data_ptr<float>()[0], ScalarType::Float) : Tensor();
    };
    if (!int8_scale_term) return 0;
    if (in_channels == groups && groups == out_channels) {
        if (int8_scale_term == 1 || int8_scale_term == 101) {
            weight_data_int8_scales = initializer.load({groups}, 1);
            bottom_blob_int8_scales = scalar_to(groups);
        } else {
            weight_data_int8_scales = scalar_to(groups);
            bottom_blob_int8_scales = scalar_to(groups);
        }
        if (int8_scale_term > 100) top_blob_int8_scales = scalar_to(groups);
    } else {
        weight_data_int8_scales = initializer.load({out_channels}, 1);
        bottom_blob_int8_scales = initializer.load({1}, 1);
        if (int8_scale_term > 100) top_blob_int8_scales = initializer.load({1}, 1);
    }
    if (!weight_data_int8_scales.defined() || !bottom_blob_int8_scales.defined()) return -1;
    if (int8_scale_term > 100 && !top_blob_int8_scales.defined()) return -1;
    return 0;
}

// Tensor/ConvolutionLayer.cpp:298-304 -> create_pipeline_int8 (:666-752)
int ConvolutionLayer::create_pipeline(const NetOption& opt) {
    if (!opt.gpu) return -1;
    if (!int8_scale_term) {
        // Tensor/ConvolutionLayer.cpp:298-503: the fp32 layer. One kernel, no weight transforms to choose from.
        if (!weight_data.defined() || weight_data.scalar_type() != ScalarType::Float) return -1;
        if (bias_term && !bias_data.defined()) return -1;
        release_gpu();
        gpu_ctx_ = opt.gpu;
        ott_conv_desc d{};
        d.cin = in_channels; d.cout = out_channels; d.kh = kernel_height; d.kw = kernel_width;
        d.sh = stride_height; d.sw = stride_width; d.ph = padding_height; d.pw = padding_width;
        d.dh = dilation_height; d.dw = dilation_width; d.groups = groups; d.bias_term = bias_term;
        d.int8_scale_term = 0; d.act_type = activation_type;
        d.act_param0 = activation_params.defined() ? activation_params.data_ptr<float>()[0] : (activation_type == 2 ? 0.1f : 0.f);
        return ott_conv_f32_create(opt.gpu, &d, weight_data.data_ptr<float>(), bias_term ? bias_data.data_ptr<float>() : nullptr, &gpu_conv_f32_);
    }
    if (weight_data.defined() && weight_data.scalar_type() != ScalarType::Byte) return -1;  // int8 layer with fp32 weights
    if (!weight_data.defined() || !weight_data_int8_scales.defined() || !bottom_blob_int8_scales.defined()) return -1;
    release_gpu();
    gpu_ctx_ = opt.gpu;
    // scale_in_data is kept as a public field like the reference's (ConvolutionLayer.cpp:667-679); the library
    // computes the same values from the same inputs for its own use
    scale_in_data = empty({out_channels}, ScalarType::Float);
    for (int p = 0; p < out_channels; ++p) {
        const float ws = weight_data_int8_scales.data_ptr<float>()[p];
        volatile float prod = bottom_blob_int8_scales.data_ptr<float>()[0] * ws;
        scale_in_data.data_ptr<float>()[p] = ws == 0.f ? 0.f : 1.f / prod;
    }
    const bool requant = int8_scale_term > 100;
    int rc = make_gpu_conv(opt, int8_scale_term, requant ? top_blob_int8_scales : Tensor(), &gpu_conv_);
    if (rc != 0) return rc;
    if (!requant && handover_scales.defined()) rc = make_gpu_conv(opt, 101, handover_scales, &gpu_conv_handover_);
    return rc;
}

int ConvolutionLayer::make_gpu_conv(const NetOption& opt, int scale_term, const Tensor& top_scales, ott_conv** out) const {
    ott_conv_desc d{};
    d.cin = in_channels; d.cout = out_channels; d.kh = kernel_height; d.kw = kernel_width;
    d.sh = stride_height; d.sw = stride_width; d.ph = padding_height; d.pw = padding_width;
    d.dh = dilation_height; d.dw = dilation_width; d.groups = groups; d.bias_term = bias_term;
    d.int8_scale_term = scale_term; d.act_type = activation_type;
    d.act_param0 = activation_params.defined() ? activation_params.data_ptr<float>()[0] : (activation_type == 2 ? 0.1f : 0.f);
    d.rounding = opt.int8_rounding;
    const bool requant = scale_term > 100;
    if (requant && !top_scales.defined()) return -1;
    return ott_conv_int8_create(opt.gpu, &d, weight_data.data_ptr<int8_t>(), bias_term ? bias_data.data_ptr<float>() : nullptr,
                                weight_data_int8_scales.data_ptr<float>(), bottom_blob_int8_scales.data_ptr<float>(),
                                (int)bottom_blob_int8_scales.numel(), requant ? top_scales.data_ptr<float>() : nullptr,
                                requant ? (int)top_scales.numel() : 0, out);
}

void ConvolutionLayer::release_gpu() {
    set_pair_fusion(NetOption(), nullptr, -1);
    if (gpu_conv_) ott_conv_int8_destroy(gpu_ctx_, gpu_conv_);
    if (gpu_conv_handover_) ott_conv_int8_destroy(gpu_ctx_, gpu_conv_handover_);
    if (gpu_conv_routed_) ott_conv_int8_destroy(gpu_ctx_, gpu_conv_routed_);
    if (gpu_conv_f32_) ott_conv_f32_destroy(gpu_ctx_, gpu_conv_f32_);
    gpu_conv_ = gpu_conv_handover_ = gpu_conv_routed_ = nullptr;
    gpu_conv_f32_ = nullptr;
}

bool ConvolutionLayer::routable_consumer() const {
    return gpu_conv_ && int8_scale_term > 0 && groups == 1 && kernel_height == 1 && kernel_width == 1 && stride_height == 1 &&
           stride_width == 1 && padding_height == 0 && padding_width == 0 && !fused_maxpool &&
           bottom_blob_int8_scales.defined() && bottom_blob_int8_scales.numel() == 1 &&
           ott_conv_int8_kernel_kind(gpu_conv_) == OTT_KERNEL_DENSE_UMMA;
}

bool ConvolutionLayer::routable_depthwise_reader() const {
    if (!gpu_conv_ || int8_scale_term <= 100 || groups <= 16 || groups != in_channels || groups != out_channels) return false;
    if (kernel_height != kernel_width || (kernel_height != 3 && kernel_height != 5) || stride_height != stride_width ||
        (stride_height != 1 && stride_height != 2) || dilation_height != 1 || dilation_width != 1)
        return false;
    if (!bottom_blob_int8_scales.defined() || !top_blob_int8_scales.defined()) return false;
    for (int64_t i = 1; i < bottom_blob_int8_scales.numel(); ++i)
        if (bottom_blob_int8_scales.data_ptr<float>()[i] != bottom_blob_int8_scales.data_ptr<float>()[0]) return false;
    return true;
}

bool ConvolutionLayer::routable_producer() const {
    if (!gpu_conv_ || int8_scale_term <= 0 || int8_scale_term >= 100 || groups != 1 || ott_nhwc_channels(out_channels) < 32) return false;
    if (fused_maxpool) return true;  // the first-layer + max-pool kernel: all of its channels or none (routes_all_or_nothing)
    return out_channels <= 1024 && ott_conv_int8_kernel_kind(gpu_conv_) == OTT_KERNEL_DENSE_UMMA;
}

// The routed twin of the layer: its input gathered from the producers' int8 tensors and / or its output channels quantized
// for their readers. Same arithmetic as the plain layer; only where the bytes come from and go to differs.
int ConvolutionLayer::set_routing(const NetOption& opt, const Routing* plan) {
    if (gpu_conv_routed_) {
        ott_conv_int8_destroy(gpu_ctx_, gpu_conv_routed_);
        gpu_conv_routed_ = nullptr;
    }
    routing_ = Routing();
    if (!plan || (!plan->gathered && !plan->routed_out) || !gpu_conv_) return 0;
    ott_conv_desc d{};
    d.cin = in_channels; d.cout = out_channels; d.kh = kernel_height; d.kw = kernel_width;
    d.sh = stride_height; d.sw = stride_width; d.ph = padding_height; d.pw = padding_width;
    d.dh = dilation_height; d.dw = dilation_width; d.groups = groups; d.bias_term = bias_term;
    d.int8_scale_term = plan->routed_out ? 101 : int8_scale_term;
    d.act_type = activation_type;
    d.act_param0 = activation_params.defined() ? activation_params.data_ptr<float>()[0] : (activation_type == 2 ? 0.1f : 0.f);
    d.rounding = opt.int8_rounding;
    const bool requant = d.int8_scale_term > 100;
    const float* out_scales = nullptr;
    int n_out = 0;
    if (plan->routed_out) {
        if ((int)plan->out_scales.size() != out_channels) return -1;
        out_scales = plan->out_scales.data();
        n_out = out_channels;
    } else if (requant) {
        if (!top_blob_int8_scales.defined()) return -1;
        out_scales = top_blob_int8_scales.data_ptr<float>();
        n_out = (int)top_blob_int8_scales.numel();
    }
    const float* bias = bias_term ? bias_data.data_ptr<float>() : nullptr;
    int rc;
    if (plan->gathered)
        rc = ott_conv_int8_create_gathered(opt.gpu, &d, weight_data.data_ptr<int8_t>(), bias, weight_data_int8_scales.data_ptr<float>(),
                                           bottom_blob_int8_scales.data_ptr<float>(), (int)bottom_blob_int8_scales.numel(), out_scales, n_out,
                                           (int)plan->source_layers.size(), plan->source_channels.data(), plan->channel_source.data(),
                                           plan->channel_index.data(), &gpu_conv_routed_);
    else
        rc = ott_conv_int8_create(opt.gpu, &d, weight_data.data_ptr<int8_t>(), bias, weight_data_int8_scales.data_ptr<float>(),
                                  bottom_blob_int8_scales.data_ptr<float>(), (int)bottom_blob_int8_scales.numel(), out_scales, n_out,
                                  &gpu_conv_routed_);
    if (rc != 0) return rc;
    routing_ = *plan;
    if (plan->gathered && groups > 1) {
        routing_.position.assign((size_t)out_channels, 0);
        ott_conv_int8_gathered_layout(gpu_conv_routed_, &routing_.stored_channels, routing_.position.data(), out_channels);
    }
    return 0;
}

// An fp32 NCHW tensor of the given logical shape none of whose planes is ever read or written: the blob of a layer all of
// whose channels travel in the int8 companion (plane tables still need a tensor to point into).
static Tensor device_shell(const NetOption& opt, std::vector<int64_t> sizes) {
    void* p = nullptr;
    if (!opt.gpu || ott_malloc(opt.gpu, 16, &p) != OTT_OK) return Tensor();
    ott_ctx* ctx = opt.gpu;
    return Tensor::wrap(p, 16, Device::CUDA, [ctx](void* q) { ott_free(ctx, q); }, std::move(sizes), ScalarType::Float, Layout::NCHW);
}

int ConvolutionLayer::routed_input(const Tensor& bottom_blob, const NetOption& opt, ott_conv_io& io, std::vector<const int8_t*>& srcs, Tensor& hold) const {
    const Routing& R = routing_;
    Tensor src = bottom_blob;
    if (R.gathered && R.direct) {
        // the output of the depthwise layer in front, in that layer's stored channel order
        if (src.scalar_type() != ScalarType::Byte || src.layout() != Layout::NHWC16 || (int)src.size(1) != R.source_channels[0]) return -1;
        srcs.assign(1, src.data_ptr<int8_t>());
        io.sources = srcs.data();
        io.n_sources = 1;
        io.in_dtype = OTT_S8_NHWC;
    } else if (R.gathered) {
        // the producers' int8 tensors, found through the plane table (or the plain tensor) the glue layers handed down; the
        // table must say exactly what the plan was made for
        const bool table = src.is_table();
        const size_t nbuf = table ? src.table_bufs().size() : 1;
        auto buf = [&](size_t b) -> const Tensor& { return table ? src.table_bufs()[b] : src; };
        srcs.assign(R.source_layers.size(), nullptr);
        for (size_t s = 0; s < R.source_layers.size(); ++s)
            for (size_t b = 0; b < nbuf; ++b)
                if (buf(b).companion_tag() == R.source_layers[s]) srcs[s] = buf(b).companion()->data_ptr<int8_t>();
        for (int i = 0; i < in_channels; ++i) {
            const uint32_t ref = table ? src.table_refs()[(size_t)i] : (uint32_t)i;
            const Tensor& b = buf(ref >> 24);
            const int s = R.channel_source[(size_t)i];
            if (!srcs[(size_t)s] || b.companion_tag() != R.source_layers[(size_t)s] || (int)(ref & 0xFFFFFFu) != R.channel_index[(size_t)i] ||
                (int)b.size(1) != R.source_channels[(size_t)s])
                return -1;  // not the graph this layer was planned for
        }
        io.sources = srcs.data();
        io.n_sources = (int)srcs.size();
        io.in_dtype = OTT_S8_NHWC;
    } else {
        if (src.is_table()) {
            src = materialize(opt, src);
            if (!src.defined()) return -100;
        }
        if (src.scalar_type() == ScalarType::Float && src.layout() == Layout::NCHW) io.in_dtype = OTT_F32_NCHW;
        else if (src.scalar_type() == ScalarType::Byte && src.layout() == Layout::NHWC16) io.in_dtype = OTT_S8_NHWC;
        else return -1;
        io.in_dev = src.raw_data();
        hold = src;
    }
    return 0;
}

int ConvolutionLayer::routed_output(const NetOption& opt, int n, int oh, int ow, ott_conv_io& io, Tensor& top_blob) const {
    const Routing& R = routing_;
    const bool requant = R.routed_out || int8_scale_term > 100;
    Tensor s8;
    if (requant) {
        s8 = device_empty(opt, {n, R.stored_channels > 0 ? R.stored_channels : out_channels, oh, ow}, ScalarType::Byte, Layout::NHWC16);
        if (!s8.defined()) return -100;
    }
    if (R.routed_out) {
        // the fp32 blob of the layer: only the planes named in f32_mask are written, which are the only ones anyone reads
        bool any = false;
        for (uint32_t m : R.f32_mask) any = any || m != 0u;
        top_blob = any ? device_empty(opt, {n, out_channels, oh, ow}, ScalarType::Float, Layout::NCHW) : device_shell(opt, {n, out_channels, oh, ow});
        if (!top_blob.defined()) return -100;
        top_blob.set_companion(s8, R.self_layer);
        io.out_dev = s8.raw_data();
        io.out_dtype = OTT_S8_NHWC;
        if (any) {
            io.out_f32_dev = top_blob.data_ptr<float>();
            io.f32_channel_mask = R.f32_mask.data();
        }
    } else if (requant) {
        top_blob = s8;
        io.out_dev = s8.raw_data();
        io.out_dtype = OTT_S8_NHWC;
    } else {
        top_blob = device_empty(opt, {n, out_channels, oh, ow}, ScalarType::Float, Layout::NCHW);
        if (!top_blob.defined()) return -100;
        io.out_dev = top_blob.raw_data();
        io.out_dtype = OTT_F32_NCHW;
    }
    return 0;
}

int ConvolutionLayer::forward_routed(const Tensor& bottom_blob, Tensor& top_blob, const NetOption& opt) const {
    const Routing& R = routing_;
    const int n = (int)bottom_blob.size(0), h = (int)bottom_blob.size(2), w = (int)bottom_blob.size(3);
    int oh = 0, ow = 0;
    ott_conv_int8_out_shape(gpu_conv_routed_, h, w, &oh, &ow);
    if (fused_maxpool) {
        // first layer + max-pool: the pooled values leave quantized for the layers that read the pooled blob
        if (bottom_blob.is_table() || bottom_blob.scalar_type() != ScalarType::Float || !R.routed_out) return -1;
        const int ph = (oh - 1) / 2 + 1, pw = (ow - 1) / 2 + 1;
        Tensor q = device_empty(opt, {n, out_channels, ph, pw}, ScalarType::Byte, Layout::NHWC16);
        top_blob = device_shell(opt, {n, out_channels, ph, pw});
        if (!q.defined() || !top_blob.defined()) return -100;
        top_blob.set_companion(q, R.self_layer);
        return ott_conv_int8_forward_maxpool_s8(opt.gpu, gpu_conv_routed_, bottom_blob.data_ptr<float>(), n, h, w, fused_maxpool == 2 ? 1 : 0,
                                                q.data_ptr<int8_t>());
    }
    ott_conv_io io{};
    std::vector<const int8_t*> srcs;
    Tensor hold;
    int rc = routed_input(bottom_blob, opt, io, srcs, hold);
    if (rc == 0) rc = routed_output(opt, n, oh, ow, io, top_blob);
    if (rc != 0) return rc;
    return ott_conv_int8_forward_io(opt.gpu, gpu_conv_routed_, &io, n, h, w, nullptr);
}

// ---- depthwise + 1x1 pair fusion ----
int ConvolutionLayer::set_pair_fusion(const NetOption& opt, ConvolutionLayer* dw, int dw_index) {
    if (pair_plain_ && pair_plain_ != pair_routed_) ott_dwpw_int8_destroy(gpu_ctx_, pair_plain_);
    if (pair_routed_) ott_dwpw_int8_destroy(gpu_ctx_, pair_routed_);
    pair_plain_ = pair_routed_ = nullptr;
    if (pair_front_) const_cast<ConvolutionLayer*>(pair_front_)->pair_next_ = nullptr;
    if (pair_next_) {  // (a depthwise layer being released: its reader must not run the pair any more)
        ConvolutionLayer* next = const_cast<ConvolutionLayer*>(pair_next_);
        pair_next_ = nullptr;
        next->pair_front_ = nullptr;
        next->set_pair_fusion(opt, nullptr, -1);
    }
    pair_front_ = nullptr;
    pair_tag_ = -1;
    if (!dw || !opt.gpu || !gpu_conv_ || !dw->gpu_conv_) return 0;
    auto make = [&](const ott_conv* dc, const ott_conv* pc, ott_dwpw** out) -> int {
        *out = nullptr;
        if (!dc || !pc) return 0;
        const int rc = ott_dwpw_int8_create(opt.gpu, dc, pc, out);
        return rc == OTT_ERR_UNSUPPORTED ? 0 : rc;  // a pair the library cannot fuse runs as two layers
    };
    // the layer objects forward() would run with routing off (a layer with an int8 hand-over twin picks per call: not fused)
    const ott_conv* p_plain = gpu_conv_handover_ ? nullptr : gpu_conv_;
    const ott_conv* d_plain = dw->gpu_conv_handover_ ? nullptr : dw->gpu_conv_;
    // ... and with routing on
    const ott_conv* p_routed = gpu_conv_routed_ ? gpu_conv_routed_ : p_plain;
    const ott_conv* d_routed = dw->gpu_conv_routed_ ? dw->gpu_conv_routed_ : d_plain;
    int rc = make(d_plain, p_plain, &pair_plain_);
    if (rc != 0) return rc;
    if (d_routed == d_plain && p_routed == p_plain) pair_routed_ = pair_plain_;
    else rc = make(d_routed, p_routed, &pair_routed_);
    if (rc != 0) return rc;
    if (pair_plain_ || pair_routed_) {
        pair_front_ = dw;
        dw->pair_next_ = this;
        pair_tag_ = dw->pair_tag_ = kDeferredTag + dw_index;
    }
    return 0;
}

// (on the depthwise layer) may this call leave the work to the 1x1 layer behind? Only when that layer's fused state exists for
// the mode of this call, nobody wants this layer's own blob, and the input is int8 already.
bool ConvolutionLayer::defers(const Tensor& bottom_blob, const NetOption& opt) const {
    if (!pair_next_ || !opt.fuse_depthwise_pointwise || tops.empty() || opt.layer_ms) return false;
    const bool routed = opt.routing_active;
    if (!pair_next_->pair_ready(routed)) return false;
    if (opt.blob_wanted == tops[0] || (opt.keep_blobs && (*opt.keep_blobs)[(size_t)tops[0]])) return false;
    if (routed && gpu_conv_routed_ && routing_.gathered && !routing_.direct) return true;  // reads its producers' int8 tensors
    return !bottom_blob.is_table() && bottom_blob.scalar_type() == ScalarType::Byte && bottom_blob.layout() == Layout::NHWC16 &&
           (int)bottom_blob.size(1) == in_channels;
}

// (on the 1x1 layer) both layers in one launch: the input side is the depthwise layer's, the output side this layer's
int ConvolutionLayer::forward_pair(const Tensor& dwb, Tensor& top_blob, const NetOption& opt) const {
    const ConvolutionLayer* dw = pair_front_;
    const bool routed = opt.routing_active;
    const ott_dwpw* pair = routed ? pair_routed_ : pair_plain_;
    if (!dw || !pair || !dwb.defined() || dwb.dim() != 4) return -1;
    const int n = (int)dwb.size(0), h = (int)dwb.size(2), w = (int)dwb.size(3);
    const int oh = (h + 2 - 3) / dw->stride_height + 1, ow = (w + 2 - 3) / dw->stride_width + 1;
    ott_conv_io io{};
    std::vector<const int8_t*> srcs;
    Tensor hold;
    int rc = 0;
    if (routed && dw->gpu_conv_routed_) {
        rc = dw->routed_input(dwb, opt, io, srcs, hold);
        if (rc == 0 && io.in_dtype != OTT_S8_NHWC) rc = -1;
    } else {
        if (dwb.is_table() || dwb.scalar_type() != ScalarType::Byte || dwb.layout() != Layout::NHWC16) return -1;
        io.in_dev = dwb.raw_data();
        io.in_dtype = OTT_S8_NHWC;
    }
    if (rc != 0) return rc;
    if (routed && gpu_conv_routed_) {
        rc = routed_output(opt, n, oh, ow, io, top_blob);
        if (rc != 0) return rc;
    } else {
        const bool requant = int8_scale_term > 100;
        top_blob = device_empty(opt, {n, out_channels, oh, ow}, requant ? ScalarType::Byte : ScalarType::Float, requant ? Layout::NHWC16 : Layout::NCHW);
        if (!top_blob.defined()) return -100;
        io.out_dev = top_blob.raw_data();
        io.out_dtype = requant ? OTT_S8_NHWC : OTT_F32_NCHW;
    }
    return ott_dwpw_int8_forward_io(opt.gpu, pair, &io, n, h, w, nullptr);
}

// The consumer quantizes its fp32 input with float2int8(v * scale) (Tensor/QuantizeX86.cpp:23-71, called from
// ConvolutionLayer.cpp:763-779); the requantizing epilogue ends with float2int8(v * scale_out) on the same fp32 v
// (Tensor/QuantizeX86.cpp:1723-1870). With scale_out = the consumer's input scale the two give the same bytes, so the fp32
// blob between the two layers need not exist.
int ConvolutionLayer::set_handover(const NetOption& opt, const Tensor& consumer_input_scales) {
    handover_scales = consumer_input_scales;
    if (gpu_conv_handover_) {
        ott_conv_int8_destroy(gpu_ctx_, gpu_conv_handover_);
        gpu_conv_handover_ = nullptr;
    }
    if (!handover_scales.defined() || !gpu_conv_ || int8_scale_term > 100) return 0;
    return make_gpu_conv(opt, 101, handover_scales, &gpu_conv_handover_);
}

bool ConvolutionLayer::can_fuse_maxpool() const {
    return int8_scale_term > 0 && int8_scale_term < 100 && groups == 1 && in_channels == 3 && kernel_height == 3 && kernel_width == 3 &&
           dilation_height == 1 && dilation_width == 1 && stride_height == stride_width && (stride_height == 1 || stride_height == 2) &&
           ott_nhwc_channels(out_channels) <= 32;
}

// Tensor/ConvolutionLayer.cpp:507-511 -> forward_int8 (:754-847). Device tensors in and out; asynchronous.
int ConvolutionLayer::forward(const Tensor& bottom_blob, Tensor& top_blob, const NetOption& opt) const {
    if (gpu_conv_f32_) {
        if (!bottom_blob.defined() || bottom_blob.device() != Device::CUDA || bottom_blob.dim() != 4 || bottom_blob.scalar_type() != ScalarType::Float ||
            (int)bottom_blob.size(1) != in_channels)
            return -1;
        Tensor src = materialize(opt, bottom_blob);
        if (!src.defined()) return -100;
        const int n = (int)src.size(0), h = (int)src.size(2), w = (int)src.size(3);
        const int oh = (h + 2 * padding_height - dilation_height * (kernel_height - 1) - 1) / stride_height + 1;
        const int ow = (w + 2 * padding_width - dilation_width * (kernel_width - 1) - 1) / stride_width + 1;
        top_blob = device_empty(opt, {n, out_channels, oh, ow}, ScalarType::Float, Layout::NCHW);
        if (!top_blob.defined()) return -100;
        return ott_conv_f32_forward(opt.gpu, gpu_conv_f32_, src.data_ptr<float>(), n, h, w, top_blob.data_ptr<float>());
    }
    if (!gpu_conv_ || !bottom_blob.defined() || bottom_blob.device() != Device::CUDA || bottom_blob.dim() != 4) return -1;
    // a deferred depthwise layer in front: its input arrives as the companion of an empty shell, and this layer runs both
    if (pair_front_ && bottom_blob.companion_tag() == pair_tag_) return forward_pair(*bottom_blob.companion(), top_blob, opt);
    const int n = (int)bottom_blob.size(0), c = (int)bottom_blob.size(1), h = (int)bottom_blob.size(2), w = (int)bottom_blob.size(3);
    if (defers(bottom_blob, opt)) {
        // this depthwise layer runs inside the 1x1 layer behind it: hand the input on
        const int oh = (h + 2 - 3) / stride_height + 1, ow = (w + 2 - 3) / stride_width + 1;
        top_blob = device_shell(opt, {n, out_channels, oh, ow});
        if (!top_blob.defined()) return -100;
        top_blob.set_companion(bottom_blob, pair_tag_);
        return 0;
    }
    if (opt.routing_active && gpu_conv_routed_) return forward_routed(bottom_blob, top_blob, opt);
    if (c != in_channels) return -1;
    int oh = 0, ow = 0;
    ott_conv_int8_out_shape(gpu_conv_, h, w, &oh, &ow);
    // int8 hand-over: the only reader of the top blob is a quantized convolution, and nobody asked for the blob itself
    const bool handover = gpu_conv_handover_ && opt.int8_handover && !tops.empty() && opt.blob_wanted != tops[0];
    const bool requant = int8_scale_term > 100 || handover;
    const ott_conv* conv = handover ? gpu_conv_handover_ : gpu_conv_;
    const int out_dtype = requant ? OTT_S8_NHWC : OTT_F32_NCHW;
    if (fused_maxpool && !bottom_blob.is_table() && bottom_blob.scalar_type() == ScalarType::Float) {
        top_blob = device_empty(opt, {n, out_channels, (oh - 1) / 2 + 1, (ow - 1) / 2 + 1}, ScalarType::Float, Layout::NCHW);
        if (!top_blob.defined()) return -100;
        return ott_conv_int8_forward_maxpool(opt.gpu, gpu_conv_, bottom_blob.data_ptr<float>(), n, h, w, fused_maxpool == 2 ? 1 : 0,
                                             top_blob.data_ptr<float>());
    }
    Tensor src = bottom_blob;
    std::vector<const float*> bufs;
    std::vector<int64_t> strides;
    if (src.is_table() && !table_arrays(src, bufs, strides)) {
        src = materialize(opt, src);  // more buffers or channels than one kernel table holds
        if (!src.defined()) return -100;
    }
    top_blob = device_empty(opt, {n, out_channels, oh, ow}, requant ? ScalarType::Byte : ScalarType::Float,
                            requant ? Layout::NHWC16 : Layout::NCHW);
    if (!top_blob.defined()) return -100;
    if (src.is_table())
        return ott_conv_int8_forward_gather(opt.gpu, conv, bufs.data(), strides.data(), (int)bufs.size(), src.table_refs().data(), n, h, w,
                                            top_blob.raw_data(), out_dtype, nullptr);
    int in_dtype;
    if (src.scalar_type() == ScalarType::Float && src.layout() == Layout::NCHW) in_dtype = OTT_F32_NCHW;
    else if (src.scalar_type() == ScalarType::Byte && src.layout() == Layout::NHWC16) in_dtype = OTT_S8_NHWC;
    else return -1;
    return ott_conv_int8_forward(opt.gpu, conv, src.raw_data(), in_dtype, n, h, w, top_blob.raw_data(), out_dtype, nullptr);
}

// ---- Input (Tensor/InputLayer.cpp:19-71): declares the shape of a graph input; the blob is set by Extractor::input ----
class InputLayer : public Layer {
public:
    InputLayer() { one_blob_only = true; support_inplace = true; }
    int parse_param(LayerOption& option, ParamDict& pd) override {
        pd.clear();
        pd.set(0, opt_find_int(option, "batchsize", 1));
        pd.set(1, opt_find_int(option, "channel", 1));
        pd.set(2, opt_find_int(option, "height", 1));
        pd.set(3, opt_find_int(option, "width", 1));
        return 0;
    }
    int compute_output_shape(ParamDict& pd) override {
        pd.set(OUTPUT_SHAPE_HINT, shape_tensor(pd.get(0, 1), pd.get(1, 1), pd.get(2, 1), pd.get(3, 1)));
        return 0;
    }
    int forward_inplace(Tensor&, const NetOption&) const override { return 0; }
    std::string type() const override { return "Input"; }
};

// ---- Split (Tensor/SplitLayer.cpp): every top is the bottom itself ----
class SplitLayer : public Layer {
public:
    SplitLayer() { one_blob_only = false; support_inplace = false; accepts_tables = true; }
    int compute_output_shape(ParamDict& pd) override {
        if (bottom_shapes.empty() || !bottom_shapes[0].defined()) return -1;
        pd.set(OUTPUT_SHAPE_HINT, bottom_shapes[0]);
        return 0;
    }
    int forward(const std::vector<Tensor>& bottom_blobs, std::vector<Tensor>& top_blobs, const NetOption&) const override {
        for (auto& t : top_blobs) t = bottom_blobs[0];
        return 0;
    }
    bool map_channels(const std::vector<std::vector<int>>& in, std::vector<std::vector<int>>& out) const override {
        if (in.size() != 1 || in[0].empty()) return false;
        for (auto& t : out) t = in[0];
        return true;
    }
    std::string type() const override { return "Split"; }
};

REGISTER_LAYER_CLASS(Convolution);
REGISTER_LAYER_CLASS(Input);
REGISTER_LAYER_CLASS(Split);

}  // namespace otter
