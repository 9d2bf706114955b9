// The fp32 glue layers of the benchmark graphs in the host-side API mirror: MaxPool, Concat, Crop,
// ChannelShuffle, ShortCut, Upsample and the stand-alone activations. Option keys and shape rules follow the reference
// layer of the same name; forward enqueues one small CUDA kernel (include/otter_b200.h, "fp32 glue layers").
// Blobs are device fp32 NCHW tensors.
#include <algorithm>
#include <cstring>
#include <sstream>

#include "otter_api.hpp"

namespace otter {

namespace {
bool is_dev_f32(const Tensor& t) {
    return t.defined() && !t.is_table() && t.device() == Device::CUDA && t.scalar_type() == ScalarType::Float &&
           t.layout() == Layout::NCHW && t.dim() == 4;
}
bool is_dev_f32_or_table(const Tensor& t) {
    return t.defined() && t.device() == Device::CUDA && t.scalar_type() == ScalarType::Float && t.layout() == Layout::NCHW && t.dim() == 4;
}
}  // namespace

// Tensor/MaxPoolLayer.cpp:28-133
class MaxPoolLayer : public Layer {
public:
    MaxPoolLayer() { one_blob_only = true; support_inplace = false; support_packing = true; }
    int parse_param(LayerOption& option, ParamDict& pd) override {
        pd.clear();
        auto pair = [&](const char* both, const char* h, const char* w, int def, int& oh, int& ow) {
            oh = opt_find_int(option, h, -1);
            ow = opt_find_int(option, w, -1);
            const int b = opt_find_int(option, both, def);
            if (oh < 0) oh = b;
            if (ow < 0) ow = b;
        };
        int sh, sw, kh, kw, ph, pw;
        pair("stride", "stride_h", "stride_w", 1, sh, sw);
        pair("kernel", "kernel_h", "kernel_w", opt_find_int(option, "stride", 1), kh, kw);
        pair("padding", "padding_h", "padding_w", 0, ph, pw);
        if (opt_check_string(option, "ceil_mode") || opt_check_string(option, "darknet_mode")) return -1;  // not needed by the int8 graphs
        if (opt_find_int(option, "dilation", 1) != 1 || opt_find_int(option, "dilation_h", 1) != 1 || opt_find_int(option, "dilation_w", 1) != 1) return -1;
        pd.set(0, kh); pd.set(1, kw); pd.set(2, sh); pd.set(3, sw); pd.set(4, ph); pd.set(5, pw);
        return 0;
    }
    int compute_output_shape(ParamDict& pd) override {
        if (bottom_shapes.empty() || !bottom_shapes[0].defined()) return -1;
        int n, c, h, w;
        read_shape(bottom_shapes[0], n, c, h, w);
        const int oh = (h + 2 * pd.get(4, 0) - pd.get(0, 3)) / pd.get(2, 1) + 1;
        const int ow = (w + 2 * pd.get(5, 0) - pd.get(1, 3)) / pd.get(3, 1) + 1;
        pd.set(OUTPUT_SHAPE_HINT, shape_tensor(n, c, oh, ow));
        return 0;
    }
    int load_param(const ParamDict& pd) override {
        kh = pd.get(0, 3); kw = pd.get(1, 3); sh = pd.get(2, 1); sw = pd.get(3, 1); ph = pd.get(4, 0); pw = pd.get(5, 0);
        return 0;
    }
    bool is_pool3x3s2p1() const override { return kh == 3 && kw == 3 && sh == 2 && sw == 2 && ph == 1 && pw == 1; }
    int forward(const Tensor& bottom, Tensor& top, const NetOption& opt) const override {
        if (!is_dev_f32(bottom)) return -1;
        if (absorbed) {  // the producing convolution already pooled (Net::compile fused the pair)
            top = bottom;
            return 0;
        }
        const int n = (int)bottom.size(0), c = (int)bottom.size(1), h = (int)bottom.size(2), w = (int)bottom.size(3);
        const int oh = (h + 2 * ph - kh) / sh + 1, ow = (w + 2 * pw - kw) / sw + 1;
        top = device_empty(opt, {n, c, oh, ow}, ScalarType::Float, Layout::NCHW);
        if (!top.defined()) return -100;
        // The reference's Net packs fp32 blobs whose channel count is a multiple of 4 (Tensor/Net.cpp:380-411), and its
        // packed 3x3 stride-2 max-pool kernels pad with zeros (Tensor/Pool.cpp:972-975, :807-810); every other case
        // goes through the plain kernel, where padding never wins.
        const bool packed_zero_pad = opt.use_packing_layout && c % 4 == 0 && kh == 3 && kw == 3 && sh == 2 && sw == 2;
        return ott_maxpool_f32_nchw(opt.gpu, bottom.data_ptr<float>(), n, c, h, w, kh, kw, sh, sw, ph, pw, packed_zero_pad ? 1 : 0,
                                    top.data_ptr<float>());
    }
    std::string type() const override { return "MaxPool"; }
    int kh = 3, kw = 3, sh = 1, sw = 1, ph = 0, pw = 0;
};

// Tensor/ConcatLayer.cpp:24-70 (channel axis only: the only use in the int8 graphs)
class ConcatLayer : public Layer {
public:
    ConcatLayer() { one_blob_only = false; support_inplace = false; support_packing = true; accepts_tables = true; }
    int parse_param(LayerOption& option, ParamDict& pd) override {
        pd.clear();
        pd.set(0, opt_find_int(option, "axis", 1));
        return 0;
    }
    int compute_output_shape(ParamDict& pd) override {
        if (pd.get(0, 1) != 1 || bottom_shapes.empty()) return -1;
        int n, c, h, w;
        read_shape(bottom_shapes[0], n, c, h, w);
        for (size_t i = 1; i < bottom_shapes.size(); ++i) {
            int n2, c2, h2, w2;
            read_shape(bottom_shapes[i], n2, c2, h2, w2);
            c += c2;
        }
        pd.set(OUTPUT_SHAPE_HINT, shape_tensor(n, c, h, w));
        return 0;
    }
    // No plane is copied: the result is a plane table over the inputs (Tensor::is_table). A consumer that reads through
    // tables (Convolution) does so; for any other consumer the Net materialises the tensor with one gather kernel.
    int forward(const std::vector<Tensor>& bottoms, std::vector<Tensor>& tops, const NetOption&) const override {
        for (const Tensor& b : bottoms)
            if (!is_dev_f32_or_table(b) || b.size(0) != bottoms[0].size(0) || b.size(2) != bottoms[0].size(2) || b.size(3) != bottoms[0].size(3)) return -1;
        tops[0] = Tensor::concat_channels(bottoms);
        return tops[0].defined() ? 0 : -1;
    }
    bool map_channels(const std::vector<std::vector<int>>& in, std::vector<std::vector<int>>& out) const override {
        if (out.size() != 1) return false;
        out[0].clear();
        for (const auto& b : in) {
            if (b.empty()) return false;
            out[0].insert(out[0].end(), b.begin(), b.end());
        }
        return true;
    }
    std::string type() const override { return "Concat"; }
};

// Tensor/CropLayer.cpp:25-76 (channel axis): a selection of channel planes, no copy
class CropLayer : public Layer {
public:
    CropLayer() { one_blob_only = true; support_inplace = false; support_packing = true; accepts_tables = true; }
    int parse_param(LayerOption& option, ParamDict& pd) override {
        pd.clear();
        pd.set(0, opt_find_int(option, "axis", 1));
        pd.set(1, opt_find_int(option, "start", -1));
        pd.set(2, opt_find_int(option, "end", -1));
        return 0;
    }
    int compute_output_shape(ParamDict& pd) override {
        if (pd.get(0, 1) != 1 || bottom_shapes.empty() || !bottom_shapes[0].defined()) return -1;
        int n, c, h, w;
        read_shape(bottom_shapes[0], n, c, h, w);
        const int e = pd.get(2, -1) == -1 ? c : pd.get(2, -1);
        pd.set(OUTPUT_SHAPE_HINT, shape_tensor(n, e - pd.get(1, 0), h, w));
        return 0;
    }
    int load_param(const ParamDict& pd) override {
        start = pd.get(1, -1);
        end = pd.get(2, -1);
        return 0;
    }
    int forward(const Tensor& bottom, Tensor& top, const NetOption&) const override {
        if (!is_dev_f32_or_table(bottom)) return -1;
        const int c = (int)bottom.size(1);
        const int e = end == -1 ? c : end;
        if (start < 0 || e > c || e <= start) return -1;
        std::vector<int> pick((size_t)(e - start));
        for (int i = start; i < e; ++i) pick[(size_t)(i - start)] = i;
        top = bottom.select_channels(pick);  // a selection of planes, as the view native::slice gives the reference
        return top.defined() ? 0 : -1;
    }
    bool map_channels(const std::vector<std::vector<int>>& in, std::vector<std::vector<int>>& out) const override {
        if (in.size() != 1 || out.size() != 1 || in[0].empty()) return false;
        const int c = (int)in[0].size(), e = end == -1 ? c : end;
        if (start < 0 || e > c || e <= start) return false;
        out[0].assign(in[0].begin() + start, in[0].begin() + e);
        return true;
    }
    std::string type() const override { return "Crop"; }
    int start = -1, end = -1;
};

// Tensor/ChannelShuffleLayer.cpp:20-41: output channel i*g + k is input channel k*(C/g) + i
class ChannelShuffleLayer : public Layer {
public:
    ChannelShuffleLayer() { one_blob_only = true; support_inplace = false; support_packing = true; accepts_tables = true; }
    int parse_param(LayerOption& option, ParamDict& pd) override {
        pd.clear();
        pd.set(0, opt_find_int(option, "groups", 1));
        return 0;
    }
    int load_param(const ParamDict& pd) override {
        groups = pd.get(0, 1);
        return 0;
    }
    // A permutation of planes: output channel i*groups + k is input channel k*(C/groups) + i. No plane is copied.
    int forward(const Tensor& bottom, Tensor& top, const NetOption&) const override {
        if (!is_dev_f32_or_table(bottom)) return -1;
        const int c = (int)bottom.size(1);
        if (groups < 1 || c % groups != 0) return -1;
        const int per = c / groups;
        std::vector<int> pick((size_t)c);
        for (int i = 0; i < per; ++i)
            for (int k = 0; k < groups; ++k) pick[(size_t)(i * groups + k)] = k * per + i;
        top = bottom.select_channels(pick);
        return top.defined() ? 0 : -1;
    }
    bool map_channels(const std::vector<std::vector<int>>& in, std::vector<std::vector<int>>& out) const override {
        if (in.size() != 1 || out.size() != 1 || in[0].empty()) return false;
        const int c = (int)in[0].size();
        if (groups < 1 || c % groups != 0) return false;
        const int per = c / groups;
        out[0].resize((size_t)c);
        for (int i = 0; i < per; ++i)
            for (int k = 0; k < groups; ++k) out[0][(size_t)(i * groups + k)] = in[0][(size_t)(k * per + i)];
        return true;
    }
    std::string type() const override { return "ChannelShuffle"; }
    int groups = 1;
};

// Tensor/ShortCutLayer.cpp (element-wise add of two blobs of the same shape). Operands that are plane tables (the result of a
// Concat in the Ghost blocks of the detector graphs) are read where their planes lie.
class ShortCutLayer : public Layer {
public:
    ShortCutLayer() { one_blob_only = false; support_inplace = false; support_packing = true; accepts_tables = true; }
    int forward(const std::vector<Tensor>& bottoms, std::vector<Tensor>& tops, const NetOption& opt) const override {
        if (bottoms.size() != 2 || !is_dev_f32_or_table(bottoms[0]) || !is_dev_f32_or_table(bottoms[1]) || bottoms[0].sizes() != bottoms[1].sizes())
            return -1;
        Tensor a = bottoms[0], b = bottoms[1];
        const int n = (int)a.size(0), c = (int)a.size(1), hw = (int)(a.size(2) * a.size(3));
        std::vector<const float*> abufs, bbufs;
        std::vector<int64_t> astr, bstr;
        std::vector<uint32_t> arefs, brefs;
        auto describe = [&](Tensor& t, std::vector<const float*>& bufs, std::vector<int64_t>& strides, std::vector<uint32_t>& refs) {
            if (t.is_table() && table_arrays(t, bufs, strides)) { refs = t.table_refs(); return true; }
            if (t.is_table()) { t = materialize(opt, t); if (!t.defined()) return false; }
            if (c > kMaxTableChannels) return false;
            bufs.assign(1, t.data_ptr<float>());
            strides.assign(1, (int64_t)c * hw);
            refs.resize((size_t)c);
            for (int i = 0; i < c; ++i) refs[(size_t)i] = (uint32_t)i;
            return true;
        };
        tops[0] = device_empty(opt, a.sizes(), ScalarType::Float, Layout::NCHW);
        if (!tops[0].defined()) return -100;
        if ((a.is_table() || b.is_table()) && describe(a, abufs, astr, arefs) && describe(b, bbufs, bstr, brefs))
            return ott_add_gather_f32(opt.gpu, abufs.data(), astr.data(), (int)abufs.size(), arefs.data(), bbufs.data(), bstr.data(), (int)bbufs.size(),
                                      brefs.data(), c, n, hw, tops[0].data_ptr<float>());
        a = materialize(opt, a);
        b = materialize(opt, b);
        if (!a.defined() || !b.defined()) return -100;
        return ott_add_f32(opt.gpu, a.data_ptr<float>(), b.data_ptr<float>(), tops[0].data_ptr<float>(), (size_t)a.numel());
    }
    std::string type() const override { return "ShortCut"; }
};

// Tensor/UpsampleLayer.cpp:26-131, the one-input form. Option keys upsample_mode, output_height/width, scale_height/width,
// stride (wins over the scales when non-zero, :80-83) and align_corner. Built: nearest and bilinear, both as the reference's
// default options run them (NetOption::use_non_lib_optimize = true -> otter::Interpolate, which never sees align_corner, so
// the flag changes nothing there and is ignored here too). Bicubic is refused by the reference's own parse_param (:50).
class UpsampleLayer : public Layer {
public:
    UpsampleLayer() { one_blob_only = true; support_inplace = false; support_packing = true; }
    int parse_param(LayerOption& option, ParamDict& pd) override {
        pd.clear();
        const std::string m = opt_find_string(option, "upsample_mode", "nearest");
        const int mode_id = m == "nearest" ? 1 : m == "bilinear" ? 2 : m == "bicubic" ? 3 : -1;
        if (mode_id > 2) return -1;  // "Unsupport upsample type" in the reference
        pd.set(0, mode_id);
        pd.set(1, opt_find_int(option, "output_height", 0));
        pd.set(2, opt_find_int(option, "output_width", 0));
        pd.set(3, opt_find_float(option, "scale_height", 1.f));
        pd.set(4, opt_find_float(option, "scale_width", 1.f));
        pd.set(5, opt_find_float(option, "stride", 1.f));
        pd.set(6, opt_find(option, "align_corner") && option["align_corner"] != "false" ? 1 : 0);
        return 0;
    }
    int compute_output_shape(ParamDict& pd) override {
        if (bottom_shapes.empty() || !bottom_shapes[0].defined()) return -1;
        int n, c, h, w;
        read_shape(bottom_shapes[0], n, c, h, w);
        int out_h = pd.get(1, 0), out_w = pd.get(2, 0);
        float sh = pd.get(3, 0.f), sw = pd.get(4, 0.f);
        const float stride = pd.get(5, 1.f);
        if (out_h && out_w) { sh = (float)(out_h / h); sw = (float)(out_w / w); }  // integer division, as in the reference (:75-78)
        if (stride != 0.f) sh = sw = stride;
        if (sh != 0.f && sw != 0.f) { out_h = (int)(h * sh); out_w = (int)(w * sw); }
        pd.set(1, out_h); pd.set(2, out_w); pd.set(3, sh); pd.set(4, sw);
        pd.set(OUTPUT_SHAPE_HINT, shape_tensor(n, c, out_h, out_w));
        return 0;
    }
    int load_param(const ParamDict& pd) override {
        mode = pd.get(0, 0); scale_height = pd.get(3, 0.f); scale_width = pd.get(4, 0.f); align_corner = pd.get(6, 0);
        return 0;
    }
    int forward(const Tensor& bottom, Tensor& top, const NetOption& opt) const override {
        if (!is_dev_f32(bottom)) return -1;
        if (mode != 1 && mode != 2) return -1;
        const int n = (int)bottom.size(0), c = (int)bottom.size(1), h = (int)bottom.size(2), w = (int)bottom.size(3);
        const int oh = (int)(h * scale_height), ow = (int)(w * scale_width);
        if (oh < 1 || ow < 1) return -1;
        top = device_empty(opt, {n, c, oh, ow}, ScalarType::Float, Layout::NCHW);
        if (!top.defined()) return -100;
        // The reference's Net hands this layer a packed blob when the channel count is a multiple of 4 (Tensor/Net.cpp:380-411),
        // and its resize of packed blobs rounds differently from its resize of plain ones (see ott_upsample_bilinear_f32_nchw).
        const bool packed = opt.use_packing_layout && c % 4 == 0;
        if (mode == 1)
            return ott_upsample_nearest_f32_nchw(opt.gpu, bottom.data_ptr<float>(), n, c, h, w, oh, ow, scale_height, scale_width, packed ? 1 : 0,
                                                 top.data_ptr<float>());
        return ott_upsample_bilinear_f32_nchw(opt.gpu, bottom.data_ptr<float>(), n, c, h, w, oh, ow, scale_height, scale_width, packed ? 1 : 0,
                                              top.data_ptr<float>());
    }
    std::string type() const override { return "Upsample"; }
    int mode = 2, align_corner = 0;
    float scale_height = 1.f, scale_width = 1.f;
};

// Tensor/NanodetPlusDetectionOutputLayer.cpp:22-110. Bottoms: the head blobs of the pyramid levels (fp32 NCHW on the device);
// top: a HOST tensor [count, 6] {label + 1, score, x, y, width, height} for image 0, as in the reference (which reads only
// the first image of each blob). Option keys prob_threshold (0.4), nms_threshold (0.5), stride ("8, 16, 32, 64").
class NanodetPlusDetectionOutputLayer : public Layer {
public:
    NanodetPlusDetectionOutputLayer() { one_blob_only = false; support_inplace = false; }
    int parse_param(LayerOption& option, ParamDict& pd) override {
        pd.clear();
        pd.set(0, opt_find_float(option, "prob_threshold", 0.4f));
        pd.set(1, opt_find_float(option, "nms_threshold", 0.5f));
        std::vector<int> st;
        if (opt_check_string(option, "stride")) {
            std::stringstream ss(option["stride"]);
            int v;
            char comma;
            while (ss >> v) { st.push_back(v); ss >> comma; }
        }
        if (st.empty()) st = {8, 16, 32, 64};
        pd.set(2, tensor(st, ScalarType::Int));
        return 0;
    }
    int compute_output_shape(ParamDict& pd) override {
        pd.set(OUTPUT_SHAPE_HINT, shape_tensor(6, 0, 0, 0));  // the reference's hint; the real shape is [count, 6]
        return 0;
    }
    int load_param(const ParamDict& pd) override {
        prob_threshold = pd.get(0, 0.45f);
        nms_threshold = pd.get(1, 0.5f);
        Tensor st = pd.get(2, Tensor());
        strides.assign(st.data_ptr<int>(), st.data_ptr<int>() + st.numel());
        return 0;
    }
    int forward(const std::vector<Tensor>& bottoms, std::vector<Tensor>& tops, const NetOption& opt) const override {
        const int levels = (int)bottoms.size();
        if (levels < 1 || levels > (int)strides.size()) return -1;
        std::vector<const float*> heads;
        std::vector<int> gh, gw;
        const int channels = (int)bottoms[0].size(1);
        const int num_class = 80;  // fixed in the reference (:120)
        if ((channels - num_class) % 4 != 0 || channels <= num_class) return -1;
        for (const Tensor& b : bottoms) {
            if (!is_dev_f32(b) || b.size(1) != channels) return -1;
            heads.push_back(b.data_ptr<float>());
            gh.push_back((int)b.size(2));
            gw.push_back((int)b.size(3));
        }
        int cells = 0;
        for (int l = 0; l < levels; ++l) cells += gh[(size_t)l] * gw[(size_t)l];
        std::vector<float> rows((size_t)cells * 6);
        int count = 0;
        // image 0 only: with n = 1 the decode reads the first image of every (batched) head blob
        const int rc = ott_nanodet_detect(opt.gpu, heads.data(), gh.data(), gw.data(), strides.data(), levels, 1, num_class, (channels - num_class) / 4,
                                          prob_threshold, nms_threshold, rows.data(), &count, cells);
        if (rc != 0) return rc;
        tops[0] = empty({count, 6}, ScalarType::Float);
        if (count > 0) std::memcpy(tops[0].raw_data(), rows.data(), (size_t)count * 6 * sizeof(float));
        return 0;
    }
    std::string type() const override { return "NanodetPlusDetectionOutput"; }
    float prob_threshold = 0.4f, nms_threshold = 0.5f;
    std::vector<int> strides{8, 16, 32, 64};
};

// Tensor/ReluLayer.cpp, Tensor/LReluLayer.cpp:28-113 (option "alpha", default 0.1), Tensor/Relu6Layer.cpp
template <int ACT>
class ActivationLayerT : public Layer {
public:
    ActivationLayerT() { one_blob_only = true; support_inplace = true; support_packing = true; }
    int parse_param(LayerOption& option, ParamDict& pd) override {
        pd.clear();
        pd.set(0, opt_find_float(option, "alpha", 0.1f));
        return 0;
    }
    int load_param(const ParamDict& pd) override {
        slope = pd.get(0, 0.1f);
        return 0;
    }
    int forward_inplace(Tensor& blob, const NetOption& opt) const override {
        if (!is_dev_f32(blob)) return -1;
        return ott_activation_f32(opt.gpu, blob.data_ptr<float>(), (size_t)blob.numel(), ACT, slope);
    }
    int forward(const Tensor& bottom, Tensor& top, const NetOption& opt) const override {
        if (!is_dev_f32(bottom)) return -1;
        top = device_empty(opt, bottom.sizes(), ScalarType::Float, Layout::NCHW);
        if (!top.defined()) return -100;
        const int c = (int)bottom.size(1);
        int rc = ott_copy_channels_f32(opt.gpu, bottom.data_ptr<float>(), c, 0, 1, top.data_ptr<float>(), c, 0, 1, c, (int)bottom.size(0),
                                       (int)(bottom.size(2) * bottom.size(3)));
        if (rc != 0) return rc;
        return forward_inplace(top, opt);
    }
    std::string type() const override { return ACT == 1 ? "Relu" : ACT == 2 ? "LRelu" : "Relu6"; }
    float slope = 0.1f;
};
using ReluLayer = ActivationLayerT<1>;
using LReluLayer = ActivationLayerT<2>;
using Relu6Layer = ActivationLayerT<3>;

REGISTER_LAYER_CLASS(MaxPool);
REGISTER_LAYER_CLASS(Concat);
REGISTER_LAYER_CLASS(Crop);
REGISTER_LAYER_CLASS(ChannelShuffle);
REGISTER_LAYER_CLASS(ShortCut);
REGISTER_LAYER_CLASS(Upsample);
REGISTER_LAYER_CLASS(NanodetPlusDetectionOutput);
REGISTER_LAYER_CLASS(Relu);
REGISTER_LAYER_CLASS(LRelu);
REGISTER_LAYER_CLASS(Relu6);

}  // namespace otter
