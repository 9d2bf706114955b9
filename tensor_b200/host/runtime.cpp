// Tensor handle, Layer base class, LayerRegistry, Net and Extractor of the host-side API mirror
// (declarations and reference citations in otter_api.hpp).
#include <algorithm>
#include <cstring>
#include <set>
#include <sstream>

#include "otter_api.hpp"

namespace otter {

// ---------------------------------------------------------------- Tensor
Tensor Tensor::wrap(void* ptr, size_t bytes, Device dev, std::function<void(void*)> deleter, std::vector<int64_t> sizes,
                    ScalarType dtype, Layout layout) {
    Tensor t;
    t.st_ = std::make_shared<Storage>();
    t.st_->ptr = ptr;
    t.st_->bytes = bytes;
    t.st_->dev = dev;
    t.st_->deleter = std::move(deleter);
    t.sizes_ = std::move(sizes);
    t.dtype_ = dtype;
    t.layout_ = layout;
    return t;
}

Tensor Tensor::view(std::vector<int64_t> sizes) const {
    int64_t known = 1, unknown = -1;
    for (size_t i = 0; i < sizes.size(); ++i) {
        if (sizes[i] == -1) unknown = (int64_t)i; else known *= sizes[i];
    }
    if (unknown >= 0) sizes[(size_t)unknown] = known ? numel() / known : 0;
    Tensor t = *this;
    t.sizes_ = std::move(sizes);
    return t;
}

Tensor Tensor::select_channels(const std::vector<int>& pick) const {
    if (!defined() || dim() != 4 || scalar_type() != ScalarType::Float || layout_ != Layout::NCHW) return Tensor();
    auto tab = std::make_shared<PlaneTable>();
    std::vector<int> remap;  // old buffer index -> new
    const int c = (int)size(1);
    if (is_table()) remap.assign(table_->bufs.size(), -1);
    for (int ch : pick) {
        if (ch < 0 || ch >= c) return Tensor();
        if (!is_table()) {
            if (tab->bufs.empty()) tab->bufs.push_back(*this);
            tab->refs.push_back((uint32_t)ch);
        } else {
            const uint32_t r = table_->refs[(size_t)ch];
            const int ob = (int)(r >> 24);
            if (remap[(size_t)ob] < 0) {
                remap[(size_t)ob] = (int)tab->bufs.size();
                tab->bufs.push_back(table_->bufs[(size_t)ob]);
            }
            tab->refs.push_back(((uint32_t)remap[(size_t)ob] << 24) | (r & 0xFFFFFFu));
        }
    }
    Tensor t;
    t.sizes_ = sizes_;
    t.sizes_[1] = (int64_t)pick.size();
    t.dtype_ = ScalarType::Float;
    t.layout_ = Layout::NCHW;
    t.table_ = tab;
    return t;
}

Tensor Tensor::concat_channels(const std::vector<Tensor>& parts) {
    if (parts.empty()) return Tensor();
    auto tab = std::make_shared<PlaneTable>();
    int64_t c = 0;
    for (const Tensor& p : parts) {
        if (!p.defined() || p.dim() != 4 || p.scalar_type() != ScalarType::Float) return Tensor();
        const uint32_t base = (uint32_t)tab->bufs.size();
        if (p.is_table()) {
            // reuse a buffer already listed (same storage) instead of listing it twice
            std::vector<uint32_t> map(p.table_->bufs.size());
            for (size_t i = 0; i < p.table_->bufs.size(); ++i) {
                size_t j = 0;
                for (; j < tab->bufs.size(); ++j)
                    if (tab->bufs[j].raw_data() == p.table_->bufs[i].raw_data()) break;
                if (j == tab->bufs.size()) tab->bufs.push_back(p.table_->bufs[i]);
                map[i] = (uint32_t)j;
            }
            for (uint32_t r : p.table_->refs) tab->refs.push_back((map[r >> 24] << 24) | (r & 0xFFFFFFu));
        } else {
            tab->bufs.push_back(p);
            for (int64_t i = 0; i < p.size(1); ++i) tab->refs.push_back((base << 24) | (uint32_t)i);
        }
        c += p.size(1);
    }
    Tensor t;
    t.sizes_ = parts[0].sizes();
    t.sizes_[1] = c;
    t.dtype_ = ScalarType::Float;
    t.layout_ = Layout::NCHW;
    t.table_ = tab;
    return t;
}

Tensor Tensor::clone() const {
    if (!defined() || device() != Device::CPU) return Tensor();
    Tensor t = empty(sizes_, dtype_);
    std::memcpy(t.raw_data(), raw_data(), (size_t)numel() * elementSize(dtype_));
    t.layout_ = layout_;
    return t;
}

Tensor empty(std::vector<int64_t> sizes, ScalarType dtype) {
    int64_t n = sizes.empty() ? 0 : 1;
    for (auto s : sizes) n *= s;
    const size_t bytes = (size_t)(n > 0 ? n : 1) * elementSize(dtype);
    void* p = ::operator new(bytes);
    std::memset(p, 0, bytes);
    return Tensor::wrap(p, bytes, Device::CPU, [](void* q) { ::operator delete(q); }, std::move(sizes), dtype);
}

Tensor from_blob(void* data, std::vector<int64_t> sizes, ScalarType dtype) {
    int64_t n = sizes.empty() ? 0 : 1;
    for (auto s : sizes) n *= s;
    return Tensor::wrap(data, (size_t)n * elementSize(dtype), Device::CPU, nullptr, std::move(sizes), dtype);
}

Tensor tensor(std::vector<int> values, ScalarType dtype) {
    Tensor t = empty({(int64_t)values.size()}, dtype);
    for (size_t i = 0; i < values.size(); ++i) {
        if (dtype == ScalarType::Float) t.data_ptr<float>()[i] = (float)values[i];
        else if (dtype == ScalarType::Int) t.data_ptr<int>()[i] = values[i];
        else t.data_ptr<int8_t>()[i] = (int8_t)values[i];
    }
    return t;
}

Tensor full(std::vector<int64_t> sizes, float value, ScalarType dtype) {
    Tensor t = empty(std::move(sizes), dtype);
    for (int64_t i = 0; i < t.numel(); ++i) {
        if (dtype == ScalarType::Float) t.data_ptr<float>()[i] = value;
        else if (dtype == ScalarType::Int) t.data_ptr<int>()[i] = (int)value;
        else t.data_ptr<int8_t>()[i] = (int8_t)value;
    }
    return t;
}

Tensor shape_tensor(int n, int c, int h, int w) { return tensor({n, c, h, w}, ScalarType::Int).view({1, -1}); }

void read_shape(const Tensor& shape, int& n, int& c, int& h, int& w) {
    const int* p = shape.data_ptr<int>();
    n = p[0]; c = p[1]; h = p[2]; w = p[3];
}

Tensor device_empty(const NetOption& opt, std::vector<int64_t> sizes, ScalarType dtype, Layout layout) {
    if (!opt.gpu) return Tensor();
    int64_t n = 1;
    for (auto s : sizes) n *= s;
    if (layout == Layout::NHWC16 && sizes.size() == 4)  // sizes are logical {N,C,H,W}; storage pads C
        n = sizes[0] * sizes[2] * sizes[3] * ott_nhwc_channels((int)sizes[1]);
    const size_t bytes = (size_t)(n > 0 ? n : 1) * elementSize(dtype);
    void* p = nullptr;
    if (ott_malloc(opt.gpu, bytes, &p) != OTT_OK) return Tensor();
    ott_ctx* ctx = opt.gpu;
    return Tensor::wrap(p, bytes, Device::CUDA, [ctx](void* q) { ott_free(ctx, q); }, std::move(sizes), dtype, layout);
}

// the arrays ott_conv_int8_forward_gather / ott_gather_channels_f32 take, from a plane table
bool table_arrays(const Tensor& t, std::vector<const float*>& bufs, std::vector<int64_t>& strides) {
    if (!t.is_table() || t.table_bufs().size() > (size_t)kMaxTableBufs || t.size(1) > kMaxTableChannels) return false;
    const int64_t hw = t.size(2) * t.size(3);
    for (const Tensor& b : t.table_bufs()) {
        bufs.push_back(b.data_ptr<float>());
        strides.push_back(b.size(1) * hw);
    }
    return true;
}

Tensor materialize(const NetOption& opt, const Tensor& t) {
    if (!t.is_table()) return t;
    const int n = (int)t.size(0), c = (int)t.size(1), hw = (int)(t.size(2) * t.size(3));
    Tensor out = device_empty(opt, t.sizes(), ScalarType::Float, Layout::NCHW);
    if (!out.defined()) return Tensor();
    std::vector<const float*> bufs;
    std::vector<int64_t> strides;
    if (table_arrays(t, bufs, strides)) {
        if (ott_gather_channels_f32(opt.gpu, bufs.data(), strides.data(), (int)bufs.size(), t.table_refs().data(), c, n, hw, out.data_ptr<float>()) != OTT_OK)
            return Tensor();
        return out;
    }
    // too many buffers or channels for one table: plane by plane runs
    const auto& refs = t.table_refs();
    int i = 0;
    while (i < c) {
        const uint32_t b = refs[(size_t)i] >> 24, p0 = refs[(size_t)i] & 0xFFFFFFu;
        int run = 1;
        while (i + run < c && (refs[(size_t)(i + run)] >> 24) == b && (refs[(size_t)(i + run)] & 0xFFFFFFu) == p0 + (uint32_t)run) ++run;
        const Tensor& src = t.table_bufs()[b];
        if (ott_copy_channels_f32(opt.gpu, src.data_ptr<float>(), (int)src.size(1), (int)p0, 1, out.data_ptr<float>(), c, i, 1, run, n, hw) != OTT_OK)
            return Tensor();
        i += run;
    }
    return out;
}

// ---------------------------------------------------------------- Layer
Layer::Layer() = default;
Layer::~Layer() = default;
int Layer::parse_param(LayerOption&, ParamDict& pd) { pd.clear(); return 0; }
int Layer::compute_output_shape(ParamDict& pd) {
    if (!bottom_shapes.empty() && bottom_shapes[0].defined()) pd.set(OUTPUT_SHAPE_HINT, bottom_shapes[0]);
    return 0;
}
int Layer::load_param(const ParamDict&) { return 0; }
int Layer::init_model() { return 0; }
int Layer::load_model(const Initializer&) { return 0; }
int Layer::create_pipeline(const NetOption&) { return 0; }
int Layer::forward(const Tensor& bottom_blob, Tensor& top_blob, const NetOption& opt) const {
    if (!support_inplace) return -1;
    top_blob = bottom_blob;
    return forward_inplace(top_blob, opt);
}
int Layer::forward(const std::vector<Tensor>& bottom_blobs, std::vector<Tensor>& top_blobs, const NetOption& opt) const {
    if (!support_inplace) return -1;
    top_blobs = bottom_blobs;
    return forward_inplace(top_blobs, opt);
}
int Layer::forward_inplace(Tensor&, const NetOption&) const { return -1; }
int Layer::forward_inplace(std::vector<Tensor>&, const NetOption&) const { return -1; }

std::map<std::string, LayerCreator>& LayerRegistry::Registry() {
    static std::map<std::string, LayerCreator> reg;
    return reg;
}
void LayerRegistry::AddCreator(const std::string& type, LayerCreator creator) { Registry()[type] = std::move(creator); }
Layer* LayerRegistry::CreateLayer(const std::string& type) {
    auto it = Registry().find(type);
    return it == Registry().end() ? nullptr : it->second();
}
std::string LayerRegistry::LayerTypeListString() {
    std::string s;
    for (auto& kv : Registry()) s += (s.empty() ? "" : ", ") + kv.first;
    return s;
}

// ---------------------------------------------------------------- Net
namespace {

std::vector<std::string> split_names(const std::string& list) {
    std::vector<std::string> out;
    std::stringstream ss(list);
    std::string item;
    while (std::getline(ss, item, ',')) {
        item.erase(std::remove_if(item.begin(), item.end(), [](unsigned char ch) { return ch == ' ' || ch == '"'; }), item.end());
        if (!item.empty()) out.push_back(item);
    }
    return out;
}

}  // namespace

Net::Net() = default;

Net::~Net() {
    for (Layer* l : layers_) delete l;
    layers_.clear();
    if (owns_ctx_ && option.gpu) {
        ott_ctx_destroy(option.gpu);
        option.gpu = nullptr;
    }
}

// Tensor/Net.cpp:40-80 (the BatchNorm / activation auto-insertion belongs to the fp32 path and is not mirrored)
void Net::addLayer(LayerOption option) {
    if (!opt_check_string(option, "name")) option["name"] = std::to_string(layer_options_.size());
    if (!opt_check_string(option, "output")) option["output"] = option["name"];
    if (!opt_check_string(option, "input_id")) option["input_id"] = "0";
    layer_options_.push_back(std::move(option));
}

// Tensor/Net.cpp:82-172: default input = previous layer's first output; a blob with several consumers gets an
// automatic Split layer whose outputs rename the consumers' inputs.
void Net::graph_construct() {
    for (size_t i = 1; i < layer_options_.size(); ++i) {
        LayerOption& l = layer_options_[i];
        if (!opt_check_string(l, "input") && l["type"] != "Input") l["input"] = split_names(layer_options_[i - 1]["output"])[0];
    }
    int extra = 0;
    for (size_t i = 0; i < layer_options_.size(); ++i) {
        const std::vector<std::string> outs = split_names(layer_options_[i]["output"]);
        for (const std::string& out : outs) {
            std::vector<std::pair<size_t, size_t>> users;  // (layer, input position)
            for (size_t j = 0; j < layer_options_.size(); ++j) {
                if (layer_options_[j]["type"] == "Input") continue;
                const auto ins = split_names(layer_options_[j]["input"]);
                for (size_t k = 0; k < ins.size(); ++k)
                    if (ins[k] == out) users.emplace_back(j, k);
            }
            if (users.size() <= 1) continue;
            LayerOption sp;
            sp["type"] = "Split";
            sp["name"] = "auto_sp_" + std::to_string(++extra);
            sp["input"] = out;
            std::string outputs;
            for (size_t u = 0; u < users.size(); ++u) {
                const std::string nm = "asp_" + std::to_string(i) + "_" + out + "_" + std::to_string(u);
                outputs += (u ? ", " : "") + nm;
                auto ins = split_names(layer_options_[users[u].first]["input"]);
                ins[users[u].second] = nm;
                std::string joined;
                for (size_t k = 0; k < ins.size(); ++k) joined += (k ? ", " : "") + ins[k];
                layer_options_[users[u].first]["input"] = joined;
            }
            sp["output"] = outputs;
            layer_options_.insert(layer_options_.begin() + (long)i + 1, sp);
        }
    }
}

int Net::find_blob_index_by_name(const std::string& name) const {
    for (size_t i = 0; i < blobs_.size(); ++i)
        if (blobs_[i].name == name) return (int)i;
    return -1;
}

int Net::find_layer_index_by_name(const std::string& name) const {
    for (size_t i = 0; i < layers_.size(); ++i)
        if (layers_[i] && layers_[i]->name == name) return (int)i;
    return -1;
}

// Tensor/Net.cpp:174-280
int Net::compile(CompileMode mode) {
    if (!option.gpu) {
        if (option.device < 0) { error_ = "NetOption::device < 0: this build has no CPU path"; return -1; }
        const int rc = ott_ctx_create(option.device, &option.gpu);
        if (rc != OTT_OK) { error_ = "no usable sm_100 GPU (ott_ctx_create failed)"; return rc; }
        owns_ctx_ = true;
    }
    graph_construct();
    if (layer_options_.empty()) { error_ = "Invalid network"; return -1; }
    size_t blob_count = 0;
    for (auto& o : layer_options_) blob_count += split_names(o["output"]).size();
    blobs_.assign(blob_count, Blob());
    layers_.assign(layer_options_.size(), nullptr);
    ParamDict pd;
    int blob_index = 0;
    for (size_t i = 0; i < layer_options_.size(); ++i) {
        LayerOption& opt = layer_options_[i];
        const std::string type = opt["type"];
        Layer* layer = LayerRegistry::CreateLayer(type);
        if (!layer) { error_ = "Unknown layer type: " + type + " (known layer types: " + LayerRegistry::LayerTypeListString() + ")"; return -1; }
        layers_[i] = layer;
        layer->name = opt["name"];
        const auto ins = type == "Input" ? std::vector<std::string>() : split_names(opt["input"]);
        const auto outs = split_names(opt["output"]);
        layer->bottoms.resize(ins.size());
        for (size_t j = 0; j < ins.size(); ++j) {
            const int b = find_blob_index_by_name(ins[j]);
            if (b < 0) { error_ = "layer " + layer->name + " consumes unknown blob " + ins[j]; return -1; }
            blobs_[(size_t)b].consumer = (int)i;
            layer->bottoms[j] = b;
        }
        layer->tops.resize(outs.size());
        for (size_t j = 0; j < outs.size(); ++j) {
            blobs_[(size_t)blob_index].name = outs[j];
            blobs_[(size_t)blob_index].producer = (int)i;
            layer->tops[j] = blob_index++;
        }
        if (layer->parse_param(opt, pd) != 0) { error_ = "ParamDict load " + layer->name + " failed"; return -1; }
        layer->bottom_shapes.resize(ins.size());
        for (size_t j = 0; j < ins.size(); ++j) layer->bottom_shapes[j] = blobs_[(size_t)layer->bottoms[j]].shape;
        layer->top_shapes.resize(outs.size());
        if (layer->compute_output_shape(pd) != 0) { error_ = "Layer " + layer->name + " output shape undefined"; return -1; }
        Tensor hints = pd.get(OUTPUT_SHAPE_HINT, Tensor());
        if (hints.defined()) {
            const int64_t rows = hints.size(0);
            for (size_t j = 0; j < outs.size(); ++j) {
                const int64_t r = rows > 1 ? (int64_t)j : 0;
                const int* p = hints.data_ptr<int>() + r * 4;
                blobs_[(size_t)layer->tops[j]].shape = shape_tensor(p[0], p[1], p[2], p[3]);
                layer->top_shapes[j] = blobs_[(size_t)layer->tops[j]].shape;
            }
        }
        if (layer->load_param(pd) != 0) { error_ = "Layer load " + layer->name + " failed"; return -1; }
        if (mode == CompileMode::Initial) {
            if (layer->init_model() != 0) { error_ = "init_model of " + layer->name + " failed"; return -1; }
            const int rc = layer->create_pipeline(option);
            if (rc != 0) { error_ = "create_pipeline of " + layer->name + " failed: " + ott_last_error(option.gpu); return rc; }
        }
    }
    blob_fused_away_.assign(blobs_.size(), 0);
    if (mode == CompileMode::Initial) {
        const int rc = plan_fusions();
        if (rc != 0) return rc;
    }
    input_names_.clear();
    output_names_.clear();
    for (Layer* l : layers_)
        if (l->type() == "Input") input_names_.push_back(blobs_[(size_t)l->tops[0]].name);
    for (const Blob& b : blobs_)
        if (b.producer != -1 && b.consumer == -1) output_names_.push_back(b.name);
    return 0;
}

// Decides whether layer `producer_layer` hands its result to its reader in int8, and (re)builds its requantizing twin.
// Holds when: both are quantized convolutions, the producer's own result is fp32, its top blob has this one reader (a blob
// read twice goes through a Split layer and stays fp32), and the reader does not run as a fused first-layer kernel.
int Net::refresh_handover(int producer_layer) {
    auto* conv = dynamic_cast<ConvolutionLayer*>(layers_[(size_t)producer_layer]);
    if (!conv || conv->tops.size() != 1) return 0;
    Tensor scales;
    const Blob& b = blobs_[(size_t)conv->tops[0]];
    if (option.int8_handover && conv->int8_scale_term > 0 && conv->int8_scale_term < 100 && !conv->fused_maxpool && b.consumer >= 0) {
        auto* reader = dynamic_cast<ConvolutionLayer*>(layers_[(size_t)b.consumer]);
        if (reader && reader->int8_scale_term > 0 && !reader->fused_maxpool && reader->bottom_blob_int8_scales.defined()) {
            const int64_t ns = reader->bottom_blob_int8_scales.numel();
            if (ns == 1 || ns == conv->out_channels) scales = reader->bottom_blob_int8_scales;
        }
    }
    if (!scales.defined() && !conv->handover_scales.defined()) return 0;
    return conv->set_handover(option, scales);
}

int Net::plan_fusions() {
    blob_fused_away_.assign(blobs_.size(), 0);
    // first layer + max-pool fusion: conv1's blob must have the pool as its only reader
    if (option.fuse_first_layer_pool) {
        for (Layer* l : layers_) {
            auto* conv = dynamic_cast<ConvolutionLayer*>(l);
            if (!conv || !conv->can_fuse_maxpool()) continue;
            const Blob& b = blobs_[(size_t)conv->tops[0]];
            if (b.consumer < 0) continue;
            Layer* pool = layers_[(size_t)b.consumer];
            if (!pool->is_pool3x3s2p1() || pool->bottoms.size() != 1) continue;
            // same rule as MaxPoolLayer::forward: the reference's packed 3x3 s2 kernels pad with zeros
            conv->fused_maxpool = (option.use_packing_layout && conv->out_channels % 4 == 0) ? 2 : 1;
            pool->absorbed = true;
            blob_fused_away_[(size_t)conv->tops[0]] = 1;
        }
    }
    for (size_t i = 0; i < layers_.size(); ++i) {
        const int rc = refresh_handover((int)i);
        if (rc != 0) { error_ = "create_pipeline (int8 hand-over) of " + layers_[i]->name + " failed: " + ott_last_error(option.gpu); return rc; }
    }
    routing_dirty_ = true;
    return 0;
}

int Net::ensure_routing() const {
    if (!routing_dirty_) return 0;
    return const_cast<Net*>(this)->plan_routing();
}

// int8 hand-over through Concat / Crop / ChannelShuffle / Split. Those layers only select and re-order channel planes, so
// every channel a convolution reads can be traced back to the output channel of the layer that computed it. A 1x1
// convolution all of whose input channels come from quantized convolutions, each of those channels read by nobody else,
// needs no quantize pass: its producers store these channels as float2int8(v * its input scale), which is what the pass
// would have computed from the fp32 v (ConvolutionLayer.cpp:763-779 after QuantizeX86.cpp:851-903), and it gathers them from
// the producers' int8 tensors. Channels with any other reader (a depthwise layer, a second branch, a graph output) stay fp32.
int Net::plan_routing() {
    // fused pairs point into the layer objects the routing plan is about to replace
    for (Layer* l : layers_)
        if (auto* conv = dynamic_cast<ConvolutionLayer*>(l)) conv->set_pair_fusion(option, nullptr, -1);
    const int rc = plan_channel_routing();
    return rc != 0 ? rc : plan_pair_fusions();
}

// A depthwise 3x3 layer whose output blob has exactly one reader, a 1x1 convolution: the two run as one kernel wherever the
// library can fuse the layer objects they would run with (ConvolutionLayer::set_pair_fusion decides; not fusable is not an error).
int Net::plan_pair_fusions() {
    if (!option.fuse_depthwise_pointwise || !option.gpu) return 0;
    for (size_t li = 0; li < layers_.size(); ++li) {
        auto* dw = dynamic_cast<ConvolutionLayer*>(layers_[li]);
        if (!dw || dw->tops.size() != 1 || dw->bottoms.size() != 1) continue;
        if (dw->groups <= 1 || dw->groups != dw->in_channels || dw->groups != dw->out_channels || dw->kernel_height != 3 || dw->kernel_width != 3) continue;
        const int next = blobs_[(size_t)dw->tops[0]].consumer;
        if (next < 0) continue;
        auto* pw = dynamic_cast<ConvolutionLayer*>(layers_[(size_t)next]);
        if (!pw || pw->bottoms.size() != 1 || pw->bottoms[0] != dw->tops[0] || pw->groups != 1 || pw->kernel_height != 1 || pw->kernel_width != 1) continue;
        const int rc = pw->set_pair_fusion(option, dw, (int)li);
        if (rc != 0) { error_ = "depthwise + 1x1 fusion of " + dw->name + " and " + pw->name + " failed: " + ott_last_error(option.gpu); return rc; }
    }
    return 0;
}

int Net::plan_channel_routing() {
    routing_dirty_ = false;
    has_routing_ = false;
    blob_needs_f32_.assign(blobs_.size(), 0);
    std::vector<ConvolutionLayer*> convs(layers_.size(), nullptr);
    for (size_t i = 0; i < layers_.size(); ++i) {
        convs[i] = dynamic_cast<ConvolutionLayer*>(layers_[i]);
        if (convs[i]) convs[i]->set_routing(option, nullptr);
    }
    if (!option.int8_routing || !option.gpu) return 0;

    // 1. where every channel of every blob was computed: id -> (layer, channel of its first top blob)
    std::vector<std::vector<int>> prov(blobs_.size());
    std::vector<std::pair<int, int>> origin;
    std::vector<char> glue(layers_.size(), 0);
    for (size_t li = 0; li < layers_.size(); ++li) {
        const Layer* l = layers_[li];
        std::vector<std::vector<int>> in, out(l->tops.size());
        for (int b : l->bottoms) in.push_back(prov[(size_t)b]);
        if (!in.empty() && l->map_channels(in, out)) {
            glue[li] = 1;
            for (size_t j = 0; j < l->tops.size(); ++j) prov[(size_t)l->tops[j]] = out[j];
            continue;
        }
        if (l->absorbed && in.size() == 1 && l->tops.size() == 1 && !in[0].empty()) {
            // a max-pool computed inside its producer's kernel: its channels are that kernel's output channels
            glue[li] = 1;
            prov[(size_t)l->tops[0]] = in[0];
            continue;
        }
        for (size_t j = 0; j < l->tops.size(); ++j) {
            const Tensor& shape = blobs_[(size_t)l->tops[j]].shape;
            const int c = shape.defined() && shape.numel() >= 4 ? shape.data_ptr<int>()[1] : 0;
            for (int ch = 0; ch < c; ++ch) {
                prov[(size_t)l->tops[j]].push_back((int)origin.size());
                origin.emplace_back(j == 0 ? (int)li : -1, ch);
            }
        }
    }
    // 2. who reads each channel: layer indices, -2 for "leaves the graph"
    std::vector<std::vector<int>> readers(origin.size());
    auto add_reader = [&](int id, int who) {
        auto& r = readers[(size_t)id];
        if (std::find(r.begin(), r.end(), who) == r.end()) r.push_back(who);
    };
    for (size_t li = 0; li < layers_.size(); ++li) {
        if (glue[li]) continue;
        for (int b : layers_[li]->bottoms)
            for (int id : prov[(size_t)b]) add_reader(id, (int)li);
    }
    for (size_t b = 0; b < blobs_.size(); ++b)
        if (blobs_[b].consumer < 0)
            for (int id : prov[b]) add_reader(id, -2);

    // 3. Readers that can take their whole input from int8 tensors: 1x1 layers (any number of sources), and depthwise
    // layers that feed a 1x1 layer directly (they run on a permuted channel order, which that layer's weights absorb). A
    // channel may have several such readers when all of them quantize it with the same scale (layers reading the same blob
    // were calibrated on the same values). Start from every layer that could, and drop layers until the set is closed.
    enum : char { kNot = 0, kPointwise = 1, kDepthwise = 2 };
    std::vector<char> cand(layers_.size(), kNot);
    auto in_scale = [&](size_t li) { return convs[li]->bottom_blob_int8_scales.data_ptr<float>()[0]; };
    for (size_t li = 0; li < layers_.size(); ++li) {
        ConvolutionLayer* conv = convs[li];
        if (!conv || conv->bottoms.size() != 1 || conv->tops.size() != 1) continue;
        const int direct = blobs_[(size_t)conv->bottoms[0]].producer;
        if (direct >= 0 && !glue[(size_t)direct]) continue;  // reads its producer's blob as it is: the plain hand-over covers that
        if ((int)prov[(size_t)conv->bottoms[0]].size() != conv->in_channels) continue;
        if (conv->routable_consumer()) cand[li] = kPointwise;
        else if (conv->routable_depthwise_reader()) {
            const int next = blobs_[(size_t)conv->tops[0]].consumer;
            if (next >= 0 && convs[(size_t)next] && convs[(size_t)next]->routable_consumer()) cand[li] = kDepthwise;
        }
    }
    for (bool changed = true; changed;) {
        changed = false;
        for (size_t li = 0; li < layers_.size(); ++li) {
            if (!cand[li]) continue;
            const std::vector<int>& ids = prov[(size_t)convs[li]->bottoms[0]];
            bool ok = std::set<int>(ids.begin(), ids.end()).size() == ids.size();
            std::set<int> sources;
            for (size_t i = 0; ok && i < ids.size(); ++i) {
                const int pl = origin[(size_t)ids[i]].first;
                const ConvolutionLayer* pc = pl >= 0 ? convs[(size_t)pl] : nullptr;
                ok = pc && pc->routable_producer();
                if (ok) sources.insert(pl);
                for (int r : readers[(size_t)ids[i]])
                    ok = ok && r >= 0 && cand[(size_t)r] && in_scale((size_t)r) == in_scale(li);
                if (ok && pc->routes_all_or_nothing())  // then every channel of that producer needs readers like these
                    for (size_t id2 = 0; ok && id2 < origin.size(); ++id2) {
                        if (origin[id2].first != pl) continue;
                        ok = !readers[id2].empty();
                        for (int r : readers[id2]) ok = ok && r >= 0 && cand[(size_t)r] && in_scale((size_t)r) == in_scale(li);
                    }
            }
            if (ok && sources.size() > 12) ok = false;
            if (ok && cand[li] == kPointwise) {
                // the 32-channel blocks the kernel would read, per source from the first to the last one it needs: at most 64
                int blocks = 0;
                for (int pl : sources) {
                    int lo = 1 << 30, hi = -1;
                    for (int id : ids)
                        if (origin[(size_t)id].first == pl) { lo = std::min(lo, origin[(size_t)id].second / 32); hi = std::max(hi, origin[(size_t)id].second / 32); }
                    blocks += hi - lo + 1;
                }
                ok = blocks <= 64;
            }
            if (!ok) { cand[li] = kNot; changed = true; }
        }
    }
    std::vector<ConvolutionLayer::Routing> plans(layers_.size());
    std::vector<int> routed_to(origin.size(), -1);
    for (size_t li = 0; li < layers_.size(); ++li) {
        if (!cand[li]) continue;
        ConvolutionLayer* conv = convs[li];
        const std::vector<int>& ids = prov[(size_t)conv->bottoms[0]];
        ConvolutionLayer::Routing plan;
        plan.self_layer = (int)li;
        plan.gathered = true;
        for (int id : ids) {
            const int pl = origin[(size_t)id].first, ch = origin[(size_t)id].second;
            size_t s = 0;
            for (; s < plan.source_layers.size(); ++s)
                if (plan.source_layers[s] == pl) break;
            if (s == plan.source_layers.size()) {
                plan.source_layers.push_back(pl);
                plan.source_channels.push_back(convs[(size_t)pl]->out_channels);
            }
            plan.channel_source.push_back((int)s);
            plan.channel_index.push_back(ch);
        }
        if (cand[li] == kDepthwise) {
            // the 1x1 layer behind the depthwise layer reads that layer's output where the permuted order put each channel
            // (filled in once the depthwise twin exists)
            ConvolutionLayer::Routing& next = plans[(size_t)blobs_[(size_t)conv->tops[0]].consumer];
            next.self_layer = blobs_[(size_t)conv->tops[0]].consumer;
            next.gathered = true;
            next.direct = true;
            next.source_layers.assign(1, (int)li);
        }
        plans[li] = plan;
        for (int id : ids) routed_to[(size_t)id] = (int)li;
    }
    // 4. their producers: per-channel output scales and the fp32 planes other readers still need
    for (size_t id = 0; id < origin.size(); ++id) {
        if (routed_to[id] < 0) continue;
        const int pl = origin[id].first;
        ConvolutionLayer::Routing& plan = plans[(size_t)pl];
        if (!plan.routed_out) {
            plan.self_layer = pl;
            plan.routed_out = true;
            plan.out_scales.assign((size_t)convs[(size_t)pl]->out_channels, 0.f);
            plan.f32_mask.assign((size_t)(convs[(size_t)pl]->out_channels + 31) / 32, 0u);
        }
        plan.out_scales[(size_t)origin[id].second] = in_scale((size_t)routed_to[id]);
    }
    for (size_t id = 0; id < origin.size(); ++id) {
        const int pl = origin[id].first;
        if (pl < 0 || !plans[(size_t)pl].routed_out || routed_to[id] >= 0 || readers[id].empty()) continue;
        plans[(size_t)pl].f32_mask[(size_t)origin[id].second >> 5] |= 1u << (origin[id].second & 31);
    }
    for (size_t li = 0; li < layers_.size(); ++li) {
        if (!convs[li] || (!plans[li].gathered && !plans[li].routed_out)) continue;
        ConvolutionLayer::Routing& plan = plans[li];
        if (plan.direct) {
            const ConvolutionLayer::Routing* dw = convs[(size_t)plan.source_layers[0]]->routing();
            if (!dw || dw->stored_channels <= 0) { error_ = "int8 hand-over: depthwise twin of " + layers_[li]->name + " is missing"; return -1; }
            plan.source_channels.assign(1, dw->stored_channels);
            plan.channel_source.assign((size_t)convs[li]->in_channels, 0);
            plan.channel_index = dw->position;
        }
        const int rc = convs[li]->set_routing(option, &plan);
        if (rc != 0) { error_ = "int8 hand-over through the glue layers: layer " + layers_[li]->name + " failed: " + ott_last_error(option.gpu); return rc; }
        has_routing_ = true;
        if (cand[li] == kDepthwise) blob_needs_f32_[(size_t)convs[li]->tops[0]] = 1;  // exists in the permuted order only
    }
    for (size_t b = 0; b < blobs_.size(); ++b)
        for (int id : prov[b])
            if (routed_to[(size_t)id] >= 0) { blob_needs_f32_[b] = 1; break; }
    return 0;
}

int Net::recreate_pipeline(int layer_index) {
    if (layer_index < 0 || layer_index >= (int)layers_.size()) return -1;
    Layer* layer = layers_[(size_t)layer_index];
    int rc = layer->create_pipeline(option);
    routing_dirty_ = true;
    // the layer's input scales are the hand-over scales of the layer before it
    if (rc == 0) rc = refresh_handover(layer_index);
    for (int b : layer->bottoms)
        if (rc == 0 && blobs_[(size_t)b].producer >= 0) rc = refresh_handover(blobs_[(size_t)b].producer);
    if (rc != 0) error_ = std::string("create_pipeline failed: ") + ott_last_error(option.gpu);
    return rc;
}

void Net::summary() const {
    printf("=============================================================\n");
    printf("Layer count: %d Blob count: %zu\n", (int)layers_.size(), blobs_.size());
    for (const Layer* l : layers_) {
        printf("%-16s %-24s", l->type().c_str(), l->name.c_str());
        for (int t : l->tops) {
            const Tensor& s = blobs_[(size_t)t].shape;
            if (s.defined()) printf(" -> %s(%d,%d,%d,%d)", blobs_[(size_t)t].name.c_str(), s.data_ptr<int>()[0], s.data_ptr<int>()[1], s.data_ptr<int>()[2], s.data_ptr<int>()[3]);
        }
        printf("\n");
    }
}

Extractor Net::create_extractor() const { return Extractor(this, blobs_.size()); }

// Tensor/Net.cpp:350-378: recursive pull of missing bottoms
int Net::forward_layer(int layer_index, std::vector<Tensor>& blob_tensors, const NetOption& opt) const {
    if (layer_index < 0) { error_ = "blob has no producer and was not given as input"; return -1; }
    const Layer* layer = layers_[(size_t)layer_index];
    for (int b : layer->bottoms) {
        if (!blob_tensors[(size_t)b].defined()) {
            const int ret = forward_layer(blobs_[(size_t)b].producer, blob_tensors, opt);
            if (ret != 0) return ret;
        }
    }
    return do_forward_layer(layer, blob_tensors, opt);
}

// Tensor/Net.cpp:413-505. Every kernel of the layer is enqueued on the Net's stream; nothing waits here.
int Net::do_forward_layer(const Layer* layer, std::vector<Tensor>& blob_tensors, const NetOption& opt) const {
    if (layer->type() == "Input") return blob_tensors[(size_t)layer->tops[0]].defined() ? 0 : -1;
    int ret = 0;
    ott_event *ev0 = nullptr, *ev1 = nullptr;
    if (opt.layer_ms) {
        ott_event_create(opt.gpu, &ev0);
        ott_event_create(opt.gpu, &ev1);
        ott_event_record(opt.gpu, ev0);
    }
    struct EventGuard {
        const Net* net; const Layer* layer; const NetOption& opt; ott_event *a, *b;
        ~EventGuard() {
            if (!a) return;
            ott_event_record(opt.gpu, b);
            float ms = 0.f;
            if (ott_event_elapsed_ms(a, b, &ms) == OTT_OK) {
                const int idx = net->find_layer_index_by_name(layer->name);
                if (idx >= 0 && idx < (int)opt.layer_ms->size()) (*opt.layer_ms)[(size_t)idx] += ms;
            }
            ott_event_destroy(a);
            ott_event_destroy(b);
        }
    } guard{this, layer, opt, ev0, ev1};
    auto prepared = [&](const Tensor& t) { return (t.is_table() && !layer->accepts_tables) ? materialize(opt, t) : t; };
    if (layer->one_blob_only) {
        Tensor bottom = prepared(blob_tensors[(size_t)layer->bottoms[0]]);
        if (!bottom.defined()) { error_ = "could not materialise the input of layer " + layer->name; return -100; }
        Tensor top;
        const bool kept = opt.keep_blobs && (*opt.keep_blobs)[(size_t)layer->bottoms[0]];
        if (opt.lightmode && layer->support_inplace && bottom.use_count() <= 2 && !kept) {  // ours + the blob table's
            top = bottom;
            ret = layer->forward_inplace(top, opt);
        } else {
            ret = layer->forward(bottom, top, opt);
        }
        if (ret != 0) { error_ = "forward of layer " + layer->name + " failed: " + ott_last_error(opt.gpu); return ret; }
        blob_tensors[(size_t)layer->tops[0]] = top;
    } else {
        std::vector<Tensor> bottoms(layer->bottoms.size()), tops(layer->tops.size());
        for (size_t i = 0; i < bottoms.size(); ++i) {
            bottoms[i] = prepared(blob_tensors[(size_t)layer->bottoms[i]]);
            if (!bottoms[i].defined()) { error_ = "could not materialise an input of layer " + layer->name; return -100; }
        }
        ret = layer->forward(bottoms, tops, opt);
        if (ret != 0) { error_ = "forward of layer " + layer->name + " failed: " + ott_last_error(opt.gpu); return ret; }
        for (size_t i = 0; i < tops.size(); ++i) blob_tensors[(size_t)layer->tops[i]] = tops[i];
    }
    if (opt.lightmode)  // Tensor/Net.cpp:449-451: a consumed blob is dropped at once (the allocator reuses it stream-ordered)
        for (int b : layer->bottoms)
            if (!(opt.keep_blobs && (*opt.keep_blobs)[(size_t)b])) blob_tensors[(size_t)b].reset();
    return 0;
}

// ---------------------------------------------------------------- Extractor (Tensor/Net.cpp:659-736)
Extractor::Extractor(const Net* net, size_t blob_count) : net_(net), blob_tensors_(blob_count), option(net->option) {}

void Extractor::clear() { for (auto& t : blob_tensors_) t.reset(); }

int Extractor::keep(const std::string& blob_name) {
    const int idx = net_->find_blob_index_by_name(blob_name);
    if (idx < 0) return -1;
    if (keep_.empty()) keep_.assign(blob_tensors_.size(), 0);
    keep_[(size_t)idx] = 1;
    return 0;
}

int Extractor::input(const std::string& blob_name, const Tensor& in) {
    const int idx = net_->find_blob_index_by_name(blob_name);
    if (idx == -1) fprintf(stderr, "Input failed!\n");
    return input(idx, in);
}

int Extractor::input(int blob_index, const Tensor& in) {
    if (blob_index < 0 || blob_index >= (int)blob_tensors_.size() || !in.defined()) return -1;
    if (is_input_.empty()) is_input_.assign(blob_tensors_.size(), 0);
    is_input_[(size_t)blob_index] = 1;
    if (in.device() == Device::CUDA) {
        blob_tensors_[(size_t)blob_index] = in;
        return 0;
    }
    if (in.scalar_type() != ScalarType::Float || in.dim() != 4) return -1;
    Tensor dev = device_empty(option, in.sizes(), ScalarType::Float, Layout::NCHW);
    if (!dev.defined()) return -100;
    const int rc = ott_memcpy_h2d(option.gpu, dev.raw_data(), in.raw_data(), (size_t)in.numel() * 4);
    if (rc != OTT_OK) return rc;
    blob_tensors_[(size_t)blob_index] = dev;
    return 0;
}

int Extractor::benchmark_info(const std::string& blob_name, std::vector<float>& ms) {
    ms.assign((size_t)net_->layer_count(), 0.f);
    option.layer_ms = &ms;
    Tensor feat;
    const int rc = extract(blob_name, feat, 1);
    option.layer_ms = nullptr;
    return rc;
}

int Extractor::extract(const std::string& blob_name, Tensor& feat, int type) {
    const int idx = net_->find_blob_index_by_name(blob_name);
    if (idx == -1) fprintf(stderr, "Extract failed!\n");
    return extract(idx, feat, type);
}

int Extractor::extract_into(const std::string& blob_name, void* host_dst) {
    Tensor dev;
    int rc = extract(blob_name, dev, 1);
    if (rc != 0) return rc;
    if (dev.layout() == Layout::NCHW) {
        rc = ott_memcpy_d2h(option.gpu, host_dst, dev.raw_data(), (size_t)dev.numel() * elementSize(dev.scalar_type()));
        if (rc == OTT_OK) rc = ott_sync(option.gpu);
        return rc;
    }
    Tensor host;
    rc = extract(blob_name, host, 0);
    if (rc != 0) return rc;
    std::memcpy(host_dst, host.raw_data(), (size_t)host.numel() * elementSize(host.scalar_type()));
    return 0;
}

int Extractor::extract(int blob_index, Tensor& feat, int type) {
    if (blob_index < 0 || blob_index >= (int)blob_tensors_.size()) return -1;
    if (net_->blob_fused_away_[(size_t)blob_index]) {
        net_->error_ = "blob " + net_->blobs_[(size_t)blob_index].name + " only exists inside a fused kernel; set NetOption::fuse_first_layer_pool = false to extract it";
        return -1;
    }
    {
        // a blob that an earlier extract left in its int8 hand-over form is computed again in the reference's type
        const int prod = net_->blobs_[(size_t)blob_index].producer;
        const auto* conv = prod >= 0 ? dynamic_cast<const ConvolutionLayer*>(net_->layers_[(size_t)prod]) : nullptr;
        const Tensor& have = blob_tensors_[(size_t)blob_index];
        if (conv && conv->int8_scale_term < 100 && have.defined() && have.scalar_type() == ScalarType::Byte) blob_tensors_[(size_t)blob_index].reset();
        // a depthwise layer's blob that an earlier extract left deferred (computed inside the next layer's kernel) likewise
        if (have.defined() && have.companion_tag() >= ConvolutionLayer::kDeferredTag) blob_tensors_[(size_t)blob_index].reset();
    }
    {
        // Routing on or off for this call: off when the wanted blob, or one the caller keeps, holds a channel that would then
        // exist in int8 only. Blobs computed under the other setting are dropped first (their fp32 planes may be partial).
        const int rc = net_->ensure_routing();
        if (rc != 0) return rc;
        bool routed = option.int8_routing && net_->has_routing_ && !net_->blob_needs_f32_[(size_t)blob_index];
        for (size_t b = 0; routed && b < keep_.size(); ++b)
            if (keep_[b] && net_->blob_needs_f32_[b]) routed = false;
        if (last_mode_ >= 0 && last_mode_ != (int)routed)
            for (size_t b = 0; b < blob_tensors_.size(); ++b)
                if (is_input_.empty() || !is_input_[b]) blob_tensors_[b].reset();
        option.routing_active = routed;
    }
    if (!blob_tensors_[(size_t)blob_index].defined()) {
        option.blob_wanted = blob_index;
        option.keep_blobs = keep_.empty() ? nullptr : &keep_;
        const int ret = net_->forward_layer(net_->blobs_[(size_t)blob_index].producer, blob_tensors_, option);
        option.blob_wanted = -1;
        if (ret != 0) return ret;
        last_mode_ = (int)option.routing_active;
    }
    if (blob_tensors_[(size_t)blob_index].is_table()) {
        Tensor dense = materialize(option, blob_tensors_[(size_t)blob_index]);
        if (!dense.defined()) return -100;
        blob_tensors_[(size_t)blob_index] = dense;
    }
    const Tensor& dev = blob_tensors_[(size_t)blob_index];
    if (type != 0 || dev.device() == Device::CPU) { feat = dev; return 0; }  // (the detection layer's result is a host tensor)
    // plain host layout, like `feat.packing(1)` of the reference (Tensor/Net.cpp:729-731)
    if (dev.layout() == Layout::NCHW) {
        feat = empty(dev.sizes(), dev.scalar_type());
        int rc = ott_memcpy_d2h(option.gpu, feat.raw_data(), dev.raw_data(), (size_t)dev.numel() * elementSize(dev.scalar_type()));
        if (rc == OTT_OK) rc = ott_sync(option.gpu);
        return rc;
    }
    const int n = (int)dev.size(0), c = (int)dev.size(1), h = (int)dev.size(2), w = (int)dev.size(3);
    const int cp = ott_nhwc_channels(c);
    const size_t es = elementSize(dev.scalar_type());
    std::vector<char> tmp((size_t)n * h * w * cp * es);
    int rc = ott_memcpy_d2h(option.gpu, tmp.data(), dev.raw_data(), tmp.size());
    if (rc == OTT_OK) rc = ott_sync(option.gpu);
    if (rc != OTT_OK) return rc;
    feat = empty(dev.sizes(), dev.scalar_type());
    char* dst = static_cast<char*>(feat.raw_data());
    for (int b = 0; b < n; ++b)
        for (int y = 0; y < h; ++y)
            for (int x = 0; x < w; ++x)
                for (int ch = 0; ch < c; ++ch)
                    std::memcpy(dst + ((((size_t)b * c + ch) * h + y) * w + x) * es, tmp.data() + ((((size_t)b * h + y) * w + x) * cp + ch) * es, es);
    return 0;
}

}  // namespace otter
