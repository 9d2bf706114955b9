// Host-side mirror of the reference's operator API for the int8 convolution path, in C++17.
//
// Same names, argument meaning and return codes as the reference, so that code written against
//   otter::Net::addLayer / compile / create_extractor          (Tensor/Net.hpp:28-55)
//   otter::Extractor::input / extract                          (Tensor/Net.hpp:92-98)
//   otter::Layer::parse_param / compute_output_shape / load_param / init_model / create_pipeline / forward
//                                                              (Tensor/Layer.hpp:30-49)
//   otter::LayerRegistry::CreateLayer, REGISTER_LAYER_CLASS    (Tensor/LayerRegistry.hpp:36-43,79-86)
//   otter::ParamDict                                           (Tensor/ParamDict.hpp:15-64)
//   otter::LayerOption (string -> string)                      (Tensor/Layer.hpp:21)
// keeps compiling and a quantized Convolution layer in a Net runs on the GPU "with no other change".
// The one new switch is NetOption::device (>= 0: the CUDA device the Net lives on).
//
// Everything below the Layer objects is the C-ABI of include/otter_b200.h; this file contains no kernel
// and no CPU arithmetic path: a Net without a GPU fails at compile().
#pragma once

#include <cstdint>
#include <cstdio>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/otter_b200.h"

namespace otter {

enum class ScalarType { Float, Byte, Int, Undefined };
enum class Device { CPU, CUDA };
// NCHW: the reference's plain layout. NHWC16: channels innermost, channel stride padded to a multiple of 16
// (device int8 blobs between a requantizing convolution and its consumer; replaces Byte8 elempack blobs).
enum class Layout { NCHW, NHWC16 };

inline size_t elementSize(ScalarType t) { return t == ScalarType::Byte ? 1 : 4; }

// A reference-counted handle over host or device memory (the subset of otter::Tensor the path needs:
// Tensor/Tensor.hpp, Tensor/TensorBase.hpp; Memory/DataPtr with a deleter as in Tensor/Allocator.hpp:67-110).
class Tensor {
public:
    Tensor() = default;
    bool defined() const { return static_cast<bool>(st_) || is_table(); }
    void reset() { st_.reset(); table_.reset(); sizes_.clear(); offset_ = 0; }
    long use_count() const { return st_.use_count(); }
    int64_t dim() const { return (int64_t)sizes_.size(); }
    int64_t size(int64_t i) const { return sizes_[(size_t)(i < 0 ? i + dim() : i)]; }
    const std::vector<int64_t>& sizes() const { return sizes_; }
    int64_t numel() const { int64_t n = 1; for (auto s : sizes_) n *= s; return sizes_.empty() ? 0 : n; }
    ScalarType scalar_type() const { return dtype_; }
    Device device() const { return st_ ? st_->dev : (is_table() ? Device::CUDA : Device::CPU); }
    Layout layout() const { return layout_; }
    size_t nbytes() const { return st_ ? st_->bytes : 0; }
    void* raw_data() const { return st_ ? static_cast<char*>(st_->ptr) + offset_ : nullptr; }
    template <typename T> T* data_ptr() const { return static_cast<T*>(raw_data()); }
    Tensor view(std::vector<int64_t> sizes) const;  // same storage, new sizes (-1 allowed once)
    Tensor clone() const;                            // host tensors only
    // A "plane table": an fp32 NCHW tensor whose channel planes live in other device tensors. Logical channel i is plane
    // (refs[i] & 0xFFFFFF) of bufs[refs[i] >> 24]. Concat, Crop and ChannelShuffle produce these instead of copying
    // planes; consumers that can read through a table (Convolution) do, for the rest the Net materialises a dense copy.
    bool is_table() const { return static_cast<bool>(table_); }
    const std::vector<Tensor>& table_bufs() const { return table_->bufs; }
    const std::vector<uint32_t>& table_refs() const { return table_->refs; }
    // logical channels `pick` (indices into this tensor's channels) of a dense tensor or of a table, as a table;
    // buffers no picked channel uses are dropped
    Tensor select_channels(const std::vector<int>& pick) const;
    static Tensor concat_channels(const std::vector<Tensor>& parts);
    // The int8 NHWC tensor a producer layer wrote beside this fp32 tensor, for readers that take their input already
    // quantized (see Net::plan_routing); tag = the producer's layer index. Travels with the handle, also inside plane tables.
    void set_companion(const Tensor& int8_tensor, int tag) { companion_ = std::make_shared<const Tensor>(int8_tensor); companion_tag_ = tag; }
    const Tensor* companion() const { return companion_.get(); }
    int companion_tag() const { return companion_ ? companion_tag_ : -1; }

    static Tensor wrap(void* ptr, size_t bytes, Device dev, std::function<void(void*)> deleter, std::vector<int64_t> sizes,
                       ScalarType dtype, Layout layout = Layout::NCHW);

private:
    struct Storage {
        void* ptr = nullptr;
        size_t bytes = 0;
        Device dev = Device::CPU;
        std::function<void(void*)> deleter;
        ~Storage() { if (deleter && ptr) deleter(ptr); }
    };
    std::shared_ptr<Storage> st_;
    size_t offset_ = 0;
    std::vector<int64_t> sizes_;
    ScalarType dtype_ = ScalarType::Undefined;
    Layout layout_ = Layout::NCHW;
    struct PlaneTable {
        std::vector<Tensor> bufs;    // dense device fp32 NCHW tensors
        std::vector<uint32_t> refs;  // per logical channel: (buffer << 24) | plane
    };
    std::shared_ptr<const PlaneTable> table_;
    std::shared_ptr<const Tensor> companion_;
    int companion_tag_ = -1;
};

Tensor empty(std::vector<int64_t> sizes, ScalarType dtype);                       // host, zero-initialised
Tensor from_blob(void* data, std::vector<int64_t> sizes, ScalarType dtype);       // host, not owned
Tensor tensor(std::vector<int> values, ScalarType dtype);                         // 1-D host tensor of ints/floats
Tensor full(std::vector<int64_t> sizes, float value, ScalarType dtype);

#define MAX_PARAM_COUNT 32
enum class ParamType { Undefined, Int, Float, Array };

// 32 numbered slots of int / float / Tensor (Tensor/ParamDict.hpp:15-64)
class ParamDict {
public:
    ParamDict() { clear(); }
    ParamType type(int id) const { return params[id].type; }
    int get(int id, int def) const { return params[id].type == ParamType::Int ? params[id].i : def; }
    float get(int id, float def) const { return params[id].type == ParamType::Float ? params[id].f : def; }
    Tensor get(int id, const Tensor& def) const { return params[id].type == ParamType::Array ? params[id].t : def; }
    void set(int id, int i) { params[id].type = ParamType::Int; params[id].i = i; }
    void set(int id, float f) { params[id].type = ParamType::Float; params[id].f = f; }
    void set(int id, const Tensor& v) { params[id].type = ParamType::Array; params[id].t = v; }
    void clear() { for (auto& p : params) { p.type = ParamType::Undefined; p.i = 0; p.t = Tensor(); } }
private:
    struct { ParamType type; union { int i; float f; }; Tensor t; } params[MAX_PARAM_COUNT];
};

// Tensor/NetOption.hpp:16-24 plus the device switch.
class NetOption {
public:
    bool lightmode = true;
    bool train = false;
    bool use_non_lib_optimize = true;
    bool use_packing_layout = true;   // kept for source compatibility; the GPU layouts do not depend on it
    bool use_fp16_storage = false;
    int openmp_blocktime = 20;
    int device = 0;                   // NEW: CUDA device of the Net
    ott_ctx* gpu = nullptr;           // set by Net::compile; what every Layer::forward launches on
    bool fuse_first_layer_pool = true;  // run conv1 -> MaxPool(3x3, s2, p1) as one kernel when nothing else reads conv1
    // a quantized convolution whose fp32 result is read by one other quantized convolution and nothing else writes that
    // reader's int8 input itself (same bytes as dequantize -> store -> load -> quantize); a blob asked for through
    // Extractor::extract is still delivered in fp32
    bool int8_handover = true;
    // the same hand-over through Concat / Crop / ChannelShuffle / Split: a producer stores each output channel already
    // quantized for the one convolution that will read it, and that convolution gathers its input channels from its producers'
    // int8 tensors (Net::plan_routing). routing_active is set per Extractor::extract call: off when the wanted blob (or a kept
    // one) contains a channel that would then exist in int8 only.
    bool int8_routing = true;
    bool routing_active = false;
    // a depthwise 3x3 layer (pad 1, stride 1 / 2) whose int8 output only the 1x1 layer behind it reads runs inside that layer's
    // kernel (ott_dwpw): one launch instead of two, the tensor between them never leaves the SM. Asking for the depthwise
    // layer's blob through Extractor::extract still delivers it (the pair then runs as two layers). Off by default: it pays
    // for small batches only (fewer launches), large batches run faster as two kernels whose epilogues overlap.
    bool fuse_depthwise_pointwise = false;
    int host_chunk = 64;  // ott_net_forward from host memory: images per chunk of the upload / compute / download pipeline
    const std::vector<char>* keep_blobs = nullptr;  // set by Extractor::keep: blobs lightmode must not release
    int blob_wanted = -1;  // set by Extractor::extract: the blob that must come out in the reference's own type
    int int8_rounding = OTT_ROUND_ADD_HALF_TRUNC;  // which reference build is mirrored (packed x86 default / aarch64)
    std::vector<float>* layer_ms = nullptr;  // when set: per-layer device time, indexed by layer (Extractor::benchmark_info)
};

// ---- weight files (Tensor/DataReader.hpp, Tensor/Initializer.hpp) ----
class DataReader {
public:
    virtual ~DataReader() = default;
    virtual size_t read(void* buf, size_t size) const = 0;
    virtual size_t remain() const = 0;  // bytes not yet read
};
class DataReaderFromStdio : public DataReader {
public:
    explicit DataReaderFromStdio(FILE* file) : file_(file) {}
    size_t read(void* buf, size_t size) const override;
    size_t remain() const override;
private:
    FILE* file_;
};
enum class InitializerType { Otter, Ncnn };
class Initializer {
public:
    virtual ~Initializer() = default;
    // type 0: a weight blob with its 4-byte storage tag in front (ncnn files); type 1: plain fp32 values
    virtual Tensor load(std::vector<int64_t> shape, int type) const = 0;
    InitializerType type = InitializerType::Otter;
};
// Tensor/Initializer.cpp:21-51: the reference's own weight files, plain fp32 throughout
class InitializerFromDataReader : public Initializer {
public:
    explicit InitializerFromDataReader(const DataReader& dr) : dr_(dr) { type = InitializerType::Otter; }
    Tensor load(std::vector<int64_t> shape, int type) const override;
private:
    const DataReader& dr_;
};
// Tensor/Initializer.cpp:57-188: ncnn model files. Tags: 0x000D4B38 int8 values (padded to 4 bytes), 0x0002C056 / 0 raw fp32.
// Half-precision (0x01306B47) and 256-entry table weights describe fp32 layers, which this build does not run: load fails.
class InitializerNcnnFromDataReader : public Initializer {
public:
    explicit InitializerNcnnFromDataReader(const DataReader& dr) : dr_(dr) { type = InitializerType::Ncnn; }
    Tensor load(std::vector<int64_t> shape, int type) const override;
private:
    const DataReader& dr_;
};

using LayerOption = std::unordered_map<std::string, std::string>;

#define OUTPUT_SHAPE_HINT 30
#define opt_find(opt, type) ((opt).find(type) != (opt).end())
#define opt_get_int(opt, type) int(atoi((opt)[type].c_str()))
#define opt_get_float(opt, type) float(atof((opt)[type].c_str()))
#define opt_find_int(opt, type, default) (((opt).find(type) == (opt).end()) ? (default) : opt_get_int(opt, type))
#define opt_find_float(opt, type, default) (((opt).find(type) == (opt).end()) ? (default) : opt_get_float(opt, type))
#define opt_find_string(opt, type, default) (((opt).find(type) == (opt).end()) ? std::string(default) : (opt)[type])
#define opt_check_string(opt, type) ((opt).find(type) != (opt).end())

// Tensor/Layer.hpp:23-62. Return 0 for success; -1 unsupported; -100 allocation failure (Tensor/Layer.cpp:50-59).
class Layer {
public:
    Layer();
    virtual ~Layer();
    virtual int parse_param(LayerOption& option, ParamDict& pd);
    virtual int compute_output_shape(ParamDict& pd);
    virtual int load_param(const ParamDict& pd);
    virtual int init_model();
    virtual int load_model(const Initializer& initializer);
    virtual int create_pipeline(const NetOption& opt);
    virtual std::string type() const { return "Undefined"; }

    virtual int forward(const Tensor& bottom_blob, Tensor& top_blob, const NetOption& opt) const;
    virtual int forward(const std::vector<Tensor>& bottom_blobs, std::vector<Tensor>& top_blobs, const NetOption& opt) const;
    virtual int forward_inplace(Tensor& bottom_top_blob, const NetOption& opt) const;
    virtual int forward_inplace(std::vector<Tensor>& bottom_top_blobs, const NetOption& opt) const;

    bool support_inplace = false;
    bool one_blob_only = false;
    bool support_packing = false;
    bool accepts_tables = false;  // extension: forward reads fp32 blobs through plane tables (see Tensor::is_table)
    // extension: a 3x3 stride-2 pad-1 max-pool can be absorbed into the first convolution layer (Net::compile decides)
    virtual bool is_pool3x3s2p1() const { return false; }
    bool absorbed = false;  // this layer's work is done by its producer; forward passes the blob through
    // extension: a layer that only selects / re-orders channel planes says which input channel each output channel is.
    // bottom_ids[b][c] is an opaque id of channel c of bottom b; top_ids gets the same ids. false for every other layer.
    virtual bool map_channels(const std::vector<std::vector<int>>& bottom_ids, std::vector<std::vector<int>>& top_ids) const {
        (void)bottom_ids; (void)top_ids;
        return false;
    }
    std::vector<int> bottoms, tops;
    std::vector<Tensor> bottom_shapes, top_shapes;  // Int tensors [1,4] {N,C,H,W}
    std::string name;
};

using LayerCreator = std::function<Layer*()>;
class LayerRegistry {
public:
    static std::map<std::string, LayerCreator>& Registry();
    static void AddCreator(const std::string& type, LayerCreator creator);
    static Layer* CreateLayer(const std::string& type);  // unknown type -> nullptr (the reference exits the process)
    static std::string LayerTypeListString();
};
struct LayerRegister {
    LayerRegister(const std::string& type, LayerCreator c) { LayerRegistry::AddCreator(type, std::move(c)); }
};
#define REGISTER_LAYER_CLASS(type) \
    static ::otter::LayerRegister g_creator_##type(#type, []() -> ::otter::Layer* { return new type##Layer(); })

// helpers shared by the layers
Tensor shape_tensor(int n, int c, int h, int w);                 // Int [1,4]
void read_shape(const Tensor& shape, int& n, int& c, int& h, int& w);
Tensor device_empty(const NetOption& opt, std::vector<int64_t> sizes, ScalarType dtype, Layout layout);  // from the ctx allocator
bool table_arrays(const Tensor& t, std::vector<const float*>& bufs, std::vector<int64_t>& strides);
Tensor materialize(const NetOption& opt, const Tensor& t);  // dense fp32 NCHW copy of a plane table (or t itself)
constexpr int kMaxTableBufs = 12, kMaxTableChannels = 512;  // limits of the kernels' plane tables

// ---- ConvolutionLayer (Tensor/ConvolutionLayer.hpp:15-99): the quantized layer, and the plain fp32 layer as one kernel ----
enum class ConvParam : int {
    In_channels, Out_channels, Kernel_height, Kernel_width, Stride_height, Stride_width, Padding_height, Padding_width,
    Dilation_height, Dilation_width, Output_padding_height, Output_padding_width, Group, Bias_term, Weight_data_size,
    Int8_scale_term, Activation_type, Activation_params
};

class ConvolutionLayer : public Layer {
public:
    ConvolutionLayer();
    ~ConvolutionLayer() override;
    int parse_param(LayerOption& option, ParamDict& pd) override;
    int compute_output_shape(ParamDict& pd) override;
    int load_param(const ParamDict& pd) override;
    int init_model() override;
    int load_model(const Initializer& initializer) override;
    int create_pipeline(const NetOption& opt) override;
    int forward(const Tensor& bottom_blob, Tensor& top_blob, const NetOption& opt) const override;
    std::string type() const override { return "Convolution"; }

    int in_channels = 1, out_channels = 1, kernel_height = 3, kernel_width = 3, stride_height = 1, stride_width = 1;
    int padding_height = 0, padding_width = 0, dilation_height = 1, dilation_width = 1;
    int output_padding_height = 0, output_padding_width = 0, groups = 1, bias_term = 0, int8_scale_term = 0;
    int weight_data_size = 0, activation_type = 0;
    Tensor activation_params;
    // the reference's own fields, host tensors: weight Byte OIHW, the rest Float
    Tensor weight_data, bias_data, weight_data_int8_scales, bottom_blob_int8_scales, top_blob_int8_scales, scale_in_data;

    // set by Net::compile when the layer's only consumer is an absorbable max-pool: 0 none, 1 pool (padding ignored),
    // 2 pool with the reference's packed zero-padding rule
    int fused_maxpool = 0;
    bool can_fuse_maxpool() const;
    // set by Net::compile when the only reader of the fp32 top blob is another quantized convolution: that layer's
    // bottom_blob_int8_scales. The layer then also owns a requantizing twin that writes the reader's int8 input directly.
    Tensor handover_scales;
    int set_handover(const NetOption& opt, const Tensor& consumer_input_scales);
    bool hands_over_int8() const { return gpu_conv_handover_ != nullptr; }

    // Hand-over through glue layers (Net::plan_routing). As a reader: logical input channel i is channel channel_index[i] of
    // the int8 tensor that layer source_layers[channel_source[i]] writes. As a producer: output channel c is stored quantized
    // with out_scales[c] (0: nobody reads it in int8) and, when bit c of f32_mask is set, also as an fp32 plane.
    struct Routing {
        int self_layer = -1;
        bool gathered = false;
        bool direct = false;  // the one source is the bottom blob itself: the output of a depthwise layer with gathered input
        std::vector<int> source_layers, source_channels, channel_source, channel_index;
        // a depthwise layer with gathered input computes and stores its channels in the order of its sources' 16-channel groups
        int stored_channels = 0;
        std::vector<int> position;
        bool routed_out = false;
        std::vector<float> out_scales;
        std::vector<uint32_t> f32_mask;
    };
    int set_routing(const NetOption& opt, const Routing* plan);  // NULL: drop the routed twin
    const Routing* routing() const { return gpu_conv_routed_ ? &routing_ : nullptr; }
    bool routable_consumer() const;
    bool routable_depthwise_reader() const;
    bool routable_producer() const;
    bool routes_all_or_nothing() const { return fused_maxpool != 0; }  // no fp32 side output: every channel in int8, or none

    // Depthwise + 1x1 pair fusion (Net::plan_pair_fusions), called on the 1x1 layer with the depthwise layer in front of it
    // (NULL: drop). Builds the fused state for the layer objects the two layers would run with routing on and with routing
    // off, wherever the library can fuse them. The depthwise layer's forward then hands its input on in a deferred tensor
    // (Tensor::companion_tag() == kDeferredTag + its layer index) and this layer's forward runs both.
    static constexpr int kDeferredTag = 1 << 28;
    int set_pair_fusion(const NetOption& opt, ConvolutionLayer* depthwise_front, int depthwise_layer_index);
    bool pair_ready(bool routed) const { return (routed ? pair_routed_ : pair_plain_) != nullptr; }

private:
    int forward_routed(const Tensor& bottom_blob, Tensor& top_blob, const NetOption& opt) const;
    // the two halves of forward_routed: where the routed twin's input bytes are, where its output goes
    int routed_input(const Tensor& bottom_blob, const NetOption& opt, ott_conv_io& io, std::vector<const int8_t*>& srcs, Tensor& hold) const;
    int routed_output(const NetOption& opt, int n, int oh, int ow, ott_conv_io& io, Tensor& top_blob) const;
    int forward_pair(const Tensor& depthwise_bottom, Tensor& top_blob, const NetOption& opt) const;
    bool defers(const Tensor& bottom_blob, const NetOption& opt) const;
    const ConvolutionLayer* pair_front_ = nullptr;  // on the 1x1 layer
    const ConvolutionLayer* pair_next_ = nullptr;   // on the depthwise layer
    int pair_tag_ = -1;                              // on both: kDeferredTag + the depthwise layer's index
    ott_dwpw* pair_routed_ = nullptr;
    ott_dwpw* pair_plain_ = nullptr;
    Routing routing_;
    ott_conv* gpu_conv_routed_ = nullptr;
    int make_gpu_conv(const NetOption& opt, int scale_term, const Tensor& top_scales, ott_conv** out) const;
    void release_gpu();
    ott_conv* gpu_conv_ = nullptr;
    ott_conv* gpu_conv_handover_ = nullptr;
    ott_conv_f32* gpu_conv_f32_ = nullptr;  // the fp32 layer (int8_scale_term == 0)
    ott_ctx* gpu_ctx_ = nullptr;
};

// ---- graph runtime (Tensor/Net.hpp, Tensor/Blob.hpp) ----
struct Blob {
    std::string name;
    int producer = -1, consumer = -1;
    Tensor shape;
};

// Tensor/NetOption.hpp:26-29. Inference: structure only, parameters come from Net::load_weight; Initial: random parameters.
enum class CompileMode { Inference, Initial };
class Extractor;
int parse_otter_text(const std::string& text, std::vector<LayerOption>& layers, std::string& err);  // the .otter reader

class Net {
    friend class Extractor;
public:
    Net();
    ~Net();
    Net(const Net&) = delete;
    Net& operator=(const Net&) = delete;

    void addLayer(LayerOption option);
    int compile(CompileMode mode = CompileMode::Initial);  // 0 on success (the reference throws on a bad graph)
    int load_otter(const char* model_structure, CompileMode mode = CompileMode::Initial);  // Tensor/Net.cpp:518-536
    enum class WeightType { Otter, Ncnn };
    // Tensor/Net.cpp:538-607: every layer's load_model in graph order, then create_pipeline. An ncnn file must be consumed to
    // its last byte (the reference returns non-zero otherwise).
    int load_weight(const char* weight_path, WeightType type = WeightType::Otter);
    int load_weight(const DataReader& dr, WeightType type);
    int load_weight(const Initializer& initializer);
    Extractor create_extractor() const;
    void summary() const;
    int find_blob_index_by_name(const std::string& name) const;
    int find_layer_index_by_name(const std::string& name) const;
    int layer_count() const { return (int)layers_.size(); }
    Layer* layer(int index) const { return layers_[(size_t)index]; }
    int recreate_pipeline(int layer_index);  // after the caller replaced a layer's weight fields
    const std::vector<std::string>& input_names() const { return input_names_; }
    const std::vector<std::string>& output_names() const { return output_names_; }
    const Blob& blob(int index) const { return blobs_[(size_t)index]; }
    const std::string& last_error() const { return error_; }
    int prepare() const { return ensure_routing(); }  // finish the lazy planning now (otherwise done by the first extract)
    ott_ctx* context() const { return option.gpu; }

    NetOption option;

private:
    void graph_construct();
    int refresh_handover(int producer_layer);
    int plan_fusions();  // first layer + max-pool, int8 hand-over: after every create_pipeline
    // Which channels travel in int8 through the glue layers: done lazily before the first forward after a change.
    int plan_routing();
    int plan_channel_routing();
    int plan_pair_fusions();
    int ensure_routing() const;
    int forward_layer(int layer_index, std::vector<Tensor>& blob_tensors, const NetOption& opt) const;
    int do_forward_layer(const Layer* layer, std::vector<Tensor>& blob_tensors, const NetOption& opt) const;

    std::vector<Layer*> layers_;
    std::vector<Blob> blobs_;
    std::vector<LayerOption> layer_options_;
    std::vector<std::string> input_names_, output_names_;
    std::vector<char> blob_fused_away_;  // blobs that exist only inside a fused kernel
    std::vector<char> blob_needs_f32_;   // blobs holding a channel that exists in int8 only while routing is active
    bool routing_dirty_ = true, has_routing_ = false;
    mutable std::string error_;
    bool owns_ctx_ = false;
};

class Extractor {
    friend class Net;
public:
    void clear();
    void set_lightmode(bool lightmode) { option.lightmode = lightmode; }
    // Blobs that will be extracted later from this Extractor: lightmode keeps them although their reader has run. (Every
    // other blob read by two layers survives anyway, through the Split layer the Net inserted.)
    int keep(const std::string& blob_name);
    // `in` may be a host fp32 NCHW tensor (copied to the GPU here) or a device tensor made by device_empty
    int input(const std::string& blob_name, const Tensor& in);
    int input(int blob_index, const Tensor& in);
    // type 0: result copied to a host tensor in the reference's plain layout (fp32 NCHW / int8 NCHW), after a
    // stream synchronisation; type 1: the device tensor as it is (asynchronous)
    int extract(const std::string& blob_name, Tensor& feat, int type = 0);
    int extract(int blob_index, Tensor& feat, int type = 0);
    // extract(..., type 0) straight into caller memory (pinned memory makes the copy run at PCIe speed): no staging tensor
    int extract_into(const std::string& blob_name, void* host_dst);
    // per-layer device times in ms of the layers that ran to produce blob_name (Tensor/Net.cpp:811-850 benchmark_info):
    // CUDA events around every layer, so the layers run serialised; ms has one entry per layer of the Net
    int benchmark_info(const std::string& blob_name, std::vector<float>& ms);
private:
    Extractor(const Net* net, size_t blob_count);
    const Net* net_;
    std::vector<Tensor> blob_tensors_;
    std::vector<char> keep_, is_input_;
    int last_mode_ = -1;  // -1 nothing computed yet, 0 / 1 = the blobs present were computed with routing off / on
    NetOption option;
};

}  // namespace otter
