// C-ABI over the host-side graph runtime (include/otter_b200_net.h).
#include <cstring>
#include <sstream>

#include "../../include/otter_b200_net.h"
#include "otter_api.hpp"

struct ott_net;
struct ott_net_graph {
    ott_net* net = nullptr;
    ott_graph* graph = nullptr;
    std::vector<otter::Tensor> outputs;  // device tensors the replays write
};

// What ott_net_forward keeps between calls with host buffers of one shape: the device input buffer and one captured forward
// per chunk of the batch (the chunks differ in where they read the input).
struct HostPipeline {
    std::string key;
    void* dev_in = nullptr;
    int chunk = 0;
    std::vector<ott_net_graph*> graphs;
};

struct ott_net {
    otter::Net net;
    std::string error;
    std::vector<HostPipeline> pipelines;
    void drop_pipelines();
    ~ott_net() { drop_pipelines(); }
};

namespace {

int fail(ott_net* n, int code, const std::string& what) {
    n->error = what;
    return code;
}

void copy_str(const std::string& s, char* dst, int cap) {
    if (!dst || cap <= 0) return;
    std::strncpy(dst, s.c_str(), (size_t)cap - 1);
    dst[cap - 1] = 0;
}

}  // namespace

extern "C" {

int ott_net_create(int device, ott_net** out) {
    if (!out) return OTT_ERR_INVALID;
    ott_net* n = new (std::nothrow) ott_net();
    if (!n) return OTT_ERR_ALLOC;
    n->net.option.device = device;
    *out = n;
    return OTT_OK;
}

int ott_net_destroy(ott_net* net) {
    delete net;
    return OTT_OK;
}

const char* ott_net_last_error(const ott_net* net) {
    if (!net) return "null net";
    return net->error.empty() ? net->net.last_error().c_str() : net->error.c_str();
}

ott_ctx* ott_net_context(ott_net* net) { return net ? net->net.context() : nullptr; }

int ott_net_load_model(ott_net* net, const char* otter_path, const char* weight_path, int weight_type) {
    if (!net || !otter_path || !weight_path || (weight_type != 0 && weight_type != 1)) return OTT_ERR_INVALID;
    net->error.clear();
    int rc = net->net.load_otter(otter_path, otter::CompileMode::Inference);
    if (rc != 0) return rc;
    return net->net.load_weight(weight_path, weight_type == 1 ? otter::Net::WeightType::Ncnn : otter::Net::WeightType::Otter);
}

int ott_net_set_option(ott_net* net, const char* key, int value) {
    if (!net || !key) return OTT_ERR_INVALID;
    otter::NetOption& o = net->net.option;
    const std::string k = key;
    if (k == "lightmode") o.lightmode = value != 0;
    else if (k == "use_packing_layout") o.use_packing_layout = value != 0;
    else if (k == "int8_rounding") o.int8_rounding = value;
    else if (k == "fuse_first_layer_pool") o.fuse_first_layer_pool = value != 0;
    else if (k == "int8_handover") o.int8_handover = value != 0;
    else if (k == "int8_routing") o.int8_routing = value != 0;
    else if (k == "fuse_depthwise_pointwise") o.fuse_depthwise_pointwise = value != 0;
    else if (k == "host_chunk") o.host_chunk = value;
    else return fail(net, OTT_ERR_INVALID, "unknown Net option: " + k);
    return OTT_OK;
}

int ott_net_add_layer(ott_net* net, const char* options) {
    if (!net || !options) return OTT_ERR_INVALID;
    otter::LayerOption opt;
    std::stringstream ss(options);
    std::string item;
    while (std::getline(ss, item, ';')) {
        const size_t eq = item.find('=');
        if (eq == std::string::npos) continue;
        auto trim = [](std::string s) {
            const size_t a = s.find_first_not_of(" \t\n"), b = s.find_last_not_of(" \t\n");
            return a == std::string::npos ? std::string() : s.substr(a, b - a + 1);
        };
        opt[trim(item.substr(0, eq))] = trim(item.substr(eq + 1));
    }
    if (!opt.count("type")) return fail(net, OTT_ERR_INVALID, "layer option without a type");
    net->net.addLayer(opt);
    return OTT_OK;
}

int ott_net_load_otter(ott_net* net, const char* path) {
    if (!net || !path) return OTT_ERR_INVALID;
    net->error.clear();
    return net->net.load_otter(path, otter::CompileMode::Initial);
}

int ott_otter_parse_text(const char* text, char* out, int cap) {
    if (!text || !out || cap <= 0) return OTT_ERR_INVALID;
    std::vector<otter::LayerOption> layers;
    std::string err;
    if (otter::parse_otter_text(text, layers, err) != 0) return OTT_ERR_INVALID;
    std::string s;
    for (auto& l : layers) {
        s += "type=" + l["type"];
        for (auto& kv : l)
            if (kv.first != "type") s += ";" + kv.first + "=" + kv.second;
        s += "\n";
    }
    if ((int)s.size() + 1 > cap) return OTT_ERR_INVALID;
    std::memcpy(out, s.c_str(), s.size() + 1);
    return (int)layers.size();
}

int ott_net_compile(ott_net* net) {
    if (!net) return OTT_ERR_INVALID;
    net->error.clear();
    return net->net.compile(otter::CompileMode::Initial);
}

int ott_net_layer_count(const ott_net* net) { return net ? net->net.layer_count() : 0; }

int ott_net_layer_info(const ott_net* net, int i, char* type, int type_cap, char* name, int name_cap, int geom[12]) {
    if (!net || i < 0 || i >= net->net.layer_count()) return OTT_ERR_INVALID;
    const otter::Layer* l = net->net.layer(i);
    copy_str(l->type(), type, type_cap);
    copy_str(l->name, name, name_cap);
    if (geom) {
        std::memset(geom, 0, sizeof(int) * 12);
        if (const auto* c = dynamic_cast<const otter::ConvolutionLayer*>(l)) {
            const int g[12] = {c->in_channels, c->out_channels, c->kernel_height, c->kernel_width, c->stride_height, c->stride_width,
                               c->padding_height, c->padding_width, c->groups, c->bias_term, c->int8_scale_term, c->activation_type};
            std::memcpy(geom, g, sizeof g);
        }
    }
    return OTT_OK;
}

int ott_net_layer_routing(ott_net* net, int i, int info[3]) {
    if (!net || !info || i < 0 || i >= net->net.layer_count()) return OTT_ERR_INVALID;
    info[0] = info[1] = info[2] = 0;
    const auto* c = dynamic_cast<const otter::ConvolutionLayer*>(net->net.layer(i));
    if (!c) return OTT_OK;
    const int rc = net->net.prepare();
    if (rc != 0) return fail(net, rc, net->net.last_error());
    if (const auto* r = c->routing()) {
        info[0] = r->gathered ? (int)r->source_layers.size() : 0;
        if (r->routed_out) {
            for (float sc : r->out_scales) info[1] += sc != 0.f;
            for (uint32_t m : r->f32_mask) info[2] += __builtin_popcount(m);
        }
    }
    return OTT_OK;
}

int ott_net_blob_shape(const ott_net* net, const char* blob, int shape[4]) {
    if (!net || !blob || !shape) return OTT_ERR_INVALID;
    const int b = net->net.find_blob_index_by_name(blob);
    if (b < 0 || !net->net.blob(b).shape.defined()) return OTT_ERR_INVALID;
    std::memcpy(shape, net->net.blob(b).shape.data_ptr<int>(), sizeof(int) * 4);
    return OTT_OK;
}

int ott_net_blob_element_size(const ott_net* net, const char* blob) {
    if (!net || !blob) return 0;
    const int b = net->net.find_blob_index_by_name(blob);
    if (b < 0) return 0;
    // a requantizing convolution's blob is int8 (Tensor/ConvolutionLayer.cpp:834-844); every other blob is fp32
    const int prod = net->net.blob(b).producer;
    const auto* c = prod >= 0 ? dynamic_cast<const otter::ConvolutionLayer*>(net->net.layer(prod)) : nullptr;
    return (c && c->int8_scale_term > 100) ? 1 : 4;
}

int ott_net_set_conv_params(ott_net* net, const char* layer, const int8_t* w_oihw, const float* bias, const float* w_scales,
                            const float* in_scales, int n_in_scales, const float* out_scales, int n_out_scales) {
    if (!net || !layer || !w_oihw || !w_scales || !in_scales) return OTT_ERR_INVALID;
    const int idx = net->net.find_layer_index_by_name(layer);
    auto* c = idx < 0 ? nullptr : dynamic_cast<otter::ConvolutionLayer*>(net->net.layer(idx));
    if (!c) return fail(net, OTT_ERR_INVALID, std::string("no Convolution layer named ") + layer);
    using otter::ScalarType;
    c->weight_data = otter::empty({c->out_channels, c->in_channels / c->groups, c->kernel_height, c->kernel_width}, ScalarType::Byte);
    std::memcpy(c->weight_data.raw_data(), w_oihw, (size_t)c->weight_data.numel());
    auto fvec = [](const float* p, int n) {
        otter::Tensor t = otter::empty({n}, ScalarType::Float);
        std::memcpy(t.raw_data(), p, sizeof(float) * (size_t)n);
        return t;
    };
    if (c->bias_term) {
        if (!bias) return fail(net, OTT_ERR_INVALID, "layer has a bias term but bias is NULL");
        c->bias_data = fvec(bias, c->out_channels);
    }
    c->weight_data_int8_scales = fvec(w_scales, c->out_channels);
    c->bottom_blob_int8_scales = fvec(in_scales, n_in_scales);
    if (c->int8_scale_term > 100) {
        if (!out_scales || n_out_scales < 1) return fail(net, OTT_ERR_INVALID, "int8 output needs top_blob_int8_scales");
        c->top_blob_int8_scales = fvec(out_scales, n_out_scales);
    }
    net->error.clear();
    net->drop_pipelines();  // captured forwards address the old parameters
    return net->net.recreate_pipeline(idx);
}

int ott_net_set_conv_params_f32(ott_net* net, const char* layer, const float* w_oihw, const float* bias) {
    if (!net || !layer || !w_oihw) return OTT_ERR_INVALID;
    const int idx = net->net.find_layer_index_by_name(layer);
    auto* c = idx < 0 ? nullptr : dynamic_cast<otter::ConvolutionLayer*>(net->net.layer(idx));
    if (!c || c->int8_scale_term != 0) return fail(net, OTT_ERR_INVALID, std::string("no fp32 Convolution layer named ") + layer);
    c->weight_data = otter::empty({c->out_channels, c->in_channels / c->groups, c->kernel_height, c->kernel_width}, otter::ScalarType::Float);
    std::memcpy(c->weight_data.raw_data(), w_oihw, (size_t)c->weight_data.numel() * sizeof(float));
    if (c->bias_term) {
        if (!bias) return fail(net, OTT_ERR_INVALID, "layer has a bias term but bias is NULL");
        c->bias_data = otter::empty({c->out_channels}, otter::ScalarType::Float);
        std::memcpy(c->bias_data.raw_data(), bias, sizeof(float) * (size_t)c->out_channels);
    }
    net->error.clear();
    net->drop_pipelines();
    return net->net.recreate_pipeline(idx);
}

int ott_net_forward(ott_net* net, const char* input_blob, const void* in, int in_on_device, int n, int c, int h, int w, int n_out,
                    const char* const* out_blobs, void* const* out_host) {
    if (!net || !input_blob || !in || n_out < 1 || !out_blobs) return OTT_ERR_INVALID;
    net->error.clear();
    // Host in, host out, large batch: run the batch in chunks so that the upload of chunk i+1 and the download of chunk i-1
    // overlap the kernels of chunk i (images are independent, so chunking changes no value). Each chunk's forward is a
    // captured CUDA graph, kept for the next call with the same shape: a chunk then costs the host one launch instead of one
    // per kernel, which is what allows chunks small enough to keep the fill and drain of the pipeline short.
    bool all_host_out = out_host != nullptr;
    for (int i = 0; all_host_out && i < n_out; ++i) all_host_out = out_host[i] != nullptr;
    const int chunk = net->net.option.host_chunk > 0 ? net->net.option.host_chunk : 64;
    if (!in_on_device && all_host_out && n >= 2 * chunk) {
        ott_ctx* ctx = net->net.context();
        const size_t img_bytes = (size_t)c * h * w * sizeof(float);
        std::string key = std::string(input_blob) + "|" + std::to_string(n) + "x" + std::to_string(c) + "x" + std::to_string(h) + "x" + std::to_string(w) +
                          "|" + std::to_string(chunk);
        for (int i = 0; i < n_out; ++i) key += std::string("|") + out_blobs[i];
        HostPipeline* pipe = nullptr;
        for (HostPipeline& p : net->pipelines)
            if (p.key == key) pipe = &p;
        int rc = OTT_OK;
        if (!pipe) {
            HostPipeline p;
            p.key = key;
            p.chunk = chunk;
            if (ott_malloc(ctx, img_bytes * n, &p.dev_in) != OTT_OK) return fail(net, OTT_ERR_ALLOC, "device allocation for the input batch failed");
            // the warm-up forward inside every capture reads the (not yet uploaded) buffer: give it defined contents
            rc = ott_memset(ctx, p.dev_in, 0, img_bytes * n);
            for (int b0 = 0; b0 < n && rc == OTT_OK; b0 += chunk) {
                const int nb = n - b0 < chunk ? n - b0 : chunk;
                ott_net_graph* g = nullptr;
                rc = ott_net_capture(net, input_blob, static_cast<char*>(p.dev_in) + img_bytes * b0, nb, c, h, w, n_out, out_blobs, &g);
                if (rc == OTT_OK) p.graphs.push_back(g);
            }
            bool dense = rc == OTT_OK;
            for (size_t gi = 0; dense && gi < p.graphs.size(); ++gi)
                for (const otter::Tensor& t : p.graphs[gi]->outputs) dense = dense && t.layout() == otter::Layout::NCHW;
            if (!dense) {  // a capture failed, or an output is an int8 NHWC blob: this shape takes the plain path below
                for (ott_net_graph* g : p.graphs) ott_net_graph_destroy(g);
                ott_free(ctx, p.dev_in);
                if (rc != OTT_OK && rc != OTT_ERR_UNSUPPORTED) return rc;
                p.graphs.clear();
                p.dev_in = nullptr;  // remembered, so that the next call does not try again
            }
            if (net->pipelines.size() >= 4) {  // a handful of shapes is kept; the oldest goes
                for (ott_net_graph* g : net->pipelines.front().graphs) ott_net_graph_destroy(g);
                if (net->pipelines.front().dev_in) ott_free(ctx, net->pipelines.front().dev_in);
                net->pipelines.erase(net->pipelines.begin());
            }
            net->pipelines.push_back(std::move(p));
            pipe = &net->pipelines.back();
            rc = OTT_OK;
        }
        if (pipe && !pipe->graphs.empty()) {
            size_t gi = 0;
            for (int b0 = 0; b0 < n && rc == OTT_OK; b0 += chunk, ++gi) {
                const int nb = n - b0 < chunk ? n - b0 : chunk;
                char* dptr = static_cast<char*>(pipe->dev_in) + img_bytes * b0;
                rc = ott_memcpy_overlapped(ctx, 0, dptr, static_cast<const char*>(in) + img_bytes * b0, img_bytes * nb);
                if (rc == OTT_OK) rc = ott_net_graph_launch(pipe->graphs[gi]);
                for (int i = 0; i < n_out && rc == OTT_OK; ++i) {
                    const otter::Tensor& t = pipe->graphs[gi]->outputs[(size_t)i];
                    const size_t per_img = (size_t)(t.numel() / t.size(0)) * otter::elementSize(t.scalar_type());
                    rc = ott_memcpy_overlapped(ctx, 1, static_cast<char*>(out_host[i]) + per_img * b0, t.raw_data(), per_img * nb);
                }
            }
            const int rc_sync = ott_sync(ctx);
            return rc != OTT_OK ? rc : rc_sync;
        }
    }
    otter::Extractor ex = net->net.create_extractor();
    otter::Tensor x;
    if (in_on_device)
        x = otter::Tensor::wrap(const_cast<void*>(in), (size_t)n * c * h * w * 4, otter::Device::CUDA, nullptr, {n, c, h, w}, otter::ScalarType::Float);
    else
        x = otter::from_blob(const_cast<void*>(in), {n, c, h, w}, otter::ScalarType::Float);
    int rc = ex.input(input_blob, x);
    if (rc != 0) return fail(net, rc, "Extractor::input failed");
    // outputs are pulled in order; a requested blob that is consumed on the way to another output must survive lightmode
    for (int i = 0; i < n_out; ++i)
        if (ex.keep(out_blobs[i]) != 0) return fail(net, OTT_ERR_INVALID, std::string("unknown blob ") + out_blobs[i]);
    std::vector<otter::Tensor> dev((size_t)n_out);
    for (int i = 0; i < n_out; ++i) {
        rc = ex.extract(out_blobs[i], dev[(size_t)i], 1);
        if (rc != 0) return rc;
    }
    for (int i = 0; i < n_out; ++i) {
        if (!out_host || !out_host[i]) continue;
        rc = ex.extract_into(out_blobs[i], out_host[i]);
        if (rc != 0) return rc;
    }
    return OTT_OK;
}

int ott_net_capture(ott_net* net, const char* input_blob, const void* in_dev, int n, int c, int h, int w, int n_out,
                    const char* const* out_blobs, ott_net_graph** out) {
    if (!net || !input_blob || !in_dev || n_out < 1 || !out_blobs || !out) return OTT_ERR_INVALID;
    net->error.clear();
    ott_ctx* ctx = net->net.context();
    if (!ctx) return fail(net, OTT_ERR_INVALID, "capture before compile");
    const otter::Tensor x = otter::Tensor::wrap(const_cast<void*>(in_dev), (size_t)n * c * h * w * 4, otter::Device::CUDA, nullptr, {n, c, h, w},
                                                otter::ScalarType::Float);
    auto run = [&](std::vector<otter::Tensor>& outs) -> int {
        otter::Extractor ex = net->net.create_extractor();
        for (int i = 0; i < n_out; ++i)
            if (ex.keep(out_blobs[i]) != 0) return fail(net, OTT_ERR_INVALID, std::string("unknown blob ") + out_blobs[i]);
        int rc = ex.input(input_blob, x);
        if (rc != 0) return fail(net, rc, "Extractor::input failed");
        outs.assign((size_t)n_out, otter::Tensor());
        for (int i = 0; i < n_out && rc == 0; ++i) rc = ex.extract(out_blobs[i], outs[(size_t)i], 1);
        for (int i = 0; i < n_out && rc == 0; ++i)
            if (outs[(size_t)i].device() != otter::Device::CUDA) rc = fail(net, OTT_ERR_UNSUPPORTED, std::string(out_blobs[i]) + " is produced on the host and cannot be captured");
        return rc;
    };
    std::vector<otter::Tensor> outs;
    int rc = run(outs);  // warm-up: every buffer size is in the allocator's cache afterwards, one-time kernel set-up is done
    if (rc == 0) rc = ott_sync(ctx);
    outs.clear();
    if (rc != 0) return rc;
    rc = ott_graph_capture_begin(ctx);
    if (rc != 0) return rc;
    rc = run(outs);
    ott_graph* g = nullptr;
    if (rc != 0) {
        ott_graph_capture_end(ctx, nullptr);
        return rc;
    }
    rc = ott_graph_capture_end(ctx, &g);
    if (rc != 0) return rc;
    // the Extractor inside run() is gone: its temporaries are back in the cache and can be set aside for the graph
    ott_graph_seal(ctx, g);
    ott_net_graph* ng = new (std::nothrow) ott_net_graph();
    if (!ng) { ott_graph_destroy(ctx, g); return OTT_ERR_ALLOC; }
    ng->net = net;
    ng->graph = g;
    ng->outputs = std::move(outs);
    *out = ng;
    return OTT_OK;
}

int ott_net_graph_launch(ott_net_graph* graph) {
    if (!graph) return OTT_ERR_INVALID;
    return ott_graph_launch(graph->net->net.context(), graph->graph);
}

int ott_net_graph_output(ott_net_graph* graph, int index, void** dev_ptr, int shape[4]) {
    if (!graph || index < 0 || index >= (int)graph->outputs.size() || !dev_ptr) return OTT_ERR_INVALID;
    const otter::Tensor& t = graph->outputs[(size_t)index];
    *dev_ptr = t.raw_data();
    if (shape)
        for (int i = 0; i < 4; ++i) shape[i] = i < t.dim() ? (int)t.size(i) : 1;
    return OTT_OK;
}

int ott_net_graph_destroy(ott_net_graph* graph) {
    if (!graph) return OTT_OK;
    ott_graph_destroy(graph->net->net.context(), graph->graph);  // synchronises, then releases the temporaries
    graph->outputs.clear();
    delete graph;
    return OTT_OK;
}

}  // extern "C"

void ott_net::drop_pipelines() {
    for (HostPipeline& p : pipelines) {
        for (ott_net_graph* g : p.graphs) ott_net_graph_destroy(g);
        if (p.dev_in && net.context()) ott_free(net.context(), p.dev_in);
    }
    pipelines.clear();
}

extern "C" {

int ott_net_forward_rows(ott_net* net, const char* input_blob, const void* in, int in_on_device, int n, int c, int h, int w, const char* out_blob,
                         float* out_host, int capacity_rows, int* rows, int* cols) {
    if (!net || !input_blob || !in || !out_blob || !out_host || !rows || !cols || capacity_rows < 0) return OTT_ERR_INVALID;
    net->error.clear();
    otter::Extractor ex = net->net.create_extractor();
    otter::Tensor x = in_on_device ? otter::Tensor::wrap(const_cast<void*>(in), (size_t)n * c * h * w * 4, otter::Device::CUDA, nullptr,
                                                          {n, c, h, w}, otter::ScalarType::Float)
                                   : otter::from_blob(const_cast<void*>(in), {n, c, h, w}, otter::ScalarType::Float);
    int rc = ex.input(input_blob, x);
    if (rc != 0) return fail(net, rc, "Extractor::input failed");
    otter::Tensor feat;
    rc = ex.extract(out_blob, feat, 0);
    if (rc != 0) return rc;
    if (feat.dim() != 2 || feat.scalar_type() != otter::ScalarType::Float) return fail(net, OTT_ERR_INVALID, std::string(out_blob) + " is not a 2-D fp32 blob");
    *rows = (int)feat.size(0);
    *cols = (int)feat.size(1);
    const int64_t take = feat.size(0) < capacity_rows ? feat.size(0) : capacity_rows;
    if (take > 0) std::memcpy(out_host, feat.raw_data(), (size_t)(take * feat.size(1)) * sizeof(float));
    return OTT_OK;
}

int ott_net_profile(ott_net* net, const char* input_blob, const void* in, int in_on_device, int n, int c, int h, int w,
                    const char* out_blob, float* ms_per_layer) {
    if (!net || !input_blob || !in || !out_blob || !ms_per_layer) return OTT_ERR_INVALID;
    net->error.clear();
    otter::Extractor ex = net->net.create_extractor();
    otter::Tensor x = in_on_device ? otter::Tensor::wrap(const_cast<void*>(in), (size_t)n * c * h * w * 4, otter::Device::CUDA, nullptr,
                                                          {n, c, h, w}, otter::ScalarType::Float)
                                   : otter::from_blob(const_cast<void*>(in), {n, c, h, w}, otter::ScalarType::Float);
    int rc = ex.input(input_blob, x);
    if (rc != 0) return fail(net, rc, "Extractor::input failed");
    std::vector<float> ms;
    rc = ex.benchmark_info(out_blob, ms);
    if (rc != 0) return rc;
    std::memcpy(ms_per_layer, ms.data(), sizeof(float) * ms.size());
    return ott_sync(net->net.context());
}

}  // extern "C"
