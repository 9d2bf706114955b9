// The C-ABI of the library (include/otter_b200.h): device context, caching allocator, and the quantized
// ConvolutionLayer's create_pipeline_int8 / forward_int8 (Tensor/ConvolutionLayer.cpp:666-752, :754-847)
// mapped onto the CUDA kernels. No CPU compute path exists here: every forward launches kernels.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "conv_object.h"
#include "ctx.h"
#include "dense_umma.h"
#include "kernels.h"

using namespace ottk;

namespace {

int out_dim(int in, int k, int s, int p, int d) { return (in + 2 * p - d * (k - 1) - 1) / s + 1; }

int upload(ott_ctx* ctx, const void* host, size_t bytes, void** dev) {
    cudaError_t e = ctx->alloc->allocate(bytes, dev);
    if (e != cudaSuccess) return ctx->fail(OTT_ERR_ALLOC, "device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(*dev, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return OTT_OK;
}

int check_status_word(ott_ctx* ctx) {
    OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    OTT_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    for (cudaStream_t a : ctx->aux_stream)
        if (a) OTT_CUDA_CHECK(ctx, cudaStreamSynchronize(a));
    if (*ctx->status_host != 0) {
        const uint32_t w = *ctx->status_host;
        cudaMemsetAsync(ctx->status_dev, 0, sizeof(uint32_t), ctx->stream);
        return ctx->fail(OTT_ERR_DEVICE_WAIT, "a kernel gave up a bounded wait (status word 0x%x)", w);
    }
    return OTT_OK;
}

size_t dtype_bytes(int dtype, int n, int c, int h, int w) {
    const size_t pix = (size_t)n * h * w;
    switch (dtype) {
        case OTT_F32_NCHW: return pix * c * 4;
        case OTT_S8_NHWC: return pix * nhwc_channels(c);
        case OTT_S32_NHWC: return pix * nhwc_channels(c) * 4;
        default: return 0;
    }
}

}  // namespace

extern "C" {

int ott_cuda_device_count(int* n) {
    if (!n) return OTT_ERR_INVALID;
    int c = 0;
    if (cudaGetDeviceCount(&c) != cudaSuccess) {
        (void)cudaGetLastError();
        *n = 0;
        return OTT_ERR_CUDA;
    }
    *n = c;
    return OTT_OK;
}

int ott_ctx_create(int device, ott_ctx** out) {
    if (!out) return OTT_ERR_INVALID;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        (void)cudaGetLastError();
        return OTT_ERR_CUDA;
    }
    if (cudaSetDevice(device) != cudaSuccess) return OTT_ERR_CUDA;
    ott_ctx* ctx = new (std::nothrow) ott_ctx();
    if (!ctx) return OTT_ERR_ALLOC;
    ctx->device = device;
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess || prop.major != 10) {
        delete ctx;
        return OTT_ERR_UNSUPPORTED;  // the kernels are sm_100a only
    }
    ctx->sm_count = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete ctx;
        return OTT_ERR_CUDA;
    }
    ctx->alloc = new DeviceCachingAllocator(device);
    if (const char* g = std::getenv("OTT_DEBUG_GUARD_BYTES")) {  // the tests' guard bands for every context, also those a Net makes
        const long v = std::atol(g);
        if (v > 0) ctx->alloc->set_guard((size_t)v);
    }
    if (cudaMalloc((void**)&ctx->status_dev, sizeof(uint32_t)) != cudaSuccess ||
        cudaMallocHost((void**)&ctx->status_host, sizeof(uint32_t)) != cudaSuccess) {
        ott_ctx_destroy(ctx);
        return OTT_ERR_ALLOC;
    }
    cudaMemsetAsync(ctx->status_dev, 0, sizeof(uint32_t), ctx->stream);
    *ctx->status_host = 0;
    *out = ctx;
    return OTT_OK;
}

int ott_ctx_destroy(ott_ctx* ctx) {
    if (!ctx) return OTT_OK;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    for (cudaStream_t a : ctx->aux_stream)
        if (a) { cudaStreamSynchronize(a); cudaStreamDestroy(a); }
    delete ctx->alloc;
    if (ctx->status_dev) cudaFree(ctx->status_dev);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    if (ctx->stage_in) cudaFreeHost(ctx->stage_in);
    if (ctx->stage_out) cudaFreeHost(ctx->stage_out);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return OTT_OK;
}

const char* ott_last_error(const ott_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }
void* ott_ctx_stream(ott_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }
uint64_t ott_launch_count(const ott_ctx* ctx) { return ctx ? ctx->launches : 0; }

int ott_sync(ott_ctx* ctx) {
    if (!ctx) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    return check_status_word(ctx);
}

int ott_set_wait_limit_ms(ott_ctx* ctx, int ms) {
    if (!ctx || ms <= 0) return OTT_ERR_INVALID;
    ctx->wait_limit_ns = (unsigned long long)ms * 1000000ull;
    return OTT_OK;
}

int ott_set_depthwise_tensor_cores(ott_ctx* ctx, int on) {
    if (!ctx) return OTT_ERR_INVALID;
    if (on < 0 || on > 2) return OTT_ERR_INVALID;
    ctx->dw_tensor_cores = on;
    return OTT_OK;
}

int ott_debug_fail_alloc_after(ott_ctx* ctx, int n) {
    if (!ctx) return OTT_ERR_INVALID;
    ctx->alloc->fail_after(n);
    return OTT_OK;
}

int ott_debug_guard_bands(ott_ctx* ctx, size_t bytes) {
    if (!ctx) return OTT_ERR_INVALID;
    ctx->alloc->set_guard(bytes);
    return OTT_OK;
}

int ott_debug_check_guards(ott_ctx* ctx, long* bad_blocks) {
    if (!ctx || !bad_blocks) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    OTT_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    size_t first = 0;
    OTT_CUDA_CHECK(ctx, ctx->alloc->check_guards(bad_blocks, &first));
    if (*bad_blocks != 0) return ctx->fail(OTT_ERR_CUDA, "%ld device block(s) written outside their bounds (first: a block of %zu bytes)", *bad_blocks, first);
    return OTT_OK;
}

int ott_debug_wait_probe(ott_ctx* ctx) {
    if (!ctx) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    OTT_CUDA_CHECK(ctx, launch_wait_probe(ctx->stream, ctx->status_dev, ctx->wait_limit_ns));
    ctx->launches += 1;
    return OTT_OK;
}

int ott_malloc(ott_ctx* ctx, size_t bytes, void** out) {
    if (!ctx || !out) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    cudaError_t e = ctx->alloc->allocate(bytes, out);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return ctx->fail(OTT_ERR_ALLOC, "device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    }
    return OTT_OK;
}

int ott_free(ott_ctx* ctx, void* p) {
    if (!ctx) return OTT_ERR_INVALID;
    return ctx->alloc->free(p) ? OTT_OK : ctx->fail(OTT_ERR_INVALID, "pointer was not allocated by this context");
}

int ott_alloc_stats(ott_ctx* ctx, uint64_t* m, uint64_t* h, uint64_t* u, uint64_t* c) {
    if (!ctx) return OTT_ERR_INVALID;
    ctx->alloc->stats(m, h, u, c);
    return OTT_OK;
}

int ott_alloc_release_cached(ott_ctx* ctx) {
    if (!ctx) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    ctx->alloc->release_cached();
    return OTT_OK;
}

int ott_host_alloc(size_t bytes, void** out) {
    if (!out) return OTT_ERR_INVALID;
    if (cudaMallocHost(out, bytes ? bytes : 1) != cudaSuccess) {
        (void)cudaGetLastError();
        return OTT_ERR_ALLOC;
    }
    return OTT_OK;
}

int ott_host_free(void* p) { return cudaFreeHost(p) == cudaSuccess ? OTT_OK : OTT_ERR_CUDA; }

int ott_memcpy_h2d(ott_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return OTT_OK;
}

int ott_memcpy_d2h(ott_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return OTT_OK;
}

int ott_memcpy_overlapped(ott_ctx* ctx, int direction, void* dst, const void* src, size_t bytes) {
    if (!ctx || !dst || !src || (direction != 0 && direction != 1)) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    cudaStream_t& aux = ctx->aux_stream[direction];
    if (!aux) OTT_CUDA_CHECK(ctx, cudaStreamCreateWithFlags(&aux, cudaStreamNonBlocking));
    cudaEvent_t ev;
    OTT_CUDA_CHECK(ctx, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    if (direction == 0) {
        // host -> device: runs beside whatever the compute stream is doing; later compute work waits for it
        OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, aux));
        OTT_CUDA_CHECK(ctx, cudaEventRecord(ev, aux));
        OTT_CUDA_CHECK(ctx, cudaStreamWaitEvent(ctx->stream, ev, 0));
    } else {
        // device -> host: waits for the compute work enqueued so far, then runs beside later compute work
        OTT_CUDA_CHECK(ctx, cudaEventRecord(ev, ctx->stream));
        OTT_CUDA_CHECK(ctx, cudaStreamWaitEvent(aux, ev, 0));
        OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, aux));
    }
    cudaEventDestroy(ev);  // released by the runtime once the recorded work has completed
    return OTT_OK;
}

// ---- CUDA graphs: a sequence of calls on the context's stream frozen into one launch ----
struct ott_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    std::vector<void*> pinned;  // allocator blocks the captured kernels address
    uint64_t launches = 0;      // kernels inside
};

int ott_graph_capture_begin(ott_ctx* ctx) {
    if (!ctx) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    if (ctx->capture_launches0 != UINT64_MAX) return ctx->fail(OTT_ERR_INVALID, "a capture is already open on this context");
    ctx->alloc->begin_log();
    // relaxed mode: the calls in between may use cudaMalloc-class routines (a cache miss in the allocator) without
    // invalidating the capture
    cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed);
    if (e != cudaSuccess) {
        (void)ctx->alloc->take_logged();
        return ctx->fail(OTT_ERR_CUDA, "cudaStreamBeginCapture: %s", cudaGetErrorString(e));
    }
    ctx->capture_launches0 = ctx->launches;
    return OTT_OK;
}

int ott_graph_capture_end(ott_ctx* ctx, ott_graph** out) {
    if (!ctx || ctx->capture_launches0 == UINT64_MAX) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    const uint64_t launches = ctx->launches - ctx->capture_launches0;
    ctx->capture_launches0 = UINT64_MAX;
    if (e != cudaSuccess || !graph || !out) {
        if (graph) cudaGraphDestroy(graph);
        ctx->alloc->give_back(ctx->alloc->take_logged());
        if (!out && e == cudaSuccess) return OTT_OK;  // capture abandoned by the caller
        return ctx->fail(OTT_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
    }
    ott_graph* g = new (std::nothrow) ott_graph();
    if (!g) { cudaGraphDestroy(graph); ctx->alloc->give_back(ctx->alloc->take_logged()); return OTT_ERR_ALLOC; }
    g->graph = graph;
    g->launches = launches;
    e = cudaGraphInstantiate(&g->exec, graph, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(graph);
        delete g;
        ctx->alloc->give_back(ctx->alloc->take_logged());
        return ctx->fail(OTT_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    }
    *out = g;
    return OTT_OK;
}

int ott_graph_seal(ott_ctx* ctx, ott_graph* g) {
    if (!ctx || !g) return OTT_ERR_INVALID;
    const std::vector<void*> taken = ctx->alloc->take_logged();
    g->pinned.insert(g->pinned.end(), taken.begin(), taken.end());
    return OTT_OK;
}

int ott_graph_launch(ott_ctx* ctx, ott_graph* g) {
    if (!ctx || !g || !g->exec) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    OTT_CUDA_CHECK(ctx, cudaGraphLaunch(g->exec, ctx->stream));
    ctx->launches += g->launches;
    return OTT_OK;
}

int ott_graph_destroy(ott_ctx* ctx, ott_graph* g) {
    if (!g) return OTT_OK;
    if (ctx) {
        cudaSetDevice(ctx->device);
        cudaStreamSynchronize(ctx->stream);  // no replay may still be addressing the blocks
        ctx->alloc->give_back(g->pinned);
    }
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    return OTT_OK;
}

int ott_memset(ott_ctx* ctx, void* dst, int value, size_t bytes) {
    if (!ctx) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    OTT_CUDA_CHECK(ctx, cudaMemsetAsync(dst, value, bytes, ctx->stream));
    return OTT_OK;
}

int ott_event_create(ott_ctx* ctx, ott_event** out) {
    if (!ctx || !out) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    ott_event* e = new (std::nothrow) ott_event();
    if (!e) return OTT_ERR_ALLOC;
    if (cudaEventCreate(&e->ev) != cudaSuccess) {
        delete e;
        return ctx->fail(OTT_ERR_CUDA, "cudaEventCreate failed");
    }
    *out = e;
    return OTT_OK;
}

int ott_event_record(ott_ctx* ctx, ott_event* ev) {
    if (!ctx || !ev) return OTT_ERR_INVALID;
    OTT_CUDA_CHECK(ctx, cudaEventRecord(ev->ev, ctx->stream));
    return OTT_OK;
}

int ott_event_elapsed_ms(ott_event* start, ott_event* stop, float* ms) {
    if (!start || !stop || !ms) return OTT_ERR_INVALID;
    if (cudaEventSynchronize(stop->ev) != cudaSuccess) return OTT_ERR_CUDA;
    return cudaEventElapsedTime(ms, start->ev, stop->ev) == cudaSuccess ? OTT_OK : OTT_ERR_CUDA;
}

int ott_event_destroy(ott_event* ev) {
    if (!ev) return OTT_OK;
    cudaEventDestroy(ev->ev);
    delete ev;
    return OTT_OK;
}

int ott_nhwc_channels(int c) { return nhwc_channels(c); }

int ott_quantize_f32_nchw_to_s8_nhwc(ott_ctx* ctx, const float* x_dev, int n, int c, int h, int w, const float* scales_host,
                                     int n_scales, int rounding, int8_t* out_dev) {
    if (!ctx || !x_dev || !out_dev || !scales_host || n < 0 || c <= 0 || h < 0 || w < 0) return OTT_ERR_INVALID;
    if (n_scales != 1 && n_scales != c) return ctx->fail(OTT_ERR_INVALID, "n_scales must be 1 or the channel count");
    cudaSetDevice(ctx->device);
    DeviceBlock sc;
    if (sc.alloc(ctx, sizeof(float) * n_scales) != cudaSuccess) return ctx->fail(OTT_ERR_ALLOC, "scale upload allocation failed");
    OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(sc.p, scales_host, sizeof(float) * n_scales, cudaMemcpyHostToDevice, ctx->stream));
    OTT_CUDA_CHECK(ctx, launch_quantize_dense(ctx->stream, x_dev, c, out_dev, (const float*)sc.p, n_scales, n, c, h, w, rounding));
    ctx->launches += (uint64_t)((nhwc_channels(c) + kGatherMaxChannels - 1) / kGatherMaxChannels);
    // the pageable scale array must stay readable until the copy has been issued; it has (pageable copies
    // are staged synchronously)
    return OTT_OK;
}

namespace {
struct GatheredInput {
    int n_sources;
    const int* source_channels;  // [n_sources]
    const int* channel_source;   // [cin]
    const int* channel_index;    // [cin]
};
int conv_create_impl(ott_ctx* ctx, const ott_conv_desc* d, const int8_t* w_oihw, const float* bias, const float* w_scales,
                     const float* in_scales, int n_in_scales, const float* out_scales, int n_out_scales, const GatheredInput* gi,
                     ott_conv** out);
}  // namespace

int ott_conv_int8_create(ott_ctx* ctx, const ott_conv_desc* d, const int8_t* w_oihw, const float* bias, const float* w_scales,
                         const float* in_scales, int n_in_scales, const float* out_scales, int n_out_scales, ott_conv** out) {
    return conv_create_impl(ctx, d, w_oihw, bias, w_scales, in_scales, n_in_scales, out_scales, n_out_scales, nullptr, out);
}

namespace {
// Depthwise layer over gathered int8 input. The kernel reads whole 16-channel groups, each from one source tensor, so the
// layer is rebuilt over the channel order "for every source, the aligned 16-channel groups that cover what is read from it":
// filters, scales and bias move to their channel's new position, every other channel of a group gets zero parameters (its
// output is 0). The output tensor has that order too (ott_conv_int8_gathered_layout tells the reader).
int create_gathered_depthwise(ott_ctx* ctx, const ott_conv_desc* d, const int8_t* w_oihw, const float* bias, const float* w_scales,
                              const float* in_scales, int n_in_scales, const float* out_scales, int n_out_scales, int n_sources,
                              const int* source_channels, const int* channel_source, const int* channel_index, ott_conv** out) {
    if (!w_oihw || !w_scales || !in_scales || !out) return OTT_ERR_INVALID;
    ConvShape probe{};
    probe.kh = d->kh; probe.kw = d->kw; probe.sh = d->sh; probe.sw = d->sw; probe.dh = d->dh; probe.dw = d->dw;
    if (!depthwise_tiled_supports(probe, d->int8_scale_term > 100 ? DT_S8_NHWC : DT_F32_NCHW) || d->int8_scale_term < 100)
        return ctx->fail(OTT_ERR_UNSUPPORTED, "gathered input: depthwise layers need a 3x3 / 5x5, stride 1 / 2, undilated filter and int8 output");
    for (int i = 1; i < n_in_scales; ++i)
        if (in_scales[i] != in_scales[0]) return ctx->fail(OTT_ERR_UNSUPPORTED, "gathered input: one input scale for all channels");
    // Granularity of the groups: 32 channels when the layer will run on the tensor cores (3x3, pad 1, stride 1 / 2: one K block
    // of the MMA per group; every source must then be at least 32 channels wide), else the CUDA-core kernel's 16.
    bool tensor = ctx->dw_tensor_cores != 0 && d->kh == 3 && d->kw == 3 && d->ph == 1 && d->pw == 1 && d->sh == d->sw && (d->sh == 1 || d->sh == 2) &&
                  d->rounding == OTT_ROUND_ADD_HALF_TRUNC;
    for (int i = 0; tensor && i < n_sources; ++i) tensor = nhwc_channels(source_channels[i]) >= 32;
    const int C = d->cin, G16 = tensor ? 32 : 16;
    std::vector<int> lo(n_sources, 1 << 30), hi(n_sources, -1), base(n_sources, 0);
    for (int i = 0; i < C; ++i) {
        const int sidx = channel_source[i], pos = channel_index[i];
        if (sidx < 0 || sidx >= n_sources || pos < 0 || pos >= source_channels[sidx])
            return ctx->fail(OTT_ERR_INVALID, "gathered input: channel %d names channel %d of source %d", i, pos, sidx);
        lo[sidx] = std::min(lo[sidx], pos / G16);
        hi[sidx] = std::max(hi[sidx], pos / G16);
    }
    std::vector<uint16_t> block_x;
    std::vector<uint8_t> block_src;
    for (int sidx = 0; sidx < n_sources; ++sidx) {
        if (hi[sidx] < 0) return ctx->fail(OTT_ERR_UNSUPPORTED, "gathered input: source %d is unused", sidx);
        base[sidx] = (int)block_x.size();
        for (int b = lo[sidx]; b <= hi[sidx]; ++b) {
            block_x.push_back((uint16_t)(b * G16));
            block_src.push_back((uint8_t)sidx);
        }
    }
    const int Cs = (int)block_x.size() * G16, taps = d->kh * d->kw;
    if ((int)block_x.size() > (tensor ? kUmmaMaxGatherBlocks : kGatherMaxChannels))
        return ctx->fail(OTT_ERR_UNSUPPORTED, "gathered input: too many channel groups");
    std::vector<int> position(C);
    std::vector<int8_t> w2((size_t)Cs * taps, 0);
    std::vector<float> ws2(Cs, 0.f), b2(Cs, 0.f), os2(Cs, 0.f);
    std::vector<char> taken(Cs, 0);
    for (int i = 0; i < C; ++i) {
        const int sidx = channel_source[i], pos = channel_index[i];
        const int p = (base[sidx] + pos / G16 - lo[sidx]) * G16 + pos % G16;
        if (taken[p]) return ctx->fail(OTT_ERR_UNSUPPORTED, "gathered input: channel %d of source %d is read twice", pos, sidx);
        taken[p] = 1;
        position[i] = p;
        std::memcpy(&w2[(size_t)p * taps], w_oihw + (size_t)i * taps, (size_t)taps);
        ws2[p] = w_scales[i];
        if (d->bias_term && bias) b2[p] = bias[i];
        if (out_scales) os2[p] = n_out_scales == 1 ? out_scales[0] : out_scales[i];
    }
    ott_conv_desc d2 = *d;
    d2.cin = d2.cout = d2.groups = Cs;
    const float in0 = in_scales[0];
    int rc = conv_create_impl(ctx, &d2, w2.data(), d->bias_term ? b2.data() : nullptr, ws2.data(), &in0, 1, out_scales ? os2.data() : nullptr,
                              out_scales ? Cs : 0, nullptr, out);
    if (rc != OTT_OK) return rc;
    ott_conv* c = *out;
    c->block_x = block_x;
    c->block_src = block_src;
    c->src_channels.assign(source_channels, source_channels + n_sources);
    c->position = position;
    c->stored_channels = Cs;
    c->gather_group = G16;
    if (tensor && !c->dw_umma) {  // the tensor-core plan did not fit: the groups are of no use to the other kernel
        ott_conv_int8_destroy(ctx, c);
        *out = nullptr;
        return ctx->fail(OTT_ERR_UNSUPPORTED, "gathered input: the depthwise layer does not fit the tensor-core kernel");
    }
    return OTT_OK;
}
}  // namespace

int ott_conv_int8_gathered_layout(const ott_conv* c, int* stored_channels, int* position, int n_position) {
    if (!c || !stored_channels) return OTT_ERR_INVALID;
    *stored_channels = c->stored_channels;
    if (position)
        for (int i = 0; i < n_position && i < (int)c->position.size(); ++i) position[i] = c->position[(size_t)i];
    return OTT_OK;
}

int ott_conv_int8_create_gathered(ott_ctx* ctx, const ott_conv_desc* d, const int8_t* w_oihw, const float* bias, const float* w_scales,
                                  const float* in_scales, int n_in_scales, const float* out_scales, int n_out_scales, int n_sources,
                                  const int* source_channels, const int* channel_source, const int* channel_index, ott_conv** out) {
    if (!ctx || !d || !source_channels || !channel_source || !channel_index) return OTT_ERR_INVALID;
    if (n_sources < 1 || n_sources > kUmmaMaxSources) return ctx->fail(OTT_ERR_UNSUPPORTED, "gathered input: 1..%d sources", kUmmaMaxSources);
    if (d->groups > 1 && d->groups == d->cin && d->groups == d->cout)
        return create_gathered_depthwise(ctx, d, w_oihw, bias, w_scales, in_scales, n_in_scales, out_scales, n_out_scales, n_sources, source_channels,
                                         channel_source, channel_index, out);
    if (d->kh != 1 || d->kw != 1 || d->sh != 1 || d->sw != 1 || d->ph != 0 || d->pw != 0 || d->groups != 1 || n_in_scales != 1)
        return ctx->fail(OTT_ERR_UNSUPPORTED, "gathered input: 1x1 stride-1 unpadded dense layers with one input scale, or depthwise layers");
    const GatheredInput gi{n_sources, source_channels, channel_source, channel_index};
    return conv_create_impl(ctx, d, w_oihw, bias, w_scales, in_scales, n_in_scales, out_scales, n_out_scales, &gi, out);
}

namespace {
int conv_create_impl(ott_ctx* ctx, const ott_conv_desc* d, const int8_t* w_oihw, const float* bias, const float* w_scales,
                     const float* in_scales, int n_in_scales, const float* out_scales, int n_out_scales, const GatheredInput* gi,
                     ott_conv** out) {
    if (!ctx || !d || !w_oihw || !w_scales || !in_scales || !out) return OTT_ERR_INVALID;
    *out = nullptr;
    if (d->cin <= 0 || d->cout <= 0 || d->kh <= 0 || d->kw <= 0 || d->sh <= 0 || d->sw <= 0 || d->dh <= 0 || d->dw <= 0 ||
        d->ph < 0 || d->pw < 0 || d->groups <= 0)
        return ctx->fail(OTT_ERR_INVALID, "bad convolution geometry");
    if (d->int8_scale_term == 0) return ctx->fail(OTT_ERR_UNSUPPORTED, "int8_scale_term == 0 is the fp32 layer; only the int8 path lives here");
    if (d->act_type < 0 || d->act_type > 3)
        return ctx->fail(OTT_ERR_UNSUPPORTED, "activation %d is not reproducible bit-for-bit on the GPU (only none/ReLU/LeakyReLU/ReLU6)", d->act_type);
    if (d->bias_term && !bias) return ctx->fail(OTT_ERR_INVALID, "bias_term set but bias is NULL");
    const bool requant = d->int8_scale_term > 100;
    if (requant && (!out_scales || (n_out_scales != 1 && n_out_scales != d->cout)))
        return ctx->fail(OTT_ERR_INVALID, "int8 output needs top_blob_int8_scales of size 1 or cout");
    const bool depthwise = d->groups == d->cin && d->groups == d->cout && d->groups > 1;
    if (!depthwise && d->groups != 1)
        return ctx->fail(OTT_ERR_UNSUPPORTED, "grouped (non-depthwise) int8 convolution is not supported");
    if (n_in_scales != 1 && n_in_scales != d->cin) return ctx->fail(OTT_ERR_INVALID, "bottom_blob_int8_scales must have 1 or cin entries");
    cudaSetDevice(ctx->device);

    ott_conv* c = new (std::nothrow) ott_conv();
    if (!c) return OTT_ERR_ALLOC;
    c->d = *d;
    c->depthwise = depthwise;
    c->cin_pad = nhwc_channels(d->cin);
    c->cout_pad = nhwc_channels(d->cout);
    c->n_in_scales = n_in_scales;

    // scale_in exactly as ConvolutionLayer.cpp:667-679: fp32 product, fp32 divide, 0 for a zero weight scale
    std::vector<float> scale_in(c->cout_pad, 0.f), bias_p(c->cout_pad, 0.f), scale_out(c->cout_pad, 0.f);
    for (int p = 0; p < d->cout; ++p) {
        volatile float prod = in_scales[0] * w_scales[p];
        scale_in[p] = w_scales[p] == 0.f ? 0.f : 1.f / prod;
        if (d->bias_term) bias_p[p] = bias[p];
        if (requant) scale_out[p] = n_out_scales == 1 ? out_scales[0] : out_scales[p];
    }

    c->w_host.assign(w_oihw, w_oihw + (size_t)d->cout * (d->cin / d->groups) * d->kh * d->kw);
    c->scale_in_host = scale_in;
    c->bias_host = bias_p;
    c->scale_out_host = scale_out;
    c->in_scale0 = in_scales[0];
    int rc = OTT_OK;
    std::vector<int8_t> wpacked;
    const int taps = d->kh * d->kw;
    if (gi) {
        // K blocks: for every source the aligned 32-channel blocks that cover the channels this layer reads from it
        std::vector<int> lo(gi->n_sources, 1 << 30), hi(gi->n_sources, -1), base(gi->n_sources, 0);
        for (int i = 0; i < d->cin; ++i) {
            const int sidx = gi->channel_source[i], pos = gi->channel_index[i];
            if (sidx < 0 || sidx >= gi->n_sources || pos < 0 || pos >= gi->source_channels[sidx]) {
                delete c;
                return ctx->fail(OTT_ERR_INVALID, "gathered input: channel %d names channel %d of source %d", i, pos, sidx);
            }
            lo[sidx] = std::min(lo[sidx], pos / kUmmaGatherBlock);
            hi[sidx] = std::max(hi[sidx], pos / kUmmaGatherBlock);
        }
        int nblocks = 0;
        for (int sidx = 0; sidx < gi->n_sources; ++sidx) {
            if (hi[sidx] < 0 || nhwc_channels(gi->source_channels[sidx]) < kUmmaGatherBlock) {
                delete c;
                return ctx->fail(OTT_ERR_UNSUPPORTED, "gathered input: source %d is unused or narrower than %d channels", sidx, kUmmaGatherBlock);
            }
            base[sidx] = nblocks;
            for (int b = lo[sidx]; b <= hi[sidx]; ++b, ++nblocks) {
                c->block_x.push_back((uint16_t)(b * kUmmaGatherBlock));
                c->block_src.push_back((uint8_t)sidx);
            }
        }
        int smem_optin = 0;
        cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, ctx->device);
        const int kk = nblocks * kUmmaGatherBlock;
        // a stage that holds the whole K extent of a tile when shared memory allows (one barrier round trip per tile)
        // (unless that would cost weight panels: every extra panel fetches the activations once more)
        ottk::UmmaPlan per_block{}, per_tile{};
        const bool ok_block = nblocks <= kUmmaMaxGatherBlocks && umma_plan_layer(kk, d->cout, 1, 1, 1, 1, 1, 1, smem_optin, &per_block, kUmmaGatherBlock, false);
        const bool ok_tile = nblocks <= kUmmaMaxGatherBlocks && umma_plan_layer(kk, d->cout, 1, 1, 1, 1, 1, 1, smem_optin, &per_tile, kUmmaGatherBlock, true);
        if (ok_tile && (!ok_block || per_tile.n_tiles <= per_block.n_tiles)) c->plan = per_tile;
        else if (ok_block) c->plan = per_block;
        if (!ok_tile && !ok_block) {
            delete c;
            return ctx->fail(OTT_ERR_UNSUPPORTED, "gathered input: %d K blocks do not fit the tensor-core kernel", nblocks);
        }
        c->plan.gather = gi->n_sources;
        c->src_channels.assign(gi->source_channels, gi->source_channels + gi->n_sources);
        c->kind = OTT_KERNEL_DENSE_UMMA;
        // the layer's weights against that K order; channels of a block that other layers read get zero weights
        std::vector<int8_t> wk((size_t)d->cout * kk, 0);
        std::vector<char> taken((size_t)kk, 0);
        for (int i = 0; i < d->cin; ++i) {
            const int sidx = gi->channel_source[i], pos = gi->channel_index[i];
            const int k = (base[sidx] + pos / kUmmaGatherBlock - lo[sidx]) * kUmmaGatherBlock + pos % kUmmaGatherBlock;
            if (taken[(size_t)k]) {
                delete c;
                return ctx->fail(OTT_ERR_UNSUPPORTED, "gathered input: channel %d of source %d is read twice", pos, sidx);
            }
            taken[(size_t)k] = 1;
            for (int o = 0; o < d->cout; ++o) wk[(size_t)o * kk + k] = w_oihw[(size_t)o * d->cin + i];
        }
        wpacked.resize((size_t)c->plan.cout_rows * c->plan.k_total);
        umma_pack_weights(c->plan, wk.data(), kk, d->cout, 1, 1, wpacked.data());
        c->w_korder = std::move(wk);
    } else if (depthwise) {
        c->kind = OTT_KERNEL_DEPTHWISE;
        // [tap][c_pad], channel innermost: what depthwise.cu reads as 32-bit words of 4 channels
        wpacked.assign((size_t)taps * c->cout_pad, 0);
        for (int ch = 0; ch < d->cout; ++ch)
            for (int t = 0; t < taps; ++t) wpacked[(size_t)t * c->cout_pad + ch] = w_oihw[(size_t)ch * taps + t];
    } else {
        int smem_optin = 0;
        cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, ctx->device);
        if (umma_plan_layer(d->cin, d->cout, d->kh, d->kw, d->sh, d->sw, d->dh, d->dw, smem_optin, &c->plan)) {
            c->kind = OTT_KERNEL_DENSE_UMMA;
            wpacked.resize((size_t)c->plan.cout_rows * c->plan.k_total);
            umma_pack_weights(c->plan, w_oihw, d->cin, d->cout, d->kh, d->kw, wpacked.data());
        } else {
            c->kind = OTT_KERNEL_DENSE_DIRECT;
            // [cout_pad][tap][cin_pad]
            wpacked.assign((size_t)c->cout_pad * taps * c->cin_pad, 0);
            for (int o = 0; o < d->cout; ++o)
                for (int ci = 0; ci < d->cin; ++ci)
                    for (int t = 0; t < taps; ++t)
                        wpacked[((size_t)o * taps + t) * c->cin_pad + ci] = w_oihw[((size_t)o * d->cin + ci) * taps + t];
        }
    }
    rc = upload(ctx, wpacked.data(), wpacked.size(), (void**)&c->w_dev);
    std::vector<uint32_t> wtiled;
    if (rc == OTT_OK && depthwise && d->kh == d->kw && (d->kh == 3 || d->kh == 5)) {
        wtiled.resize((size_t)c->cout_pad * depthwise_tiled_weight_words(d->kh));
        depthwise_tiled_pack_weights(w_oihw, d->cout, c->cout_pad, d->kh, wtiled.data());
        rc = upload(ctx, wtiled.data(), wtiled.size() * 4, (void**)&c->w_tiled_dev);
    }
    if (rc == OTT_OK && depthwise && !gi && d->kh == 3 && d->kw == 3 && d->ph == 1 && d->pw == 1 && d->dh == 1 && d->dw == 1 && d->sh == d->sw &&
        (d->sh == 1 || d->sh == 2) && d->rounding == OTT_ROUND_ADD_HALF_TRUNC) {
        int smem_optin = 0;
        cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, ctx->device);
        if (dw_umma_plan(d->cout, d->sh, smem_optin, &c->dw_plan)) {
            std::vector<int8_t> wd(dw_umma_weight_bytes(c->dw_plan));
            dw_umma_pack_weights(c->dw_plan, w_oihw, d->cout, wd.data());
            rc = upload(ctx, wd.data(), wd.size(), (void**)&c->w_dwu_dev);
            if (rc == OTT_OK) {
                rc = cudaStreamSynchronize(ctx->stream) == cudaSuccess ? OTT_OK : ctx->fail(OTT_ERR_CUDA, "upload failed");  // wd dies here
                const char* err = rc == OTT_OK ? dw_umma_encode_weight_map(c->dw_plan, c->w_dwu_dev, c->weight_map_dw) : nullptr;
                if (err) rc = ctx->fail(OTT_ERR_CUDA, "%s", err);
                c->dw_umma = rc == OTT_OK;
            }
        }
    }
    if (rc == OTT_OK) rc = upload(ctx, scale_in.data(), sizeof(float) * c->cout_pad, (void**)&c->scale_in_dev);
    if (rc == OTT_OK) rc = upload(ctx, bias_p.data(), sizeof(float) * c->cout_pad, (void**)&c->bias_dev);
    if (rc == OTT_OK) rc = upload(ctx, scale_out.data(), sizeof(float) * c->cout_pad, (void**)&c->scale_out_dev);
    if (rc == OTT_OK) rc = upload(ctx, in_scales, sizeof(float) * n_in_scales, (void**)&c->in_scales_dev);
    if (rc == OTT_OK && c->kind == OTT_KERNEL_DENSE_UMMA) {
        const char* err = umma_encode_weight_map(c->plan, c->w_dev, c->weight_map);
        if (err) rc = ctx->fail(OTT_ERR_CUDA, "%s", err);
    }
    // host staging vectors die at return: make sure the uploads have consumed them
    if (rc == OTT_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = ctx->fail(OTT_ERR_CUDA, "upload failed");
    if (rc != OTT_OK) {
        ott_conv_int8_destroy(ctx, c);
        return rc;
    }
    *out = c;
    return OTT_OK;
}
}  // namespace

int ott_conv_int8_destroy(ott_ctx* ctx, ott_conv* c) {
    if (!c) return OTT_OK;
    if (ctx) {
        ctx->alloc->free(c->w_dev);
        ctx->alloc->free(c->w_tiled_dev);
        ctx->alloc->free(c->w_dwu_dev);
        ctx->alloc->free(c->scale_in_dev);
        ctx->alloc->free(c->bias_dev);
        ctx->alloc->free(c->scale_out_dev);
        ctx->alloc->free(c->in_scales_dev);
        ctx->alloc->free(c->plane_map_dev);
    }
    delete c;
    return OTT_OK;
}

// ---- the fp32 layer (int8_scale_term == 0) ----
struct ott_conv_f32 {
    ott_conv_desc d{};
    bool depthwise = false;
    float* w_dev = nullptr;
    float* bias_dev = nullptr;
};

int ott_conv_f32_create(ott_ctx* ctx, const ott_conv_desc* d, const float* w_oihw, const float* bias, ott_conv_f32** out) {
    if (!ctx || !d || !w_oihw || !out) return OTT_ERR_INVALID;
    *out = nullptr;
    if (d->cin <= 0 || d->cout <= 0 || d->kh <= 0 || d->kw <= 0 || d->sh <= 0 || d->sw <= 0 || d->dh <= 0 || d->dw <= 0 || d->ph < 0 || d->pw < 0 ||
        d->groups <= 0)
        return ctx->fail(OTT_ERR_INVALID, "bad convolution geometry");
    if (d->int8_scale_term != 0) return ctx->fail(OTT_ERR_INVALID, "ott_conv_f32_create is the fp32 layer (int8_scale_term == 0)");
    if (d->act_type < 0 || d->act_type > 3) return ctx->fail(OTT_ERR_UNSUPPORTED, "activation %d is not supported (none/ReLU/LeakyReLU/ReLU6)", d->act_type);
    if (d->bias_term && !bias) return ctx->fail(OTT_ERR_INVALID, "bias_term set but bias is NULL");
    const bool depthwise = d->groups > 1 && d->groups == d->cin && d->groups == d->cout;
    if (!depthwise && d->groups != 1) return ctx->fail(OTT_ERR_UNSUPPORTED, "grouped (non-depthwise) fp32 convolution is not supported");
    cudaSetDevice(ctx->device);
    ott_conv_f32* c = new (std::nothrow) ott_conv_f32();
    if (!c) return OTT_ERR_ALLOC;
    c->d = *d;
    c->depthwise = depthwise;
    const int cp = conv_f32_channel_stride(d->cout), taps = d->kh * d->kw, cin_g = d->cin / d->groups;
    std::vector<float> wp((size_t)(depthwise ? 1 : cin_g) * taps * cp), bp((size_t)cp, 0.f);
    conv_f32_pack_weights(w_oihw, cin_g, d->cout, taps, depthwise, wp.data());
    for (int i = 0; i < d->cout && d->bias_term; ++i) bp[(size_t)i] = bias[i];
    int rc = upload(ctx, wp.data(), wp.size() * sizeof(float), (void**)&c->w_dev);
    if (rc == OTT_OK) rc = upload(ctx, bp.data(), bp.size() * sizeof(float), (void**)&c->bias_dev);
    if (rc == OTT_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = ctx->fail(OTT_ERR_CUDA, "upload failed");
    if (rc != OTT_OK) {
        ott_conv_f32_destroy(ctx, c);
        return rc;
    }
    *out = c;
    return OTT_OK;
}

int ott_conv_f32_destroy(ott_ctx* ctx, ott_conv_f32* c) {
    if (!c) return OTT_OK;
    if (ctx) {
        ctx->alloc->free(c->w_dev);
        ctx->alloc->free(c->bias_dev);
    }
    delete c;
    return OTT_OK;
}

int ott_conv_f32_forward(ott_ctx* ctx, const ott_conv_f32* c, const float* in_dev, int n, int h, int w, float* out_dev) {
    if (!ctx || !c || !in_dev || !out_dev || n < 0 || h <= 0 || w <= 0) return OTT_ERR_INVALID;
    const ott_conv_desc& d = c->d;
    ConvShape s{};
    s.n = n; s.h = h; s.w = w;
    s.oh = out_dim(h, d.kh, d.sh, d.ph, d.dh);
    s.ow = out_dim(w, d.kw, d.sw, d.pw, d.dw);
    if (s.oh <= 0 || s.ow <= 0) return ctx->fail(OTT_ERR_INVALID, "empty output");
    s.cin = d.cin; s.cout = d.cout; s.cin_pad = d.cin; s.cout_pad = d.cout;
    s.kh = d.kh; s.kw = d.kw; s.sh = d.sh; s.sw = d.sw; s.ph = d.ph; s.pw = d.pw; s.dh = d.dh; s.dw = d.dw;
    if (n == 0) return OTT_OK;
    cudaSetDevice(ctx->device);
    OTT_CUDA_CHECK(ctx, launch_conv_f32(ctx->stream, s, c->depthwise ? 1 : 0, in_dev, c->w_dev, c->bias_dev, d.act_type, d.act_param0, out_dev));
    ctx->launches += 1;
    return OTT_OK;
}

int ott_conv_int8_kernel_kind(const ott_conv* c) { return c ? c->kind : OTT_ERR_INVALID; }

const char* ott_conv_int8_kernel_name(const ott_ctx* ctx, const ott_conv* c, int in_dtype, int out_dtype, int h, int w) {
    if (!ctx || !c) return "";
    const ott_conv_desc& d = c->d;
    ConvShape s{};
    s.h = h; s.w = w;
    s.oh = out_dim(h, d.kh, d.sh, d.ph, d.dh);
    s.ow = out_dim(w, d.kw, d.sw, d.pw, d.dw);
    s.cin = d.cin; s.cout = d.cout; s.cin_pad = c->cin_pad; s.cout_pad = c->cout_pad;
    s.kh = d.kh; s.kw = d.kw; s.sh = d.sh; s.sw = d.sw; s.ph = d.ph; s.pw = d.pw; s.dh = d.dh; s.dw = d.dw;
    if (c->kind == OTT_KERNEL_DENSE_UMMA) return "dense_umma_kernel";
    if (c->kind == OTT_KERNEL_DENSE_DIRECT) return dense_stem_supports(s, in_dtype, out_dtype) ? "dense_stem_kernel" : "dense_direct_kernel";
    const bool gathered = !c->src_channels.empty();
    const bool tc_wins = c->dw_plan.ncb_total <= 2 || (long)s.h * s.w >= 2048;
    if (c->dw_umma && (ctx->dw_tensor_cores == 2 || (ctx->dw_tensor_cores == 1 && tc_wins)) && !gathered && in_dtype == OTT_S8_NHWC && out_dtype != OTT_S32_NHWC)
        return "dw_umma_kernel";
    if (c->w_tiled_dev && depthwise_tiled_supports(s, out_dtype)) return "depthwise_tiled_kernel";
    return "depthwise_kernel";
}

int ott_conv_int8_out_shape(const ott_conv* c, int h, int w, int* oh, int* ow) {
    if (!c || !oh || !ow) return OTT_ERR_INVALID;
    *oh = out_dim(h, c->d.kh, c->d.sh, c->d.ph, c->d.dh);
    *ow = out_dim(w, c->d.kw, c->d.sw, c->d.pw, c->d.dw);
    return OTT_OK;
}

namespace {
int conv_forward_impl(ott_ctx* ctx, const ott_conv* c, const void* in_dev, const PlaneGather* gather, int in_dtype, int n, int h, int w,
                      void* out_dev, int out_dtype, uint32_t* status_word_dev, const int8_t* const* sources = nullptr, int n_sources = 0,
                      const UmmaMixedOut* mixed = nullptr);
}

int ott_conv_int8_forward(ott_ctx* ctx, const ott_conv* c, const void* in_dev, int in_dtype, int n, int h, int w, void* out_dev,
                          int out_dtype, uint32_t* status_word_dev) {
    if (!in_dev) return OTT_ERR_INVALID;
    return conv_forward_impl(ctx, c, in_dev, nullptr, in_dtype, n, h, w, out_dev, out_dtype, status_word_dev);
}

int ott_conv_int8_forward_ex(ott_ctx* ctx, const ott_conv* c, const void* in_dev, int in_dtype, int in_channels_total, int n, int h, int w,
                             void* out_dev, int out_dtype, uint32_t* status_word_dev) {
    if (!ctx || !c || !in_dev) return OTT_ERR_INVALID;
    if (in_channels_total < c->d.cin || (in_dtype != OTT_F32_NCHW && in_channels_total != c->d.cin))
        return ctx->fail(OTT_ERR_INVALID, "in_channels_total must be >= cin (and == cin for int8 NHWC input)");
    if (in_dtype != OTT_F32_NCHW || in_channels_total == c->d.cin)
        return conv_forward_impl(ctx, c, in_dev, nullptr, in_dtype, n, h, w, out_dev, out_dtype, status_word_dev);
    if (c->d.cin > kGatherMaxChannels) return ctx->fail(OTT_ERR_UNSUPPORTED, "channel-range input with more than %d channels", kGatherMaxChannels);
    PlaneGather g;
    gather_identity(&g, static_cast<const float*>(in_dev), c->d.cin, in_channels_total, (long)h * w);
    return conv_forward_impl(ctx, c, in_dev, &g, in_dtype, n, h, w, out_dev, out_dtype, status_word_dev);
}

int ott_conv_int8_forward_gather(ott_ctx* ctx, const ott_conv* c, const float* const* buffers, const int64_t* image_strides, int n_buffers,
                                 const uint32_t* plane_refs, int n, int h, int w, void* out_dev, int out_dtype, uint32_t* status_word_dev) {
    if (!ctx || !c || !buffers || !image_strides || !plane_refs) return OTT_ERR_INVALID;
    if (n_buffers < 1 || n_buffers > kGatherMaxBufs || c->d.cin > kGatherMaxChannels)
        return ctx->fail(OTT_ERR_UNSUPPORTED, "gathered input: at most %d buffers and %d channels", kGatherMaxBufs, kGatherMaxChannels);
    PlaneGather g;
    for (int i = 0; i < n_buffers; ++i) {
        if (!buffers[i]) return ctx->fail(OTT_ERR_INVALID, "null buffer in the plane table");
        g.base[i] = buffers[i];
        g.img_stride[i] = image_strides[i];
    }
    for (int i = 0; i < c->d.cin; ++i) {
        if ((int)(plane_refs[i] >> 24) >= n_buffers) return ctx->fail(OTT_ERR_INVALID, "plane reference %d names buffer %u of %d", i, plane_refs[i] >> 24, n_buffers);
        g.ref[i] = plane_refs[i];
    }
    return conv_forward_impl(ctx, c, buffers[0], &g, OTT_F32_NCHW, n, h, w, out_dev, out_dtype, status_word_dev);
}

int ott_conv_int8_set_f32_plane_map(ott_ctx* ctx, ott_conv* c, const int* plane_of_channel, int planes_total) {
    if (!ctx || !c || !plane_of_channel || planes_total <= 0 || planes_total > 32767) return OTT_ERR_INVALID;
    std::vector<int16_t> m((size_t)c->cout_pad, 0);
    for (int i = 0; i < c->d.cout; ++i) {
        if (plane_of_channel[i] >= planes_total) return ctx->fail(OTT_ERR_INVALID, "plane %d of %d", plane_of_channel[i], planes_total);
        m[(size_t)i] = (int16_t)(plane_of_channel[i] < 0 ? 0 : plane_of_channel[i]);
    }
    ctx->alloc->free(c->plane_map_dev);
    c->plane_map_dev = nullptr;
    int rc = upload(ctx, m.data(), m.size() * sizeof(int16_t), (void**)&c->plane_map_dev);
    if (rc == OTT_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = ctx->fail(OTT_ERR_CUDA, "upload failed");
    if (rc == OTT_OK) c->f32_planes = planes_total;
    return rc;
}

int ott_conv_int8_forward_io(ott_ctx* ctx, const ott_conv* c, const ott_conv_io* io, int n, int h, int w, uint32_t* status_word_dev) {
    if (!ctx || !c || !io) return OTT_ERR_INVALID;
    UmmaMixedOut mixed{};
    void* out_dev = io->out_dev;
    if (io->n_chunks > 0) {
        if (!io->chunk_dst || !io->chunk_pitch || io->out_dtype != OTT_S8_NHWC || io->n_chunks != c->cout_pad / 16 || io->n_chunks > 64 ||
            c->kind != OTT_KERNEL_DENSE_UMMA)
            return ctx->fail(OTT_ERR_INVALID, "scattered output: int8 launch of the tensor-core kernel, one destination per 16 output channels (at most 64)");
        mixed.n_chunks = io->n_chunks;
        for (int i = 0; i < io->n_chunks; ++i) {
            mixed.dst[i] = io->chunk_dst[i];
            mixed.pitch[i] = io->chunk_pitch[i];
            if (mixed.dst[i] && ((reinterpret_cast<uintptr_t>(mixed.dst[i]) | mixed.pitch[i]) & 15u))
                return ctx->fail(OTT_ERR_INVALID, "scattered output: destinations and pitches must be multiples of 16 bytes");
            if (mixed.dst[i] && !out_dev) out_dev = mixed.dst[i];
        }
        for (int i = 0; i + 1 < io->n_chunks; i += 2)
            if (mixed.dst[i] && mixed.dst[i + 1] == mixed.dst[i] + 16 && mixed.pitch[i] == mixed.pitch[i + 1] &&
                ((reinterpret_cast<uintptr_t>(mixed.dst[i]) | mixed.pitch[i]) & 31u) == 0)
                mixed.pair_ok |= 1ull << (i >> 1);
        if (!out_dev) return OTT_OK;  // nobody reads any channel in int8
    }
    if (c->plane_map_dev && io->out_f32_dev) {
        mixed.plane_of_col = c->plane_map_dev;
        mixed.f32_planes = c->f32_planes;
    }
    if (io->out_f32_dev) {
        if (!io->f32_channel_mask) return ctx->fail(OTT_ERR_INVALID, "out_f32_dev without f32_channel_mask");
        if (c->d.cout > 1024) return ctx->fail(OTT_ERR_UNSUPPORTED, "an fp32 side output is limited to 1024 output channels");
        mixed.out_f32 = io->out_f32_dev;
        for (int i = 0; i < (c->d.cout + 31) / 32 && i < 32; ++i) mixed.mask[i] = io->f32_channel_mask[i];
        if (c->d.cout % 32) mixed.mask[c->d.cout / 32] &= (1u << (c->d.cout % 32)) - 1u;  // never a channel past cout
    }
    return conv_forward_impl(ctx, c, io->in_dev, nullptr, io->in_dtype, n, h, w, out_dev, io->out_dtype, status_word_dev, io->sources,
                             io->sources ? io->n_sources : 0, (io->out_f32_dev || mixed.n_chunks > 0) ? &mixed : nullptr);
}

namespace {
int forward_maxpool_impl(ott_ctx* ctx, const ott_conv* c, const float* in_dev, int n, int h, int w, int pad_with_zero, void* out_dev, int out_dtype);
}

int ott_conv_int8_forward_maxpool(ott_ctx* ctx, const ott_conv* c, const float* in_dev, int n, int h, int w, int pad_with_zero, float* out_dev) {
    return forward_maxpool_impl(ctx, c, in_dev, n, h, w, pad_with_zero, out_dev, OTT_F32_NCHW);
}

int ott_conv_int8_forward_maxpool_s8(ott_ctx* ctx, const ott_conv* c, const float* in_dev, int n, int h, int w, int pad_with_zero, int8_t* out_dev) {
    return forward_maxpool_impl(ctx, c, in_dev, n, h, w, pad_with_zero, out_dev, OTT_S8_NHWC);
}

namespace {
int forward_maxpool_impl(ott_ctx* ctx, const ott_conv* c, const float* in_dev, int n, int h, int w, int pad_with_zero, void* out_dev, int out_dtype) {
    if (!ctx || !c || !in_dev || !out_dev || n < 0 || h <= 0 || w <= 0) return OTT_ERR_INVALID;
    const ott_conv_desc& d = c->d;
    ConvShape s{};
    s.n = n; s.h = h; s.w = w;
    s.oh = out_dim(h, d.kh, d.sh, d.ph, d.dh);
    s.ow = out_dim(w, d.kw, d.sw, d.pw, d.dw);
    s.cin = d.cin; s.cout = d.cout; s.cin_pad = c->cin_pad; s.cout_pad = c->cout_pad;
    s.kh = d.kh; s.kw = d.kw; s.sh = d.sh; s.sw = d.sw; s.ph = d.ph; s.pw = d.pw; s.dh = d.dh; s.dw = d.dw;
    if ((d.int8_scale_term > 100) != (out_dtype == OTT_S8_NHWC) || c->kind != OTT_KERNEL_DENSE_DIRECT ||
        !dense_stem_supports(s, OTT_F32_NCHW, OTT_F32_NCHW) || s.oh < 1 || s.ow < 1)
        return ctx->fail(OTT_ERR_UNSUPPORTED, "the fused max-pool exists for the 3-channel 3x3 first layer (fp32 output: int8_scale_term < 100, int8: > 100)");
    if (n == 0) return OTT_OK;
    cudaSetDevice(ctx->device);
    EpilogueParams ep{};
    ep.scale_in = c->scale_in_dev; ep.bias = c->bias_dev; ep.scale_out = c->scale_out_dev;
    ep.has_bias = d.bias_term ? 1 : 0;
    ep.act_type = d.act_type; ep.act_param0 = d.act_param0; ep.rounding = d.rounding;
    OTT_CUDA_CHECK(ctx, launch_dense_stem_pool(ctx->stream, s, in_dev, c->w_host.data(), c->scale_in_host.data(), c->bias_host.data(),
                                                c->scale_out_host.data(), c->in_scale0, ep, out_dev, out_dtype, pad_with_zero, ctx->status_dev));
    ctx->launches += 1;
    return OTT_OK;
}
}  // namespace

int ott_gather_channels_f32(ott_ctx* ctx, const float* const* buffers, const int64_t* image_strides, int n_buffers, const uint32_t* plane_refs,
                            int channels, int n, int hw, float* dst_dev) {
    if (!ctx || !buffers || !image_strides || !plane_refs || !dst_dev || channels < 0 || n < 0 || hw < 0) return OTT_ERR_INVALID;
    if (n_buffers < 1 || n_buffers > kGatherMaxBufs || channels > kGatherMaxChannels)
        return ctx->fail(OTT_ERR_UNSUPPORTED, "gather: at most %d buffers and %d channels", kGatherMaxBufs, kGatherMaxChannels);
    PlaneGather g;
    for (int i = 0; i < n_buffers; ++i) { g.base[i] = buffers[i]; g.img_stride[i] = image_strides[i]; }
    for (int i = 0; i < channels; ++i) {
        if ((int)(plane_refs[i] >> 24) >= n_buffers) return ctx->fail(OTT_ERR_INVALID, "plane reference names a buffer that was not given");
        g.ref[i] = plane_refs[i];
    }
    cudaSetDevice(ctx->device);
    OTT_CUDA_CHECK(ctx, launch_gather_planes(ctx->stream, g, dst_dev, n, channels, hw));
    ctx->launches += 1;
    return OTT_OK;
}

int ott_add_gather_f32(ott_ctx* ctx, const float* const* a_buffers, const int64_t* a_image_strides, int a_n_buffers, const uint32_t* a_plane_refs,
                       const float* const* b_buffers, const int64_t* b_image_strides, int b_n_buffers, const uint32_t* b_plane_refs, int channels,
                       int n, int hw, float* dst_dev) {
    if (!ctx || !a_buffers || !a_image_strides || !a_plane_refs || !b_buffers || !b_image_strides || !b_plane_refs || !dst_dev || channels < 0 ||
        n < 0 || hw < 0)
        return OTT_ERR_INVALID;
    if (a_n_buffers < 1 || a_n_buffers > kGatherMaxBufs || b_n_buffers < 1 || b_n_buffers > kGatherMaxBufs || channels > kGatherMaxChannels)
        return ctx->fail(OTT_ERR_UNSUPPORTED, "gather: at most %d buffers and %d channels", kGatherMaxBufs, kGatherMaxChannels);
    PlaneGather ga, gb;
    for (int i = 0; i < a_n_buffers; ++i) { ga.base[i] = a_buffers[i]; ga.img_stride[i] = a_image_strides[i]; }
    for (int i = 0; i < b_n_buffers; ++i) { gb.base[i] = b_buffers[i]; gb.img_stride[i] = b_image_strides[i]; }
    for (int i = 0; i < channels; ++i) {
        if ((int)(a_plane_refs[i] >> 24) >= a_n_buffers || (int)(b_plane_refs[i] >> 24) >= b_n_buffers)
            return ctx->fail(OTT_ERR_INVALID, "plane reference names a buffer that was not given");
        ga.ref[i] = a_plane_refs[i];
        gb.ref[i] = b_plane_refs[i];
    }
    cudaSetDevice(ctx->device);
    OTT_CUDA_CHECK(ctx, launch_add_planes(ctx->stream, ga, gb, dst_dev, n, channels, hw));
    ctx->launches += 1;
    return OTT_OK;
}

}  // extern "C"

namespace {
int conv_forward_impl(ott_ctx* ctx, const ott_conv* c, const void* in_dev, const PlaneGather* gather, int in_dtype, int n, int h, int w,
                      void* out_dev, int out_dtype, uint32_t* status_word_dev, const int8_t* const* sources, int n_sources,
                      const UmmaMixedOut* mixed) {
    if (!ctx || !c || !out_dev || n < 0 || h <= 0 || w <= 0) return OTT_ERR_INVALID;
    const ott_conv_desc& d = c->d;
    const bool gathered = !c->src_channels.empty();
    if (gathered != (sources != nullptr) || (gathered && n_sources != (int)c->src_channels.size()))
        return ctx->fail(OTT_ERR_INVALID, "a layer created with gathered input runs on exactly its %d int8 sources, any other layer on one input",
                         (int)c->src_channels.size());
    if (!gathered && !in_dev) return OTT_ERR_INVALID;
    if (mixed && (c->kind != OTT_KERNEL_DENSE_UMMA || out_dtype != OTT_S8_NHWC || d.cout > 1024))
        return ctx->fail(OTT_ERR_UNSUPPORTED, "an fp32 side output needs an int8 launch of the tensor-core kernel with at most 1024 output channels");
    if (gathered) in_dtype = OTT_S8_NHWC;
    if (in_dtype != OTT_F32_NCHW && in_dtype != OTT_S8_NHWC) return ctx->fail(OTT_ERR_INVALID, "input must be fp32 NCHW or int8 NHWC");
    const bool requant = d.int8_scale_term > 100;
    if (out_dtype == OTT_S8_NHWC && !requant) return ctx->fail(OTT_ERR_INVALID, "int8 output needs int8_scale_term > 100");
    if (out_dtype == OTT_F32_NCHW && requant) return ctx->fail(OTT_ERR_INVALID, "fp32 output needs int8_scale_term < 100");
    if (out_dtype != OTT_S8_NHWC && out_dtype != OTT_F32_NCHW && out_dtype != OTT_S32_NHWC) return ctx->fail(OTT_ERR_INVALID, "bad output dtype");
    cudaSetDevice(ctx->device);

    ConvShape s{};
    s.n = n; s.h = h; s.w = w;
    s.oh = out_dim(h, d.kh, d.sh, d.ph, d.dh);
    s.ow = out_dim(w, d.kw, d.sw, d.pw, d.dw);
    if (s.oh <= 0 || s.ow <= 0) return ctx->fail(OTT_ERR_INVALID, "empty output");
    s.cin = d.cin; s.cout = d.cout; s.cin_pad = c->cin_pad; s.cout_pad = c->cout_pad;
    s.kh = d.kh; s.kw = d.kw; s.sh = d.sh; s.sw = d.sw; s.ph = d.ph; s.pw = d.pw; s.dh = d.dh; s.dw = d.dw;
    if (n == 0) return OTT_OK;

    EpilogueParams ep{};
    ep.scale_in = c->scale_in_dev; ep.bias = c->bias_dev; ep.scale_out = c->scale_out_dev;
    ep.has_bias = d.bias_term ? 1 : 0;
    ep.act_type = d.act_type; ep.act_param0 = d.act_param0; ep.rounding = d.rounding;

    uint32_t* status = status_word_dev ? status_word_dev : ctx->status_dev;
    PlaneGather groups8;  // depthwise over gathered int8 input: where each 16-channel group lies
    if (gathered && c->kind == OTT_KERNEL_DEPTHWISE && c->gather_group == 32) {
        for (int i = 0; i < n_sources; ++i)
            if (!sources[i]) return ctx->fail(OTT_ERR_INVALID, "null source tensor");
        in_dev = sources[0];
    } else if (gathered && c->kind == OTT_KERNEL_DEPTHWISE) {
        if (!c->w_tiled_dev || !depthwise_tiled_supports(s, out_dtype)) return ctx->fail(OTT_ERR_UNSUPPORTED, "gathered depthwise layer: tiled kernel only");
        for (int i = 0; i < n_sources; ++i) {
            if (!sources[i]) return ctx->fail(OTT_ERR_INVALID, "null source tensor");
            groups8.base[i] = reinterpret_cast<const float*>(sources[i]);
            groups8.img_stride[i] = nhwc_channels(c->src_channels[(size_t)i]);
        }
        for (size_t g = 0; g < c->block_x.size(); ++g) groups8.ref[g] = ((uint32_t)c->block_src[g] << 24) | c->block_x[g];
        gather = &groups8;
        in_dev = sources[0];
    }
    // int8 NHWC input: the multiply-adds can go to the tensor cores as the data lies, no byte transposes. Every tap costs one
    // 128-row MMA per 32 channels and 8 x 16 pixel tile, so this wins for narrow layers (at most 64 channels) and for wide
    // layers on input maps large enough for the tiles to fit well (256 channels, 56 x 56, 64 images: stride 1 41.8 us against
    // 49.1, stride 2 16.3 against 22.2; 116 channels on 20 x 20 lose, 18.5 against 13.6 and 10.5 against 9.2); elsewhere the CUDA cores do.
    // A layer with gathered input that was laid out in 32-channel groups always runs here (its groups are the MMA's K blocks).
    const bool dw_tc_wins = c->dw_plan.ncb_total <= 2 || (long)s.h * s.w >= 2048;
    const bool dw_gathered_tc = gathered && c->kind == OTT_KERNEL_DEPTHWISE && c->gather_group == 32;
    if (c->kind == OTT_KERNEL_DEPTHWISE && c->dw_umma && in_dtype == OTT_S8_NHWC && out_dtype != OTT_S32_NHWC &&
        (dw_gathered_tc || (!gathered && (ctx->dw_tensor_cores == 2 || (ctx->dw_tensor_cores == 1 && dw_tc_wins))))) {
        UmmaSources us{};
        if (gathered) {
            us.n_src = n_sources;
            for (int i = 0; i < n_sources; ++i) {
                us.src[i] = sources[i];
                us.src_cpad[i] = nhwc_channels(c->src_channels[(size_t)i]);
            }
            for (size_t b = 0; b < c->block_x.size(); ++b) { us.block_x[b] = c->block_x[b]; us.block_src[b] = c->block_src[b]; }
        }
        const char* err = launch_dw_umma(ctx->stream, ctx->sm_count, c->dw_plan, c->weight_map_dw, s, static_cast<const int8_t*>(in_dev), gathered ? &us : nullptr,
                                         ep, out_dev, out_dtype, status, ctx->wait_limit_ns);
        if (err) return ctx->fail(OTT_ERR_CUDA, "%s: %s", err, cudaGetErrorString(cudaGetLastError()));
        ctx->launches += 1;
        return OTT_OK;
    }
    if (c->kind == OTT_KERNEL_DEPTHWISE && c->w_tiled_dev && depthwise_tiled_supports(s, out_dtype) &&
        (in_dtype != OTT_F32_NCHW || d.cin <= kGatherMaxChannels)) {
        // one pass over HBM: quantize (when the input is fp32), depthwise and epilogue in the same kernel
        OTT_CUDA_CHECK(ctx, launch_depthwise_tiled(ctx->stream, s, in_dev, gather, in_dtype, c->w_tiled_dev, c->in_scales_dev, c->n_in_scales, ep,
                                                    out_dev, out_dtype));
        ctx->launches += 1;
        return OTT_OK;
    }
    if (c->kind == OTT_KERNEL_DENSE_DIRECT && !gather && dense_stem_supports(s, in_dtype, out_dtype)) {
        OTT_CUDA_CHECK(ctx, launch_dense_stem(ctx->stream, s, static_cast<const float*>(in_dev), c->w_host.data(), c->scale_in_host.data(),
                                               c->bias_host.data(), c->scale_out_host.data(), c->in_scale0, ep, out_dev, out_dtype));
        ctx->launches += 1;
        return OTT_OK;
    }
    DeviceBlock xq;  // scratch: the quantized activations when the input arrives as fp32
    const int8_t* x = static_cast<const int8_t*>(in_dev);
    if (in_dtype == OTT_F32_NCHW) {
        if (xq.alloc(ctx, (size_t)n * h * w * c->cin_pad) != cudaSuccess) {
            (void)cudaGetLastError();
            return ctx->fail(OTT_ERR_ALLOC, "scratch allocation for quantized activations failed");
        }
        if (gather) {
            OTT_CUDA_CHECK(ctx, launch_quantize_nchw_to_nhwc(ctx->stream, *gather, (int8_t*)xq.p, c->in_scales_dev, c->n_in_scales, n, d.cin, h, w,
                                                              d.rounding));
        } else {
            OTT_CUDA_CHECK(ctx, launch_quantize_dense(ctx->stream, static_cast<const float*>(in_dev), d.cin, (int8_t*)xq.p, c->in_scales_dev,
                                                       c->n_in_scales, n, d.cin, h, w, d.rounding));
        }
        ctx->launches += gather ? 1u : (uint64_t)((c->cin_pad + kGatherMaxChannels - 1) / kGatherMaxChannels);
        x = (const int8_t*)xq.p;
    }
    switch (c->kind) {
        case OTT_KERNEL_DEPTHWISE:
            OTT_CUDA_CHECK(ctx, launch_depthwise(ctx->stream, s, x, c->w_dev, ep, out_dev, out_dtype));
            break;
        case OTT_KERNEL_DENSE_DIRECT:
            OTT_CUDA_CHECK(ctx, launch_dense_direct(ctx->stream, s, x, c->w_dev, ep, out_dev, out_dtype));
            break;
        case OTT_KERNEL_DENSE_UMMA: {
            UmmaSources us{};
            if (gathered && c->plan.gather != n_sources) return ctx->fail(OTT_ERR_INVALID, "corrupt gathered layer");
            if (gathered) {
                us.n_src = n_sources;
                for (int i = 0; i < n_sources; ++i) {
                    if (!sources[i]) return ctx->fail(OTT_ERR_INVALID, "null source tensor");
                    us.src[i] = sources[i];
                    us.src_cpad[i] = nhwc_channels(c->src_channels[(size_t)i]);
                }
                for (size_t kb = 0; kb < c->block_x.size(); ++kb) {
                    us.block_x[kb] = c->block_x[kb];
                    us.block_src[kb] = c->block_src[kb];
                }
            }
            const char* err = launch_dense_umma(ctx->stream, ctx->sm_count, c->plan, c->weight_map, s, x, ep, out_dev, out_dtype, status,
                                                gathered ? &us : nullptr, mixed, ctx->wait_limit_ns);
            if (err) return ctx->fail(OTT_ERR_CUDA, "%s: %s", err, cudaGetErrorString(cudaGetLastError()));
            break;
        }
        default: return ctx->fail(OTT_ERR_INVALID, "corrupt layer object");
    }
    ctx->launches += 1;
    return OTT_OK;
}
}  // namespace

extern "C" {

int ott_conv_int8_forward_host(ott_ctx* ctx, const ott_conv* c, const void* in_host, int in_dtype, int n, int h, int w,
                               void* out_host, int out_dtype) {
    if (!ctx || !c || !in_host || !out_host) return OTT_ERR_INVALID;
    cudaSetDevice(ctx->device);
    int oh = 0, ow = 0;
    ott_conv_int8_out_shape(c, h, w, &oh, &ow);
    const size_t in_bytes = dtype_bytes(in_dtype, n, c->d.cin, h, w), out_bytes = dtype_bytes(out_dtype, n, c->d.cout, oh, ow);
    if (in_bytes == 0 || out_bytes == 0) return ctx->fail(OTT_ERR_INVALID, "bad dtype or empty tensor");
    DeviceBlock din, dout;
    if (din.alloc(ctx, in_bytes) != cudaSuccess || dout.alloc(ctx, out_bytes) != cudaSuccess) {
        (void)cudaGetLastError();
        return ctx->fail(OTT_ERR_ALLOC, "device allocation failed");
    }
    OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(din.p, in_host, in_bytes, cudaMemcpyHostToDevice, ctx->stream));
    int rc = ott_conv_int8_forward(ctx, c, din.p, in_dtype, n, h, w, dout.p, out_dtype, nullptr);
    if (rc != OTT_OK) return rc;
    OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(out_host, dout.p, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return check_status_word(ctx);
}

}  // extern "C"
