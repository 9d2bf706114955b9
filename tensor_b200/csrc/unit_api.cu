// C-ABI of the fused unit kernel (unit_umma.cu): ott_unit_int8_create builds, from three existing layer objects, the state of
// the chain 1x1 convolution -> depthwise 3x3 -> 1x1 convolution; ott_unit_int8_forward_io runs it as one launch.
#include <cstring>
#include <new>
#include <vector>

#include "conv_object.h"
#include "ctx.h"
#include "unit_umma.h"

using namespace ottk;

struct ott_unit {
    UnitPlan plan{};
    UnitWeights maps{};
    int cin1 = 0, cm = 0, cout2 = 0;
    bool requant2 = false;
    int act = 0;
    float act_p1 = 0.f, act_p2 = 0.f;
    // the first layer's input: K block kb = 32 channels from block_x[kb] of source block_src[kb]
    std::vector<uint16_t> block_x;
    std::vector<uint8_t> block_src;
    std::vector<int> src_channels;
    bool gathered = false;
    // device state, owned
    int8_t *w1 = nullptr, *wdw = nullptr, *w2 = nullptr;
    float* params = nullptr;  // si1 bi1 so1 [cm] | sid bid sod [cm]
    // the second layer's epilogue arrays stay with that layer (the caller keeps it alive)
    const ott_conv* pw2 = nullptr;
};

namespace {
int upload(ott_ctx* ctx, const void* host, size_t bytes, void** dev) {
    cudaError_t e = ctx->alloc->allocate(bytes, dev);
    if (e != cudaSuccess) return ctx->fail(OTT_ERR_ALLOC, "device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(*dev, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return OTT_OK;
}
bool is_pointwise(const ott_conv_desc& d) {
    return d.groups == 1 && d.kh == 1 && d.kw == 1 && d.sh == 1 && d.sw == 1 && d.ph == 0 && d.pw == 0;
}
}  // namespace

extern "C" {

int ott_unit_int8_destroy(ott_ctx* ctx, ott_unit* u) {
    if (!u) return OTT_OK;
    if (ctx) {
        ctx->alloc->free(u->w1);
        ctx->alloc->free(u->wdw);
        ctx->alloc->free(u->w2);
        ctx->alloc->free(u->params);
    }
    delete u;
    return OTT_OK;
}

int ott_unit_int8_create(ott_ctx* ctx, const ott_conv* pw1, const ott_conv* dw, const ott_conv* pw2, ott_unit** out) {
    if (!ctx || !pw1 || !dw || !pw2 || !out) return OTT_ERR_INVALID;
    *out = nullptr;
    const ott_conv_desc &d1 = pw1->d, &dd = dw->d, &d2 = pw2->d;
    const char* why = nullptr;
    if (!is_pointwise(d1) || !is_pointwise(d2)) why = "the first and the last layer must be 1x1, stride 1, unpadded, ungrouped";
    else if (!dw->depthwise || dd.kh != 3 || dd.kw != 3 || dd.sh != 1 || dd.sw != 1 || dd.ph != 1 || dd.pw != 1 || dd.dh != 1 || dd.dw != 1)
        why = "the middle layer must be a depthwise 3x3, stride 1, pad 1";
    else if (d1.cout != dd.cin || dd.cout != d2.cin) why = "channel counts of the three layers do not chain";
    else if (d1.int8_scale_term <= 100 || dd.int8_scale_term <= 100) why = "the first two layers must requantize (int8_scale_term > 100)";
    else if (!d1.bias_term || !dd.bias_term || !d2.bias_term) why = "all three layers need a bias term";
    else if (dd.act_type != 0 || d1.act_type != d2.act_type) why = "the 1x1 layers must share one activation and the depthwise layer have none";
    else if (d1.rounding != OTT_ROUND_ADD_HALF_TRUNC || dd.rounding != OTT_ROUND_ADD_HALF_TRUNC || d2.rounding != OTT_ROUND_ADD_HALF_TRUNC)
        why = "only the add-half-truncate rounding rule";
    else if (pw1->n_in_scales != 1 || !pw2->src_channels.empty() || pw2->plane_map_dev) why = "unsupported input / output form";
    for (int i = 1; !why && i < dw->n_in_scales; ++i) (void)i;  // (per-channel input scales of the depthwise layer play no part: its input is int8)
    if (why) return ctx->fail(OTT_ERR_UNSUPPORTED, "fused unit: %s", why);
    cudaSetDevice(ctx->device);
    ott_unit* u = new (std::nothrow) ott_unit();
    if (!u) return OTT_ERR_ALLOC;
    u->cin1 = d1.cin; u->cm = d1.cout; u->cout2 = d2.cout;
    u->requant2 = d2.int8_scale_term > 100;
    u->act = d1.act_type; u->act_p1 = d1.act_param0; u->act_p2 = d2.act_param0;
    u->pw2 = pw2;
    std::vector<int8_t> wk;  // first layer's weights against its K order
    if (!pw1->src_channels.empty()) {
        u->gathered = true;
        u->block_x = pw1->block_x;
        u->block_src = pw1->block_src;
        u->src_channels = pw1->src_channels;
        wk = pw1->w_korder;
    } else {
        const int nb = (pw1->cin_pad + kUnitBlock - 1) / kUnitBlock;
        for (int b = 0; b < nb; ++b) { u->block_x.push_back((uint16_t)(b * kUnitBlock)); u->block_src.push_back(0); }
        u->src_channels.assign(1, d1.cin);
        wk.assign((size_t)d1.cout * nb * kUnitBlock, 0);
        for (int o = 0; o < d1.cout; ++o)
            for (int c = 0; c < d1.cin; ++c) wk[(size_t)o * nb * kUnitBlock + c] = pw1->w_host[(size_t)o * d1.cin + c];
    }
    int smem_optin = 0;
    cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, ctx->device);
    if ((int)u->block_x.size() > kUmmaMaxGatherBlocks || wk.size() != (size_t)d1.cout * u->block_x.size() * kUnitBlock ||
        !unit_plan((int)u->block_x.size(), d1.cout, d2.cout, smem_optin, &u->plan)) {
        delete u;
        return ctx->fail(OTT_ERR_UNSUPPORTED, "fused unit: %d K blocks x %d -> %d channels do not fit one SM's shared / tensor memory", (int)pw1->block_x.size(),
                         d1.cout, d2.cout);
    }
    const UnitPlan& p = u->plan;
    std::vector<int8_t> w1(unit_w1_bytes(p)), wd(unit_wdw_bytes(p)), w2(unit_w2_bytes(p));
    unit_pack_w1(p, wk.data(), d1.cout, w1.data());
    unit_pack_wdw(p, dw->w_host.data(), dd.cout, wd.data());
    unit_pack_w2(p, pw2->w_host.data(), d2.cout, d2.cin, w2.data());
    std::vector<float> prm((size_t)6 * p.cm, 0.f);
    for (int i = 0; i < d1.cout; ++i) {
        prm[(size_t)i] = pw1->scale_in_host[(size_t)i];
        prm[(size_t)p.cm + i] = pw1->bias_host[(size_t)i];
        prm[(size_t)2 * p.cm + i] = pw1->scale_out_host[(size_t)i];
        prm[(size_t)3 * p.cm + i] = dw->scale_in_host[(size_t)i];
        prm[(size_t)4 * p.cm + i] = dw->bias_host[(size_t)i];
        prm[(size_t)5 * p.cm + i] = dw->scale_out_host[(size_t)i];
    }
    int rc = upload(ctx, w1.data(), w1.size(), (void**)&u->w1);
    if (rc == OTT_OK) rc = upload(ctx, wd.data(), wd.size(), (void**)&u->wdw);
    if (rc == OTT_OK) rc = upload(ctx, w2.data(), w2.size(), (void**)&u->w2);
    if (rc == OTT_OK) rc = upload(ctx, prm.data(), prm.size() * sizeof(float), (void**)&u->params);
    if (rc == OTT_OK) {
        const char* err = unit_encode_weight_maps(p, u->w1, u->wdw, u->w2, &u->maps);
        if (err) rc = ctx->fail(OTT_ERR_CUDA, "%s", err);
    }
    if (rc == OTT_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = ctx->fail(OTT_ERR_CUDA, "upload failed");
    if (rc != OTT_OK) {
        ott_unit_int8_destroy(ctx, u);
        return rc;
    }
    *out = u;
    return OTT_OK;
}

int ott_unit_int8_forward_io(ott_ctx* ctx, const ott_unit* u, const ott_conv_io* io, int n, int h, int w, uint32_t* status_word_dev) {
    if (!ctx || !u || !io || n < 0 || h <= 0 || w <= 0) return OTT_ERR_INVALID;
    if (io->n_chunks > 0) return ctx->fail(OTT_ERR_UNSUPPORTED, "fused unit: no scattered output");
    if (!io->out_dev) return OTT_ERR_INVALID;
    if (io->out_dtype == OTT_S8_NHWC ? !u->requant2 : (io->out_dtype != OTT_F32_NCHW || u->requant2))
        return ctx->fail(OTT_ERR_INVALID, "fused unit: output type does not match the last layer's int8_scale_term");
    UmmaSources us{};
    if (u->gathered) {
        if (!io->sources || io->n_sources != (int)u->src_channels.size())
            return ctx->fail(OTT_ERR_INVALID, "fused unit: the first layer reads exactly its %d int8 sources", (int)u->src_channels.size());
        for (int i = 0; i < io->n_sources; ++i) {
            if (!io->sources[i]) return ctx->fail(OTT_ERR_INVALID, "null source tensor");
            us.src[i] = io->sources[i];
        }
    } else {
        if (!io->in_dev || io->in_dtype != OTT_S8_NHWC) return ctx->fail(OTT_ERR_INVALID, "fused unit: int8 NHWC input");
        us.src[0] = static_cast<const int8_t*>(io->in_dev);
    }
    us.n_src = (int)u->src_channels.size();
    for (int i = 0; i < us.n_src; ++i) us.src_cpad[i] = nhwc_channels(u->src_channels[(size_t)i]);
    for (size_t kb = 0; kb < u->block_x.size(); ++kb) { us.block_x[kb] = u->block_x[kb]; us.block_src[kb] = u->block_src[kb]; }
    UmmaMixedOut mixed{};
    if (io->out_f32_dev) {
        if (!io->f32_channel_mask || io->out_dtype != OTT_S8_NHWC) return ctx->fail(OTT_ERR_INVALID, "out_f32_dev needs f32_channel_mask and an int8 launch");
        if (u->cout2 > 1024) return ctx->fail(OTT_ERR_UNSUPPORTED, "an fp32 side output is limited to 1024 output channels");
        mixed.out_f32 = io->out_f32_dev;
        for (int i = 0; i < (u->cout2 + 31) / 32 && i < 32; ++i) mixed.mask[i] = io->f32_channel_mask[i];
        if (u->cout2 % 32) mixed.mask[u->cout2 / 32] &= (1u << (u->cout2 % 32)) - 1u;
    }
    if (n == 0) return OTT_OK;
    cudaSetDevice(ctx->device);
    UnitEpilogues ep{};
    const int cm = u->plan.cm;
    ep.e1.scale_in = u->params; ep.e1.bias = u->params + cm; ep.e1.scale_out = u->params + 2 * cm;
    ep.e1.has_bias = 1; ep.e1.act_type = u->act; ep.e1.act_param0 = u->act_p1;
    ep.edw.scale_in = u->params + 3 * cm; ep.edw.bias = u->params + 4 * cm; ep.edw.scale_out = u->params + 5 * cm;
    ep.edw.has_bias = 1;
    ep.e2.scale_in = u->pw2->scale_in_dev; ep.e2.bias = u->pw2->bias_dev; ep.e2.scale_out = u->pw2->scale_out_dev;
    ep.e2.has_bias = 1; ep.e2.act_type = u->act; ep.e2.act_param0 = u->act_p2;
    const char* err = launch_unit_umma(ctx->stream, ctx->sm_count, u->plan, u->maps, us, n, h, w, u->cout2, ep, io->out_dev, io->out_dtype,
                                       status_word_dev ? status_word_dev : ctx->status_dev, io->out_f32_dev ? &mixed : nullptr, ctx->wait_limit_ns);
    if (err) return ctx->fail(OTT_ERR_CUDA, "%s: %s", err, cudaGetErrorString(cudaGetLastError()));
    ctx->launches += 1;
    return OTT_OK;
}

}  // extern "C"
