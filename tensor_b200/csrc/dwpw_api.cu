// C-ABI of the fused depthwise 3x3 -> 1x1 kernel (dwpw_umma.cu): ott_dwpw_int8_create builds, from two existing layer objects,
// the state of the pair; ott_dwpw_int8_forward_io runs both layers as one launch.
#include <cstring>
#include <new>
#include <vector>

#include "conv_object.h"
#include "ctx.h"
#include "dwpw_umma.h"

using namespace ottk;

struct ott_dwpw {
    DwPwPlan plan{};
    DwPwWeights maps{};
    int cout2 = 0;
    bool requant2 = false;
    int8_t* wpw = nullptr;  // device, owned: the 1x1 layer's weights against the depthwise layer's stored channel order
    // everything else stays with the two layers (the caller keeps them alive): the depthwise layer's diagonal weight panel and
    // where its channel blocks come from, both layers' epilogue arrays
    const ott_conv* dw = nullptr;
    const ott_conv* pw = nullptr;
};

namespace {
bool is_pointwise(const ott_conv_desc& d) {
    return d.groups == 1 && d.kh == 1 && d.kw == 1 && d.sh == 1 && d.sw == 1 && d.ph == 0 && d.pw == 0;
}
}  // namespace

extern "C" {

int ott_dwpw_int8_destroy(ott_ctx* ctx, ott_dwpw* f) {
    if (!f) return OTT_OK;
    if (ctx) ctx->alloc->free(f->wpw);
    delete f;
    return OTT_OK;
}

int ott_dwpw_int8_create(ott_ctx* ctx, const ott_conv* dw, const ott_conv* pw, ott_dwpw** out) {
    if (!ctx || !dw || !pw || !out) return OTT_ERR_INVALID;
    *out = nullptr;
    const ott_conv_desc &dd = dw->d, &dp = pw->d;
    const bool dw_gathered = !dw->src_channels.empty();
    const bool pw_gathered = !pw->src_channels.empty();
    const int dw_stored = dw_gathered ? dw->stored_channels : dd.cout;  // channels of the depthwise layer's output tensor
    const char* why = nullptr;
    if (!dw->depthwise || !dw->dw_umma) why = "the first layer must be a depthwise 3x3, pad 1, stride 1 or 2, add-half-truncate rounding";
    else if (dw_gathered && dw->gather_group != 32) why = "a depthwise layer with gathered input must be laid out in 32-channel groups";
    else if (!is_pointwise(dp)) why = "the second layer must be 1x1, stride 1, unpadded, ungrouped";
    else if (dd.int8_scale_term <= 100) why = "the depthwise layer must requantize (int8_scale_term > 100)";
    else if (dd.act_type != 0) why = "the depthwise layer must have no activation";
    else if (!dd.bias_term || !dp.bias_term) why = "both layers need a bias term";
    else if (dp.rounding != OTT_ROUND_ADD_HALF_TRUNC) why = "only the add-half-truncate rounding rule";
    else if (pw->n_in_scales != 1) why = "the 1x1 layer needs one input scale";
    else if (pw->plane_map_dev) why = "no scattered output";
    else if (pw_gathered ? (pw->src_channels.size() != 1 || pw->src_channels[0] != dw_stored) : (dw_gathered || dp.cin != dd.cout))
        why = "the 1x1 layer must read exactly the depthwise layer's output tensor";
    if (why) return ctx->fail(OTT_ERR_UNSUPPORTED, "fused depthwise + 1x1: %s", why);
    cudaSetDevice(ctx->device);
    int smem_optin = 0;
    cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, ctx->device);
    DwPwPlan p{};
    if (!dwpw_plan(dw_stored, dd.sh, dp.cout, smem_optin, &p) || p.ncb != dw->dw_plan.ncb_total)
        return ctx->fail(OTT_ERR_UNSUPPORTED, "fused depthwise + 1x1: %d -> %d channels do not fit one SM's shared / tensor memory", dw_stored, dp.cout);
    // the 1x1 layer's weights against the stored channel order of the depthwise layer's output: [c2][dwcols], zeros elsewhere
    std::vector<int8_t> w2(dwpw_wpw_bytes(p), 0);
    if (pw_gathered) {
        const size_t kk = pw->block_x.size() * 32;
        if (pw->w_korder.size() != (size_t)dp.cout * kk) return ctx->fail(OTT_ERR_INVALID, "fused depthwise + 1x1: the 1x1 layer keeps no K-ordered weights");
        for (size_t b = 0; b < pw->block_x.size(); ++b) {
            const int c0 = pw->block_x[b];  // first stored channel of the depthwise output this K block reads
            if (c0 % 32 != 0 || c0 + 32 > p.dwcols) return ctx->fail(OTT_ERR_UNSUPPORTED, "fused depthwise + 1x1: K block outside the depthwise layer's channels");
            for (int o = 0; o < dp.cout; ++o) std::memcpy(&w2[(size_t)o * p.dwcols + c0], &pw->w_korder[(size_t)o * kk + b * 32], 32);
        }
    } else {
        for (int o = 0; o < dp.cout; ++o) std::memcpy(&w2[(size_t)o * p.dwcols], &pw->w_host[(size_t)o * dp.cin], (size_t)dp.cin);
    }
    ott_dwpw* f = new (std::nothrow) ott_dwpw();
    if (!f) return OTT_ERR_ALLOC;
    f->plan = p;
    f->cout2 = dp.cout;
    f->requant2 = dp.int8_scale_term > 100;
    f->dw = dw;
    f->pw = pw;
    void* dev = nullptr;
    cudaError_t e = ctx->alloc->allocate(w2.size(), &dev);
    if (e != cudaSuccess) {
        delete f;
        return ctx->fail(OTT_ERR_ALLOC, "device allocation of %zu bytes failed: %s", w2.size(), cudaGetErrorString(e));
    }
    f->wpw = static_cast<int8_t*>(dev);
    int rc = OTT_OK;
    if (cudaMemcpyAsync(f->wpw, w2.data(), w2.size(), cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess ||
        cudaStreamSynchronize(ctx->stream) != cudaSuccess)
        rc = ctx->fail(OTT_ERR_CUDA, "upload failed");
    if (rc == OTT_OK) {
        const char* err = dwpw_encode_weight_maps(p, dw->w_dwu_dev, f->wpw, &f->maps);
        if (err) rc = ctx->fail(OTT_ERR_CUDA, "%s", err);
    }
    if (rc != OTT_OK) {
        ott_dwpw_int8_destroy(ctx, f);
        return rc;
    }
    *out = f;
    return OTT_OK;
}

int ott_dwpw_int8_forward_io(ott_ctx* ctx, const ott_dwpw* f, const ott_conv_io* io, int n, int h, int w, uint32_t* status_word_dev) {
    if (!ctx || !f || !io || n < 0 || h <= 0 || w <= 0) return OTT_ERR_INVALID;
    if (io->n_chunks > 0) return ctx->fail(OTT_ERR_UNSUPPORTED, "fused depthwise + 1x1: no scattered output");
    if (!io->out_dev) return OTT_ERR_INVALID;
    if (io->out_dtype == OTT_S8_NHWC ? !f->requant2 : (io->out_dtype != OTT_F32_NCHW || f->requant2))
        return ctx->fail(OTT_ERR_INVALID, "fused depthwise + 1x1: output type does not match the 1x1 layer's int8_scale_term");
    const ott_conv* dw = f->dw;
    const bool gathered = !dw->src_channels.empty();
    UmmaSources us{};
    const int8_t* x = nullptr;
    if (gathered) {
        if (!io->sources || io->n_sources != (int)dw->src_channels.size())
            return ctx->fail(OTT_ERR_INVALID, "fused depthwise + 1x1: the depthwise layer reads exactly its %d int8 sources", (int)dw->src_channels.size());
        us.n_src = io->n_sources;
        for (int i = 0; i < io->n_sources; ++i) {
            if (!io->sources[i]) return ctx->fail(OTT_ERR_INVALID, "null source tensor");
            us.src[i] = io->sources[i];
            us.src_cpad[i] = nhwc_channels(dw->src_channels[(size_t)i]);
        }
        for (size_t b = 0; b < dw->block_x.size(); ++b) { us.block_x[b] = dw->block_x[b]; us.block_src[b] = dw->block_src[b]; }
    } else {
        if (!io->in_dev || io->in_dtype != OTT_S8_NHWC) return ctx->fail(OTT_ERR_INVALID, "fused depthwise + 1x1: int8 NHWC input");
        x = static_cast<const int8_t*>(io->in_dev);
    }
    UmmaMixedOut mixed{};
    if (io->out_f32_dev) {
        if (!io->f32_channel_mask || io->out_dtype != OTT_S8_NHWC) return ctx->fail(OTT_ERR_INVALID, "out_f32_dev needs f32_channel_mask and an int8 launch");
        if (f->cout2 > 1024) return ctx->fail(OTT_ERR_UNSUPPORTED, "an fp32 side output is limited to 1024 output channels");
        mixed.out_f32 = io->out_f32_dev;
        for (int i = 0; i < (f->cout2 + 31) / 32 && i < 32; ++i) mixed.mask[i] = io->f32_channel_mask[i];
        if (f->cout2 % 32) mixed.mask[f->cout2 / 32] &= (1u << (f->cout2 % 32)) - 1u;
    }
    const ott_conv_desc& dd = dw->d;
    ConvShape s{};
    s.n = n; s.h = h; s.w = w;
    s.oh = (h + 2 - 3) / dd.sh + 1;
    s.ow = (w + 2 - 3) / dd.sw + 1;
    if (s.oh <= 0 || s.ow <= 0) return ctx->fail(OTT_ERR_INVALID, "empty output");
    s.cin = dd.cin; s.cout = dd.cout; s.cin_pad = dw->cin_pad; s.cout_pad = dw->cout_pad;
    s.kh = s.kw = 3; s.sh = dd.sh; s.sw = dd.sw; s.ph = s.pw = 1; s.dh = s.dw = 1;
    if (n == 0) return OTT_OK;
    cudaSetDevice(ctx->device);
    DwPwEpilogues ep{};
    ep.dw.scale_in = dw->scale_in_dev; ep.dw.bias = dw->bias_dev; ep.dw.scale_out = dw->scale_out_dev;
    ep.dw.has_bias = 1;
    ep.pw.scale_in = f->pw->scale_in_dev; ep.pw.bias = f->pw->bias_dev; ep.pw.scale_out = f->pw->scale_out_dev;
    ep.pw.has_bias = 1; ep.pw.act_type = f->pw->d.act_type; ep.pw.act_param0 = f->pw->d.act_param0;
    const char* err = launch_dwpw_umma(ctx->stream, ctx->sm_count, f->plan, f->maps, s, x, gathered ? &us : nullptr, f->cout2, ep, io->out_dev, io->out_dtype,
                                       status_word_dev ? status_word_dev : ctx->status_dev, io->out_f32_dev ? &mixed : nullptr, ctx->wait_limit_ns);
    if (err) return ctx->fail(OTT_ERR_CUDA, "%s: %s", err, cudaGetErrorString(cudaGetLastError()));
    ctx->launches += 1;
    return OTT_OK;
}

}  // extern "C"
