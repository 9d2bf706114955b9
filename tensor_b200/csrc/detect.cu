// Detection decode of the NanoDet-Plus head: NanodetPlusDetectionOutputLayer (Tensor/NanodetPlusDetectionOutputLayer.cpp:65-260).
// The per-cell work of generate_proposals (:111-190) — best class logit, sigmoid, threshold, softmax over the distance bins
// of the four box sides, box — runs on the GPU for every image and pyramid level; the proposals that pass the threshold
// are compacted per image with an atomic counter. Sorting by score and the greedy NMS (:208-243) see only those few rows and
// run on the host, per image, with the reference's formulas.
// Floating point: expf/division here and in the reference's -Ofast build round differently in the last place, so scores
// agree to 1-2 ulp and box coordinates to about 1e-4 pixels; labels, order and counts are the same unless a score sits
// within that distance of the threshold or of another score.
#include <algorithm>
#include <cfloat>
#include <vector>

#include "ctx.h"

namespace {

constexpr int kMaxRegBins = 32;
struct Proposal {
    float label, score, x, y, w, h;
    int order, pad;  // order = position in the reference's proposal list (level, row, column): the sort's tie-break
};

__global__ void nanodet_proposals_kernel(const float* __restrict__ pred, int n, int num_class, int reg_bins, int gh, int gw, int stride,
                                         float prob_threshold, int order_base, Proposal* __restrict__ props, int* __restrict__ counts,
                                         int capacity) {
    const long cell = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long plane = (long)gh * gw;
    if (cell >= (long)n * plane) return;
    const int img = (int)(cell / plane);
    const int p = (int)(cell - (long)img * plane);
    const float* base = pred + (long)img * (num_class + 4 * reg_bins) * plane + p;
    int label = -1;
    float score = -FLT_MAX;
    for (int k = 0; k < num_class; ++k) {
        const float s = __ldg(base + k * plane);
        if (s > score) { label = k; score = s; }
    }
    score = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-score)));
    if (!(score >= prob_threshold)) return;
    float ltrb[4];
    for (int side = 0; side < 4; ++side) {
        float v[kMaxRegBins], m = -FLT_MAX, sum = 0.f, dis = 0.f;
        for (int b = 0; b < reg_bins; ++b) {
            v[b] = __ldg(base + (num_class + side * reg_bins + b) * plane);
            m = fmaxf(m, v[b]);
        }
        for (int b = 0; b < reg_bins; ++b) { v[b] = expf(__fsub_rn(v[b], m)); sum = __fadd_rn(sum, v[b]); }
        for (int b = 0; b < reg_bins; ++b) dis = __fadd_rn(dis, __fmul_rn((float)b, __fdiv_rn(v[b], sum)));
        ltrb[side] = __fmul_rn(dis, (float)stride);
    }
    const int i = p / gw, j = p - i * gw;
    const float cx = (float)(j * stride), cy = (float)(i * stride);
    const float x0 = __fsub_rn(cx, ltrb[0]), y0 = __fsub_rn(cy, ltrb[1]), x1 = __fadd_rn(cx, ltrb[2]), y1 = __fadd_rn(cy, ltrb[3]);
    const int slot = atomicAdd(counts + img, 1);
    if (slot >= capacity) return;
    Proposal q;
    q.label = (float)(label + 1);  // +1: the reference prepends a background class
    q.score = score;
    q.x = x0; q.y = y0; q.w = __fsub_rn(x1, x0); q.h = __fsub_rn(y1, y0);
    q.order = order_base + p; q.pad = 0;
    props[(long)img * capacity + slot] = q;
}

float intersection(const Proposal& a, const Proposal& b) {
    const float axmax = a.x + a.w, aymax = a.y + a.h, bxmax = b.x + b.w, bymax = b.y + b.h;
    if (a.x > bxmax || axmax < b.x || a.y > bymax || aymax < b.y) return 0.f;
    const float iw = std::min(axmax, bxmax) - std::max(a.x, b.x);
    const float ih = std::min(aymax, bymax) - std::max(a.y, b.y);
    return iw * ih;
}

}  // namespace

extern "C" int ott_nanodet_detect(ott_ctx* ctx, const float* const* heads_dev, const int* grid_h, const int* grid_w, const int* strides,
                                  int n_levels, int n, int num_class, int reg_bins, float prob_threshold, float nms_threshold,
                                  float* out_host, int* counts_host, int max_det) {
    if (!ctx || !heads_dev || !grid_h || !grid_w || !strides || !out_host || !counts_host || n_levels < 1 || n < 0 || num_class < 1 ||
        max_det < 0)
        return OTT_ERR_INVALID;
    if (reg_bins < 1 || reg_bins > kMaxRegBins) return ctx->fail(OTT_ERR_UNSUPPORTED, "detection decode: 1..%d distance bins per box side", kMaxRegBins);
    if (n == 0) return OTT_OK;
    cudaSetDevice(ctx->device);
    long cells = 0;
    for (int l = 0; l < n_levels; ++l) {
        if (!heads_dev[l] || grid_h[l] < 1 || grid_w[l] < 1) return OTT_ERR_INVALID;
        cells += (long)grid_h[l] * grid_w[l];
    }
    if (cells > 0x7fffffffL / (long)sizeof(Proposal)) return ctx->fail(OTT_ERR_UNSUPPORTED, "detection decode: too many grid cells");
    const int capacity = (int)cells;  // every cell of an image may pass the threshold
    DeviceBlock props, counts;
    if (props.alloc(ctx, (size_t)n * capacity * sizeof(Proposal)) != cudaSuccess || counts.alloc(ctx, (size_t)n * sizeof(int)) != cudaSuccess) {
        (void)cudaGetLastError();
        return ctx->fail(OTT_ERR_ALLOC, "device allocation for the proposals failed");
    }
    OTT_CUDA_CHECK(ctx, cudaMemsetAsync(counts.p, 0, (size_t)n * sizeof(int), ctx->stream));
    int order_base = 0;
    for (int l = 0; l < n_levels; ++l) {
        const long total = (long)n * grid_h[l] * grid_w[l];
        nanodet_proposals_kernel<<<(unsigned)((total + 127) / 128), 128, 0, ctx->stream>>>(heads_dev[l], n, num_class, reg_bins, grid_h[l], grid_w[l],
                                                                                         strides[l], prob_threshold, order_base,
                                                                                         static_cast<Proposal*>(props.p), static_cast<int*>(counts.p),
                                                                                         capacity);
        OTT_CUDA_CHECK(ctx, cudaGetLastError());
        ctx->launches += 1;
        order_base += grid_h[l] * grid_w[l];
    }
    std::vector<int> cnt((size_t)n);
    OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(cnt.data(), counts.p, (size_t)n * sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    OTT_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    std::vector<Proposal> host;
    std::vector<int> picked;
    for (int img = 0; img < n; ++img) {
        const int c = std::min(cnt[(size_t)img], capacity);
        host.resize((size_t)c);
        if (c > 0) {
            OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(host.data(), static_cast<Proposal*>(props.p) + (long)img * capacity, (size_t)c * sizeof(Proposal),
                                                cudaMemcpyDeviceToHost, ctx->stream));
            OTT_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
        }
        // highest score first (:72-73); equal scores in proposal order (the reference's quicksort leaves them unspecified)
        std::sort(host.begin(), host.end(), [](const Proposal& a, const Proposal& b) { return a.score != b.score ? a.score > b.score : a.order < b.order; });
        picked.clear();
        for (int i = 0; i < c; ++i) {  // nms_sorted_bboxes (:208-243)
            bool keep = true;
            const float area_i = host[(size_t)i].w * host[(size_t)i].h;
            for (int j : picked) {
                const Proposal& b = host[(size_t)j];
                const float inter = intersection(host[(size_t)i], b);
                const float uni = area_i + b.w * b.h - inter;
                if (inter / uni > nms_threshold) keep = false;
            }
            if (keep) picked.push_back(i);
        }
        counts_host[img] = (int)picked.size();
        float* o = out_host + (size_t)img * max_det * 6;
        for (int i = 0; i < (int)picked.size() && i < max_det; ++i) {
            const Proposal& r = host[(size_t)picked[(size_t)i]];
            o[6 * i + 0] = r.label; o[6 * i + 1] = r.score; o[6 * i + 2] = r.x; o[6 * i + 3] = r.y; o[6 * i + 4] = r.w; o[6 * i + 5] = r.h;
        }
    }
    return OTT_OK;
}
