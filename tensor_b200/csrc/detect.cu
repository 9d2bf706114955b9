// Detection decode of the NanoDet-Plus head: NanodetPlusDetectionOutputLayer (Tensor/NanodetPlusDetectionOutputLayer.cpp:65-260).
// The per-cell work of generate_proposals (:111-190) — best class logit, sigmoid, threshold, softmax over the distance bins
// of the four box sides, box — runs on the GPU for every image and pyramid level; the proposals that pass the threshold
// are compacted per image with an atomic counter. Sorting by score and the greedy NMS (:208-243) run on the GPU as well, one
// CTA per image (bitonic sort of the image's proposals in shared memory, then the greedy pass as "every kept box strikes the
// later boxes it overlaps"), with the reference's formulas in the reference's operand order; one copy brings all images'
// rows back. An image with more proposals than the CTA's shared memory holds (4096) is sorted and filtered on the host.
// Floating point: expf/division here and in the reference's -Ofast build round differently in the last place, so scores
// agree to 1-2 ulp and box coordinates to about 1e-4 pixels; labels, order and counts are the same unless a score sits
// within that distance of the threshold or of another score.
#include <algorithm>
#include <cfloat>
#include <mutex>
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

__host__ __device__ inline float intersection(const Proposal& a, const Proposal& b) {
    const float axmax = a.x + a.w, aymax = a.y + a.h, bxmax = b.x + b.w, bymax = b.y + b.h;
    if (a.x > bxmax || axmax < b.x || a.y > bymax || aymax < b.y) return 0.f;
    const float iw = fminf(axmax, bxmax) - fmaxf(a.x, b.x);
    const float ih = fminf(aymax, bymax) - fmaxf(a.y, b.y);
    return iw * ih;
}

constexpr int kNmsThreads = 256, kNmsMaxProposals = 4096;

// One CTA per image. slots = power of two >= the image's proposal count (at most kNmsMaxProposals). Shared memory: the sort
// keys (score bits, then ~order: scores are positive, so their bit patterns order like the values), the proposal index
// behind each key, the sorted boxes, and one "struck" flag per box.
__global__ void __launch_bounds__(kNmsThreads)
nanodet_nms_kernel(const Proposal* __restrict__ props, const int* __restrict__ counts, int capacity, int slots, float nms_threshold, int max_det,
                   float* __restrict__ out, int* __restrict__ out_counts) {
    extern __shared__ unsigned long long nms_smem[];
    unsigned long long* key = nms_smem;
    int* idx = reinterpret_cast<int*>(key + slots);
    Proposal* box = reinterpret_cast<Proposal*>(idx + slots);
    unsigned char* struck = reinterpret_cast<unsigned char*>(box + slots);
    const int img = blockIdx.x;
    const int c = counts[img] < capacity ? counts[img] : capacity;
    if (c > slots) {  // more than this launch was sized for: the caller finishes this image on the host
        if (threadIdx.x == 0) out_counts[img] = -1;
        return;
    }
    const Proposal* mine = props + (long)img * capacity;
    int used = 32;  // the sort runs over the power of two that holds this image's proposals, not over the launch's maximum
    while (used < c) used <<= 1;
    slots = used;
    for (int i = threadIdx.x; i < slots; i += kNmsThreads) {
        if (i < c) {
            key[i] = ((unsigned long long)__float_as_uint(mine[i].score) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)mine[i].order);
            idx[i] = i;
        } else {
            key[i] = 0ull;  // below every real key (a proposal's score passed a positive threshold)
            idx[i] = -1;
        }
    }
    __syncthreads();
    // bitonic sort, descending
    for (int k = 2; k <= slots; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < slots; i += kNmsThreads) {
                const int l = i ^ j;
                if (l > i) {
                    const bool desc = (i & k) == 0;
                    const unsigned long long a = key[i], b = key[l];
                    if (desc ? a < b : a > b) {
                        key[i] = b; key[l] = a;
                        const int t = idx[i]; idx[i] = idx[l]; idx[l] = t;
                    }
                }
            }
            __syncthreads();
        }
    for (int i = threadIdx.x; i < c; i += kNmsThreads) {
        box[i] = mine[idx[i]];
        struck[i] = 0;
    }
    __syncthreads();
    // greedy NMS (:208-243): box i is kept unless an earlier kept box overlaps it by more than the threshold
    int kept = 0;
    float* o = out + (long)img * max_det * 6;
    for (int i = 0; i < c; ++i) {
        if (struck[i]) continue;  // block-uniform: every thread reads the same flag after the barrier below
        const Proposal a = box[i];
        if (threadIdx.x == 0 && kept < max_det) {
            o[6 * kept + 0] = a.label; o[6 * kept + 1] = a.score; o[6 * kept + 2] = a.x; o[6 * kept + 3] = a.y; o[6 * kept + 4] = a.w; o[6 * kept + 5] = a.h;
        }
        ++kept;
        const float area_a = a.w * a.h;
        for (int j = i + 1 + (int)threadIdx.x; j < c; j += kNmsThreads) {
            if (struck[j]) continue;
            const Proposal b = box[j];
            const float inter = intersection(b, a);
            const float uni = __fsub_rn(__fadd_rn(__fmul_rn(b.w, b.h), area_a), inter);
            if (__fdiv_rn(inter, uni) > nms_threshold) struck[j] = 1;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out_counts[img] = kept;
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
    // sort + NMS per image on the GPU, rows and counts back in one go
    int slots = 32;
    while (slots < capacity && slots < kNmsMaxProposals) slots <<= 1;
    const size_t nms_smem = (size_t)slots * (sizeof(unsigned long long) + sizeof(int) + sizeof(Proposal) + 1);
    DeviceBlock rows_dev, kept_dev;
    if (rows_dev.alloc(ctx, (size_t)n * (max_det > 0 ? max_det : 1) * 6 * sizeof(float)) != cudaSuccess || kept_dev.alloc(ctx, (size_t)n * sizeof(int)) != cudaSuccess) {
        (void)cudaGetLastError();
        return ctx->fail(OTT_ERR_ALLOC, "device allocation for the detections failed");
    }
    {
        static std::mutex mu;  // several host threads may drive different GPUs through this function at once
        std::lock_guard<std::mutex> lock(mu);
        OTT_CUDA_CHECK(ctx, cudaFuncSetAttribute(nanodet_nms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kNmsMaxProposals * (8 + 4 + sizeof(Proposal) + 1))));
    }
    nanodet_nms_kernel<<<(unsigned)n, kNmsThreads, nms_smem, ctx->stream>>>(static_cast<const Proposal*>(props.p), static_cast<const int*>(counts.p), capacity, slots,
                                                                          nms_threshold, max_det, static_cast<float*>(rows_dev.p), static_cast<int*>(kept_dev.p));
    OTT_CUDA_CHECK(ctx, cudaGetLastError());
    ctx->launches += 1;
    OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(counts_host, kept_dev.p, (size_t)n * sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    if (max_det > 0)
        OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(out_host, rows_dev.p, (size_t)n * max_det * 6 * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    OTT_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    // images whose proposals did not fit the CTA's shared memory (count marked -1): same steps on the host
    std::vector<Proposal> host;
    std::vector<int> picked;
    for (int img = 0; img < n; ++img) {
        if (counts_host[img] >= 0) continue;
        int c = 0;
        OTT_CUDA_CHECK(ctx, cudaMemcpyAsync(&c, static_cast<int*>(counts.p) + img, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
        OTT_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
        c = std::min(c, capacity);
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
