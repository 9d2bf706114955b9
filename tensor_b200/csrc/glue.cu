// The fp32 glue layers between the int8 convolutions of the benchmark graphs, as small bandwidth-bound
// CUDA kernels on the Net's stream: channel-plane copies (Concat, Crop, ChannelShuffle), MaxPool,
// element-wise add (ShortCut) and the stand-alone activations. All tensors are fp32 NCHW on the device.
// Reference: Tensor/ConcatLayer.cpp:55-70, Tensor/CropLayer.cpp:67-75, Tensor/ChannelShuffleLayer.cpp:37-41,
// Tensor/MaxPoolLayer.cpp:123-133 + Tensor/Pool.cpp:1166-1201, Tensor/ShortCutLayer.cpp, Tensor/ReluLayer.cpp,
// Tensor/LReluLayer.cpp, Tensor/Relu6Layer.cpp, Tensor/UpsampleLayer.cpp:113-131.
#include "ctx.h"
#include "launch.cuh"

namespace {

// dst[b][dst_c0 + j*dst_cs][p] = src[b][src_c0 + j*src_cs][p], j < count, p < hw
template <typename V>
__global__ void copy_channels_kernel(const V* __restrict__ src, V* __restrict__ dst, int src_channels, int src_c0, int src_cs,
                                     int dst_channels, int dst_c0, int dst_cs, int count, long hwv, long total) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long p = i % hwv;
        const long r = i / hwv;
        const int j = (int)(r % count);
        const long b = r / count;
        dst[(b * dst_channels + dst_c0 + (long)j * dst_cs) * hwv + p] = __ldg(src + (b * src_channels + src_c0 + (long)j * src_cs) * hwv + p);
    }
}

// pad_zero: out-of-image taps count as 0 (the reference's packed 3x3 s2 path pads the input with zeros,
// Tensor/Pool.cpp:972-975); otherwise they are ignored (its plain path, -inf padding).
__global__ void maxpool_kernel(const float* __restrict__ x, float* __restrict__ y, int c, int h, int w, int oh, int ow, int kh,
                               int kw, int sh, int sw, int ph, int pw, int pad_zero, long total) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int ox = (int)(i % ow);
    long r = i / ow;
    const int oy = (int)(r % oh);
    const long plane = r / oh;  // b*c + ch
    const float* xp = x + plane * h * w;
    float m = -INFINITY;
    for (int ky = 0; ky < kh; ++ky) {
        const int iy = oy * sh - ph + ky;
        for (int kx = 0; kx < kw; ++kx) {
            const int ix = ox * sw - pw + kx;
            const bool in = iy >= 0 && iy < h && ix >= 0 && ix < w;
            if (in) m = fmaxf(m, __ldg(xp + (long)iy * w + ix));
            else if (pad_zero) m = fmaxf(m, 0.f);
        }
    }
    y[i] = m;
}

__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ o, long n) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) o[i] = __fadd_rn(a[i], b[i]);
}
__global__ void add4_kernel(const float4* __restrict__ a, const float4* __restrict__ b, float4* __restrict__ o, long n4) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
        const float4 u = __ldg(a + i), v = __ldg(b + i);
        o[i] = make_float4(__fadd_rn(u.x, v.x), __fadd_rn(u.y, v.y), __fadd_rn(u.z, v.z), __fadd_rn(u.w, v.w));
    }
}

__global__ void activation_kernel(float* __restrict__ x, long n, int act, float p0) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        float v = x[i];
        if (act == 1) v = v > 0.f ? v : 0.f;
        else if (act == 2) v = v < 0.f ? __fmul_rn(v, p0) : v;
        else if (act == 3) v = fminf(fmaxf(v, 0.f), 6.f);
        x[i] = v;
    }
}

// One axis of the bilinear resize: the two source indices and their weights for output index d.
// rule 1 (the reference's packed blobs, Tensor/TensorInterpolation.cpp:16-46): source position in double, floor, and a
// border clamp that moves the pair inside the row with weights (1,0) / (0,1).
// rule 0 (its plain blobs, Tensor/UpSample.hpp:53-94,133-158): scale and position in float, negative positions clamped to 0,
// the second index clamped to the last element.
struct AxisTap {
    int i0, i1;
    float w0, w1;
};
__device__ __forceinline__ AxisTap axis_tap(int d, int in, int out, double user_scale, int rule) {
    AxisTap t;
    if (rule == 1) {
        const double scale = (double)in / out;
        float f = (float)(((double)d + 0.5) * scale - 0.5);
        int s = (int)floorf(f);
        f -= (float)s;
        if (s < 0) { s = 0; f = 0.f; }
        if (s >= in - 1) { s = in - 2; f = 1.f; }
        t.i0 = s; t.i1 = s + 1;
        t.w0 = __fsub_rn(1.f, f); t.w1 = f;
    } else {
        if (out == in) { t.i0 = t.i1 = d; t.w0 = 1.f; t.w1 = 0.f; return t; }
        const float ratio = user_scale > 0. ? (float)(1.0 / user_scale) : (float)in / (float)out;
        float real = (float)((double)ratio * ((double)d + 0.5) - 0.5);
        if (real < 0.f) real = 0.f;
        t.i0 = (int)real;
        t.i1 = t.i0 + (t.i0 < in - 1 ? 1 : 0);
        t.w1 = __fsub_rn(real, (float)t.i0);
        t.w0 = __fsub_rn(1.f, t.w1);
    }
    return t;
}

// Bilinear resize of fp32 NCHW planes, align_corners = false. Both rules resize along x first, then along y, with one
// rounding per product and one per fused multiply-add, in the operand order of the reference build:
//   rule 1: fma(S1, w1, S0 * w0)      (Tensor/TensorInterpolation.cpp:199-207,251-259)
//   rule 0: fma(S0, w0, S1 * w1)      (Tensor/UpSampleKernel.cpp:125-139 as compiled with -Ofast -mfma)
// Thread = one output position (ox, oy) of kUpsamplePlanes consecutive planes. The taps depend on the position only and need
// double-precision arithmetic, so one thread per row and per column of the block computes them once into shared memory.
constexpr int kUpsamplePlanes = 32;
__global__ void __launch_bounds__(256)
upsample_bilinear_kernel(const float* __restrict__ x, float* __restrict__ y, int h, int w, int oh, int ow, double scale_h,
                         double scale_w, int rule, long planes) {
    __shared__ AxisTap taps_x[32], taps_y[8];
    ottk::pdl_launch_dependents();  // the taps below depend on the sizes only; the previous kernel is awaited after them
    const int tid = threadIdx.y * 32 + threadIdx.x;
    if (tid < 32) {
        const int ox = blockIdx.x * 32 + tid;
        if (ox < ow) taps_x[tid] = axis_tap(ox, w, ow, scale_w, rule);
    } else if (tid < 40) {
        const int oy = blockIdx.y * 8 + (tid - 32);
        if (oy < oh) taps_y[tid - 32] = axis_tap(oy, h, oh, scale_h, rule);
    }
    __syncthreads();
    ottk::pdl_wait();
    const int ox = blockIdx.x * 32 + threadIdx.x;
    const int oy = blockIdx.y * 8 + threadIdx.y;
    if (ox >= ow || oy >= oh) return;
    const AxisTap tx = taps_x[threadIdx.x], ty = taps_y[threadIdx.y];
    const int o00 = ty.i0 * w + tx.i0, o01 = ty.i0 * w + tx.i1, o10 = ty.i1 * w + tx.i0, o11 = ty.i1 * w + tx.i1;
    const long p0 = (long)blockIdx.z * kUpsamplePlanes;
    const long p1 = p0 + kUpsamplePlanes < planes ? p0 + kUpsamplePlanes : planes;
    const long in_plane = (long)h * w, out_plane = (long)oh * ow;
    const float* xp = x + p0 * in_plane;
    float* yp = y + p0 * out_plane + (long)oy * ow + ox;
#pragma unroll 4
    for (long p = p0; p < p1; ++p, xp += in_plane, yp += out_plane) {
        const float a00 = __ldg(xp + o00), a01 = __ldg(xp + o01), a10 = __ldg(xp + o10), a11 = __ldg(xp + o11);
        float v;
        if (rule == 1) {
            const float r0 = __fmaf_rn(a01, tx.w1, __fmul_rn(a00, tx.w0));
            const float r1 = __fmaf_rn(a11, tx.w1, __fmul_rn(a10, tx.w0));
            v = __fmaf_rn(r1, ty.w1, __fmul_rn(r0, ty.w0));
        } else {
            const float r0 = __fmaf_rn(a00, tx.w0, __fmul_rn(a01, tx.w1));
            const float r1 = __fmaf_rn(a10, tx.w0, __fmul_rn(a11, tx.w1));
            v = __fmaf_rn(r0, ty.w0, __fmul_rn(r1, ty.w1));
        }
        *yp = v;
    }
}

// Source index of the nearest resize along one axis: rule 1 is the reference's packed resize (ratio in / out in fp32, product
// truncated: Tensor/TensorInterpolation.cpp:660-676), rule 0 its plain resize (copy for equal sizes, index >> 1 for a doubled
// size, else floor(d * (float)(1 / scale)): Tensor/UpSampleKernel.cpp:41-60, Tensor/UpSample.hpp:30-51).
__device__ __forceinline__ int nearest_index(int d, int in, int out, double user_scale, int rule) {
    int i;
    if (rule == 1) {
        i = (int)__fmul_rn((float)d, __fdiv_rn((float)in, (float)out));
    } else {
        if (out == in) return d;
        if (out == 2 * in) return d >> 1;
        const float ratio = user_scale > 0. ? (float)(1.0 / user_scale) : __fdiv_rn((float)in, (float)out);
        i = (int)floorf(__fmul_rn((float)d, ratio));
    }
    return i < in - 1 ? i : in - 1;
}

// Nearest resize of fp32 NCHW planes: the same thread layout as the bilinear kernel (one output position of kUpsamplePlanes
// consecutive planes per thread; the source indices are computed once per block row and column).
__global__ void __launch_bounds__(256)
upsample_nearest_kernel(const float* __restrict__ x, float* __restrict__ y, int h, int w, int oh, int ow, double scale_h, double scale_w,
                        int rule, long planes) {
    __shared__ int src_x[32], src_y[8];
    ottk::pdl_launch_dependents();
    const int tid = threadIdx.y * 32 + threadIdx.x;
    if (tid < 32) {
        const int ox = blockIdx.x * 32 + tid;
        if (ox < ow) src_x[tid] = nearest_index(ox, w, ow, scale_w, rule);
    } else if (tid < 40) {
        const int oy = blockIdx.y * 8 + (tid - 32);
        if (oy < oh) src_y[tid - 32] = nearest_index(oy, h, oh, scale_h, rule);
    }
    __syncthreads();
    ottk::pdl_wait();
    const int ox = blockIdx.x * 32 + threadIdx.x;
    const int oy = blockIdx.y * 8 + threadIdx.y;
    if (ox >= ow || oy >= oh) return;
    const int src = src_y[threadIdx.y] * w + src_x[threadIdx.x];
    const long p0 = (long)blockIdx.z * kUpsamplePlanes;
    const long p1 = p0 + kUpsamplePlanes < planes ? p0 + kUpsamplePlanes : planes;
    const long in_plane = (long)h * w, out_plane = (long)oh * ow;
    const float* xp = x + p0 * in_plane + src;
    float* yp = y + p0 * out_plane + (long)oy * ow + ox;
#pragma unroll 4
    for (long p = p0; p < p1; ++p, xp += in_plane, yp += out_plane) *yp = __ldg(xp);
}

unsigned grid_for(const ott_ctx* ctx, long total, int block) {
    long g = (total + block - 1) / block;
    const long cap = (long)ctx->sm_count * 16;
    return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

extern "C" {

int ott_copy_channels_f32(ott_ctx* ctx, const float* src, int src_channels, int src_c0, int src_cstride, float* dst, int dst_channels,
                          int dst_c0, int dst_cstride, int count, int n, int hw) {
    if (!ctx || !src || !dst || count < 0 || n < 0 || hw < 0) return OTT_ERR_INVALID;
    if (src_c0 < 0 || dst_c0 < 0 || (count > 0 && (src_c0 + (long)(count - 1) * src_cstride >= src_channels ||
                                                   dst_c0 + (long)(count - 1) * dst_cstride >= dst_channels)))
        return ctx->fail(OTT_ERR_INVALID, "channel range outside the tensor");
    const long total = (long)n * count * hw;
    if (total == 0) return OTT_OK;
    cudaSetDevice(ctx->device);
    const bool vec = hw % 4 == 0 && ((uintptr_t)src % 16 == 0) && ((uintptr_t)dst % 16 == 0);
    if (vec) {
        const long tv = total / 4;
        copy_channels_kernel<float4><<<grid_for(ctx, tv, 256), 256, 0, ctx->stream>>>(
            reinterpret_cast<const float4*>(src), reinterpret_cast<float4*>(dst), src_channels, src_c0, src_cstride, dst_channels, dst_c0,
            dst_cstride, count, hw / 4, tv);
    } else {
        copy_channels_kernel<float><<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(src, dst, src_channels, src_c0, src_cstride,
                                                                                      dst_channels, dst_c0, dst_cstride, count, hw, total);
    }
    OTT_CUDA_CHECK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return OTT_OK;
}

int ott_maxpool_f32_nchw(ott_ctx* ctx, const float* in, int n, int c, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw,
                         int pad_with_zero, float* out) {
    if (!ctx || !in || !out || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0) return OTT_ERR_INVALID;
    const int oh = (h + 2 * ph - kh) / sh + 1, ow = (w + 2 * pw - kw) / sw + 1;
    const long total = (long)n * c * oh * ow;
    if (total <= 0) return OTT_OK;
    cudaSetDevice(ctx->device);
    maxpool_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(in, out, c, h, w, oh, ow, kh, kw, sh, sw, ph, pw, pad_with_zero, total);
    OTT_CUDA_CHECK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return OTT_OK;
}

int ott_upsample_bilinear_f32_nchw(ott_ctx* ctx, const float* in, int n, int c, int h, int w, int oh, int ow, double scale_h, double scale_w,
                                   int packed_rule, float* out) {
    if (!ctx || !in || !out || n < 0 || c < 0 || h < 1 || w < 1 || oh < 1 || ow < 1) return OTT_ERR_INVALID;
    if (packed_rule && (h < 2 || w < 2)) return ctx->fail(OTT_ERR_UNSUPPORTED, "bilinear resize of a packed blob needs at least 2 rows and 2 columns");
    const long planes = (long)n * c;
    if (planes == 0) return OTT_OK;
    const long zblocks = (planes + kUpsamplePlanes - 1) / kUpsamplePlanes;
    if (zblocks > 65535 || (oh + 7) / 8 > 65535) return ctx->fail(OTT_ERR_UNSUPPORTED, "Upsample: more than 2097120 planes or 524280 rows in one call");
    cudaSetDevice(ctx->device);
    const dim3 block(32, 8), grid((unsigned)((ow + 31) / 32), (unsigned)((oh + 7) / 8), (unsigned)zblocks);
    OTT_CUDA_CHECK(ctx, ottk::launch_overlapped(upsample_bilinear_kernel, grid, block, 0, ctx->stream, in, out, h, w, oh, ow, scale_h, scale_w,
                                                packed_rule ? 1 : 0, planes));
    ctx->launches += 1;
    return OTT_OK;
}

int ott_upsample_nearest_f32_nchw(ott_ctx* ctx, const float* in, int n, int c, int h, int w, int oh, int ow, double scale_h, double scale_w,
                                  int packed_rule, float* out) {
    if (!ctx || !in || !out || n < 0 || c < 0 || h < 1 || w < 1 || oh < 1 || ow < 1) return OTT_ERR_INVALID;
    const long planes = (long)n * c;
    if (planes == 0) return OTT_OK;
    const long zblocks = (planes + kUpsamplePlanes - 1) / kUpsamplePlanes;
    if (zblocks > 65535 || (oh + 7) / 8 > 65535) return ctx->fail(OTT_ERR_UNSUPPORTED, "Upsample: more than 2097120 planes or 524280 rows in one call");
    cudaSetDevice(ctx->device);
    const dim3 block(32, 8), grid((unsigned)((ow + 31) / 32), (unsigned)((oh + 7) / 8), (unsigned)zblocks);
    OTT_CUDA_CHECK(ctx, ottk::launch_overlapped(upsample_nearest_kernel, grid, block, 0, ctx->stream, in, out, h, w, oh, ow, scale_h, scale_w,
                                                packed_rule ? 1 : 0, planes));
    ctx->launches += 1;
    return OTT_OK;
}

int ott_add_f32(ott_ctx* ctx, const float* a, const float* b, float* out, size_t count) {
    if (!ctx || !a || !b || !out) return OTT_ERR_INVALID;
    if (count == 0) return OTT_OK;
    cudaSetDevice(ctx->device);
    if (count % 4 == 0 && ((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) % 16 == 0)
        add4_kernel<<<grid_for(ctx, (long)(count / 4), 256), 256, 0, ctx->stream>>>(reinterpret_cast<const float4*>(a), reinterpret_cast<const float4*>(b),
                                                                                 reinterpret_cast<float4*>(out), (long)(count / 4));
    else
        add_kernel<<<grid_for(ctx, (long)count, 256), 256, 0, ctx->stream>>>(a, b, out, (long)count);
    OTT_CUDA_CHECK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return OTT_OK;
}

int ott_activation_f32(ott_ctx* ctx, float* x, size_t count, int act_type, float param0) {
    if (!ctx || !x || act_type < 0 || act_type > 3) return OTT_ERR_INVALID;
    if (count == 0 || act_type == 0) return OTT_OK;
    cudaSetDevice(ctx->device);
    activation_kernel<<<grid_for(ctx, (long)count, 256), 256, 0, ctx->stream>>>(x, (long)count, act_type, param0);
    OTT_CUDA_CHECK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return OTT_OK;
}

}  // extern "C"
