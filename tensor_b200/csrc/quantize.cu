// fp32 NCHW -> int8 NHWC quantization: otter::quantize_to_int8 (Tensor/Quantize.cpp:52-58,
// Tensor/QuantizeX86.cpp:47-644) moved to the GPU, together with the layout change the reference does in
// Net::convert_layout (Tensor/Net.cpp:380-411).
//
// HBM-bound: 4 bytes read + 1 byte written per element. Each CTA moves a [64 channels x 128 pixels] tile
// of one image: reads are float4 along W (the contiguous axis of NCHW), the channel/pixel transpose of
// 4x4 blocks happens in registers, 32-bit words of 4 channels go through shared memory, and writes are
// 16-byte groups of channels (the contiguous axis of NHWC).
#include "kernels.h"
#include "launch.cuh"

namespace ottk {

constexpr int QT_C = 64;    // channels per tile
constexpr int QT_P = 128;   // pixels per tile
constexpr int QT_THREADS = 256;
constexpr int QT_PITCH = 17;  // words per pixel row in shared memory (16 used): odd, so columns spread over banks

// pixel p of the tile lives in row (p%4)*33 + p/4: the four pixels a thread produces from one float4 land in
// four row groups, and the 32 lanes of a warp land in 32 consecutive rows of a group (no bank conflicts).
__device__ __forceinline__ int qt_row(int p) { return (p & 3) * 33 + (p >> 2); }

__global__ void __launch_bounds__(QT_THREADS)
quantize_nchw_to_nhwc_kernel(const __grid_constant__ PlaneGather G, int8_t* __restrict__ out, const float* __restrict__ scales,
                             int n_scales, int c, int cpad, int hw, int tiles_p, int tiles_c, int rounding, int out_stride, int scale_base, int flat,
                             long total_px) {
    __shared__ uint32_t tile[4 * 33 * QT_PITCH];
    pdl_launch_dependents();
    pdl_wait();
    const long tile_id = blockIdx.x;
    const int tc = (int)(tile_id % tiles_c);
    const int tp = (int)((tile_id / tiles_c) % tiles_p);
    // flat: the pixel axis runs over all images (hw % 4 == 0, so a thread's 4 pixels never straddle two images) and no
    // tile is wasted on the tail of an image; otherwise tiles are per image
    const int img_tile = flat ? 0 : (int)(tile_id / ((long)tiles_c * tiles_p));
    const int c0 = tc * QT_C;
    const long p0 = (long)tp * QT_P;                     // first pixel of the tile (global when flat, in-image otherwise)
    const long px_end = flat ? total_px : (long)hw;      // pixels beyond this do not exist

    // phase 1: a thread quantizes 4 consecutive pixels of 4 consecutive channels and packs, per pixel, the
    // 4 channels into one word. Lanes run along pixels (512 contiguous bytes per channel row per warp).
    const int pq = threadIdx.x & 31, cq = threadIdx.x >> 5;
    const bool vec_ok = (hw % 4 == 0);
    const long gp = p0 + pq * 4;
    const int img = flat ? (int)(gp / hw) : img_tile;
    const int p = flat ? (int)(gp - (long)img * hw) : (int)gp;
#pragma unroll
    for (int pass = 0; pass < QT_C / 32; ++pass) {
        if (c0 + 32 * pass >= cpad) break;  // narrow tensors: nothing of this half of the tile is ever stored
        const int cword = cq + 8 * pass;
        uint32_t cw[4];  // channel i: its 4 pixels packed
        float4 v[4];
        float sc[4];
        const bool fast = vec_ok && gp + 3 < px_end && c0 + cword * 4 + 3 < c && rounding == ROUND_ADD_HALF_TRUNC;
        if (fast) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int cg = c0 + cword * 4 + i;
                sc[i] = n_scales == 1 ? __ldg(scales) : __ldg(scales + scale_base + cg);
                v[i] = __ldg(reinterpret_cast<const float4*>(G.plane(cg, img, hw) + p));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) cw[i] = quantize4_pack(v[i].x, v[i].y, v[i].z, v[i].w, sc[i]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int cg = c0 + cword * 4 + i;
                int q[4] = {0, 0, 0, 0};
                if (cg < c) {
                    const float s = n_scales == 1 ? __ldg(scales) : __ldg(scales + scale_base + cg);
                    const float* row = G.plane(cg, img, hw);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (gp + j < px_end) q[j] = quantize1(__ldg(row + p + j), s, rounding);
                }
                cw[i] = pack4(q[0], q[1], q[2], q[3]);
            }
        }
        uint32_t pw[4];  // pixel j: its 4 channels packed
        transpose4x4(cw[0], cw[1], cw[2], cw[3], pw);
#pragma unroll
        for (int j = 0; j < 4; ++j) tile[(j * 33 + pq) * QT_PITCH + cword] = pw[j];
    }
    __syncthreads();
    // phase 2: 16-byte channel groups; consecutive threads -> consecutive groups of one pixel
    int8_t* dst = out + (long)img_tile * hw * out_stride;
    for (int i = threadIdx.x; i < QT_P * (QT_C / 16); i += QT_THREADS) {
        const int pl = i >> 2, g = i & 3;
        const long pg = p0 + pl;
        const int cg = c0 + g * 16;
        if (pg < px_end && cg < cpad) {
            const uint32_t* r = tile + qt_row(pl) * QT_PITCH + g * 4;
            *reinterpret_cast<uint4*>(dst + pg * out_stride + cg) = make_uint4(r[0], r[1], r[2], r[3]);
        }
    }
}

void gather_identity(PlaneGather* g, const float* x, int c, int c_total, long hw) {
    g->base[0] = x;
    g->img_stride[0] = (long long)c_total * hw;
    for (int i = 0; i < c && i < kGatherMaxChannels; ++i) g->ref[i] = (uint32_t)i;
}

cudaError_t launch_quantize_nchw_to_nhwc(cudaStream_t stream, const PlaneGather& src, int8_t* out, const float* scales_dev,
                                         int n_scales, int n, int c, int h, int w, int rounding) {
    const int hw = h * w, cpad = nhwc_channels(c);
    if (n == 0 || hw == 0) return cudaSuccess;
    if (c > kGatherMaxChannels) return cudaErrorInvalidValue;
    const int flat = hw % 4 == 0 ? 1 : 0;
    const long total_px = (long)n * hw;
    const int tiles_p = flat ? (int)((total_px + QT_P - 1) / QT_P) : (hw + QT_P - 1) / QT_P, tiles_c = (cpad + QT_C - 1) / QT_C;
    const long blocks = (long)(flat ? 1 : n) * tiles_p * tiles_c;
    return launch_overlapped(quantize_nchw_to_nhwc_kernel, dim3((unsigned)blocks), dim3(QT_THREADS), 0, stream, src, out, scales_dev, n_scales, c, cpad,
                             hw, tiles_p, tiles_c, rounding, cpad, 0, flat, total_px);
}

// A plain tensor of any channel count: the plane table holds kGatherMaxChannels entries, so wider tensors are
// quantized in channel chunks, each launch writing its slice of the NHWC rows.
cudaError_t launch_quantize_dense(cudaStream_t stream, const float* x, int c_total, int8_t* out, const float* scales_dev, int n_scales,
                                  int n, int c, int h, int w, int rounding) {
    const int hw = h * w, cpad = nhwc_channels(c);
    if (n == 0 || hw == 0) return cudaSuccess;
    const int flat = hw % 4 == 0 ? 1 : 0;
    const long total_px = (long)n * hw;
    const int tiles_p = flat ? (int)((total_px + QT_P - 1) / QT_P) : (hw + QT_P - 1) / QT_P;
    for (int base = 0; base < cpad; base += kGatherMaxChannels) {
        const int chunk_pad = cpad - base < kGatherMaxChannels ? cpad - base : kGatherMaxChannels;  // channels written by this launch
        const int chunk = c - base < chunk_pad ? (c - base > 0 ? c - base : 0) : chunk_pad;          // of which real ones
        PlaneGather g;
        g.base[0] = x;
        g.img_stride[0] = (long long)c_total * hw;
        for (int i = 0; i < chunk; ++i) g.ref[i] = (uint32_t)(base + i);
        const int tiles_c = (chunk_pad + QT_C - 1) / QT_C;
        const long blocks = (long)(flat ? 1 : n) * tiles_p * tiles_c;
        cudaError_t e = launch_overlapped(quantize_nchw_to_nhwc_kernel, dim3((unsigned)blocks), dim3(QT_THREADS), 0, stream, g, out + base, scales_dev,
                                          n_scales, chunk, chunk_pad, hw, tiles_p, tiles_c, rounding, cpad, base, flat, total_px);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// dst[img][c][p] = plane(c, img)[p]
__global__ void gather_planes_kernel(const __grid_constant__ PlaneGather G, float* __restrict__ dst, int c, long hw, long total4, int vec) {
    pdl_launch_dependents();
    pdl_wait();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (long)gridDim.x * blockDim.x) {
        const long per = vec ? hw / 4 : hw;
        const long p = i % per;
        const long r = i / per;
        const int ch = (int)(r % c);
        const int img = (int)(r / c);
        const float* src = G.plane(ch, img, hw);
        if (vec) reinterpret_cast<float4*>(dst)[i] = __ldg(reinterpret_cast<const float4*>(src) + p);
        else dst[i] = __ldg(src + p);
    }
}

// dst[img][c][p] = A.plane(c, img)[p] + B.plane(c, img)[p]: the reference's ShortCut (Tensor/ShortCutLayer.cpp) reading both
// operands where their planes lie. Block = one plane (or a slice of one), so the table look-up is per block, not per element.
__global__ void add_planes_kernel(const __grid_constant__ PlaneGather A, const __grid_constant__ PlaneGather B, float* __restrict__ dst, int c,
                                  long hw, int slices, int vec) {
    pdl_launch_dependents();
    pdl_wait();
    const long plane = blockIdx.x / slices;
    const int slice = (int)(blockIdx.x % slices);
    const int ch = (int)(plane % c);
    const int img = (int)(plane / c);
    const float* a = A.plane(ch, img, hw);
    const float* b = B.plane(ch, img, hw);
    float* o = dst + plane * hw;
    const long per = vec ? hw / 4 : hw;
    const long lo = per * slice / slices, hi = per * (slice + 1) / slices;
    if (vec) {
        for (long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            const float4 u = __ldg(reinterpret_cast<const float4*>(a) + i), v = __ldg(reinterpret_cast<const float4*>(b) + i);
            reinterpret_cast<float4*>(o)[i] = make_float4(__fadd_rn(u.x, v.x), __fadd_rn(u.y, v.y), __fadd_rn(u.z, v.z), __fadd_rn(u.w, v.w));
        }
    } else {
        for (long i = lo + threadIdx.x; i < hi; i += blockDim.x) o[i] = __fadd_rn(__ldg(a + i), __ldg(b + i));
    }
}

cudaError_t launch_add_planes(cudaStream_t stream, const PlaneGather& a, const PlaneGather& b, float* dst, int n, int c, long hw) {
    if (n == 0 || c == 0 || hw == 0) return cudaSuccess;
    if (c > kGatherMaxChannels) return cudaErrorInvalidValue;
    const int vec = hw % 4 == 0 ? 1 : 0;
    const long per = vec ? hw / 4 : hw;
    const int threads = per >= 256 ? 256 : (per >= 128 ? 128 : 64);
    int slices = (int)((per + 4L * threads - 1) / (4L * threads));  // about four elements (vectors) per thread
    if (slices < 1) slices = 1;
    const long blocks = (long)n * c * slices;
    if (blocks > 0x7fffffffL) return cudaErrorInvalidValue;
    return launch_overlapped(add_planes_kernel, dim3((unsigned)blocks), dim3(threads), 0, stream, a, b, dst, c, hw, slices, vec);
}

cudaError_t launch_gather_planes(cudaStream_t stream, const PlaneGather& src, float* dst, int n, int c, long hw) {
    if (n == 0 || c == 0 || hw == 0) return cudaSuccess;
    if (c > kGatherMaxChannels) return cudaErrorInvalidValue;
    const int vec = hw % 4 == 0 ? 1 : 0;
    const long total = (long)n * c * (vec ? hw / 4 : hw);
    long grid = (total + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    return launch_overlapped(gather_planes_kernel, dim3((unsigned)grid), dim3(256), 0, stream, src, dst, c, hw, total, vec);
}

}  // namespace ottk
