// fp32 NCHW -> int8 NHWC quantization: otter::quantize_to_int8 (Tensor/Quantize.cpp:52-58,
// Tensor/QuantizeX86.cpp:47-644) moved to the GPU, together with the layout change the reference does in
// Net::convert_layout (Tensor/Net.cpp:380-411).
//
// HBM-bound: 4 bytes read + 1 byte written per element. Each CTA moves a [64 channels x 128 pixels] tile
// of one image through shared memory: reads are float4 along W (the contiguous axis of NCHW), writes are
// 16-byte groups of channels (the contiguous axis of NHWC).
#include "kernels.h"

namespace ottk {

constexpr int QT_C = 64;    // channels per tile
constexpr int QT_P = 128;   // pixels per tile
constexpr int QT_THREADS = 256;

__global__ void __launch_bounds__(QT_THREADS)
quantize_nchw_to_nhwc_kernel(const float* __restrict__ x, int8_t* __restrict__ out, const float* __restrict__ scales,
                             int n_scales, int c, int cpad, int hw, int tiles_p, int tiles_c, int rounding) {
    __shared__ __align__(16) int8_t tile[QT_P][QT_C + 16];  // +16 keeps rows 16-byte aligned and spreads banks
    const long tile_id = blockIdx.x;
    const int tc = (int)(tile_id % tiles_c);
    const int tp = (int)((tile_id / tiles_c) % tiles_p);
    const int img = (int)(tile_id / ((long)tiles_c * tiles_p));
    const int c0 = tc * QT_C, p0 = tp * QT_P;
    const float* src = x + (long)img * c * hw;

    // phase 1: each warp takes channels, each lane 4 consecutive pixels
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec_ok = (hw % 4 == 0);
    for (int ch = warp; ch < QT_C; ch += QT_THREADS / 32) {
        const int cg = c0 + ch;
        const int p = p0 + lane * 4;
        int q[4] = {0, 0, 0, 0};
        if (cg < c) {
            const float s = n_scales == 1 ? scales[0] : scales[cg];
            const float* row = src + (long)cg * hw;
            if (vec_ok && p + 3 < hw) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(row + p));
                q[0] = quantize1(v.x, s, rounding);
                q[1] = quantize1(v.y, s, rounding);
                q[2] = quantize1(v.z, s, rounding);
                q[3] = quantize1(v.w, s, rounding);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (p + j < hw) q[j] = quantize1(__ldg(row + p + j), s, rounding);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) tile[lane * 4 + j][ch] = (int8_t)q[j];
    }
    __syncthreads();
    // phase 2: 16-byte channel groups, consecutive threads -> consecutive groups of one pixel
    const int groups = QT_C / 16;
    int8_t* dst = out + (long)img * hw * cpad;
    for (int i = threadIdx.x; i < QT_P * groups; i += QT_THREADS) {
        const int pl = i / groups, g = i % groups;
        const int p = p0 + pl, cg = c0 + g * 16;
        if (p < hw && cg < cpad) {
            const uint4 v = *reinterpret_cast<const uint4*>(&tile[pl][g * 16]);
            *reinterpret_cast<uint4*>(dst + (long)p * cpad + cg) = v;
        }
    }
}

cudaError_t launch_quantize_nchw_to_nhwc(cudaStream_t stream, const float* x, int8_t* out, const float* scales_dev,
                                         int n_scales, int n, int c, int h, int w, int rounding) {
    const int hw = h * w, cpad = nhwc_channels(c);
    if (n == 0 || hw == 0) return cudaSuccess;
    const int tiles_p = (hw + QT_P - 1) / QT_P, tiles_c = (cpad + QT_C - 1) / QT_C;
    const long blocks = (long)n * tiles_p * tiles_c;
    quantize_nchw_to_nhwc_kernel<<<(unsigned)blocks, QT_THREADS, 0, stream>>>(x, out, scales_dev, n_scales, c, cpad, hw,
                                                                            tiles_p, tiles_c, rounding);
    return cudaGetLastError();
}

}  // namespace ottk
