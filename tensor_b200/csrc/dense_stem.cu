// First-layer ("stem") int8 convolution: 3 input channels, 3x3, stride 1 or 2, fp32 NCHW image in, with the
// quantize prologue (Tensor/QuantizeX86.cpp:47-644) and the dequantize/requantize epilogue fused.
// Reference kernels: conv2d_3x3s2_int8_pack1to4 (Tensor/ConvolutionMM2DInt8X86Pack.cpp:2569-2651) and the generic
// pack1to4 im2col path (:2225-2261).
//
// HBM-bound (12 B of image per input pixel in, Cout*4 or Cout bytes per output pixel out). One CTA computes a
// 32x8 tile of output pixels for all output channels:
//  1. the fp32 input halo tile is quantized once into shared memory as int8 channel planes;
//  2. each thread gathers the 27 taps of its output pixel into 7 registers (4 taps per register, K order
//     channel-row-column) with funnel shifts and byte permutes;
//  3. 7 dp4a per output channel against the packed filter, which lives in the kernel parameter bank so every
//     multiply reads its weights as an immediate constant operand (warp-uniform, no loads);
//  4. epilogue per channel; fp32 NCHW stores are coalesced along the tile row, int8 NHWC stores are 16-byte vectors.
#include "store.cuh"

namespace ottk {

namespace {

constexpr int ST_TX = 32, ST_TY = 8;  // output tile
constexpr int ST_COUT_MAX = 32;

struct StemParams {
    uint32_t w[ST_COUT_MAX][7];  // packed filters: byte k of the 28 = tap (c, ky, kx) with k = c*9 + ky*3 + kx
    float scale_in[ST_COUT_MAX], bias[ST_COUT_MAX], scale_out[ST_COUT_MAX];
};

template <int S, int OUT, int ACT>
__global__ void __launch_bounds__(ST_TX * ST_TY)
dense_stem_kernel(const float* __restrict__ x, const __grid_constant__ StemParams P, float in_scale, int has_bias, float act_p0,
                  int rounding, void* __restrict__ out, ConvShape s, int tiles_x, int tiles_y) {
    constexpr int IW = (ST_TX - 1) * S + 3, IH = (ST_TY - 1) * S + 3;  // input halo tile
    constexpr int RP = (IW + 3 + 3) / 4 + 1;                            // words per row (tile origin rounded down to 4)
    __shared__ uint32_t tin[3][IH][RP];

    int b = blockIdx.x;
    const int tx = b % tiles_x; b /= tiles_x;
    const int ty = b % tiles_y;
    const int img = b / tiles_y;
    const int ox0 = tx * ST_TX, oy0 = ty * ST_TY;
    const int iy0 = oy0 * S - s.ph, ix_first = ox0 * S - s.pw;
    const int ix_al = (ix_first >= 0 ? ix_first : ix_first - 3) / 4 * 4;
    const int sh = ix_first - ix_al;  // 0..3

    // ---- 1. quantize the halo tile ----
    const float* ximg = x + (long)img * 3 * s.h * s.w;
    const bool vec_ok = (s.w % 4 == 0) && rounding == ROUND_ADD_HALF_TRUNC;
    for (int i = threadIdx.x; i < 3 * IH * RP; i += ST_TX * ST_TY) {
        const int xw = i % RP, r = (i / RP) % IH, c = i / (RP * IH);
        const int iy = iy0 + r, ix = ix_al + xw * 4;
        uint32_t word = 0;
        if (iy >= 0 && iy < s.h && ix + 3 >= 0 && ix < s.w) {
            const float* row = ximg + ((long)c * s.h + iy) * s.w;
            if (vec_ok && ix >= 0 && ix + 3 < s.w) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(row + ix));
                word = quantize4_pack(v.x, v.y, v.z, v.w, in_scale);
            } else {
                int q[4] = {0, 0, 0, 0};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (ix + j >= 0 && ix + j < s.w) q[j] = quantize1(__ldg(row + ix + j), in_scale, rounding);
                word = pack4(q[0], q[1], q[2], q[3]);
            }
        }
        tin[c][r][xw] = word;
    }
    __syncthreads();

    // ---- 2. gather the 27 taps of this thread's pixel ----
    const int lx = threadIdx.x % ST_TX, ly = threadIdx.x / ST_TX;
    const int ox = ox0 + lx, oy = oy0 + ly;
    const int boff = sh + lx * S;  // byte offset of the pixel's first tap column in a tile row
    const int wi = boff >> 2, bs = (boff & 3) * 8;
    uint32_t win[9];  // (c, ky): bytes 0..2 = taps kx 0..2
#pragma unroll
    for (int c = 0; c < 3; ++c)
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
            const uint32_t* p = &tin[c][ly * S + ky][wi];
            win[c * 3 + ky] = __funnelshift_r(p[0], p[1], bs);
        }
    // K words: byte k = win[k / 3] byte (k % 3)
    uint32_t kw[7];
    kw[0] = __byte_perm(win[0], win[1], 0x4210);  // k0..3  = w0.b0 w0.b1 w0.b2 w1.b0
    kw[1] = __byte_perm(win[1], win[2], 0x5421);  // k4..7  = w1.b1 w1.b2 w2.b0 w2.b1
    kw[2] = __byte_perm(win[2], win[3], 0x6542);  // k8..11 = w2.b2 w3.b0 w3.b1 w3.b2
    kw[3] = __byte_perm(win[4], win[5], 0x4210);
    kw[4] = __byte_perm(win[5], win[6], 0x5421);
    kw[5] = __byte_perm(win[6], win[7], 0x6542);
    kw[6] = __byte_perm(win[8], 0u, 0x4210);      // k24..26, byte 3 = 0

    // ---- 3. multiply + 4. epilogue ----
    const bool valid = ox < s.ow && oy < s.oh;
    const long oplane = (long)s.oh * s.ow;
    float* of32 = reinterpret_cast<float*>(out) + (long)img * s.cout * oplane + (long)oy * s.ow + ox;
    int8_t* os8 = reinterpret_cast<int8_t*>(out) + (((long)img * s.oh + oy) * s.ow + ox) * s.cout_pad;
#pragma unroll
    for (int g = 0; g < ST_COUT_MAX / 4; ++g) {
        if (g * 4 >= s.cout_pad) break;
        int qv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int co = g * 4 + j;
            int acc = 0;
#pragma unroll
            for (int k = 0; k < 7; ++k) acc = __dp4a((int)kw[k], (int)P.w[co][k], acc);
            const float a = __int2float_rn(acc);
            float v = has_bias ? __fmaf_rn(a, P.scale_in[co], P.bias[co]) : __fmul_rn(a, P.scale_in[co]);
            v = activate_t<ACT>(v, act_p0);
            if (OUT == DT_F32_NCHW) {
                if (valid && co < s.cout) of32[(long)co * oplane] = v;
            } else {
                qv[j] = float2int8(__fmul_rn(v, P.scale_out[co]), rounding);
            }
        }
        if (OUT == DT_S8_NHWC && valid) *reinterpret_cast<uint32_t*>(os8 + g * 4) = pack4(qv[0], qv[1], qv[2], qv[3]);
    }
}

template <int S, int OUT>
cudaError_t launch_act(cudaStream_t stream, const float* x, const StemParams& P, float in_scale, const EpilogueParams& ep, void* out,
                       const ConvShape& s) {
    const int tiles_x = (s.ow + ST_TX - 1) / ST_TX, tiles_y = (s.oh + ST_TY - 1) / ST_TY;
    const long blocks = (long)s.n * tiles_x * tiles_y;
    if (blocks == 0) return cudaSuccess;
    const dim3 grid((unsigned)blocks), block(ST_TX * ST_TY);
#define OTT_STEM_LAUNCH(ACT) \
    dense_stem_kernel<S, OUT, ACT><<<grid, block, 0, stream>>>(x, P, in_scale, ep.has_bias, ep.act_param0, ep.rounding, out, s, tiles_x, tiles_y)
    switch (ep.act_type) {
        case ACT_RELU: OTT_STEM_LAUNCH(ACT_RELU); break;
        case ACT_LRELU: OTT_STEM_LAUNCH(ACT_LRELU); break;
        case ACT_RELU6: OTT_STEM_LAUNCH(ACT_RELU6); break;
        default: OTT_STEM_LAUNCH(ACT_NONE); break;
    }
#undef OTT_STEM_LAUNCH
    return cudaGetLastError();
}

}  // namespace

bool dense_stem_supports(const ConvShape& s, int in_dtype, int out_dtype) {
    return in_dtype == DT_F32_NCHW && (out_dtype == DT_F32_NCHW || out_dtype == DT_S8_NHWC) && s.cin == 3 && s.kh == 3 && s.kw == 3 &&
           s.dh == 1 && s.dw == 1 && s.sh == s.sw && (s.sh == 1 || s.sh == 2) && s.cout_pad <= ST_COUT_MAX;
}

// Host-side parameter block: filters OIHW int8 [cout][3][3][3] and the per-channel epilogue vectors.
cudaError_t launch_dense_stem(cudaStream_t stream, const ConvShape& s, const float* x, const int8_t* w_oihw_host, const float* scale_in_host,
                              const float* bias_host, const float* scale_out_host, float in_scale, const EpilogueParams& ep, void* out,
                              int out_dtype) {
    StemParams P{};
    for (int o = 0; o < s.cout; ++o) {
        for (int k = 0; k < 27; ++k) P.w[o][k / 4] |= (uint32_t)(uint8_t)w_oihw_host[o * 27 + k] << (8 * (k % 4));
        P.scale_in[o] = scale_in_host[o];
        P.bias[o] = bias_host ? bias_host[o] : 0.f;
        P.scale_out[o] = scale_out_host ? scale_out_host[o] : 0.f;
    }
    if (s.sh == 1) {
        return out_dtype == DT_F32_NCHW ? launch_act<1, DT_F32_NCHW>(stream, x, P, in_scale, ep, out, s)
                                        : launch_act<1, DT_S8_NHWC>(stream, x, P, in_scale, ep, out, s);
    }
    return out_dtype == DT_F32_NCHW ? launch_act<2, DT_F32_NCHW>(stream, x, P, in_scale, ep, out, s)
                                    : launch_act<2, DT_S8_NHWC>(stream, x, P, in_scale, ep, out, s);
}

}  // namespace ottk
