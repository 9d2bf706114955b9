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

// ---- stem convolution followed by a 3x3 stride-2 pad-1 max-pool, in one kernel ----
// The pool is the only consumer of the first layer's output in the benchmark graphs (conv1 -> pool1), and that output is
// the largest tensor of the whole network; here it never leaves the SM. One CTA produces a 16x7 tile of POOLED pixels for
// all channels: it computes the 33x15 convolution outputs under that tile into shared memory (fp32, after the
// dequantize epilogue and activation, exactly the values the separate layer would have stored) and max-reduces them.
// pad_zero selects the reference's packed max-pool rule (padding counts as 0, Tensor/Pool.cpp:972-975) or its plain
// rule (padding never wins).
constexpr int SP_PX = 16, SP_PY = 7;                       // pooled tile: 33x15 = 495 convolution outputs ~ 2 x 256 threads
constexpr int SP_CX = 2 * SP_PX + 1, SP_CY = 2 * SP_PY + 1;  // convolution outputs under it

template <int S, int ACT, int NCO>
__global__ void __launch_bounds__(256)
dense_stem_pool_kernel(const float* __restrict__ x, const __grid_constant__ StemParams P, float in_scale, int has_bias, float act_p0,
                       int rounding, float* __restrict__ out, ConvShape s, int ph_out, int pw_out, int tiles_x, int tiles_y, int pad_zero) {
    constexpr int IW = (SP_CX - 1) * S + 3, IH = (SP_CY - 1) * S + 3;
    constexpr int RP = (IW + 3 + 3) / 4 + 1;
    extern __shared__ uint32_t smem_sp[];
    uint32_t(*tin)[IH][RP] = reinterpret_cast<uint32_t(*)[IH][RP]>(smem_sp);  // [3][IH][RP]
    float* conv = reinterpret_cast<float*>(smem_sp + 3 * IH * RP);            // [cout][SP_CY][SP_CX]

    int b = blockIdx.x;
    const int tx = b % tiles_x; b /= tiles_x;
    const int ty = b % tiles_y;
    const int img = b / tiles_y;
    const int px0 = tx * SP_PX, py0 = ty * SP_PY;     // first pooled pixel of the tile
    const int cx0 = px0 * 2 - 1, cy0 = py0 * 2 - 1;   // first convolution output under it (pool pad 1)
    const int iy0 = cy0 * S - s.ph, ix_first = cx0 * S - s.pw;
    const int ix_al = (ix_first >= 0 ? ix_first : ix_first - 3) / 4 * 4;
    const int sh = ix_first - ix_al;

    const float* ximg = x + (long)img * 3 * s.h * s.w;
    const bool vec_ok = (s.w % 4 == 0) && rounding == ROUND_ADD_HALF_TRUNC;
    for (int i = threadIdx.x; i < 3 * IH * RP; i += 256) {
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

    const float outside = pad_zero ? 0.f : -INFINITY;
    for (int p = threadIdx.x; p < SP_CX * SP_CY; p += 256) {
        const int lx = p % SP_CX, ly = p / SP_CX;
        const int ox = cx0 + lx, oy = cy0 + ly;
        const bool inside = ox >= 0 && ox < s.ow && oy >= 0 && oy < s.oh;
        const int boff = sh + lx * S;
        const int wi = boff >> 2, bs = (boff & 3) * 8;
        uint32_t win[9];
#pragma unroll
        for (int c = 0; c < 3; ++c)
#pragma unroll
            for (int ky = 0; ky < 3; ++ky) {
                const uint32_t* q = &tin[c][ly * S + ky][wi];
                win[c * 3 + ky] = __funnelshift_r(q[0], q[1], bs);
            }
        uint32_t kw[7];
        kw[0] = __byte_perm(win[0], win[1], 0x4210);
        kw[1] = __byte_perm(win[1], win[2], 0x5421);
        kw[2] = __byte_perm(win[2], win[3], 0x6542);
        kw[3] = __byte_perm(win[4], win[5], 0x4210);
        kw[4] = __byte_perm(win[5], win[6], 0x5421);
        kw[5] = __byte_perm(win[6], win[7], 0x6542);
        kw[6] = __byte_perm(win[8], 0u, 0x4210);
        // NCO (the channel count rounded up to 8) is a template parameter so that the channel loop unrolls completely:
        // four independent accumulator chains at a time, weights as immediate constant-bank operands
#pragma unroll
        for (int g = 0; g < NCO / 4; ++g) {
            int acc[4] = {0, 0, 0, 0};
#pragma unroll
            for (int k = 0; k < 7; ++k)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j] = __dp4a((int)kw[k], (int)P.w[g * 4 + j][k], acc[j]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int co = g * 4 + j;
                const float a = __int2float_rn(acc[j]);
                float v = has_bias ? __fmaf_rn(a, P.scale_in[co], P.bias[co]) : __fmul_rn(a, P.scale_in[co]);
                v = activate_t<ACT>(v, act_p0);
                if (co < s.cout) conv[(co * SP_CY + ly) * SP_CX + lx] = inside ? v : outside;
            }
        }
    }
    __syncthreads();

    const long pplane = (long)ph_out * pw_out;
    for (int i = threadIdx.x; i < s.cout * SP_PY * SP_PX; i += 256) {
        const int lx = i % SP_PX, ly = (i / SP_PX) % SP_PY, co = i / (SP_PX * SP_PY);
        const int px = px0 + lx, py = py0 + ly;
        if (px >= pw_out || py >= ph_out) continue;
        const float* cp = conv + (co * SP_CY + 2 * ly) * SP_CX + 2 * lx;
        float m = cp[0];
#pragma unroll
        for (int dy = 0; dy < 3; ++dy)
#pragma unroll
            for (int dx = 0; dx < 3; ++dx) m = fmaxf(m, cp[dy * SP_CX + dx]);
        out[((long)img * s.cout + co) * pplane + (long)py * pw_out + px] = m;
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

static void fill_stem_params(StemParams& P, const ConvShape& s, const int8_t* w, const float* scale_in, const float* bias, const float* scale_out) {
    for (int o = 0; o < s.cout; ++o) {
        for (int k = 0; k < 27; ++k) P.w[o][k / 4] |= (uint32_t)(uint8_t)w[o * 27 + k] << (8 * (k % 4));
        P.scale_in[o] = scale_in[o];
        P.bias[o] = bias ? bias[o] : 0.f;
        P.scale_out[o] = scale_out ? scale_out[o] : 0.f;
    }
}

template <int S>
static cudaError_t launch_pool_s(cudaStream_t stream, const float* x, const StemParams& P, float in_scale, const EpilogueParams& ep, float* out,
                                 const ConvShape& s, int pad_zero) {
    const int ph_out = (s.oh + 2 - 3) / 2 + 1, pw_out = (s.ow + 2 - 3) / 2 + 1;
    const int tiles_x = (pw_out + SP_PX - 1) / SP_PX, tiles_y = (ph_out + SP_PY - 1) / SP_PY;
    const long blocks = (long)s.n * tiles_x * tiles_y;
    if (blocks <= 0) return cudaSuccess;
    constexpr int IW = (SP_CX - 1) * S + 3, IH = (SP_CY - 1) * S + 3, RP = (IW + 3 + 3) / 4 + 1;
    const size_t smem = (size_t)3 * IH * RP * 4 + (size_t)s.cout * SP_CY * SP_CX * 4;
    const int nco = (s.cout + 7) / 8 * 8;
#define OTT_STEMPOOL_LAUNCH(ACT)                                                                                          \
    {                                                                                                                     \
        auto kernel = nco <= 8 ? dense_stem_pool_kernel<S, ACT, 8> : nco <= 16 ? dense_stem_pool_kernel<S, ACT, 16>      \
                      : nco <= 24 ? dense_stem_pool_kernel<S, ACT, 24> : dense_stem_pool_kernel<S, ACT, 32>;              \
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);            \
        if (e != cudaSuccess) return e;                                                                                   \
        kernel<<<(unsigned)blocks, 256, smem, stream>>>(x, P, in_scale, ep.has_bias, ep.act_param0, ep.rounding, out, s, ph_out, pw_out,  \
                                                        tiles_x, tiles_y, pad_zero);                                      \
    }
    switch (ep.act_type) {
        case ACT_RELU: OTT_STEMPOOL_LAUNCH(ACT_RELU) break;
        case ACT_LRELU: OTT_STEMPOOL_LAUNCH(ACT_LRELU) break;
        case ACT_RELU6: OTT_STEMPOOL_LAUNCH(ACT_RELU6) break;
        default: OTT_STEMPOOL_LAUNCH(ACT_NONE) break;
    }
#undef OTT_STEMPOOL_LAUNCH
    return cudaGetLastError();
}

// first layer (fp32 output) + MaxPool 3x3 s2 p1 of its result; out is [n][cout][(oh+1)/2... pooled] fp32 NCHW
cudaError_t launch_dense_stem_pool(cudaStream_t stream, const ConvShape& s, const float* x, const int8_t* w_oihw_host, const float* scale_in_host,
                                   const float* bias_host, float in_scale, const EpilogueParams& ep, float* out, int pad_zero) {
    StemParams P{};
    fill_stem_params(P, s, w_oihw_host, scale_in_host, bias_host, nullptr);
    return s.sh == 1 ? launch_pool_s<1>(stream, x, P, in_scale, ep, out, s, pad_zero) : launch_pool_s<2>(stream, x, P, in_scale, ep, out, s, pad_zero);
}

// Host-side parameter block: filters OIHW int8 [cout][3][3][3] and the per-channel epilogue vectors.
cudaError_t launch_dense_stem(cudaStream_t stream, const ConvShape& s, const float* x, const int8_t* w_oihw_host, const float* scale_in_host,
                              const float* bias_host, const float* scale_out_host, float in_scale, const EpilogueParams& ep, void* out,
                              int out_dtype) {
    StemParams P{};
    fill_stem_params(P, s, w_oihw_host, scale_in_host, bias_host, scale_out_host);
    if (s.sh == 1) {
        return out_dtype == DT_F32_NCHW ? launch_act<1, DT_F32_NCHW>(stream, x, P, in_scale, ep, out, s)
                                        : launch_act<1, DT_S8_NHWC>(stream, x, P, in_scale, ep, out, s);
    }
    return out_dtype == DT_F32_NCHW ? launch_act<2, DT_F32_NCHW>(stream, x, P, in_scale, ep, out, s)
                                    : launch_act<2, DT_S8_NHWC>(stream, x, P, in_scale, ep, out, s);
}

}  // namespace ottk
