// Depthwise int8 convolution, shared-memory tiled: depthwise_conv2d_int8_x86_pack8_out
// (Tensor/DepthwiseConvKernelInt8X86Pack.cpp:19-119) with the layer's quantize prologue
// (Tensor/QuantizeX86.cpp:396-549) and requantize/dequantize epilogue (Tensor/QuantizeX86.cpp:1723-1870,
// :851-903) fused into one pass over HBM.
//
// One CTA = one image x 32 channels x a band of TY output rows x TXO output columns.
//  1. load: the input halo tile goes to shared memory as int8 *channel planes* (pixels of one channel are
//     consecutive bytes). From fp32 NCHW it is quantized on the way (float4 loads along W); from int8 NHWC
//     the 16-byte channel vectors of 4 neighbouring pixels are transposed in registers (4x4 byte transposes).
//  2. compute: thread = (channel = lane, 4 consecutive output columns). Because pixels are consecutive
//     bytes, one 32-bit window holds 4 horizontal taps of one channel and a dp4a against the packed filter
//     row does 4 multiply-adds; the windows of the last K input rows stay in a register ring while the
//     thread walks down the band. Sums are exact s32.
//  3. epilogue in registers (epilogue.cuh). int8 results are packed 4 pixels to a word into shared-memory
//     channel planes, transposed back to channel-innermost 16-byte vectors and stored along the NHWC
//     channel axis; fp32 NCHW results are stored directly.
//
// This header holds the kernel template; depthwise_tiled_k*s*.cu instantiate it per (kernel size, stride)
// so the variants compile in parallel.
#pragma once

#include <mutex>

#include "launch.cuh"
#include "store.cuh"

namespace ottk {
namespace dwt {

constexpr int CG = 32;  // channels per CTA (one warp's lanes)
constexpr int THREADS = 256;
enum : int { EPI_S8 = 0, EPI_S8_HALF_AWAY = 1, EPI_F32 = 2 };

struct Tile {
    int ty, txo;      // output rows / columns per CTA (txo % 4 == 0)
    int ir, rp, ps;   // input tile: rows, row pitch and plane stride in 32-bit words (ps odd)
    int orp, ops;     // output staging planes: row pitch (= txo/4) and plane stride in words (ops odd)
    int tiles_y, tiles_x, cgroups;
    int threads;      // CTA size: one warp per group of 4 output columns, at most 8 warps
};

template <int K, int S>
struct Geo {
    static constexpr int KK = (K + 3) / 4;               // packed filter words per filter row
    static constexpr int NW = (3 * S + 4 * KK + 3) / 4;  // aligned words a thread needs per input row
};

// Windows of one input row for the thread's 4 outputs: dstw[t][kk] = bytes [t*S + 4*kk, +4) counted from the
// first input column of output 0. `sh` (0..3) is the byte offset of that column inside its aligned word.
template <int K, int S>
__device__ __forceinline__ void load_row_windows(const uint32_t* __restrict__ p, int sh8, uint32_t dstw[4][Geo<K, S>::KK]) {
    constexpr int KK = Geo<K, S>::KK, NW = Geo<K, S>::NW;
    uint32_t raw[NW + 1], al[NW];
#pragma unroll
    for (int i = 0; i < NW + 1; ++i) raw[i] = p[i];
#pragma unroll
    for (int i = 0; i < NW; ++i) al[i] = __funnelshift_r(raw[i], raw[i + 1], sh8);
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int kk = 0; kk < KK; ++kk) {
            const int bo = t * S + 4 * kk;  // compile-time after unrolling
            const int wi = bo >> 2, bs = (bo & 3) * 8;
            dstw[t][kk] = bs == 0 ? al[wi] : __funnelshift_r(al[wi], wi + 1 < NW ? al[wi + 1] : 0u, bs);
        }
}

template <int EPI, int ACT>
__device__ __forceinline__ int epi_s8(int acc, float si, float bi, float so, int has_bias, float p0) {
    const float a = __int2float_rn(acc);
    float v = has_bias ? __fmaf_rn(a, si, bi) : __fmul_rn(a, si);
    v = activate_t<ACT>(v, p0);
    const float t = __fmul_rn(v, so);
    if (EPI == EPI_S8_HALF_AWAY) return float2int8(t, ROUND_HALF_AWAY);
    if (ACT == ACT_RELU || ACT == ACT_RELU6) return f2i8_nonneg(t);
    return f2i8_lo_clamped(t);
}

// Four accumulators of one channel -> four int8 in one word, the arithmetic as packed pairs (each lane rounds like epi_s8).
template <int EPI, int ACT>
__device__ __forceinline__ uint32_t epi_s8x4(const int (&acc)[4], float si, float bi, float so, int has_bias, float p0) {
    if (EPI == EPI_S8_HALF_AWAY)
        return pack_sat_s8x4(epi_s8<EPI, ACT>(acc[0], si, bi, so, has_bias, p0), epi_s8<EPI, ACT>(acc[1], si, bi, so, has_bias, p0),
                             epi_s8<EPI, ACT>(acc[2], si, bi, so, has_bias, p0), epi_s8<EPI, ACT>(acc[3], si, bi, so, has_bias, p0));
    const float2 s2 = make_float2(si, si), b2 = make_float2(bi, bi), o2 = make_float2(so, so);
    int q[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float2 a = make_float2(__int2float_rn(acc[2 * h]), __int2float_rn(acc[2 * h + 1]));
        const float2 v = has_bias ? __ffma2_rn(a, s2, b2) : __fmul2_rn(a, s2);
        const float2 t = __fmul2_rn(make_float2(activate_t<ACT>(v.x, p0), activate_t<ACT>(v.y, p0)), o2);
        if (ACT == ACT_RELU || ACT == ACT_RELU6) {
            const float2 r = __fadd2_rn(t, make_float2(0.5f, 0.5f));
            q[2 * h] = __float2int_rz(r.x);
            q[2 * h + 1] = __float2int_rz(r.y);
        } else {
            const float2 r = __fadd2_rn(t, make_float2(half_signed(t.x), half_signed(t.y)));
            q[2 * h] = __float2int_rz(fmaxf(r.x, -127.5f));
            q[2 * h + 1] = __float2int_rz(fmaxf(r.y, -127.5f));
        }
    }
    return pack_sat_s8x4(q[0], q[1], q[2], q[3]);
}

// One output row for the thread. R = (output row index) % K selects, at compile time, which ring slots hold
// the K input rows: input row r lives in slot r % K, and output row oy needs rows oy*S + ky.
template <int K, int S, int EPI, int ACT, int R>
__device__ __forceinline__ void row_step(int oy, const uint32_t* __restrict__ plane, const Tile& T, int xq, int sh8,
                                         uint32_t (&win)[K][4][Geo<K, S>::KK], const uint32_t (&wk)[K][Geo<K, S>::KK],
                                         float si, float bi, float so, const EpilogueParams& ep, uint32_t* __restrict__ oplane_s,
                                         float* __restrict__ of32, int ow_left) {
    constexpr int KK = Geo<K, S>::KK;
    constexpr int base = (R * S) % K;
    // the S rows this output row needs beyond those of the previous one
#pragma unroll
    for (int ky = K - S; ky < K; ++ky) load_row_windows<K, S>(plane + (oy * S + ky) * T.rp + xq * S, sh8, win[(base + ky) % K]);
    int acc[4] = {0, 0, 0, 0};
#pragma unroll
    for (int ky = 0; ky < K; ++ky)
#pragma unroll
        for (int kk = 0; kk < KK; ++kk)
#pragma unroll
            for (int t = 0; t < 4; ++t) acc[t] = __dp4a((int)win[(base + ky) % K][t][kk], (int)wk[ky][kk], acc[t]);
    if (EPI != EPI_F32) {
        oplane_s[oy * T.orp + xq] = epi_s8x4<EPI, ACT>(acc, si, bi, so, ep.has_bias, ep.act_param0);
    } else if (of32) {
        float v[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const float a = __int2float_rn(acc[t]);
            v[t] = activate_t<ACT>(ep.has_bias ? __fmaf_rn(a, si, bi) : __fmul_rn(a, si), ep.act_param0);
        }
        if (ow_left >= 4 && (reinterpret_cast<uintptr_t>(of32) & 15) == 0) {
            *reinterpret_cast<float4*>(of32) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
            for (int t = 0; t < 4; ++t)
                if (t < ow_left) of32[t] = v[t];
        }
    }
}

template <int K, int S, bool IN_F32, int EPI, int ACT>
__global__ void __launch_bounds__(THREADS)
depthwise_tiled_kernel(const void* __restrict__ xin, const __grid_constant__ PlaneGather G, const uint32_t* __restrict__ wq,
                       const float* __restrict__ in_scales, int n_in_scales, EpilogueParams ep, void* __restrict__ out, ConvShape s, Tile T) {
    constexpr int KK = Geo<K, S>::KK;
    extern __shared__ uint32_t smem[];
    pdl_launch_dependents();
    pdl_wait();
    uint32_t* tin = smem;                  // [32][ir][rp] (+pad): int8 channel planes of the input tile
    uint32_t* tout = smem + CG * T.ps;     // [32][ty][orp] (+pad): int8 channel planes of the output tile

    int b = blockIdx.x;
    const int cg = b % T.cgroups; b /= T.cgroups;
    const int tx = b % T.tiles_x; b /= T.tiles_x;
    const int tyi = b % T.tiles_y;
    const int img = b / T.tiles_y;
    const int c0 = cg * CG;
    const int oy0 = tyi * T.ty, ox0 = tx * T.txo;
    const int iy0 = oy0 * S - s.ph;
    const int ix_first = ox0 * S - s.pw;                                   // first input column the tile needs
    const int ix_al = (ix_first >= 0 ? ix_first : ix_first - 3) / 4 * 4;   // rounded down to a multiple of 4
    const int sh8 = (ix_first - ix_al) * 8;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // ---- 1. load the input tile ----
    if (IN_F32) {
        // warp = channel (4 per warp), lanes run over the (row, word) positions of the channel's plane
        const bool vec_ok = (s.w % 4 == 0) && ep.rounding == ROUND_ADD_HALF_TRUNC;
        const int per_plane = T.ir * T.rp;
        const float inv_rp = 1.0f / (float)T.rp;
        for (int cl = warp; cl < CG; cl += (int)blockDim.x / 32) {
            const int c = c0 + cl;
            uint32_t* dst = tin + cl * T.ps;
            if (c >= s.cin) {
                for (int i = lane; i < per_plane; i += 32) dst[i] = 0u;
                continue;
            }
            const float sc = n_in_scales == 1 ? __ldg(in_scales) : __ldg(in_scales + c);
            const float* xc = G.plane(c, img, (long)s.h * s.w);
            if (vec_ok) {
                // every aligned float4 is either wholly inside the image or wholly outside (w % 4 == 0, ix % 4 == 0);
                // four independent loads per thread are issued before any is used
                for (int i0 = lane; i0 < per_plane; i0 += 128) {
                    float4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int i = i0 + 32 * u;
                        const int r = (int)(((float)i + 0.5f) * inv_rp);
                        const int xw = i - r * T.rp;
                        const int iy = iy0 + r, ix = ix_al + xw * 4;
                        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (i < per_plane && iy >= 0 && iy < s.h && ix >= 0 && ix < s.w)
                            v[u] = __ldg(reinterpret_cast<const float4*>(xc + (long)iy * s.w + ix));
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int i = i0 + 32 * u;
                        if (i < per_plane) dst[i] = quantize4_pack(v[u].x, v[u].y, v[u].z, v[u].w, sc);
                    }
                }
            } else {
                int r = lane / T.rp, xw = lane - r * T.rp;
                for (int i = lane; i < per_plane; i += 32) {
                    const int iy = iy0 + r, ix = ix_al + xw * 4;
                    uint32_t word = 0;
                    if (iy >= 0 && iy < s.h && ix + 3 >= 0 && ix < s.w) {
                        const float* row = xc + (long)iy * s.w;
                        int q[4] = {0, 0, 0, 0};
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (ix + j >= 0 && ix + j < s.w) q[j] = quantize1(__ldg(row + ix + j), sc, ep.rounding);
                        word = pack4(q[0], q[1], q[2], q[3]);
                    }
                    dst[i] = word;
                    xw += 32;
                    while (xw >= T.rp) { xw -= T.rp; ++r; }
                }
            }
        }
    } else {
        // Each 16-channel group is read from one tensor: the layer's own input, or (a layer created with gathered input)
        // 16 channels of one of several source tensors, named by the table: ref = (tensor << 24) | first channel, and
        // img_stride[tensor] = that tensor's channel stride.
        const int half = threadIdx.x & 1;  // blockDim.x is even: a thread stays on its half
        const int c = c0 + half * 16;
        const int8_t* x = static_cast<const int8_t*>(xin) + (long)img * s.h * s.w * s.cin_pad + c;
        long pitch = s.cin_pad;
        if (G.base[0] != nullptr && c < s.cin_pad) {
            const uint32_t ref = G.ref[c >> 4];
            pitch = (long)G.img_stride[ref >> 24];
            x = reinterpret_cast<const int8_t*>(G.base[ref >> 24]) + (long)img * s.h * s.w * pitch + (ref & 0xFFFFFFu);
        }
        const int items = T.ir * T.rp * 2;  // (pixel quad, 16-channel half)
        for (int i = threadIdx.x; i < items; i += (int)blockDim.x) {
            const int xw = (i >> 1) % T.rp;
            const int r = (i >> 1) / T.rp;
            const int iy = iy0 + r, ix = ix_al + xw * 4;
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[j] = make_uint4(0, 0, 0, 0);
                if (c < s.cin_pad && iy >= 0 && iy < s.h && ix + j >= 0 && ix + j < s.w)
                    v[j] = __ldg(reinterpret_cast<const uint4*>(x + ((long)iy * s.w + ix + j) * pitch));
            }
            uint32_t* dst = tin + (half * 16) * T.ps + r * T.rp + xw;
            uint32_t o[4];
            transpose4x4(v[0].x, v[1].x, v[2].x, v[3].x, o);
#pragma unroll
            for (int k = 0; k < 4; ++k) dst[(0 + k) * T.ps] = o[k];
            transpose4x4(v[0].y, v[1].y, v[2].y, v[3].y, o);
#pragma unroll
            for (int k = 0; k < 4; ++k) dst[(4 + k) * T.ps] = o[k];
            transpose4x4(v[0].z, v[1].z, v[2].z, v[3].z, o);
#pragma unroll
            for (int k = 0; k < 4; ++k) dst[(8 + k) * T.ps] = o[k];
            transpose4x4(v[0].w, v[1].w, v[2].w, v[3].w, o);
#pragma unroll
            for (int k = 0; k < 4; ++k) dst[(12 + k) * T.ps] = o[k];
        }
    }
    __syncthreads();

    // ---- 2. compute + 3. epilogue ----
    const int c = c0 + lane;
    const bool c_ok = c < s.cout_pad;
    uint32_t wk[K][KK];
#pragma unroll
    for (int ky = 0; ky < K; ++ky)
#pragma unroll
        for (int kk = 0; kk < KK; ++kk) wk[ky][kk] = c_ok ? __ldg(wq + ((long)c * K + ky) * KK + kk) : 0u;
    const float p_si = c_ok ? __ldg(ep.scale_in + c) : 0.f;
    const float p_bi = c_ok ? __ldg(ep.bias + c) : 0.f;
    const float p_so = c_ok ? __ldg(ep.scale_out + c) : 0.f;
    const uint32_t* plane = tin + lane * T.ps;
    uint32_t* oplane_s = tout + lane * T.ops;
    const int rows_out = min(T.ty, s.oh - oy0);
    const long oplane = (long)s.oh * s.ow;

    for (int xq = warp; xq < T.txo / 4; xq += (int)blockDim.x / 32) {
        const int ox = ox0 + xq * 4;
        if (ox >= s.ow) break;
        uint32_t win[K][4][KK];
        // prime the ring with the first K-S input rows (slot = row % K)
#pragma unroll
        for (int r = 0; r < K - S; ++r) load_row_windows<K, S>(plane + r * T.rp + xq * S, sh8, win[r % K]);
        float* of32 = nullptr;
        if (EPI == EPI_F32 && c < s.cout)
            of32 = reinterpret_cast<float*>(out) + ((long)img * s.cout + c) * oplane + (long)oy0 * s.ow + ox;
        const int ow_left = s.ow - ox;
#define OTT_DW_STEP(R)                                                                                                  \
    if (oy + R < rows_out)                                                                                              \
        row_step<K, S, EPI, ACT, R>(oy + R, plane, T, xq, sh8, win, wk, p_si, p_bi, p_so, ep, oplane_s,                  \
                                    of32 ? of32 + (long)(oy + R) * s.ow : nullptr, ow_left);
        for (int oy = 0; oy < rows_out; oy += K) {
            OTT_DW_STEP(0) OTT_DW_STEP(1) OTT_DW_STEP(2)
            if (K > 3) { OTT_DW_STEP(3) OTT_DW_STEP(4) }
        }
#undef OTT_DW_STEP
    }
    if (EPI != EPI_F32) {
        __syncthreads();
        // planes -> channel-innermost: a thread takes 4 pixels x 16 channels (16 words), transposes, stores 4 x 16 B
        int8_t* o = reinterpret_cast<int8_t*>(out);
        const int items = rows_out * T.orp * 2;
        for (int i = threadIdx.x; i < items; i += (int)blockDim.x) {
            const int half = i & 1;
            const int xq = (i >> 1) % T.orp, oy = (i >> 1) / T.orp;
            const int cc = c0 + half * 16;
            const int ox = ox0 + xq * 4;
            if (ox >= s.ow || cc >= s.cout_pad) continue;
            const uint32_t* src = tout + (half * 16) * T.ops + oy * T.orp + xq;
            uint32_t px[4][4];  // [pixel][word of 4 channels]
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t t4[4];
                transpose4x4(src[(g * 4 + 0) * T.ops], src[(g * 4 + 1) * T.ops], src[(g * 4 + 2) * T.ops], src[(g * 4 + 3) * T.ops], t4);
#pragma unroll
                for (int j = 0; j < 4; ++j) px[j][g] = t4[j];
            }
            int8_t* dst = o + (((long)img * s.oh + oy0 + oy) * s.ow + ox) * s.cout_pad + cc;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (ox + j < s.ow) *reinterpret_cast<uint4*>(dst + (long)j * s.cout_pad) = make_uint4(px[j][0], px[j][1], px[j][2], px[j][3]);
        }
    }
}

template <int K, int S>
inline Tile plan_tile(const ConvShape& s) {
    constexpr int NW = Geo<K, S>::NW;
    Tile T{};
    const int ow4 = (s.ow + 3) / 4 * 4;
    T.txo = S == 1 ? (ow4 < 64 ? ow4 : 64) : (ow4 < 32 ? ow4 : 32);
    const int ty_max = S == 1 ? (K == 3 ? 14 : 12) : (K == 3 ? 7 : 6);
    // bands of equal height (20 rows -> 10 + 10, not 14 + 6), so no CTA is mostly idle
    const int bands = (s.oh + ty_max - 1) / ty_max;
    T.ty = (s.oh + bands - 1) / bands;
    T.ir = (T.ty - 1) * S + K;
    T.rp = (T.txo / 4 - 1) * S + NW + 1 + 1;  // +1 realignment word, +1 because the tile origin is rounded down
    T.ps = T.ir * T.rp;
    if (T.ps % 2 == 0) T.ps += 1;
    T.orp = T.txo / 4;
    T.ops = T.ty * T.orp;
    if (T.ops % 2 == 0) T.ops += 1;
    T.tiles_y = (s.oh + T.ty - 1) / T.ty;
    T.tiles_x = (s.ow + T.txo - 1) / T.txo;
    T.cgroups = (s.cout_pad + CG - 1) / CG;
    const int nxq = T.txo / 4;
    T.threads = 32 * (nxq < 8 ? nxq : 8);
    return T;
}

template <int K, int S, bool IN_F32, int EPI, int ACT>
cudaError_t launch_t(cudaStream_t stream, const ConvShape& s, const void* x, const PlaneGather& G, const uint32_t* wq, const float* in_scales,
                     int n_in_scales, const EpilogueParams& ep, void* out) {
    const Tile T = plan_tile<K, S>(s);
    const size_t smem = ((size_t)CG * T.ps + (EPI != EPI_F32 ? (size_t)CG * T.ops : 0)) * 4;
    auto kernel = depthwise_tiled_kernel<K, S, IN_F32, EPI, ACT>;
    static std::mutex mu;  // several host threads may drive different GPUs through this function at once
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64) {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set[dev]) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            if (e != cudaSuccess) return e;
            attr_set[dev] = true;
        }
    }
    const long blocks = (long)s.n * T.tiles_y * T.tiles_x * T.cgroups;
    if (blocks == 0) return cudaSuccess;
    return launch_overlapped(kernel, dim3((unsigned)blocks), dim3(T.threads), smem, stream, x, G, wq, in_scales, n_in_scales, ep, out, s, T);
}

template <int K, int S, bool IN_F32, int EPI>
cudaError_t launch_act(cudaStream_t stream, const ConvShape& s, const void* x, const PlaneGather& G, const uint32_t* wq, const float* in_scales,
                       int n_in_scales, const EpilogueParams& ep, void* out) {
    switch (ep.act_type) {
        case ACT_RELU: return launch_t<K, S, IN_F32, EPI, ACT_RELU>(stream, s, x, G, wq, in_scales, n_in_scales, ep, out);
        case ACT_LRELU: return launch_t<K, S, IN_F32, EPI, ACT_LRELU>(stream, s, x, G, wq, in_scales, n_in_scales, ep, out);
        case ACT_RELU6: return launch_t<K, S, IN_F32, EPI, ACT_RELU6>(stream, s, x, G, wq, in_scales, n_in_scales, ep, out);
        default: return launch_t<K, S, IN_F32, EPI, ACT_NONE>(stream, s, x, G, wq, in_scales, n_in_scales, ep, out);
    }
}

template <int K, int S>
cudaError_t launch_ks(cudaStream_t stream, const ConvShape& s, const void* x, const PlaneGather& G, int in_dtype, const uint32_t* wq,
                      const float* in_scales, int n_in_scales, const EpilogueParams& ep, void* out, int out_dtype) {
    const bool f32in = in_dtype == DT_F32_NCHW;
    if (out_dtype == DT_F32_NCHW)
        return f32in ? launch_act<K, S, true, EPI_F32>(stream, s, x, G, wq, in_scales, n_in_scales, ep, out)
                     : launch_act<K, S, false, EPI_F32>(stream, s, x, G, wq, in_scales, n_in_scales, ep, out);
    if (ep.rounding == ROUND_HALF_AWAY)
        return f32in ? launch_act<K, S, true, EPI_S8_HALF_AWAY>(stream, s, x, G, wq, in_scales, n_in_scales, ep, out)
                     : launch_act<K, S, false, EPI_S8_HALF_AWAY>(stream, s, x, G, wq, in_scales, n_in_scales, ep, out);
    return f32in ? launch_act<K, S, true, EPI_S8>(stream, s, x, G, wq, in_scales, n_in_scales, ep, out)
                 : launch_act<K, S, false, EPI_S8>(stream, s, x, G, wq, in_scales, n_in_scales, ep, out);
}

}  // namespace dwt

// defined one per file (depthwise_tiled_k3s1.cu ...)
cudaError_t launch_depthwise_tiled_k3s1(cudaStream_t, const ConvShape&, const void*, const PlaneGather&, int, const uint32_t*, const float*, int, const EpilogueParams&, void*, int);
cudaError_t launch_depthwise_tiled_k3s2(cudaStream_t, const ConvShape&, const void*, const PlaneGather&, int, const uint32_t*, const float*, int, const EpilogueParams&, void*, int);
cudaError_t launch_depthwise_tiled_k5s1(cudaStream_t, const ConvShape&, const void*, const PlaneGather&, int, const uint32_t*, const float*, int, const EpilogueParams&, void*, int);
cudaError_t launch_depthwise_tiled_k5s2(cudaStream_t, const ConvShape&, const void*, const PlaneGather&, int, const uint32_t*, const float*, int, const EpilogueParams&, void*, int);

}  // namespace ottk
