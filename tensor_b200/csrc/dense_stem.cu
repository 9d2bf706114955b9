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
#include "launch.cuh"
#include "store.cuh"
#include "umma_primitives.cuh"

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

// The multiply-adds run on the tensor cores: the 27 taps of a convolution pixel, gathered into 7 registers with funnel shifts
// and byte permutes exactly as in the kernel above, are written out as one 32-byte row of an im2col tile in shared memory,
// and four tcgen05 MMAs (M = 128 pixels, N = 32 channels, K = 32) produce the exact s32 accumulators of the CTA's 495
// convolution pixels in TMEM. (A dp4a version of this kernel was measured first: 0.333 ms for 256 images of 320x320 against
// 0.323 ms here; both are bound by the instruction count of the quantize, epilogue and pooling phases, not by the
// multiply-adds.) One CTA = one pooled tile, no pipeline: build, fence, issue, wait (bounded), read, pool.
// Shared memory per CTA is above a third of the SM's, so at most three CTAs (3 x 128 TMEM columns) are ever resident.
constexpr int SPM_ROWS = 512;                 // im2col rows: 495 convolution pixels rounded up to 4 MMA tiles
constexpr uint32_t SPM_TMEM_COLS = 128;       // 4 accumulators of 32 columns

// OUT8: the pooled values leave quantized, float2int8(v * scale_out[channel]), as an int8 NHWC tensor (what the quantize pass of
// the layers reading the pooled blob would compute from the fp32 values) instead of fp32 NCHW planes.
// C24: the instance for the usual first layer (24 output channels, a bias, the add-half-truncate rounding rule): channel-group
// counts, the accumulator tile's pitch, the bias switch and the rounding rule are compile-time constants there, so the
// channel loops unroll and their addresses are immediates (a fifth fewer instructions in a kernel bound by instruction issue).
template <int S, int ACT, bool OUT8, bool C24>
__global__ void __launch_bounds__(256)
dense_stem_pool_mma_kernel(const float* __restrict__ x, const __grid_constant__ StemParams P, float in_scale, int has_bias_arg, float act_p0,
                           int rounding_arg, void* __restrict__ out_any, ConvShape s_arg, int ph_out, int pw_out, int tiles_x, int tiles_y, int pad_zero,
                           uint32_t* __restrict__ status) {
    using namespace umma;
    const int has_bias = C24 ? 1 : has_bias_arg;
    const int rounding = C24 ? (int)ROUND_ADD_HALF_TRUNC : rounding_arg;
    ConvShape s = s_arg;
    if (C24) { s.cout = 24; s.cout_pad = 32; }
    constexpr int IW = (SP_CX - 1) * S + 3, IH = (SP_CY - 1) * S + 3;
    constexpr int RP = (IW + 3 + 3) / 4 + 1;
    extern __shared__ uint8_t smem_spm[];
    const uint32_t base = (smem_u32(smem_spm) + 1023u) & ~1023u;
    uint8_t* bp = smem_spm + (base - smem_u32(smem_spm));
    uint8_t* sA = bp;                                   // [512 rows][32 B], 32-byte swizzle
    uint8_t* sB = bp + SPM_ROWS * 32;                   // [32 output channels][32 B]
    uint32_t(*tin)[IH][RP] = reinterpret_cast<uint32_t(*)[IH][RP]>(bp + SPM_ROWS * 32 + 1024);  // [3][IH][RP]
    // The s32 accumulators of the convolution tile, [pixel][pitch]: written once the MMAs have completed, over the im2col
    // rows, the filter rows and the input planes, which are all dead by then.
    int* cacc = reinterpret_cast<int*>(bp);
    const int cout4 = (s.cout + 3) >> 2;   // 4-channel groups
    const int pitch = cout4 * 4 + 4;       // s32 per pixel row: 4 mod 8 words, so the 16-byte accesses of both phases spread over the banks
    __shared__ __align__(16) float sprm[3][ST_COUT_MAX];  // scale_in, bias, scale_out
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const uint32_t bar = smem_u32(&bar_storage);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    int b = blockIdx.x;
    const int tx = b % tiles_x; b /= tiles_x;
    const int ty = b % tiles_y;
    const int img = b / tiles_y;
    const int px0 = tx * SP_PX, py0 = ty * SP_PY;     // first pooled pixel of the tile
    const int cx0 = px0 * 2 - 1, cy0 = py0 * 2 - 1;   // first convolution output under it (pool pad 1)
    const int iy0 = cy0 * S - s.ph, ix_first = cx0 * S - s.pw;
    const int ix_al = (ix_first >= 0 ? ix_first : ix_first - 3) / 4 * 4;
    const int sh = ix_first - ix_al;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x >= 64 && threadIdx.x < 64 + ST_COUT_MAX) {
        const int o = threadIdx.x - 64;
        sprm[0][o] = P.scale_in[o];
        sprm[1][o] = P.bias[o];
        sprm[2][o] = P.scale_out[o];
    }
    if (warp == 7) {  // the warp that pools nothing (224 of the 256 threads do): its de-allocation below delays nobody
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(SPM_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // filters: row = output channel, 28 bytes of taps + 4 zero bytes, swizzled like the im2col rows
    if (threadIdx.x < 64) {
        const int o = threadIdx.x >> 1, j = threadIdx.x & 1;
        const uint4 w4 = j == 0 ? make_uint4(P.w[o][0], P.w[o][1], P.w[o][2], P.w[o][3]) : make_uint4(P.w[o][4], P.w[o][5], P.w[o][6], 0u);
        *reinterpret_cast<uint4*>(sB + o * 32 + ((j ^ ((o >> 2) & 1)) << 4)) = w4;
    }
    pdl_wait();  // set-up above overlaps the previous kernel; the image is read and the output written after it
    // quantized input halo tile, as int8 channel planes. All of a thread's loads are issued before the first is used: the CTA
    // runs its phases one after the other, so this phase's DRAM latency must be paid once, not once per loop trip.
    const float* ximg = x + (long)img * 3 * s.h * s.w;
    const bool vec_ok = (s.w % 4 == 0) && rounding == ROUND_ADD_HALF_TRUNC;
    constexpr int TIN_WORDS = 3 * IH * RP, TIN_TRIPS = (TIN_WORDS + 255) / 256;
    if (vec_ok) {
        float4 v[TIN_TRIPS];
#pragma unroll
        for (int u = 0; u < TIN_TRIPS; ++u) {
            const int i = threadIdx.x + 256 * u;
            const int xw = i % RP, r = (i / RP) % IH, c = i / (RP * IH);
            const int iy = iy0 + r, ix = ix_al + xw * 4;
            // w % 4 == 0 and ix % 4 == 0: an aligned float4 is wholly inside the row or wholly outside
            v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < TIN_WORDS && iy >= 0 && iy < s.h && ix >= 0 && ix < s.w)
                v[u] = __ldg(reinterpret_cast<const float4*>(ximg + ((long)c * s.h + iy) * s.w + ix));
        }
#pragma unroll
        for (int u = 0; u < TIN_TRIPS; ++u) {
            const int i = threadIdx.x + 256 * u;
            if (i < TIN_WORDS) (&tin[0][0][0])[i] = quantize4_pack(v[u].x, v[u].y, v[u].z, v[u].w, in_scale);
        }
    } else {
        for (int i = threadIdx.x; i < TIN_WORDS; i += 256) {
            const int xw = i % RP, r = (i / RP) % IH, c = i / (RP * IH);
            const int iy = iy0 + r, ix = ix_al + xw * 4;
            uint32_t word = 0;
            if (iy >= 0 && iy < s.h && ix + 3 >= 0 && ix < s.w) {
                const float* row = ximg + ((long)c * s.h + iy) * s.w;
                int q[4] = {0, 0, 0, 0};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (ix + j >= 0 && ix + j < s.w) q[j] = quantize1(__ldg(row + ix + j), in_scale, rounding);
                word = pack4(q[0], q[1], q[2], q[3]);
            }
            (&tin[0][0][0])[i] = word;
        }
    }
    __syncthreads();

    // im2col rows: pixel p of the 33x15 convolution tile -> row p (byte k = tap (c, ky, kx), k = c*9 + ky*3 + kx)
    for (int p = threadIdx.x; p < SPM_ROWS; p += 256) {
        uint4 c0 = make_uint4(0, 0, 0, 0), c1 = make_uint4(0, 0, 0, 0);
        if (p < SP_CX * SP_CY) {
            const int lx = p % SP_CX, ly = p / SP_CX;
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
            c0.x = __byte_perm(win[0], win[1], 0x4210);
            c0.y = __byte_perm(win[1], win[2], 0x5421);
            c0.z = __byte_perm(win[2], win[3], 0x6542);
            c0.w = __byte_perm(win[4], win[5], 0x4210);
            c1.x = __byte_perm(win[5], win[6], 0x5421);
            c1.y = __byte_perm(win[6], win[7], 0x6542);
            c1.z = __byte_perm(win[8], 0u, 0x4210);
        }
        const int swz = (p >> 2) & 1;
        *reinterpret_cast<uint4*>(sA + p * 32 + ((0 ^ swz) << 4)) = c0;
        *reinterpret_cast<uint4*>(sA + p * 32 + ((1 ^ swz) << 4)) = c1;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA's reads
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (threadIdx.x == 32) {
        // D = s32, A = B = signed int8, both K-major, N = 32, M = 128
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((32u >> 3) << 17) | ((128u >> 4) << 24);
        const uint64_t bdesc = make_smem_desc(smem_u32(sB), 32);
#pragma unroll
        for (int t = 0; t < SPM_ROWS / 128; ++t) umma_i8(tmem_base + 32u * t, make_smem_desc(smem_u32(sA) + 4096u * t, 32), bdesc, idesc, 0u);
        umma_commit(bar);
    }
    const bool ok = mbar_wait(bar, 0, &abort_flag, status, 32u);
    tc_fence_after();

    if (ok) {
        // Accumulators -> shared memory as they are (one 16-byte store per four channels). Max-pooling happens on these exact
        // s32 sums: dequantize + activation is non-decreasing in the sum for the non-negative scales the layer is prepared with,
        // so the maximum of the window's outputs is the output of the window's maximum, bit for bit, and the float epilogue
        // runs once per pooled value instead of once per convolution output. Pixels outside the image never win.
        const int q = warp & 3;  // TMEM lane quarter this warp may read
#pragma unroll
        for (int rep = 0; rep < 2; ++rep) {
            const int t = (warp >> 2) + 2 * rep;
            const int p = t * 128 + q * 32 + lane;
            const int lx = p % SP_CX, ly = p / SP_CX;
            const int ox = cx0 + lx, oy = cy0 + ly;
            const bool inside = ox >= 0 && ox < s.ow && oy >= 0 && oy < s.oh;
            const uint32_t taddr = tmem_base + 32u * t + ((uint32_t)(q * 32) << 16);
            int v[32];
            __syncwarp();
            tmem_ld16(taddr, *reinterpret_cast<int(*)[16]>(&v[0]));
            if (s.cout > 16) tmem_ld16(taddr + 16u, *reinterpret_cast<int(*)[16]>(&v[16]));  // warp-uniform
            tmem_wait_ld16(*reinterpret_cast<int(*)[16]>(&v[0]));
            tmem_wait_ld16(*reinterpret_cast<int(*)[16]>(&v[16]));
            if (p >= SP_CX * SP_CY) continue;
            int4* dst = reinterpret_cast<int4*>(cacc + p * pitch);
            if (inside) {
#pragma unroll
                for (int g = 0; g < ST_COUT_MAX / 4; ++g)
                    if (g < cout4) dst[g] = make_int4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
            } else {
#pragma unroll
                for (int g = 0; g < ST_COUT_MAX / 4; ++g)
                    if (g < cout4) dst[g] = make_int4(INT_MIN, INT_MIN, INT_MIN, INT_MIN);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 7) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(SPM_TMEM_COLS) : "memory");
    }
    if (!ok) return;

    // thread = (pooled pixel, half of the channels): the two threads of a pixel are neighbours, so its channels leave together
    const int half_groups = (cout4 + 1) >> 1;
    const long pplane = (long)ph_out * pw_out;
    for (int i = threadIdx.x; i < 2 * SP_PY * SP_PX; i += 256) {
        const int g = i & 1, lx = (i >> 1) % SP_PX, ly = (i >> 1) / SP_PX;
        const int px = px0 + lx, py = py0 + ly;
        if (px >= pw_out || py >= ph_out) continue;
        // the reference's packed max-pool lets the padding take part as 0 (Tensor/Pool.cpp:972-975); its plain one never lets it win
        const bool pad_counts = pad_zero && (2 * py - 1 < 0 || 2 * py + 1 >= s.oh || 2 * px - 1 < 0 || 2 * px + 1 >= s.ow);
        const int* cp = cacc + ((2 * ly) * SP_CX + 2 * lx) * pitch;
        const int q_end = g == 0 ? half_groups : cout4;
        for (int q4 = g == 0 ? 0 : half_groups; q4 < q_end; ++q4) {
            const int4* w0 = reinterpret_cast<const int4*>(cp + 4 * q4);
            int4 v[9];
#pragma unroll
            for (int dy = 0; dy < 3; ++dy)
#pragma unroll
                for (int dx = 0; dx < 3; ++dx) v[dy * 3 + dx] = *reinterpret_cast<const int4*>(reinterpret_cast<const int*>(w0) + (dy * SP_CX + dx) * pitch);
            int m[4];
#define OTT_MAX9(F) __vimax3_s32(__vimax3_s32(v[0].F, v[1].F, v[2].F), __vimax3_s32(v[3].F, v[4].F, v[5].F), __vimax3_s32(v[6].F, v[7].F, v[8].F))
            m[0] = OTT_MAX9(x); m[1] = OTT_MAX9(y); m[2] = OTT_MAX9(z); m[3] = OTT_MAX9(w);
#undef OTT_MAX9
            const float4 si = *reinterpret_cast<const float4*>(&sprm[0][4 * q4]);
            const float4 bi = *reinterpret_cast<const float4*>(&sprm[1][4 * q4]);
            const float sia[4] = {si.x, si.y, si.z, si.w}, bia[4] = {bi.x, bi.y, bi.z, bi.w};
            float y[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float a = __int2float_rn(m[j]);
                y[j] = activate_t<ACT>(has_bias ? __fmaf_rn(a, sia[j], bia[j]) : __fmul_rn(a, sia[j]), act_p0);
                if (ACT != ACT_RELU && ACT != ACT_RELU6 && pad_counts) y[j] = fmaxf(y[j], 0.f);  // (after a ReLU nothing is below the padding's 0)
            }
            if (OUT8) {
                const float4 so = *reinterpret_cast<const float4*>(&sprm[2][4 * q4]);
                const float soa[4] = {so.x, so.y, so.z, so.w};
                int qv[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float t = __fmul_rn(y[j], soa[j]);
                    // after ReLU / ReLU6 t >= 0 (scales are positive): trunc(t + 0.5), the saturating pack clamps at 127
                    qv[j] = 4 * q4 + j >= s.cout ? 0
                            : ((ACT == ACT_RELU || ACT == ACT_RELU6) && rounding == ROUND_ADD_HALF_TRUNC) ? f2i8_nonneg(t) : float2int8(t, rounding);
                }
                *reinterpret_cast<uint32_t*>(static_cast<int8_t*>(out_any) + (((long)img * ph_out + py) * pw_out + px) * s.cout_pad + 4 * q4) =
                    pack_sat_s8x4(qv[0], qv[1], qv[2], qv[3]);
            } else {
                float* o = static_cast<float*>(out_any) + ((long)img * s.cout + 4 * q4) * pplane + (long)py * pw_out + px;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (4 * q4 + j < s.cout) o[j * pplane] = y[j];
            }
        }
        if (OUT8 && g == 1)  // padding channels of the int8 row (the stride is a multiple of 16 channels): zeros
            for (int c4 = cout4; c4 < s.cout_pad / 4; ++c4)
                *reinterpret_cast<uint32_t*>(static_cast<int8_t*>(out_any) + (((long)img * ph_out + py) * pw_out + px) * s.cout_pad + 4 * c4) = 0u;
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
        // The kernels assume scale_in >= 0 (it is 1 / (positive scales)). Should one ever be negative, the channel's filter and
        // scale are negated together: (-acc) * (-scale) is the same product, exactly.
        const int sign = scale_in[o] < 0.f ? -1 : 1;
        for (int k = 0; k < 27; ++k) P.w[o][k / 4] |= (uint32_t)(uint8_t)(int8_t)(sign * w[o * 27 + k]) << (8 * (k % 4));
        P.scale_in[o] = sign * scale_in[o];
        P.bias[o] = bias ? bias[o] : 0.f;
        P.scale_out[o] = scale_out ? scale_out[o] : 0.f;
    }
}

template <int S, bool OUT8>
static cudaError_t launch_pool_s(cudaStream_t stream, const float* x, const StemParams& P, float in_scale, const EpilogueParams& ep, void* out,
                                 const ConvShape& s, int pad_zero, uint32_t* status) {
    const int ph_out = (s.oh + 2 - 3) / 2 + 1, pw_out = (s.ow + 2 - 3) / 2 + 1;
    const int tiles_x = (pw_out + SP_PX - 1) / SP_PX, tiles_y = (ph_out + SP_PY - 1) / SP_PY;
    const long blocks = (long)s.n * tiles_x * tiles_y;
    if (blocks <= 0) return cudaSuccess;
    constexpr int IW = (SP_CX - 1) * S + 3, IH = (SP_CY - 1) * S + 3, RP = (IW + 3 + 3) / 4 + 1;
    // alignment slack + the larger of (im2col rows + filter rows + input tile) and the s32 convolution tile that later overlays them
    const size_t front = (size_t)SPM_ROWS * 32 + 1024 + (size_t)3 * IH * RP * 4;
    const size_t tile = (size_t)SP_CY * SP_CX * (((s.cout + 3) / 4) * 4 + 4) * 4;
    const size_t smem = 1024 + (front > tile ? front : tile);
    const bool c24 = s.cout == 24 && s.cout_pad == 32 && ep.has_bias && ep.rounding == ROUND_ADD_HALF_TRUNC;
#define OTT_STEMPOOL_LAUNCH(ACT)                                                                                          \
    {                                                                                                                     \
        auto kernel = c24 ? dense_stem_pool_mma_kernel<S, ACT, OUT8, true> : dense_stem_pool_mma_kernel<S, ACT, OUT8, false>;    \
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);            \
        if (e != cudaSuccess) return e;                                                                                   \
        e = launch_overlapped(kernel, dim3((unsigned)blocks), dim3(256), smem, stream, x, P, in_scale, ep.has_bias, ep.act_param0,        \
                              ep.rounding, out, s, ph_out, pw_out, tiles_x, tiles_y, pad_zero, status);                    \
        if (e != cudaSuccess) return e;                                                                                   \
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
                                   const float* bias_host, const float* scale_out_host, float in_scale, const EpilogueParams& ep, void* out,
                                   int out_dtype, int pad_zero, uint32_t* status) {
    StemParams P{};
    fill_stem_params(P, s, w_oihw_host, scale_in_host, bias_host, out_dtype == DT_S8_NHWC ? scale_out_host : nullptr);
    if (out_dtype == DT_S8_NHWC)
        return s.sh == 1 ? launch_pool_s<1, true>(stream, x, P, in_scale, ep, out, s, pad_zero, status)
                         : launch_pool_s<2, true>(stream, x, P, in_scale, ep, out, s, pad_zero, status);
    return s.sh == 1 ? launch_pool_s<1, false>(stream, x, P, in_scale, ep, out, s, pad_zero, status)
                     : launch_pool_s<2, false>(stream, x, P, in_scale, ep, out, s, pad_zero, status);
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
