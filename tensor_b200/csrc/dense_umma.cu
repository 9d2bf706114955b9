// Dense int8 convolution as an implicit GEMM on the sm_100a tensor cores.
//
// Replaces the reference's im2col + sgemm int8 path (Tensor/ConvolutionMM2DInt8X86Pack.cpp:2369-2445 builds
// the im2col matrix, :1656-2223 is the s8 x s8 -> s32 GEMM, :2533-2556 the 1x1 shortcut) and the epilogue
// passes that follow it (Tensor/QuantizeX86.cpp:851-903 dequantize, :1723-1870 requantize). No im2col
// matrix, no s32 tensor and no padded copy ever reach HBM:
//
//   D[128 pixels, BN out-channels] (s32, in TMEM)  +=  A[128 pixels, 32..128 in-channels] * B[BN, same]^T
//
// * A tiles come straight from the NHWC int8 activations with 4-D TMA boxes {channels, TW, TH, 1};
//   out-of-image rows/columns are zero-filled by TMA, which is the reference's constant_pad
//   (Tensor/Padding.cpp:22-36). 1x1 convolutions view the activations as a flat [pixels, channels] matrix so
//   tiles never straddle anything. k x k convolutions load, per pixel tile of 8 x 16 and channel block, ONE box
//   that holds the tile and its halo; filter tap (ky, kx) is an MMA whose A descriptor starts (ky, kx) pixels
//   into that box and steps one halo row per 8-row group (the swizzle is a function of the shared-memory
//   address, so shifted views read what TMA wrote). Dilated layers load one shifted box per tap instead.
// * B (the layer's weights for this CTA's BN output channels, all taps) is loaded once per CTA and stays in
//   shared memory while the CTA walks over its pixel tiles (persistent, weight-stationary).
// * tcgen05.mma.kind::i8 accumulates exact s32 in TMEM; two accumulators are double-buffered so the
//   epilogue of tile i overlaps the loads and MMAs of tile i+1.
// * The epilogue warps read TMEM (tcgen05.ld), apply fma(acc, scale_in, bias) -> activation -> requantize
//   (epilogue.cuh) and store int8 NHWC / fp32 NCHW / s32 NHWC.
//
// Warp roles (320 threads): warp 0 = TMA producer (one lane), warp 1 = TMEM owner + MMA issuer (one lane),
// warps 2..9 = epilogue: warp w reads TMEM lanes 32*(w%4)..+31 (the hardware's lane window of a warp) and
// takes every other 32-column chunk, so two warps share each lane quarter.
// Every mbarrier wait is bounded in time: on expiry the waiter raises a CTA-wide abort flag, ORs a code
// into the status word, and all roles fall through to the common teardown, which frees TMEM.
#include <cuda.h>

#include <type_traits>

#include <mutex>

#include "dense_umma.h"
#include "launch.cuh"
#include "umma_primitives.cuh"

namespace ottk {

namespace {

constexpr int kMaxEpiWarps = 8;                     // 2 per TMEM lane quarter
constexpr int kMaxThreads = 64 + 32 * kMaxEpiWarps;  // UmmaPlan::epi_warps is 4 or 8 (16 in the wide-tile build)
constexpr int kTileM = 128;
constexpr int kMaxAccBufs = 4;
constexpr int kHaloTw = 8, kHaloTh = 16;  // pixel tile of the halo mode: 8 wide so that a tile row is one 8-row operand group
using namespace umma;

// Activation tensor maps of one launch: one for an ordinary layer; one per source tensor for a layer whose K blocks are
// gathered from several int8 tensors.
struct KernelMaps {
    CUtensorMap tm[kUmmaMaxSources];
    uint16_t block_x[kUmmaMaxGatherBlocks];
    uint8_t block_src[kUmmaMaxGatherBlocks];
};

struct SmemLayout {
    uint32_t b_panel, a_stages, bars, tmem_slot, abort_flag, params, total;
};

__host__ __device__ inline SmemLayout smem_layout(const UmmaPlan& p) {
    SmemLayout L;
    L.b_panel = 0;
    L.a_stages = (uint32_t)p.nkb * p.bn * p.bkc;
    L.bars = L.a_stages + (uint32_t)p.stages * (uint32_t)p.a_stage_bytes;
    // barriers: full[stages], empty[stages], b_full, tmem_full[kMaxAccBufs], tmem_empty[kMaxAccBufs]
    L.tmem_slot = L.bars + 8u * (2u * p.stages + 1u + 2u * kMaxAccBufs);
    L.abort_flag = L.tmem_slot + 8;
    L.params = (L.abort_flag + 8 + 15u) & ~15u;  // scale_in[bn], bias[bn], scale_out[bn]; read as float4
    L.total = L.params + 3u * 4u * p.bn;
    return L;
}

// BUILD 1: compiled for two resident CTAs per SM (at most 102 registers per thread), which small layers need to hide latency;
// BUILD 2: 576 threads (sixteen epilogue warps) for wide tiles with one CTA per SM; BUILD 0: 320 threads, one CTA per SM;
// the one-CTA-per-SM plans of large layers use the build without that register limit.
template <int OUT, int ACT, bool BIAS, int ROUND, int BUILD>
__global__ void __launch_bounds__(BUILD == 2 ? 64 + 32 * 16 : kMaxThreads, BUILD == 1 ? 2 : 1)
dense_umma_kernel(const __grid_constant__ KernelMaps maps, const __grid_constant__ CUtensorMap tmB, const UmmaPlan P,
                  const ConvShape s, const EpilogueParams ep, void* __restrict__ out, uint32_t* __restrict__ status,
                  const __grid_constant__ UmmaMixedOut mixed) {
    extern __shared__ uint8_t smem_raw[];
    pdl_launch_dependents();
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const SmemLayout L = smem_layout(P);
    const uint32_t sB = base + L.b_panel, sA = base + L.a_stages;
    const uint32_t bar_full = base + L.bars, bar_empty = bar_full + 8u * P.stages, bar_b = bar_empty + 8u * P.stages;
    const uint32_t bar_tfull = bar_b + 8, bar_tempty = bar_tfull + 8u * kMaxAccBufs;
    const uint32_t acc_mask = (uint32_t)P.acc_bufs - 1u, acc_shift = P.acc_bufs == 4 ? 2u : 1u;  // 2 or 4 accumulators in TMEM
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + L.tmem_slot);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L.abort_flag);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tile = blockIdx.x % P.n_tiles;
    const int m_first = blockIdx.x / P.n_tiles, m_step = gridDim.x / P.n_tiles;
    const uint32_t a_stage_bytes = (uint32_t)P.a_stage_bytes, b_tile_bytes = (uint32_t)P.bn * P.bkc;
    // halo mode: the 8 pixels of one tile row are one 8-row operand group; groups (tile rows) are one halo row apart
    const int halo_w = kHaloTw + s.kw - 1, halo_h = kHaloTh + s.kh - 1;
    // pipeline stages one pixel tile consumes (a gathered layer's stage holds all the K blocks of a tile: one barrier round
    // trip per tile instead of one per 32-channel block)
    const int loads_per_tile = P.halo ? P.ncb : (P.gather && P.gather_whole ? 1 : P.nkb);

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmB);
        for (int i = 0; i < (P.gather > 0 ? P.gather : 1); ++i) prefetch_tensormap(&maps.tm[i]);
        for (int i = 0; i < P.stages; ++i) {
            mbar_init(bar_full + 8u * i, 1);
            mbar_init(bar_empty + 8u * i, 1);
        }
        mbar_init(bar_b, 1);
        for (int i = 0; i < P.acc_bufs; ++i) {
            mbar_init(bar_tfull + 8u * i, 1);
            mbar_init(bar_tempty + 8u * i, (uint32_t)P.epi_warps);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // the weight panel does not depend on the previous kernel: start loading it before waiting for that kernel
        mbar_expect_tx(bar_b, (uint32_t)P.nkb * b_tile_bytes);
        for (int kb = 0; kb < P.nkb; ++kb) tma_load_2d(&tmB, bar_b, sB + kb * b_tile_bytes, kb * P.bkc, n_tile * P.bn);
    }
    {
        float* sp = reinterpret_cast<float*>(base_ptr + L.params);
        for (int i = threadIdx.x; i < P.bn; i += (int)blockDim.x) {
            const int c = n_tile * P.bn + i;
            const bool in = c < s.cout_pad;
            sp[i] = in ? ep.scale_in[c] : 0.f;
            sp[P.bn + i] = in ? ep.bias[c] : 0.f;
            sp[2 * P.bn + i] = in ? ep.scale_out[c] : 0.f;
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                     "r"((uint32_t)P.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();  // from here on the kernel reads activations and writes outputs: the previous kernel must be complete

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer (activations; the weights were requested during set-up) ----
            uint32_t it = 0;
            bool ok = true;
            for (int m = m_first; ok && m < P.m_tiles; m += m_step) {
                int img, y0, x0;
                if (P.flat) {
                    img = 0; y0 = 0; x0 = m * kTileM;
                } else {
                    const int per_img = P.tiles_x * P.tiles_y;
                    img = m / per_img;
                    const int r = m - img * per_img;
                    y0 = (r / P.tiles_x) * P.th * s.sh - s.ph;
                    x0 = (r % P.tiles_x) * P.tw * s.sw - s.pw;
                }
                for (int kb = 0; kb < loads_per_tile; ++kb, ++it) {
                    const uint32_t st = it % P.stages, ph = (it / P.stages) & 1u;
                    if (!mbar_wait(bar_empty + 8u * st, ph ^ 1u, abort_flag, status, 1u, P.wait_ns)) { ok = false; break; }
                    if (P.gather && P.gather_whole) {
                        mbar_expect_tx(bar_full + 8u * st, (uint32_t)(kTileM * P.bkc * P.nkb));
                        for (int g = 0; g < P.nkb; ++g)
                            tma_load_4d(&maps.tm[maps.block_src[g]], bar_full + 8u * st, sA + st * a_stage_bytes + (uint32_t)(g * kTileM * P.bkc),
                                        (int)maps.block_x[g], x0, 0, 0);
                    } else if (P.gather) {
                        // K block kb = 32 channels of one of the source tensors (channels past that tensor's end arrive as zeros)
                        mbar_expect_tx(bar_full + 8u * st, (uint32_t)kTileM * P.bkc);
                        tma_load_4d(&maps.tm[maps.block_src[kb]], bar_full + 8u * st, sA + st * a_stage_bytes, (int)maps.block_x[kb], x0, 0, 0);
                    } else if (P.halo) {
                        // the (8 + kw - 1) x (16 + kh - 1) pixels under the tile, one channel block; out-of-image pixels arrive as zeros
                        mbar_expect_tx(bar_full + 8u * st, (uint32_t)(halo_w * halo_h * P.bkc));
                        tma_load_4d(&maps.tm[0], bar_full + 8u * st, sA + st * a_stage_bytes, kb * P.bkc, x0, y0, img);
                    } else {
                        const int tap = kb / P.ncb, cb = kb - tap * P.ncb;
                        const int ky = tap / s.kw, kx = tap - ky * s.kw;
                        mbar_expect_tx(bar_full + 8u * st, (uint32_t)kTileM * P.bkc);
                        tma_load_4d(&maps.tm[0], bar_full + 8u * st, sA + st * a_stage_bytes, cb * P.bkc, x0 + kx * s.dw, y0 + ky * s.dh, img);
                    }
                }
            }
            if (!ok) {
                // let bulk copies already in flight land before the CTA's shared memory is released
                const unsigned long long t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 1000000ull) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ----
            bool ok = mbar_wait(bar_b, 0, abort_flag, status, 16u, P.wait_ns);
            tc_fence_after();
            uint32_t it = 0, tile_i = 0;
            for (int m = m_first; ok && m < P.m_tiles; m += m_step, ++tile_i) {
                const uint32_t buf = tile_i & acc_mask, use = tile_i >> acc_shift;
                if (!mbar_wait(bar_tempty + 8u * buf, (use & 1u) ^ 1u, abort_flag, status, 4u, P.wait_ns)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d = tmem_base + buf * (uint32_t)P.acc_stride;
                for (int kb = 0; kb < loads_per_tile; ++kb, ++it) {
                    const uint32_t st = it % P.stages, ph = (it / P.stages) & 1u;
                    if (!mbar_wait(bar_full + 8u * st, ph, abort_flag, status, 2u, P.wait_ns)) { ok = false; break; }
                    tc_fence_after();
                    if (P.halo) {
                        // every filter tap reads the same halo tile through a view shifted by (ky, kx) pixels
                        // (one thread issues all of these back to back, so the per-tap descriptors are the base descriptors plus
                        // an offset in their 16-byte address field, not rebuilt from scratch)
                        const uint64_t a0 = make_smem_desc(sA + st * a_stage_bytes, P.bkc, halo_w * P.bkc);
                        const uint64_t b0 = make_smem_desc(sB + kb * b_tile_bytes, P.bkc);
                        const uint32_t b_tap_step = ((uint32_t)P.ncb * b_tile_bytes) >> 4, a_px_step = (uint32_t)P.bkc >> 4;
                        uint32_t accumulate = kb != 0 ? 1u : 0u, a_row = 0, b_off = 0;
                        if (s.kh == 3 && s.kw == 3) {
                            // the common filter: all loops unrolled, every descriptor the base's low word plus a constant (the
                            // address field cannot carry), so that the one issuing thread spends its time issuing
                            const uint32_t a_lo = (uint32_t)a0, b_lo = (uint32_t)b0;
                            const uint64_t a_hi = a0 & 0xFFFFFFFF00000000ull, b_hi = b0 & 0xFFFFFFFF00000000ull;
                            const uint32_t row_step = (uint32_t)(kHaloTw + 2) * a_px_step;
                            auto taps = [&](auto steps) {
                                constexpr int J = decltype(steps)::value;
#pragma unroll
                                for (int tap = 0; tap < 9; ++tap) {
                                    const uint32_t ao = (uint32_t)(tap / 3) * row_step + (uint32_t)(tap % 3) * a_px_step, bo = (uint32_t)tap * b_tap_step;
#pragma unroll
                                    for (int j = 0; j < J; ++j) {
                                        umma_i8(d, a_hi | (uint64_t)(a_lo + ao + 2u * j), b_hi | (uint64_t)(b_lo + bo + 2u * j), P.idesc, accumulate);
                                        accumulate = 1u;
                                    }
                                }
                            };
                            if (P.bkc == 128) taps(std::integral_constant<int, 4>{});
                            else if (P.bkc == 64) taps(std::integral_constant<int, 2>{});
                            else taps(std::integral_constant<int, 1>{});
                        } else
                        for (int ky = 0; ky < s.kh; ++ky, a_row += (uint32_t)halo_w * a_px_step) {
                            uint32_t a_off = a_row;
                            for (int kx = 0; kx < s.kw; ++kx, a_off += a_px_step, b_off += b_tap_step) {
                                for (int j = 0; j < P.bkc / 32; ++j) {
                                    umma_i8(d, a0 + a_off + 2u * j, b0 + b_off + 2u * j, P.idesc, accumulate);
                                    accumulate = 1u;
                                }
                            }
                        }
                    } else if (P.gather && P.gather_whole) {
                        // one stage holds all the K blocks of the tile; per block only the low words of the two descriptors move
                        const uint64_t a0 = make_smem_desc(sA + st * a_stage_bytes, P.bkc), b0 = make_smem_desc(sB, P.bkc);
                        const uint32_t a_lo = (uint32_t)a0, b_lo = (uint32_t)b0;
                        const uint64_t a_hi = a0 & 0xFFFFFFFF00000000ull, b_hi = b0 & 0xFFFFFFFF00000000ull;
                        const uint32_t a_step = (uint32_t)(kTileM * P.bkc) >> 4, b_step = b_tile_bytes >> 4;
                        uint32_t ao = 0, bo = 0;
                        for (int g = 0; g < P.nkb; ++g, ao += a_step, bo += b_step)
                            for (int j = 0; j < P.bkc / 32; ++j)
                                umma_i8(d, a_hi | (uint64_t)(a_lo + ao + 2u * j), b_hi | (uint64_t)(b_lo + bo + 2u * j), P.idesc, (g | j) != 0 ? 1u : 0u);
                    } else {
                        const uint64_t adesc = make_smem_desc(sA + st * a_stage_bytes, P.bkc);
                        const uint64_t bdesc = make_smem_desc(sB + kb * b_tile_bytes, P.bkc);
                        const uint32_t a_lo = (uint32_t)adesc, b_lo = (uint32_t)bdesc;
                        const uint64_t a_hi = adesc & 0xFFFFFFFF00000000ull, b_hi = bdesc & 0xFFFFFFFF00000000ull;
                        auto steps = [&](auto n) {
                            constexpr int J = decltype(n)::value;
#pragma unroll
                            for (int j = 0; j < J; ++j) umma_i8(d, a_hi | (uint64_t)(a_lo + 2u * j), b_hi | (uint64_t)(b_lo + 2u * j), P.idesc, (kb | j) != 0 ? 1u : 0u);
                        };
                        if (P.bkc == 128) steps(std::integral_constant<int, 4>{});
                        else if (P.bkc == 64) steps(std::integral_constant<int, 2>{});
                        else steps(std::integral_constant<int, 1>{});
                    }
                    umma_commit(bar_empty + 8u * st);  // frees the A stage once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(bar_tfull + 8u * buf);  // accumulator complete
            }
        }
    } else {
        // ---- epilogue warps ----
        const int q = warp & 3;            // TMEM lane quarter this warp may read
        const int sub = (warp - 2) >> 2;   // which of the epi_warps/4 warps sharing that quarter
        const int col_step = 16 * (P.epi_warps / 4);
        const int row = q * 32 + lane;
        const long plane = (long)s.oh * s.ow;
        const long total_pix = (long)s.n * plane;
        const float* s_si = reinterpret_cast<const float*>(base_ptr + L.params);
        const float* s_bi = s_si + P.bn;
        const float* s_so = s_bi + P.bn;
        uint32_t tile_i = 0;
        bool ok = true;
        for (int m = m_first; ok && m < P.m_tiles; m += m_step, ++tile_i) {
            const uint32_t buf = tile_i & acc_mask, use = tile_i >> acc_shift;
            if (!mbar_wait(bar_tfull + 8u * buf, use & 1u, abort_flag, status, 8u, P.wait_ns)) { ok = false; break; }
            tc_fence_after();
            // which output pixel this thread's TMEM lane holds
            long pix;  // linear (img, oy, ox) index
            bool valid;
            if (P.flat) {
                pix = (long)m * kTileM + row;
                valid = pix < total_pix;
            } else {
                const int per_img = P.tiles_x * P.tiles_y;
                const int img = m / per_img;
                const int r = m - img * per_img;
                const int oy = (r / P.tiles_x) * P.th + row / P.tw;
                const int ox = (r % P.tiles_x) * P.tw + row % P.tw;
                valid = oy < s.oh && ox < s.ow;
                pix = (long)img * plane + (long)oy * s.ow + ox;
            }
            const uint32_t taddr = tmem_base + buf * (uint32_t)P.acc_stride + ((uint32_t)(q * 32) << 16);
            int8_t* out_s8 = reinterpret_cast<int8_t*>(out) + pix * s.cout_pad + n_tile * P.bn;
            int32_t* out_s32 = reinterpret_cast<int32_t*>(out) + pix * s.cout_pad + n_tile * P.bn;
            float* out_f32 = nullptr;
            if (OUT == DT_F32_NCHW || (OUT == DT_S8_NHWC && mixed.out_f32 != nullptr)) {
                // (a 64-bit division costs about a hundred instructions per thread and tile; 32 bits cover any real tensor)
                long img, inimg;
                if (total_pix <= 0xFFFFFFFFll) {
                    const uint32_t q32 = (uint32_t)pix / (uint32_t)plane;
                    img = (long)q32;
                    inimg = (long)((uint32_t)pix - q32 * (uint32_t)plane);
                } else {
                    img = pix / plane;
                    inimg = pix - img * plane;
                }
                if (OUT == DT_S8_NHWC && mixed.plane_of_col != nullptr)
                    out_f32 = mixed.out_f32 + img * mixed.f32_planes * plane + inimg;  // plane chosen per column below
                else
                    out_f32 = (OUT == DT_F32_NCHW ? reinterpret_cast<float*>(out) : mixed.out_f32) + (img * s.cout + n_tile * P.bn) * plane + inimg;
            }
            // 16 accumulator columns -> 16 outputs of this thread's pixel. int8 results come back as 4 packed words in wds
            // (the caller stores them); the other output kinds are stored here.
            auto emit16 = [&](const int (&v)[16], int col0, uint32_t (&wds)[4]) {
                const int c0 = n_tile * P.bn + col0;  // first global output channel of this chunk
                if (OUT == DT_S32_NHWC) {
                    int4* o = reinterpret_cast<int4*>(out_s32 + col0);
#pragma unroll
                    for (int g = 0; g < 4; ++g) o[g] = make_int4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                    return;
                }
                // two fp32 lanes per instruction (fma.rn.f32x2 and friends): each lane rounds exactly like the scalar form
                float y[16];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const float4 si = *reinterpret_cast<const float4*>(s_si + col0 + g * 4);
                    const float4 bi = *reinterpret_cast<const float4*>(s_bi + col0 + g * 4);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float2 a = make_float2(__int2float_rn(v[g * 4 + 2 * h]), __int2float_rn(v[g * 4 + 2 * h + 1]));
                        const float2 s2 = h ? make_float2(si.z, si.w) : make_float2(si.x, si.y);
                        const float2 b2 = h ? make_float2(bi.z, bi.w) : make_float2(bi.x, bi.y);
                        const float2 t = BIAS ? __ffma2_rn(a, s2, b2) : __fmul2_rn(a, s2);
                        y[g * 4 + 2 * h] = activate_t<ACT>(t.x, ep.act_param0);
                        y[g * 4 + 2 * h + 1] = activate_t<ACT>(t.y, ep.act_param0);
                    }
                }
                if (OUT == DT_F32_NCHW) {
                    // one plane further per channel: a pointer that walks, and one bounds test per chunk where the chunk is whole
                    float* o = out_f32 + (long)col0 * plane;
                    if (c0 + 16 <= s.cout) {
#pragma unroll
                        for (int j = 0; j < 16; ++j, o += plane) *o = y[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j, o += plane)
                            if (c0 + j < s.cout) *o = y[j];
                    }
                } else {
                    if (out_f32 != nullptr) {
                        // channels that some reader wants in fp32: the planes an fp32-output layer would have written
                        const uint32_t m = (mixed.mask[(c0 >> 5) & 31] >> (c0 & 31)) & 0xFFFFu;
                        if (m != 0u) {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if ((m >> j) & 1u) {
                                    const long pl = mixed.plane_of_col != nullptr ? (long)mixed.plane_of_col[c0 + j] : (long)(col0 + j);
                                    out_f32[pl * plane] = y[j];
                                }
                        }
                    }
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const float4 so = *reinterpret_cast<const float4*>(s_so + col0 + g * 4);
                        int qv[4];
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const float2 t = __fmul2_rn(make_float2(y[g * 4 + 2 * h], y[g * 4 + 2 * h + 1]),
                                                        h ? make_float2(so.z, so.w) : make_float2(so.x, so.y));
                            if (ROUND == ROUND_HALF_AWAY) {
                                qv[2 * h] = float2int8(t.x, ROUND_HALF_AWAY);
                                qv[2 * h + 1] = float2int8(t.y, ROUND_HALF_AWAY);
                            } else if (ACT == ACT_RELU || ACT == ACT_RELU6) {
                                // t >= 0 (or -0): trunc(t + 0.5), the upper clamp is the saturating pack
                                const float2 r = __fadd2_rn(t, make_float2(0.5f, 0.5f));
                                qv[2 * h] = __float2int_rz(r.x);
                                qv[2 * h + 1] = __float2int_rz(r.y);
                            } else {
                                const float2 r = __fadd2_rn(t, make_float2(half_signed(t.x), half_signed(t.y)));
                                qv[2 * h] = __float2int_rz(fmaxf(r.x, -127.5f));
                                qv[2 * h + 1] = __float2int_rz(fmaxf(r.y, -127.5f));
                            }
                        }
                        wds[g] = pack_sat_s8x4(qv[0], qv[1], qv[2], qv[3]);
                    }
                }
            };
            // Chunks of 32 columns: two TMEM loads in flight, and int8 rows leave as one 32-byte store per thread, a whole
            // DRAM sector (two 16-byte stores from different warps would each touch half of it).
            const bool wide_ok = OUT == DT_S8_NHWC && ((s.cout_pad | (n_tile * P.bn)) & 31) == 0;
            for (int col0 = sub * 32; col0 < P.bn; col0 += 2 * col_step) {
                int va[16], vb[16];
                const bool two = col0 + 16 < P.bn;
                __syncwarp();  // tcgen05.ld is warp-collective
                tmem_ld16(taddr + (uint32_t)col0, va);
                if (two) tmem_ld16(taddr + (uint32_t)(col0 + 16), vb);
                tmem_wait_ld16(va);
                tmem_wait_ld16(vb);
                if (!valid) continue;
                uint32_t wa[4], wb[4];
                const bool a_ok = n_tile * P.bn + col0 < s.cout_pad, b_ok = two && n_tile * P.bn + col0 + 16 < s.cout_pad;
                if (a_ok) emit16(va, col0, wa);
                if (b_ok) emit16(vb, col0 + 16, wb);
                if (OUT == DT_S8_NHWC && mixed.n_chunks > 0) {
                    // scattered output: each 16-column chunk has its own destination tensor
                    const int ch = (n_tile * P.bn + col0) >> 4;
                    int8_t* da = a_ok ? mixed.dst[ch] : nullptr;
                    int8_t* db = b_ok ? mixed.dst[ch + 1] : nullptr;
                    if (da != nullptr && db != nullptr && ((mixed.pair_ok >> (ch >> 1)) & 1ull) != 0ull && (ch & 1) == 0) {
                        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(da + pix * mixed.pitch[ch]), "r"(wa[0]),
                                     "r"(wa[1]), "r"(wa[2]), "r"(wa[3]), "r"(wb[0]), "r"(wb[1]), "r"(wb[2]), "r"(wb[3])
                                     : "memory");
                    } else {
                        if (da != nullptr) *reinterpret_cast<uint4*>(da + pix * mixed.pitch[ch]) = make_uint4(wa[0], wa[1], wa[2], wa[3]);
                        if (db != nullptr) *reinterpret_cast<uint4*>(db + pix * mixed.pitch[ch + 1]) = make_uint4(wb[0], wb[1], wb[2], wb[3]);
                    }
                } else if (OUT == DT_S8_NHWC) {
                    if (a_ok && b_ok && wide_ok) {
                        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(out_s8 + col0), "r"(wa[0]), "r"(wa[1]),
                                     "r"(wa[2]), "r"(wa[3]), "r"(wb[0]), "r"(wb[1]), "r"(wb[2]), "r"(wb[3])
                                     : "memory");
                    } else {
                        if (a_ok) *reinterpret_cast<uint4*>(out_s8 + col0) = make_uint4(wa[0], wa[1], wa[2], wa[3]);
                        if (b_ok) *reinterpret_cast<uint4*>(out_s8 + col0 + 16) = make_uint4(wb[0], wb[1], wb[2], wb[3]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8u * buf);
        }
    }

    // ---- teardown (every path ends here) ----
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)P.tmem_cols) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    // initialised once, by whichever host thread comes first (function-local statics are thread-safe)
    static const EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            return reinterpret_cast<EncodeTiledFn>(p);
        return nullptr;
    }();
    return fn;
}

CUtensorMapSwizzle swizzle_for(int bkc) {
    return bkc == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (bkc == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

template <int OUT, int ACT, bool BIAS, int ROUND, int BUILD>
const char* launch_variant(cudaStream_t stream, int sm_count, const KernelMaps& maps, const CUtensorMap& tmB, const UmmaPlan& p,
                           const ConvShape& s, const EpilogueParams& ep, void* out, uint32_t* status, const UmmaMixedOut& mixed) {
    // per-device, per-instantiation set-up; several host threads may drive different GPUs through this function at once
    static std::mutex mu;
    static bool attr_set[64] = {};
    static int regs_per_thread[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = dense_umma_kernel<OUT, ACT, BIAS, ROUND, BUILD>;
    int regs = 128;
    if (dev >= 0 && dev < 64) {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set[dev]) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
                return "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed";
            cudaFuncAttributes fa{};
            regs_per_thread[dev] = cudaFuncGetAttributes(&fa, kernel) == cudaSuccess && fa.numRegs > 0 ? fa.numRegs : 128;
            attr_set[dev] = true;
        }
        regs = regs_per_thread[dev];
    }
    // Tiles are dealt statically to the CTAs of the grid, so a grid larger than what is resident at once runs in waves.
    // The plan bounds residency by shared memory and TMEM; registers and threads are bounded here.
    const int threads = 64 + 32 * p.epi_warps;
    const int regs_per_warp = (regs * 32 + 255) / 256 * 256;
    int resident = 65536 / (regs_per_warp * (threads / 32));
    if (resident > 2048 / threads) resident = 2048 / threads;
    if (resident < 1) resident = 1;
    const int per_sm = resident < p.ctas_per_sm ? resident : p.ctas_per_sm;
    int per_n = sm_count * per_sm / p.n_tiles;
    if (per_n < 1) per_n = 1;
    if (per_n > p.m_tiles) per_n = p.m_tiles;
    const int grid = per_n * p.n_tiles;
    if (launch_overlapped(kernel, dim3(grid), dim3(threads), (size_t)p.smem_bytes, stream, maps, tmB, p, s, ep, out, status, mixed) != cudaSuccess)
        return "dense_umma_kernel launch failed";
    return nullptr;
}

}  // namespace

static int round_up(int a, int b) { return (a + b - 1) / b * b; }

bool umma_plan_layer(int cin, int cout, int kh, int kw, int sh, int sw, int dh, int dw, int smem_budget, UmmaPlan* plan, int bkc_override,
                     bool whole_tile_stages) {
    UmmaPlan p{};
    const int cin_pad = nhwc_channels(cin), cout_pad = nhwc_channels(cout);
    if (sh < 1 || sw < 1 || sh > 4 || sw > 4) return false;
    if (cin_pad < 32) return false;        // a TMA box may not be wider than the tensor
    p.bkc = cin_pad >= 128 ? 128 : (cin_pad >= 64 ? 64 : 32);
    if (bkc_override == 32 || bkc_override == 64 || bkc_override == 128) p.bkc = bkc_override;
    p.ncb = (cin_pad + p.bkc - 1) / p.bkc;
    p.taps = kh * kw;
    p.nkb = p.taps * p.ncb;
    const long k_total = (long)p.nkb * p.bkc;
    // largest BN (multiple of 16, <= 256) whose weight panel leaves room for at least 3 A stages,
    // preferring a split of cout_pad into equal tiles
    // strided and dilated layers load one box per filter tap (a strided layer's box takes every sw-th / sh-th pixel: TMA
    // element strides); undilated stride-1 k x k layers load one halo tile per pixel tile
    p.halo = (p.taps > 1 && dh == 1 && dw == 1 && sh == 1 && sw == 1) ? 1 : 0;
    const bool whole = whole_tile_stages && !p.halo && p.taps == 1;
    p.gather_whole = whole ? 1 : 0;
    const long a_stage = p.halo ? ((long)p.bkc * (kHaloTw + kw - 1) * (kHaloTh + kh - 1) + 1023) / 1024 * 1024
                                : (long)kTileM * p.bkc * (whole ? p.nkb : 1);
    p.a_stage_bytes = (int)a_stage;
    const long avail = (long)smem_budget - 1024 /*alignment slack*/ - 4096 /*barriers + epilogue parameters*/ - (whole ? 2 : 3) * a_stage;
    if (avail <= 0) return false;
    long bn_max = avail / k_total;
    bn_max = bn_max > 256 ? 256 : bn_max;
    bn_max = bn_max / 16 * 16;
    if (bn_max < 16) return false;
    p.n_tiles = (cout_pad + (int)bn_max - 1) / (int)bn_max;
    p.bn = round_up((cout_pad + p.n_tiles - 1) / p.n_tiles, 16);
    if (p.bkc == 32) p.bn = round_up(p.bn, 32);  // keeps every weight tile on a 1 KiB boundary
    if (p.bn > 256 || (long)p.bn * k_total > avail) return false;
    const long left = (long)smem_budget - 1024 - 4096 - (long)p.bn * k_total;
    p.stages = (int)(left / a_stage);
    if (p.stages > 8) p.stages = 8;
    // Small layers (few k-blocks, narrow panels) are latency-bound with one CTA per SM: keep the pipeline short so that
    // several CTAs fit an SM and overlap each other's TMA / MMA / epilogue latencies.
    if ((p.nkb <= 2 || whole) && p.stages > 4) p.stages = 4;
    if (whole && p.stages > 2) p.stages = 2;  // two whole tiles in flight, and room for a second CTA on the SM
    // a halo stage feeds all the taps of a whole pixel tile and channel block: three are a deep enough pipeline
    if (p.halo && p.stages > 3) p.stages = 3;
    if (p.stages < 2) return false;
    // two accumulators of bn columns each; TMEM allocations are powers of two >= 32 columns
    p.acc_stride = p.bn <= 32 ? 32 : (p.bn <= 64 ? 64 : (p.bn <= 128 ? 128 : 256));
    // narrow tiles finish quickly; four accumulators let the MMA issuer run three tiles ahead of the epilogue
    p.acc_bufs = p.acc_stride <= 64 ? 4 : 2;
    p.tmem_cols = p.acc_bufs * p.acc_stride;
    // instruction descriptor: D=s32 (2<<4), A=B=signed int8 (1<<7, 1<<10), both K-major, N>>3 at bit 17, M>>4 at bit 24
    p.idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
    p.k_total = (int)k_total;
    p.cout_rows = p.n_tiles * p.bn;
    SmemLayout L = smem_layout(p);
    p.smem_bytes = (int)L.total + 1024;
    // CTAs per SM: TMEM has 512 columns per SM and the hardware scheduler does not account for them, so the shared-memory
    // request is padded until no more CTAs fit an SM than TMEM can serve (a CTA that cannot get its columns would wait
    // inside tcgen05.alloc for a neighbour to finish).
    // eight epilogue warps, two per TMEM lane quarter (sixteen for wide single-CTA tiles, below)
    p.epi_warps = 8;
    int by_tmem = 512 / p.tmem_cols;
    int by_smem = smem_budget / p.smem_bytes;
    p.ctas_per_sm = by_tmem < by_smem ? by_tmem : by_smem;
    if (p.ctas_per_sm > 4) p.ctas_per_sm = 4;
    if (p.ctas_per_sm < 1) p.ctas_per_sm = 1;
    // Wide tiles with one CTA per SM: sixteen epilogue warps (four per lane quarter, 576 threads, the build without a register
    // cap). Requantizing a 128 x 256 tile costs the CUDA cores as much as its MMAs cost the tensor pipe, and eight warps reach
    // only two thirds of the SM's requantize rate (measured: 512 -> 1024: 1660 -> 1837 TOP/s; 256 -> 512: 881 -> 1025; with
    // 128-column tiles it loses, 3x3 128 -> 128: 1938 -> 1865).
    if (p.ctas_per_sm == 1 && p.bn > 128) p.epi_warps = 16;
    const int min_smem = smem_budget / (p.ctas_per_sm + 1) + 1;
    if (p.smem_bytes < min_smem) p.smem_bytes = min_smem;
    *plan = p;
    return true;
}

void umma_pack_weights(const UmmaPlan& p, const int8_t* w_oihw, int cin, int cout, int kh, int kw, int8_t* dst) {
    // dst[cout_rows][k_total], k = (tap*ncb + cb)*bkc + (channel - cb*bkc); zero elsewhere
    const long kt = p.k_total;
    for (long i = 0; i < (long)p.cout_rows * kt; ++i) dst[i] = 0;
    for (int o = 0; o < cout; ++o)
        for (int c = 0; c < cin; ++c)
            for (int t = 0; t < kh * kw; ++t) {
                const int cb = c / p.bkc, ci = c % p.bkc;
                dst[o * kt + ((long)t * p.ncb + cb) * p.bkc + ci] = w_oihw[((long)o * cin + c) * kh * kw + t];
            }
}

const char* umma_encode_weight_map(const UmmaPlan& p, const int8_t* w_dev, void* map_out) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return "cuTensorMapEncodeTiled entry point not available";
    cuuint64_t dims[2] = {(cuuint64_t)p.k_total, (cuuint64_t)p.cout_rows};
    cuuint64_t strides[1] = {(cuuint64_t)p.k_total};
    cuuint32_t box[2] = {(cuuint32_t)p.bkc, (cuuint32_t)p.bn};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(reinterpret_cast<CUtensorMap*>(map_out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)w_dev, dims, strides, box,
                     estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(p.bkc), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? nullptr : "cuTensorMapEncodeTiled(weights) failed";
}

const char* launch_dense_umma(cudaStream_t stream, int sm_count, const UmmaPlan& plan_in, const void* weight_map,
                              const ConvShape& s, const int8_t* x, const EpilogueParams& ep, void* out, int out_dtype,
                              uint32_t* status, const UmmaSources* sources, const UmmaMixedOut* mixed_in, unsigned long long wait_limit_ns) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return "cuTensorMapEncodeTiled entry point not available";
    UmmaPlan p = plan_in;
    p.wait_ns = wait_limit_ns;
    const long pixels = (long)s.n * s.oh * s.ow;
    if (pixels == 0) return nullptr;
    KernelMaps km;  // only the entries the plan uses are filled in
    CUtensorMap& tmA = km.tm[0];
    UmmaMixedOut mixed{};
    if (mixed_in) {
        if (out_dtype != DT_S8_NHWC || s.cout > 1024) return "fp32 side output needs an int8 launch with at most 1024 output channels";
        mixed = *mixed_in;
    }
    const bool flat = s.kh == 1 && s.kw == 1 && s.ph == 0 && s.pw == 0 && s.sh == 1 && s.sw == 1;
    p.flat = flat ? 1 : 0;
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = CUDA_SUCCESS;
    if ((p.gather > 0) != (sources != nullptr)) return "gathered layer launched without its sources (or the reverse)";
    if (p.gather > 0) {
        if (!flat || sources->n_src != p.gather || p.nkb > kUmmaMaxGatherBlocks || p.bkc != kUmmaGatherBlock) return "bad gathered launch";
        p.tw = kTileM; p.th = 1; p.tiles_x = (int)((pixels + kTileM - 1) / kTileM); p.tiles_y = 1;
        p.m_tiles = p.tiles_x;
        for (int i = 0; i < sources->n_src && r == CUDA_SUCCESS; ++i) {
            const cuuint64_t cp = (cuuint64_t)sources->src_cpad[i];
            cuuint64_t dims[4] = {cp, (cuuint64_t)pixels, 1, 1};
            cuuint64_t strides[3] = {cp, cp * pixels, cp * pixels};
            cuuint32_t box[4] = {(cuuint32_t)p.bkc, (cuuint32_t)kTileM, 1, 1};
            r = enc(&km.tm[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)sources->src[i], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle_for(p.bkc), CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        }
        for (int kb = 0; kb < p.nkb; ++kb) {
            km.block_x[kb] = sources->block_x[kb];
            km.block_src[kb] = sources->block_src[kb];
        }
    } else if (flat) {
        p.tw = kTileM; p.th = 1; p.tiles_x = (int)((pixels + kTileM - 1) / kTileM); p.tiles_y = 1;
        p.m_tiles = p.tiles_x;
        cuuint64_t dims[4] = {(cuuint64_t)s.cin_pad, (cuuint64_t)pixels, 1, 1};
        cuuint64_t strides[3] = {(cuuint64_t)s.cin_pad, (cuuint64_t)s.cin_pad * pixels, (cuuint64_t)s.cin_pad * pixels};
        cuuint32_t box[4] = {(cuuint32_t)p.bkc, (cuuint32_t)kTileM, 1, 1};
        r = enc(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)x, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                swizzle_for(p.bkc), CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        // rectangle of 128 output pixels with the least padding waste (halo mode: always 8 x 16)
        long best = -1;
        for (int tw = 8; tw <= 128; tw *= 2) {
            const int th = kTileM / tw;
            if ((tw - 1) * s.sw + 1 > 256 || (th - 1) * s.sh + 1 > 256) continue;  // a TMA box spans at most 256 elements per dimension
            const long cover = (long)((s.ow + tw - 1) / tw) * tw * ((s.oh + th - 1) / th) * th;
            if (best < 0 || cover < best) { best = cover; p.tw = tw; p.th = th; }
        }
        if (p.halo) { p.tw = kHaloTw; p.th = kHaloTh; }
        p.tiles_x = (s.ow + p.tw - 1) / p.tw;
        p.tiles_y = (s.oh + p.th - 1) / p.th;
        p.m_tiles = s.n * p.tiles_x * p.tiles_y;
        cuuint64_t dims[4] = {(cuuint64_t)s.cin_pad, (cuuint64_t)s.w, (cuuint64_t)s.h, (cuuint64_t)s.n};
        cuuint64_t strides[3] = {(cuuint64_t)s.cin_pad, (cuuint64_t)s.cin_pad * s.w, (cuuint64_t)s.cin_pad * s.w * s.h};
        // a strided layer's box spans (tw - 1) * sw + 1 columns of which the traversal takes every sw-th: tw land in shared memory
        cuuint32_t box[4] = {(cuuint32_t)p.bkc, (cuuint32_t)(p.halo ? p.tw + s.kw - 1 : (p.tw - 1) * s.sw + 1),
                             (cuuint32_t)(p.halo ? p.th + s.kh - 1 : (p.th - 1) * s.sh + 1), 1};
        estr[1] = (cuuint32_t)s.sw;
        estr[2] = (cuuint32_t)s.sh;
        r = enc(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)x, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                swizzle_for(p.bkc), CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return "cuTensorMapEncodeTiled(activations) failed";

    const CUtensorMap& tmB = *reinterpret_cast<const CUtensorMap*>(weight_map);
    const char* err = nullptr;
#define OTT_UMMA_LAUNCH(OUT, ACT, BIAS, ROUND)                                                                       \
    err = p.ctas_per_sm > 1   ? launch_variant<OUT, ACT, BIAS, ROUND, 1>(stream, sm_count, km, tmB, p, s, ep, out, status, mixed) \
          : p.epi_warps == 16 ? launch_variant<OUT, ACT, BIAS, ROUND, 2>(stream, sm_count, km, tmB, p, s, ep, out, status, mixed) \
                              : launch_variant<OUT, ACT, BIAS, ROUND, 0>(stream, sm_count, km, tmB, p, s, ep, out, status, mixed)
#define OTT_UMMA_ACT(OUT, BIAS, ROUND)                                   \
    switch (ep.act_type) {                                               \
        case ACT_RELU: OTT_UMMA_LAUNCH(OUT, ACT_RELU, BIAS, ROUND); break;   \
        case ACT_LRELU: OTT_UMMA_LAUNCH(OUT, ACT_LRELU, BIAS, ROUND); break; \
        case ACT_RELU6: OTT_UMMA_LAUNCH(OUT, ACT_RELU6, BIAS, ROUND); break; \
        default: OTT_UMMA_LAUNCH(OUT, ACT_NONE, BIAS, ROUND); break;         \
    }
    if (out_dtype == DT_S32_NHWC) {
        OTT_UMMA_LAUNCH(DT_S32_NHWC, ACT_NONE, false, ROUND_ADD_HALF_TRUNC);
    } else if (out_dtype == DT_F32_NCHW) {
        if (ep.has_bias) { OTT_UMMA_ACT(DT_F32_NCHW, true, ROUND_ADD_HALF_TRUNC) } else { OTT_UMMA_ACT(DT_F32_NCHW, false, ROUND_ADD_HALF_TRUNC) }
    } else if (ep.rounding == ROUND_HALF_AWAY) {
        if (ep.has_bias) { OTT_UMMA_ACT(DT_S8_NHWC, true, ROUND_HALF_AWAY) } else { OTT_UMMA_ACT(DT_S8_NHWC, false, ROUND_HALF_AWAY) }
    } else {
        if (ep.has_bias) { OTT_UMMA_ACT(DT_S8_NHWC, true, ROUND_ADD_HALF_TRUNC) } else { OTT_UMMA_ACT(DT_S8_NHWC, false, ROUND_ADD_HALF_TRUNC) }
    }
#undef OTT_UMMA_ACT
#undef OTT_UMMA_LAUNCH
    if (err) return err;
    return cudaGetLastError() == cudaSuccess ? nullptr : "dense_umma_kernel launch failed";
}

}  // namespace ottk
