// One ShuffleNetV2 unit branch in one kernel: 1x1 convolution -> depthwise 3x3 (stride 1, pad 1) -> 1x1 convolution, each
// with its own fused requantize epilogue, i.e. three consecutive ConvolutionLayer::forward_int8 calls
// (Tensor/ConvolutionLayer.cpp:754-847; in the reference's shipped int8 graph the chain conv_4 (int8_scale_term 102) ->
// conv_5 (101) -> conv_6 (2)). Run as three launches, the two intermediate int8 tensors cross HBM twice and every launch
// pays its own fill and drain; here they never leave the SM:
//
//   per tile of 8 x 16 output pixels
//   X   TMA: the 10 x 18 input pixels under the tile and its one-pixel halo, as 32-channel K blocks gathered from the source
//       tensors (out-of-image pixels arrive as zeros)
//   1   tcgen05.mma: acc1[180 px, cm] = X * W1^T (two M = 128 blocks)            -> TMEM
//       epilogue 1: fma(acc, scale_in, bias) -> activation -> float2int8(v * scale_out) -> Y1 in shared memory, laid out as
//       the K-major operand of the next MMA; pixels outside the image are written as zeros (the depthwise layer's padding)
//   2   tcgen05.mma: acc2[128 px, cm]: the depthwise 3x3 as nine taps x (cm/32) block-diagonal 32 x 32 weight matrices; tap
//       (ky, kx) reads Y1 through an operand view shifted by (ky, kx) pixels, 8-row groups one halo row apart
//       epilogue 2: requantize -> Y2 in shared memory (operand layout again)
//   3   tcgen05.mma: acc3[128 px, c2] = Y2 * W2^T
//       epilogue 3: the second 1x1 layer's ordinary output stage (int8 NHWC with per-channel scales, chosen channels also as
//       fp32 planes; or fp32 NCHW)
//
// All sums are exact s32 and every epilogue is the same arithmetic as the separate layers', so the result is identical to
// theirs bit for bit. The depthwise multiply-adds run on the tensor cores with 31 of 32 weights zero: that is 32 times the
// useful work and still far from the tensor pipe's limit, while the CUDA cores keep to the three epilogues.
//
// Warp roles: warp 0 = TMA producer (one lane), warp 1 = TMEM owner + MMA issuer (one lane), warps 2.. = epilogue (warp w
// reads TMEM lanes 32*(w%4)..+31; warps sharing a lane quarter split the columns). The issuer runs the first 1x1 layer of
// the next tile ahead of the current tile's depthwise stage. Every wait is bounded, as in dense_umma.cu.
#include <cuda.h>

#include <mutex>

#include "launch.cuh"
#include "umma_epilogue.cuh"
#include "umma_primitives.cuh"
#include "unit_umma.h"

namespace ottk {

namespace {

using namespace umma;
constexpr int kTileM = 128;
constexpr int kMaxEpiWarps = 8;
constexpr int kMaxThreads = 64 + 32 * kMaxEpiWarps;

struct UnitMaps {
    CUtensorMap tm[kUmmaMaxSources];
    uint16_t block_x[kUmmaMaxGatherBlocks];
    uint8_t block_src[kUmmaMaxGatherBlocks];
};

struct UnitGeom {
    int n, h, w;
    int cout2, c2pad;  // second layer's real output channels and the channel stride of its int8 output tensor
};

enum : uint32_t { B_W = 0, B_XFULL = 1, B_XEMPTY = 3, B_ACC1 = 5, B_Y1 = 6, B_ACC2 = 7, B_Y2 = 8, B_ACC3 = 9, B_COUNT = 10 };

template <int ACT, int OUT, bool MULTI>
__global__ void __launch_bounds__(kMaxThreads, MULTI ? 2 : 1)
unit_umma_kernel(const __grid_constant__ UnitMaps maps, const __grid_constant__ CUtensorMap tmW1, const __grid_constant__ CUtensorMap tmWdw,
                 const __grid_constant__ CUtensorMap tmW2, const UnitPlan P, const UnitGeom G, const UnitEpilogues ep, void* __restrict__ out,
                 uint32_t* __restrict__ status, const __grid_constant__ UmmaMixedOut mixed) {
    extern __shared__ uint8_t smem_raw[];
    pdl_launch_dependents();
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sW1 = base + P.w1, sWdw = base + P.wdw, sW2 = base + P.w2, sY1 = base + P.y1, sY2 = base + P.y2;
    const uint32_t bars = base + P.bars;
    auto bar = [&](uint32_t i) { return bars + 8u * i; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + P.tmem_slot);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + P.abort_flag);
    float* sp = reinterpret_cast<float*>(base_ptr + P.params);  // si1 bi1 so1 [cm] | sid bid sod [cm] | si2 bi2 so2 [c2]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ncm = P.cm / kUnitBlock;
    const uint32_t w1_block = (uint32_t)P.cm * kUnitBlock, w2_block = (uint32_t)P.c2 * kUnitBlock;

    if (threadIdx.x == 0) {
        mbar_init(bar(B_W), 1);
        for (uint32_t s = 0; s < 2; ++s) {
            mbar_init(bar(B_XFULL + s), 1);
            mbar_init(bar(B_XEMPTY + s), 1);
        }
        mbar_init(bar(B_ACC1), 1);
        mbar_init(bar(B_Y1), (uint32_t)P.epi_warps);
        mbar_init(bar(B_ACC2), 1);
        mbar_init(bar(B_Y2), (uint32_t)P.epi_warps);
        mbar_init(bar(B_ACC3), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // the three weight panels do not depend on the previous kernel
        mbar_expect_tx(bar(B_W), (uint32_t)P.nkb1 * w1_block + (uint32_t)ncm * 9u * 1024u + (uint32_t)ncm * w2_block);
        for (int kb = 0; kb < P.nkb1; ++kb) tma_load_2d(&tmW1, bar(B_W), sW1 + kb * w1_block, kb * kUnitBlock, 0);
        for (int i = 0; i < ncm * 9; ++i) tma_load_2d(&tmWdw, bar(B_W), sWdw + i * 1024u, 0, i * kUnitBlock);
        for (int cb = 0; cb < ncm; ++cb) tma_load_2d(&tmW2, bar(B_W), sW2 + cb * w2_block, cb * kUnitBlock, 0);
    }
    for (int i = threadIdx.x; i < P.cm; i += (int)blockDim.x) {
        sp[i] = ep.e1.scale_in[i];
        sp[P.cm + i] = ep.e1.bias[i];
        sp[2 * P.cm + i] = ep.e1.scale_out[i];
        sp[3 * P.cm + i] = ep.edw.scale_in[i];
        sp[4 * P.cm + i] = ep.edw.bias[i];
        sp[5 * P.cm + i] = ep.edw.scale_out[i];
    }
    for (int i = threadIdx.x; i < P.c2; i += (int)blockDim.x) {
        const bool in = i < G.c2pad;
        sp[6 * P.cm + i] = in ? ep.e2.scale_in[i] : 0.f;
        sp[6 * P.cm + P.c2 + i] = in ? ep.e2.bias[i] : 0.f;
        sp[6 * P.cm + 2 * P.c2 + i] = in ? ep.e2.scale_out[i] : 0.f;
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
    const uint32_t t_acc1 = tmem_base, t_acc2 = tmem_base + 2u * P.cm, t_acc3 = tmem_base + 3u * P.cm;
    pdl_wait();  // from here on the kernel reads activations and writes outputs

    const int per_img = P.tiles_x * P.tiles_y;
    const int m_first = blockIdx.x, m_step = gridDim.x;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer: the halo tile of every pixel tile, K block by K block ----
            uint32_t it = 0;
            bool ok = true;
            for (int m = m_first; ok && m < P.m_tiles; m += m_step, ++it) {
                const int img = m / per_img, r = m - img * per_img;
                const int y0 = (r / P.tiles_x) * kUnitTh - 1, x0 = (r % P.tiles_x) * kUnitTw - 1;
                const uint32_t st = it & 1u, ph = (it >> 1) & 1u;
                if (!mbar_wait(bar(B_XEMPTY + st), ph ^ 1u, abort_flag, status, 1u, P.wait_ns)) { ok = false; break; }
                mbar_expect_tx(bar(B_XFULL + st), (uint32_t)P.nkb1 * (uint32_t)(kUnitHaloPixels * kUnitBlock));
                for (int g = 0; g < P.nkb1; ++g)
                    tma_load_4d(&maps.tm[maps.block_src[g]], bar(B_XFULL + st), base + P.x_stage[st] + (uint32_t)g * kUnitHaloBlockBytes,
                                (int)maps.block_x[g], x0, y0, img);
            }
            if (!ok) {
                const unsigned long long t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 1000000ull) {}  // let bulk copies in flight land before shared memory is released
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ----
            bool ok = mbar_wait(bar(B_W), 0, abort_flag, status, 16u, P.wait_ns);
            tc_fence_after();
            uint32_t it1 = 0;  // tiles whose first 1x1 layer has been issued
            auto issue_pw1 = [&]() -> bool {
                const uint32_t st = it1 & 1u, ph = (it1 >> 1) & 1u;
                if (!mbar_wait(bar(B_XFULL + st), ph, abort_flag, status, 2u, P.wait_ns)) return false;
                tc_fence_after();
                const uint32_t xs = base + P.x_stage[st];
#pragma unroll 1
                for (int mb = 0; mb < 2; ++mb)
                    for (int g = 0; g < P.nkb1; ++g)
                        umma_i8(t_acc1 + (uint32_t)(mb * P.cm), make_smem_desc(xs + (uint32_t)g * kUnitHaloBlockBytes + (uint32_t)(mb * kTileM * kUnitBlock), kUnitBlock),
                                make_smem_desc(sW1 + g * w1_block, kUnitBlock), P.idesc1, g != 0 ? 1u : 0u);
                umma_commit(bar(B_XEMPTY + st));
                umma_commit(bar(B_ACC1));
                ++it1;
                return true;
            };
            int m = m_first;
            if (ok && m < P.m_tiles) ok = issue_pw1();
            for (uint32_t ti = 0; ok && m < P.m_tiles; m += m_step, ++ti) {
                const uint32_t ph = ti & 1u;
                // depthwise stage: Y1 of this tile is complete (and with it, every epilogue warp is done with acc1, acc2, acc3)
                if (!mbar_wait(bar(B_Y1), ph, abort_flag, status, 4u, P.wait_ns)) { ok = false; break; }
                tc_fence_after();
                for (int cb = 0; cb < ncm; ++cb) {
                    const uint64_t a0 = make_smem_desc(sY1 + (uint32_t)cb * kUnitHaloBlockBytes, kUnitBlock, kUnitHaloW * kUnitBlock);
                    const uint64_t b0 = make_smem_desc(sWdw + (uint32_t)cb * 9u * 1024u, kUnitBlock);
#pragma unroll
                    for (int tap = 0; tap < 9; ++tap) {
                        const uint32_t a_off = (uint32_t)((tap / 3) * kUnitHaloW + tap % 3) * (kUnitBlock >> 4);  // pixels -> 16-byte units
                        umma_i8(t_acc2 + (uint32_t)(cb * kUnitBlock), a0 + a_off, b0 + (uint32_t)tap * (1024u >> 4), P.idesc_dw, tap != 0 ? 1u : 0u);
                    }
                }
                umma_commit(bar(B_ACC2));
                // the next tile's first layer runs ahead: acc1 is free, its input stage has usually landed
                if (m + m_step < P.m_tiles && !issue_pw1()) { ok = false; break; }
                if (!mbar_wait(bar(B_Y2), ph, abort_flag, status, 4u, P.wait_ns)) { ok = false; break; }
                tc_fence_after();
                for (int cb = 0; cb < ncm; ++cb)
                    umma_i8(t_acc3, make_smem_desc(sY2 + (uint32_t)cb * (kTileM * kUnitBlock), kUnitBlock), make_smem_desc(sW2 + cb * w2_block, kUnitBlock), P.idesc2,
                            cb != 0 ? 1u : 0u);
                umma_commit(bar(B_ACC3));
            }
        }
    } else {
        // ---- epilogue warps ----
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        const int sub = (warp - 2) >> 2;        // which of the warps sharing that quarter
        const int nsub = P.epi_warps >> 2;
        const int row = q * 32 + lane;
        const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
        const float* s1 = sp;
        const float* sd = sp + 3 * P.cm;
        const float* s2 = sp + 6 * P.cm;
        const long plane = (long)G.h * G.w;
        bool ok = true;
        uint32_t ti = 0;
        for (int m = m_first; ok && m < P.m_tiles; m += m_step, ++ti) {
            const uint32_t ph = ti & 1u;
            const int img = m / per_img, r = m - img * per_img;
            const int ty0 = (r / P.tiles_x) * kUnitTh, tx0 = (r % P.tiles_x) * kUnitTw;
            // ---- epilogue 1: acc1 (two blocks of 128 halo pixels) -> Y1 ----
            if (!mbar_wait(bar(B_ACC1), ph, abort_flag, status, 8u, P.wait_ns)) { ok = false; break; }
            tc_fence_after();
#pragma unroll 1
            for (int mb = 0; mb < 2; ++mb) {
                if (mb == 1 && q * 32 >= kUnitHaloPixels - kTileM) continue;  // rows 128 + 32q.. lie past the 180 halo pixels: warp-uniform
                const int p = mb * kTileM + row;
                const int hy = p / kUnitHaloW, hx = p - hy * kUnitHaloW;
                const int iy = ty0 - 1 + hy, ix = tx0 - 1 + hx;
                const bool store = p < kUnitHaloPixels;
                const bool inside = iy >= 0 && iy < G.h && ix >= 0 && ix < G.w;
                for (int c0 = sub * 32; c0 < P.cm; c0 += nsub * 32) {
                    int va[16], vb[16];
                    __syncwarp();
                    tmem_ld16(t_acc1 + lane_sel + (uint32_t)(mb * P.cm + c0), va);
                    tmem_ld16(t_acc1 + lane_sel + (uint32_t)(mb * P.cm + c0 + 16), vb);
                    tmem_wait_ld16(va);
                    tmem_wait_ld16(vb);
                    if (!store) continue;
                    uint32_t wa[4] = {0u, 0u, 0u, 0u}, wb[4] = {0u, 0u, 0u, 0u};
                    if (inside) {
                        requant16<ACT>(va, s1 + c0, s1 + P.cm + c0, s1 + 2 * P.cm + c0, ep.e1.act_param0, wa);
                        requant16<ACT>(vb, s1 + c0 + 16, s1 + P.cm + c0 + 16, s1 + 2 * P.cm + c0 + 16, ep.e1.act_param0, wb);
                    }
                    const uint32_t blk = sY1 + (uint32_t)(c0 >> 5) * kUnitHaloBlockBytes;
                    st_shared_v4(swz32(blk, p, 0), wa[0], wa[1], wa[2], wa[3]);
                    st_shared_v4(swz32(blk, p, 1), wb[0], wb[1], wb[2], wb[3]);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // these generic-proxy stores -> visible to the MMA's reads
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_Y1));
            // ---- epilogue 2: acc2 (depthwise sums of the 128 output pixels) -> Y2 ----
            if (!mbar_wait(bar(B_ACC2), ph, abort_flag, status, 8u, P.wait_ns)) { ok = false; break; }
            tc_fence_after();
            for (int c0 = sub * 32; c0 < P.cm; c0 += nsub * 32) {
                int va[16], vb[16];
                __syncwarp();
                tmem_ld16(t_acc2 + lane_sel + (uint32_t)c0, va);
                tmem_ld16(t_acc2 + lane_sel + (uint32_t)(c0 + 16), vb);
                tmem_wait_ld16(va);
                tmem_wait_ld16(vb);
                uint32_t wa[4], wb[4];
                requant16<ACT_NONE>(va, sd + c0, sd + P.cm + c0, sd + 2 * P.cm + c0, 0.f, wa);
                requant16<ACT_NONE>(vb, sd + c0 + 16, sd + P.cm + c0 + 16, sd + 2 * P.cm + c0 + 16, 0.f, wb);
                const uint32_t blk = sY2 + (uint32_t)(c0 >> 5) * (kTileM * kUnitBlock);
                st_shared_v4(swz32(blk, row, 0), wa[0], wa[1], wa[2], wa[3]);
                st_shared_v4(swz32(blk, row, 1), wb[0], wb[1], wb[2], wb[3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_Y2));
            // ---- epilogue 3: acc3 -> the second 1x1 layer's output ----
            if (!mbar_wait(bar(B_ACC3), ph, abort_flag, status, 8u, P.wait_ns)) { ok = false; break; }
            tc_fence_after();
            const int oy = ty0 + (row >> 3), ox = tx0 + (row & 7);
            store_accumulator_row<ACT, OUT>(t_acc3 + lane_sel, P.c2, sub, nsub, oy < G.h && ox < G.w, img, (long)oy * G.w + ox, plane, s2, s2 + P.c2,
                                            s2 + 2 * P.c2, ep.e2.act_param0, G.c2pad, G.cout2, out, mixed);
            tc_fence_before();
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static const EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            return reinterpret_cast<EncodeTiledFn>(p);
        return nullptr;
    }();
    return fn;
}

uint32_t idesc_for(int n) { return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24); }

template <int ACT, int OUT, bool MULTI>
const char* launch_variant(cudaStream_t stream, int grid, const UnitMaps& maps, const UnitWeights& wts, const UnitPlan& p, const UnitGeom& g,
                           const UnitEpilogues& ep, void* out, uint32_t* status, const UmmaMixedOut& mixed) {
    static std::mutex mu;  // several host threads may drive different GPUs through this function at once
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = unit_umma_kernel<ACT, OUT, MULTI>;
    if (dev >= 0 && dev < 64) {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set[dev]) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
                return "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed";
            attr_set[dev] = true;
        }
    }
    const int threads = 64 + 32 * p.epi_warps;
    if (launch_overlapped(kernel, dim3(grid), dim3(threads), (size_t)p.smem_bytes, stream, maps, *reinterpret_cast<const CUtensorMap*>(wts.map_w1),
                          *reinterpret_cast<const CUtensorMap*>(wts.map_wdw), *reinterpret_cast<const CUtensorMap*>(wts.map_w2), p, g, ep, out, status,
                          mixed) != cudaSuccess)
        return "unit_umma_kernel launch failed";
    return nullptr;
}

}  // namespace

bool unit_plan(int cin1_blocks, int cm_real, int cout2, int smem_budget, UnitPlan* plan) {
    UnitPlan p{};
    if (cin1_blocks < 1 || cin1_blocks > kUmmaMaxGatherBlocks || cm_real < 1 || cout2 < 1) return false;
    p.nkb1 = cin1_blocks;
    p.cm = (cm_real + 31) / 32 * 32;
    p.c2 = (nhwc_channels(cout2) + 31) / 32 * 32;  // the epilogue walks over 32-column chunks
    if (p.cm > 128 || p.c2 > 256) return false;   // acc1 (two blocks), acc2 and acc3 must fit the 512 TMEM columns together
    const int cols = 3 * p.cm + p.c2;
    p.tmem_cols = cols <= 32 ? 32 : cols <= 64 ? 64 : cols <= 128 ? 128 : cols <= 256 ? 256 : 512;
    if (cols > 512) return false;
    p.idesc1 = idesc_for(p.cm);
    p.idesc_dw = idesc_for(kUnitBlock);
    p.idesc2 = idesc_for(p.c2);
    const int ncm = p.cm / kUnitBlock;
    uint32_t off = 0;
    auto take = [&](uint32_t bytes) { const uint32_t at = off; off += (bytes + 1023u) & ~1023u; return at; };
    p.w1 = take((uint32_t)p.nkb1 * p.cm * kUnitBlock);
    p.wdw = take((uint32_t)ncm * 9u * 1024u);
    p.w2 = take((uint32_t)ncm * p.c2 * kUnitBlock);
    // an M = 128 block of the first layer starting at halo pixel 128 reads 128 rows: up to row 255 of the last K block
    const uint32_t x_bytes = (uint32_t)(p.nkb1 - 1) * kUnitHaloBlockBytes + 256u * kUnitBlock;
    p.x_stage[0] = take(x_bytes);
    p.x_stage[1] = take(x_bytes);
    // the last depthwise tap view of the last block reads 128 rows from pixel 22 on, 8-row groups 10 pixels apart: within 180 pixels
    p.y1 = take((uint32_t)ncm * kUnitHaloBlockBytes);
    p.y2 = take((uint32_t)ncm * kTileM * kUnitBlock);
    p.bars = take(8u * B_COUNT + 16u);
    p.tmem_slot = p.bars + 8u * B_COUNT;
    p.abort_flag = p.tmem_slot + 8u;
    p.params = take((uint32_t)(6 * p.cm + 3 * p.c2) * 4u);
    p.total = off;
    p.smem_bytes = (int)p.total + 1024;
    if (p.smem_bytes > smem_budget) return false;
    p.epi_warps = 8;
    const int by_tmem = 512 / p.tmem_cols, by_smem = smem_budget / p.smem_bytes;
    p.ctas_per_sm = by_tmem < by_smem ? by_tmem : by_smem;
    if (p.ctas_per_sm > 2) p.ctas_per_sm = 2;
    if (p.ctas_per_sm < 1) p.ctas_per_sm = 1;
    // pad the shared-memory request so that no more CTAs become resident than TMEM can serve (see dense_umma.cu)
    const int min_smem = smem_budget / (p.ctas_per_sm + 1) + 1;
    if (p.smem_bytes < min_smem) p.smem_bytes = min_smem;
    *plan = p;
    return true;
}

size_t unit_w1_bytes(const UnitPlan& p) { return (size_t)p.cm * p.nkb1 * kUnitBlock; }
size_t unit_wdw_bytes(const UnitPlan& p) { return (size_t)(p.cm / kUnitBlock) * 9 * 1024; }
size_t unit_w2_bytes(const UnitPlan& p) { return (size_t)p.c2 * p.cm; }

void unit_pack_w1(const UnitPlan& p, const int8_t* w_korder, int cout1, int8_t* dst) {
    const long kt = (long)p.nkb1 * kUnitBlock;
    for (long i = 0; i < (long)p.cm * kt; ++i) dst[i] = 0;
    for (int o = 0; o < cout1; ++o)
        for (long k = 0; k < kt; ++k) dst[o * kt + k] = w_korder[o * kt + k];
}

void unit_pack_wdw(const UnitPlan& p, const int8_t* w_dw, int c, int8_t* dst) {
    const size_t total = unit_wdw_bytes(p);
    for (size_t i = 0; i < total; ++i) dst[i] = 0;
    for (int ch = 0; ch < c; ++ch) {
        const int cb = ch / kUnitBlock, n = ch % kUnitBlock;
        for (int tap = 0; tap < 9; ++tap) dst[((size_t)(cb * 9 + tap) * kUnitBlock + n) * kUnitBlock + n] = w_dw[ch * 9 + tap];
    }
}

void unit_pack_w2(const UnitPlan& p, const int8_t* w2, int cout2, int cin2, int8_t* dst) {
    for (long i = 0; i < (long)p.c2 * p.cm; ++i) dst[i] = 0;
    for (int o = 0; o < cout2; ++o)
        for (int c = 0; c < cin2; ++c) dst[(long)o * p.cm + c] = w2[(long)o * cin2 + c];
}

const char* unit_encode_weight_maps(const UnitPlan& p, const int8_t* w1_dev, const int8_t* wdw_dev, const int8_t* w2_dev, UnitWeights* out) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return "cuTensorMapEncodeTiled entry point not available";
    cuuint32_t estr[2] = {1, 1};
    auto encode2d = [&](unsigned char* map, const int8_t* ptr, cuuint64_t inner, cuuint64_t rows, cuuint32_t box_rows) {
        cuuint64_t dims[2] = {inner, rows};
        cuuint64_t strides[1] = {inner};
        cuuint32_t box[2] = {(cuuint32_t)kUnitBlock, box_rows};
        return enc(reinterpret_cast<CUtensorMap*>(map), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    };
    if (encode2d(out->map_w1, w1_dev, (cuuint64_t)p.nkb1 * kUnitBlock, (cuuint64_t)p.cm, (cuuint32_t)p.cm) != CUDA_SUCCESS) return "cuTensorMapEncodeTiled(w1) failed";
    if (encode2d(out->map_wdw, wdw_dev, (cuuint64_t)kUnitBlock, (cuuint64_t)(p.cm / kUnitBlock) * 9 * kUnitBlock, (cuuint32_t)kUnitBlock) != CUDA_SUCCESS)
        return "cuTensorMapEncodeTiled(wdw) failed";
    if (encode2d(out->map_w2, w2_dev, (cuuint64_t)p.cm, (cuuint64_t)p.c2, (cuuint32_t)p.c2) != CUDA_SUCCESS) return "cuTensorMapEncodeTiled(w2) failed";
    return nullptr;
}

const char* launch_unit_umma(cudaStream_t stream, int sm_count, const UnitPlan& plan_in, const UnitWeights& wts, const UmmaSources& sources, int n, int h,
                             int w, int cout2, const UnitEpilogues& ep, void* out, int out_dtype, uint32_t* status, const UmmaMixedOut* mixed_in,
                             unsigned long long wait_limit_ns) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return "cuTensorMapEncodeTiled entry point not available";
    if (n == 0) return nullptr;
    if (out_dtype != DT_S8_NHWC && out_dtype != DT_F32_NCHW) return "the fused unit writes int8 NHWC or fp32 NCHW";
    if (mixed_in && (out_dtype != DT_S8_NHWC || mixed_in->n_chunks > 0)) return "the fused unit has no scattered output";
    UnitPlan p = plan_in;
    p.wait_ns = wait_limit_ns;
    p.tiles_x = (w + kUnitTw - 1) / kUnitTw;
    p.tiles_y = (h + kUnitTh - 1) / kUnitTh;
    p.m_tiles = n * p.tiles_x * p.tiles_y;
    UnitMaps km;
    if (sources.n_src < 1 || sources.n_src > kUmmaMaxSources) return "bad source count";
    cuuint32_t estr[4] = {1, 1, 1, 1};
    for (int i = 0; i < sources.n_src; ++i) {
        const cuuint64_t cp = (cuuint64_t)sources.src_cpad[i];
        cuuint64_t dims[4] = {cp, (cuuint64_t)w, (cuuint64_t)h, (cuuint64_t)n};
        cuuint64_t strides[3] = {cp, cp * w, cp * w * h};
        cuuint32_t box[4] = {(cuuint32_t)kUnitBlock, (cuuint32_t)kUnitHaloW, (cuuint32_t)kUnitHaloH, 1};
        if (enc(&km.tm[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)sources.src[i], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return "cuTensorMapEncodeTiled(activations) failed";
    }
    for (int kb = 0; kb < p.nkb1; ++kb) {
        km.block_x[kb] = sources.block_x[kb];
        km.block_src[kb] = sources.block_src[kb];
    }
    UnitGeom g{n, h, w, cout2, nhwc_channels(cout2)};
    UmmaMixedOut mixed{};
    if (mixed_in) mixed = *mixed_in;
    int grid = sm_count * p.ctas_per_sm;
    if (grid > p.m_tiles) grid = p.m_tiles;
    const int act = ep.e1.act_type;
    const char* err = nullptr;
#define OTT_UNIT_LAUNCH(ACT, OUT)                                                                                           \
    err = p.ctas_per_sm > 1 ? launch_variant<ACT, OUT, true>(stream, grid, km, wts, p, g, ep, out, status, mixed)             \
                            : launch_variant<ACT, OUT, false>(stream, grid, km, wts, p, g, ep, out, status, mixed)
#define OTT_UNIT_ACT(OUT)                                       \
    switch (act) {                                              \
        case ACT_RELU: OTT_UNIT_LAUNCH(ACT_RELU, OUT); break;   \
        case ACT_LRELU: OTT_UNIT_LAUNCH(ACT_LRELU, OUT); break; \
        case ACT_RELU6: OTT_UNIT_LAUNCH(ACT_RELU6, OUT); break; \
        default: OTT_UNIT_LAUNCH(ACT_NONE, OUT); break;         \
    }
    if (out_dtype == DT_F32_NCHW) { OTT_UNIT_ACT(DT_F32_NCHW) } else { OTT_UNIT_ACT(DT_S8_NHWC) }
#undef OTT_UNIT_ACT
#undef OTT_UNIT_LAUNCH
    if (err) return err;
    return cudaGetLastError() == cudaSuccess ? nullptr : "unit_umma_kernel launch failed";
}

}  // namespace ottk
