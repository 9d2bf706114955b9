// Depthwise 3x3 (stride 1 or 2, pad 1) followed by a 1x1 convolution, each with its fused requantize / dequantize epilogue, as
// one kernel: two consecutive ConvolutionLayer::forward_int8 calls (Tensor/ConvolutionLayer.cpp:754-847; in the reference's
// shipped int8 graph the pairs conv_5 -> conv_6, conv_8 -> conv_9, ... : int8_scale_term 101 then 2). Run as two launches the
// int8 tensor between them crosses HBM twice and both launches pay their own fill and drain; here it stays in shared memory.
//
//   per tile of 8 x 16 output pixels
//   X    TMA: the input pixels under the tile and its halo, 32-channel blocks (from one tensor, or gathered from several), in
//        chunks of `bpc` blocks through a ring of shared-memory stages (out-of-image pixels arrive as zeros); stride 2 as two
//        boxes taking every other column, exactly as in dw_umma.cu
//   1    tcgen05.mma: accD[128 px, 32 ch] per block = sum over the nine taps of A_tap * diag(w[:, tap])    (M 128, N 32, K 32)
//        epilogue A: requantize (the depthwise layer's scales, bias; rounding rule add-half-truncate) -> Y in shared memory,
//        laid out as the K-major operand of the next MMA
//   2    tcgen05.mma: accP[128 px, c2] = Y * W2^T, one MMA per 32-channel block
//        epilogue B: the 1x1 layer's ordinary output stage (int8 NHWC with per-channel scales, chosen channels also as fp32
//        planes; or fp32 NCHW)
//
// All sums are exact s32 and both epilogues are the arithmetic of the separate layers, so the result equals theirs bit for bit.
// Warp roles: warp 0 = TMA producer (one lane); warp 1 = TMEM owner and MMA issuers (lane l issues the depthwise MMAs of
// block l of each chunk, lane 0 also the 1x1 layer's); warps 2.. = epilogue (warp w reads TMEM lanes 32*(w%4)..+31, the two
// warps of a lane quarter split the columns). The issuers run the depthwise stage of tile t+1 before the 1x1 stage of tile t,
// and the epilogue warps run A(t+1) before B(t), so that with two accumulators of each kind the tensor pipe never waits for an
// epilogue. Every wait is bounded, as in dense_umma.cu.
#include <cuda.h>

#include <mutex>

#include "dwpw_umma.h"
#include "launch.cuh"
#include "umma_epilogue.cuh"
#include "umma_primitives.cuh"

namespace ottk {

namespace {

using namespace umma;
constexpr int kTileM = 128, kTw = 8, kTh = 16, kBlock = 32;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr uint32_t kYBlockBytes = kTileM * kBlock;  // one 32-channel block of the operand tile between the layers

struct DwPwMaps {
    CUtensorMap tm[kUmmaMaxSources];
    uint16_t block_x[kUmmaMaxGatherBlocks];
    uint8_t block_src[kUmmaMaxGatherBlocks];
};

struct DwPwGeom {
    int n, h, w, oh, ow;
    int dw_cpad;        // channel stride of the depthwise layer's parameter arrays (entries past it read as zero)
    int cout2, c2pad;   // the 1x1 layer's real output channels and the channel stride of its int8 output tensor
};

// barrier slots (8 bytes each)
enum : uint32_t { B_W = 0, B_FULL = 1, B_EMPTY = B_FULL + kDwPwStagesMax, B_DFULL = B_EMPTY + kDwPwStagesMax, B_DEMPTY = B_DFULL + 2, B_YFULL = B_DEMPTY + 2,
                  B_YEMPTY = B_YFULL + 2, B_PFULL = B_YEMPTY + 2, B_PEMPTY = B_PFULL + 2, B_COUNT = B_PEMPTY + 2 };

template <int ACT, int OUT, bool MULTI>
__global__ void __launch_bounds__(kThreads, MULTI ? 2 : 1)
dwpw_umma_kernel(const __grid_constant__ DwPwMaps maps, const __grid_constant__ CUtensorMap tmWdw, const __grid_constant__ CUtensorMap tmWpw, const DwPwPlan P,
                 const DwPwGeom G, const DwPwEpilogues ep, void* __restrict__ out, uint32_t* __restrict__ status, const __grid_constant__ UmmaMixedOut mixed) {
    extern __shared__ uint8_t smem_raw[];
    pdl_launch_dependents();
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sWdw = base + P.w_dw, sWpw = base + P.w_pw, sX = base + P.x, sY = base + P.y;
    const uint32_t bars = base + P.bars;
    auto bar = [&](uint32_t i) { return bars + 8u * i; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + P.tmem_slot);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + P.abort_flag);
    float* sp = reinterpret_cast<float*>(base_ptr + P.params);  // sid bid sod [dwcols] | si2 bi2 so2 [c2]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t wpw_block = (uint32_t)P.c2 * kBlock;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmWdw);
        prefetch_tensormap(&tmWpw);
        for (int cb = 0; cb < P.ncb; ++cb) prefetch_tensormap(&maps.tm[maps.block_src[cb]]);
        mbar_init(bar(B_W), 1);
        for (int i = 0; i < P.stages; ++i) {
            mbar_init(bar(B_FULL + i), 1);
            mbar_init(bar(B_EMPTY + i), (uint32_t)P.bpc);  // one commit per issuing lane
        }
        for (uint32_t i = 0; i < 2; ++i) {
            mbar_init(bar(B_DFULL + i), (uint32_t)P.bpc);
            mbar_init(bar(B_DEMPTY + i), kEpiWarps);
            mbar_init(bar(B_YFULL + i), kEpiWarps);
            mbar_init(bar(B_YEMPTY + i), 1);
            mbar_init(bar(B_PFULL + i), 1);
            mbar_init(bar(B_PEMPTY + i), kEpiWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // both weight panels do not depend on the previous kernel
        mbar_expect_tx(bar(B_W), (uint32_t)P.ncb * 9u * 1024u + (uint32_t)P.ncb * wpw_block);
        for (int i = 0; i < P.ncb * 9; ++i) tma_load_2d(&tmWdw, bar(B_W), sWdw + i * 1024u, 0, i * kBlock);
        for (int cb = 0; cb < P.ncb; ++cb) tma_load_2d(&tmWpw, bar(B_W), sWpw + cb * wpw_block, cb * kBlock, 0);
    }
    for (int i = threadIdx.x; i < P.dwcols; i += (int)blockDim.x) {
        const bool in = i < G.dw_cpad;
        sp[i] = in ? ep.dw.scale_in[i] : 0.f;
        sp[P.dwcols + i] = in ? ep.dw.bias[i] : 0.f;
        sp[2 * P.dwcols + i] = in ? ep.dw.scale_out[i] : 0.f;
    }
    for (int i = threadIdx.x; i < P.c2; i += (int)blockDim.x) {
        const bool in = i < G.c2pad;
        sp[3 * P.dwcols + i] = in ? ep.pw.scale_in[i] : 0.f;
        sp[3 * P.dwcols + P.c2 + i] = in ? ep.pw.bias[i] : 0.f;
        sp[3 * P.dwcols + 2 * P.c2 + i] = in ? ep.pw.scale_out[i] : 0.f;
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
    const uint32_t t_dw = tmem_base, t_pw = tmem_base + (uint32_t)(P.dw_bufs * P.dwcols);
    pdl_wait();  // from here on the kernel reads activations and writes outputs

    const int per_img = P.tiles_x * P.tiles_y;
    const int m_first = blockIdx.x, m_step = gridDim.x;
    const int n_mine = m_first < P.m_tiles ? (P.m_tiles - m_first + m_step - 1) / m_step : 0;
    const uint32_t dmask = (uint32_t)P.dw_bufs - 1u, ymask = (uint32_t)P.y_bufs - 1u, pmask = (uint32_t)P.pw_bufs - 1u;
    // log2 of the buffer counts (1 or 2 each): use count of a buffer = t >> shift
    const uint32_t dsh = dmask, ysh = ymask, psh = pmask;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer: per tile, the chunks of channel blocks ----
            uint32_t cnt = 0;
            bool ok = true;
            for (int m = m_first; ok && m < P.m_tiles; m += m_step) {
                const int img = m / per_img, r = m - img * per_img;
                const int y0 = (r / P.tiles_x) * kTh * P.stride - 1, x0 = (r % P.tiles_x) * kTw * P.stride - 1;
                for (int c = 0; c < P.nchunks; ++c, ++cnt) {
                    const uint32_t st = cnt % (uint32_t)P.stages, ph = (cnt / (uint32_t)P.stages) & 1u;
                    if (!mbar_wait(bar(B_EMPTY + st), ph ^ 1u, abort_flag, status, 1u, P.wait_ns)) { ok = false; break; }
                    const int cb0 = c * P.bpc;
                    const int nb = P.ncb - cb0 < P.bpc ? P.ncb - cb0 : P.bpc;
                    mbar_expect_tx(bar(B_FULL + st), (uint32_t)(nb * P.sets * P.set_load_bytes));
                    for (int b = 0; b < nb; ++b)
                        for (int s = 0; s < P.sets; ++s)
                            tma_load_4d(&maps.tm[maps.block_src[cb0 + b]], bar(B_FULL + st),
                                        sX + st * (uint32_t)P.chunk_bytes + (uint32_t)(b * P.block_bytes + s * P.set_bytes), (int)maps.block_x[cb0 + b], x0 + s, y0,
                                        img);
                }
            }
            if (!ok) {
                const unsigned long long t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 1000000ull) {}  // let bulk copies in flight land before shared memory is released
            }
        }
    } else if (warp == 1) {
        if (lane < P.bpc) {
            // ---- MMA issuers ----
            bool ok = mbar_wait(bar(B_W), 0, abort_flag, status, 16u, P.wait_ns);
            tc_fence_after();
            const uint32_t sbo = (uint32_t)(P.stride * P.set_w * kBlock);
            // offset of each tap's shifted input view inside a block, in 16-byte units (stride 2: the taps kx = 1 read the second
            // column set, kx = 2 one column on), worked out once
            uint32_t aoff[9];
#pragma unroll
            for (int tap = 0; tap < 9; ++tap) {
                const int ky = tap / 3, kx = tap % 3;
                const int col = P.stride == 1 ? kx : (kx >> 1);
                aoff[tap] = (uint32_t)((ky * P.set_w + col) * (kBlock >> 4)) + ((P.stride == 2 && kx == 1) ? (uint32_t)(P.set_bytes >> 4) : 0u);
            }
            uint32_t cnt = 0;
            // depthwise stage of this CTA's tile number t: lane l issues the nine taps of block l of every chunk
            auto issue_dw = [&](uint32_t t) -> bool {
                const uint32_t buf = t & dmask, use = t >> dsh;
                if (!mbar_wait(bar(B_DEMPTY + buf), (use & 1u) ^ 1u, abort_flag, status, 4u, P.wait_ns)) return false;
                for (int c = 0; c < P.nchunks; ++c, ++cnt) {
                    const uint32_t st = cnt % (uint32_t)P.stages, ph = (cnt / (uint32_t)P.stages) & 1u;
                    if (!mbar_wait(bar(B_FULL + st), ph, abort_flag, status, 2u, P.wait_ns)) return false;
                    tc_fence_after();
                    const int cb = c * P.bpc + lane;
                    if (cb < P.ncb) {
                        const uint32_t d = t_dw + buf * (uint32_t)P.dwcols + (uint32_t)(cb * kBlock);
                        const uint32_t blk = sX + st * (uint32_t)P.chunk_bytes + (uint32_t)(lane * P.block_bytes);
                        const uint64_t b0 = make_smem_desc(sWdw + (uint32_t)cb * 9u * 1024u, kBlock);
                        const uint64_t a_base = make_smem_desc(blk, kBlock, (int)sbo);
                        const uint32_t a_lo = (uint32_t)a_base;
                        const uint64_t a_hi = a_base & 0xFFFFFFFF00000000ull;
#pragma unroll
                        for (int tap = 0; tap < 9; ++tap)
                            umma_i8(d, a_hi | (uint64_t)(a_lo + aoff[tap]), b0 + (uint32_t)tap * (1024u >> 4), P.idesc_dw, tap != 0 ? 1u : 0u);
                    }
                    umma_commit(bar(B_EMPTY + st));
                }
                umma_commit(bar(B_DFULL + buf));
                return true;
            };
            // 1x1 stage of tile t: lane 0 alone
            auto issue_pw = [&](uint32_t t) -> bool {
                const uint32_t yb = t & ymask, pb = t & pmask;
                if (!mbar_wait(bar(B_YFULL + yb), (t >> ysh) & 1u, abort_flag, status, 32u, P.wait_ns)) return false;
                if (!mbar_wait(bar(B_PEMPTY + pb), ((t >> psh) & 1u) ^ 1u, abort_flag, status, 64u, P.wait_ns)) return false;
                tc_fence_after();
                const uint32_t d = t_pw + pb * (uint32_t)P.c2;
                const uint32_t yt = sY + yb * (uint32_t)P.ncb * kYBlockBytes;
                for (int cb = 0; cb < P.ncb; ++cb)
                    umma_i8(d, make_smem_desc(yt + (uint32_t)cb * kYBlockBytes, kBlock), make_smem_desc(sWpw + (uint32_t)cb * wpw_block, kBlock), P.idesc_pw,
                            cb != 0 ? 1u : 0u);
                umma_commit(bar(B_YEMPTY + yb));
                umma_commit(bar(B_PFULL + pb));
                return true;
            };
            if (ok && n_mine > 0) ok = issue_dw(0);
            for (uint32_t t = 0; ok && t < (uint32_t)n_mine; ++t) {
                if (t + 1 < (uint32_t)n_mine) ok = issue_dw(t + 1);
                if (ok && lane == 0) ok = issue_pw(t);
            }
        }
    } else {
        // ---- epilogue warps ----
        const int q = warp & 3, sub = (warp - 2) >> 2, nsub = kEpiWarps >> 2;
        const int row = q * 32 + lane;
        const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
        const float* sd = sp;
        const float* s2 = sp + 3 * P.dwcols;
        const long plane = (long)G.oh * G.ow;
        // A: depthwise accumulators of tile t -> requantized operand tile Y
        auto epi_a = [&](uint32_t t) -> bool {
            const uint32_t buf = t & dmask, yb = t & ymask;
            if (!mbar_wait(bar(B_DFULL + buf), (t >> dsh) & 1u, abort_flag, status, 8u, P.wait_ns)) return false;
            if (!mbar_wait(bar(B_YEMPTY + yb), ((t >> ysh) & 1u) ^ 1u, abort_flag, status, 128u, P.wait_ns)) return false;
            tc_fence_after();
            const uint32_t acc = t_dw + buf * (uint32_t)P.dwcols + lane_sel;
            const uint32_t yt = sY + yb * (uint32_t)P.ncb * kYBlockBytes;
            for (int c0 = sub * 32; c0 < P.dwcols; c0 += nsub * 32) {
                int va[16], vb[16];
                __syncwarp();
                tmem_ld16(acc + (uint32_t)c0, va);
                tmem_ld16(acc + (uint32_t)(c0 + 16), vb);
                tmem_wait_ld16(va);
                tmem_wait_ld16(vb);
                uint32_t wa[4], wb[4];
                requant16<ACT_NONE>(va, sd + c0, sd + P.dwcols + c0, sd + 2 * P.dwcols + c0, 0.f, wa);
                requant16<ACT_NONE>(vb, sd + c0 + 16, sd + P.dwcols + c0 + 16, sd + 2 * P.dwcols + c0 + 16, 0.f, wb);
                const uint32_t blk = yt + (uint32_t)(c0 >> 5) * kYBlockBytes;
                st_shared_v4(swz32(blk, row, 0), wa[0], wa[1], wa[2], wa[3]);
                st_shared_v4(swz32(blk, row, 1), wb[0], wb[1], wb[2], wb[3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // these generic-proxy stores -> visible to the MMA's reads
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar(B_DEMPTY + buf));
                mbar_arrive(bar(B_YFULL + yb));
            }
            return true;
        };
        // B: the 1x1 layer's accumulators of tile t -> its output
        auto epi_b = [&](uint32_t t) -> bool {
            const uint32_t pb = t & pmask;
            if (!mbar_wait(bar(B_PFULL + pb), (t >> psh) & 1u, abort_flag, status, 256u, P.wait_ns)) return false;
            tc_fence_after();
            const int m = m_first + (int)t * m_step;
            const int img = m / per_img, r = m - img * per_img;
            const int oy = (r / P.tiles_x) * kTh + (row >> 3), ox = (r % P.tiles_x) * kTw + (row & 7);
            store_accumulator_row<ACT, OUT>(t_pw + pb * (uint32_t)P.c2 + lane_sel, P.c2, sub, nsub, oy < G.oh && ox < G.ow, img, (long)oy * G.ow + ox, plane, s2,
                                            s2 + P.c2, s2 + 2 * P.c2, ep.pw.act_param0, G.c2pad, G.cout2, out, mixed);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_PEMPTY + pb));
            return true;
        };
        bool ok = n_mine > 0 ? epi_a(0) : true;
        for (uint32_t t = 0; ok && t < (uint32_t)n_mine; ++t) {
            if (t + 1 < (uint32_t)n_mine) ok = epi_a(t + 1);
            if (ok) ok = epi_b(t);
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
const char* launch_variant(cudaStream_t stream, int grid, const DwPwMaps& maps, const DwPwWeights& wts, const DwPwPlan& p, const DwPwGeom& g,
                           const DwPwEpilogues& ep, void* out, uint32_t* status, const UmmaMixedOut& mixed) {
    static std::mutex mu;  // several host threads may drive different GPUs through this function at once
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = dwpw_umma_kernel<ACT, OUT, MULTI>;
    if (dev >= 0 && dev < 64) {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set[dev]) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
                return "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed";
            attr_set[dev] = true;
        }
    }
    if (launch_overlapped(kernel, dim3(grid), dim3(kThreads), (size_t)p.smem_bytes, stream, maps, *reinterpret_cast<const CUtensorMap*>(wts.map_wdw),
                          *reinterpret_cast<const CUtensorMap*>(wts.map_wpw), p, g, ep, out, status, mixed) != cudaSuccess)
        return "dwpw_umma_kernel launch failed";
    return nullptr;
}

// shared-memory layout and TMEM budget for given buffer counts; false if it does not fit `budget`
bool layout(DwPwPlan& p, int budget) {
    p.chunk_bytes = p.bpc * p.block_bytes;
    p.nchunks = (p.ncb + p.bpc - 1) / p.bpc;
    const int cols = p.dw_bufs * p.dwcols + p.pw_bufs * p.c2;
    if (cols > 512) return false;
    p.tmem_cols = cols <= 32 ? 32 : cols <= 64 ? 64 : cols <= 128 ? 128 : cols <= 256 ? 256 : 512;
    uint32_t off = 0;
    auto take = [&](uint32_t bytes) { const uint32_t at = off; off += (bytes + 1023u) & ~1023u; return at; };
    p.w_dw = take((uint32_t)p.ncb * 9u * 1024u);
    p.w_pw = take((uint32_t)p.ncb * (uint32_t)p.c2 * kBlock);
    p.y = take((uint32_t)p.y_bufs * (uint32_t)p.ncb * kYBlockBytes);
    p.bars = take(8u * B_COUNT + 16u);
    p.tmem_slot = p.bars + 8u * B_COUNT;
    p.abort_flag = p.tmem_slot + 8u;
    p.params = take((uint32_t)(3 * p.dwcols + 3 * p.c2) * 4u);
    p.x = off;
    const int left = budget - 1024 - (int)off;
    if (left < 2 * p.chunk_bytes) return false;
    p.stages = left / p.chunk_bytes;
    if (p.stages > kDwPwStagesMax) p.stages = kDwPwStagesMax;
    // at least one whole tile in flight beyond the one being consumed, where that is cheap
    off += (uint32_t)p.stages * (uint32_t)p.chunk_bytes;
    p.smem_bytes = (int)off + 1024;
    return true;
}

}  // namespace

bool dwpw_plan(int dw_channels, int stride, int pw_cout, int smem_budget, DwPwPlan* plan) {
    DwPwPlan p{};
    if (dw_channels < 1 || pw_cout < 1 || (stride != 1 && stride != 2)) return false;
    p.stride = stride;
    p.ncb = (dw_channels + kBlock - 1) / kBlock;
    p.dwcols = p.ncb * kBlock;
    p.c2 = (nhwc_channels(pw_cout) + 31) / 32 * 32;  // the output stage walks over 32-column chunks
    if (p.ncb > 8 || p.c2 > 256) return false;
    p.idesc_dw = idesc_for(kBlock);
    p.idesc_pw = idesc_for(p.c2);
    if (stride == 1) {
        p.sets = 1; p.set_w = kTw + 2; p.tile_rows = kTh + 2;
    } else {
        p.sets = 2; p.set_w = kTw + 1; p.tile_rows = 2 * kTh + 1;
    }
    p.set_load_bytes = p.set_w * p.tile_rows * kBlock;
    p.set_bytes = (p.set_load_bytes + 1023) / 1024 * 1024;
    p.block_bytes = p.sets * p.set_bytes;
    // Preferred: everything double-buffered and two CTAs per SM (narrow layers); then double-buffered with one CTA; then
    // single accumulators (the widest layers: 256 + 256 columns).
    const int bpc_pref = stride == 1 ? (p.ncb < 4 ? p.ncb : 4) : (p.ncb < 2 ? p.ncb : 2);
    bool found = false;
    for (int attempt = 0; attempt < 3 && !found; ++attempt) {
        p.dw_bufs = p.pw_bufs = p.y_bufs = attempt < 2 ? 2 : 1;
        const int ctas = attempt == 0 ? 2 : 1;
        if (ctas * (p.dw_bufs * p.dwcols + p.pw_bufs * p.c2) > 512) continue;
        for (int bpc = bpc_pref; bpc >= 1 && !found; bpc >>= 1) {
            p.bpc = bpc;
            if (!layout(p, smem_budget / ctas)) continue;
            // the ring should hold more than one tile's chunks unless a tile is a single chunk and there are three stages
            if (p.stages < 2) continue;
            p.ctas_per_sm = ctas;
            found = true;
        }
    }
    if (!found) return false;
    if (p.ctas_per_sm * p.tmem_cols > 512) p.ctas_per_sm = 1;
    // pad the request so that no more CTAs become resident than TMEM can serve (see dense_umma.cu)
    const int min_smem = smem_budget / (p.ctas_per_sm + 1) + 1;
    if (p.smem_bytes < min_smem) p.smem_bytes = min_smem;
    if (p.smem_bytes > smem_budget) return false;
    *plan = p;
    return true;
}

size_t dwpw_wdw_bytes(const DwPwPlan& p) { return (size_t)p.ncb * 9 * 1024; }
size_t dwpw_wpw_bytes(const DwPwPlan& p) { return (size_t)p.c2 * p.dwcols; }

void dwpw_pack_wdw(const DwPwPlan& p, const int8_t* w_dw, int channels, int8_t* dst) {
    const size_t total = dwpw_wdw_bytes(p);
    for (size_t i = 0; i < total; ++i) dst[i] = 0;
    for (int ch = 0; ch < channels && ch < p.dwcols; ++ch) {
        const int cb = ch / kBlock, n = ch % kBlock;
        for (int tap = 0; tap < 9; ++tap) dst[((size_t)(cb * 9 + tap) * kBlock + n) * kBlock + n] = w_dw[ch * 9 + tap];
    }
}

const char* dwpw_encode_weight_maps(const DwPwPlan& p, const int8_t* wdw_dev, const int8_t* wpw_dev, DwPwWeights* out) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return "cuTensorMapEncodeTiled entry point not available";
    cuuint32_t estr[2] = {1, 1};
    auto encode2d = [&](unsigned char* map, const int8_t* ptr, cuuint64_t inner, cuuint64_t rows, cuuint32_t box_rows) {
        cuuint64_t dims[2] = {inner, rows};
        cuuint64_t strides[1] = {inner};
        cuuint32_t box[2] = {(cuuint32_t)kBlock, box_rows};
        return enc(reinterpret_cast<CUtensorMap*>(map), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    };
    if (encode2d(out->map_wdw, wdw_dev, (cuuint64_t)kBlock, (cuuint64_t)p.ncb * 9 * kBlock, (cuuint32_t)kBlock) != CUDA_SUCCESS)
        return "cuTensorMapEncodeTiled(depthwise weights) failed";
    if (encode2d(out->map_wpw, wpw_dev, (cuuint64_t)p.dwcols, (cuuint64_t)p.c2, (cuuint32_t)p.c2) != CUDA_SUCCESS) return "cuTensorMapEncodeTiled(1x1 weights) failed";
    return nullptr;
}

const char* launch_dwpw_umma(cudaStream_t stream, int sm_count, const DwPwPlan& plan_in, const DwPwWeights& wts, const ConvShape& s, const int8_t* x,
                             const UmmaSources* sources, int pw_cout, const DwPwEpilogues& ep, void* out, int out_dtype, uint32_t* status,
                             const UmmaMixedOut* mixed_in, unsigned long long wait_limit_ns) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return "cuTensorMapEncodeTiled entry point not available";
    if (s.n == 0) return nullptr;
    if (out_dtype != DT_S8_NHWC && out_dtype != DT_F32_NCHW) return "the fused depthwise + 1x1 kernel writes int8 NHWC or fp32 NCHW";
    if (mixed_in && (out_dtype != DT_S8_NHWC || mixed_in->n_chunks > 0)) return "the fused depthwise + 1x1 kernel has no scattered output";
    DwPwPlan p = plan_in;
    p.wait_ns = wait_limit_ns;
    p.tiles_x = (s.ow + kTw - 1) / kTw;
    p.tiles_y = (s.oh + kTh - 1) / kTh;
    p.m_tiles = s.n * p.tiles_x * p.tiles_y;
    DwPwMaps km;
    const int n_src = sources ? sources->n_src : 1;
    if (n_src < 1 || n_src > kUmmaMaxSources) return "bad source count";
    // stride 2: the box spans 17 columns and the traversal takes every other one (9 land in shared memory)
    cuuint32_t box[4] = {(cuuint32_t)kBlock, (cuuint32_t)(p.stride == 1 ? p.set_w : 2 * p.set_w - 1), (cuuint32_t)p.tile_rows, 1};
    cuuint32_t estr[4] = {1, (cuuint32_t)p.stride, 1, 1};
    for (int i = 0; i < n_src; ++i) {
        const cuuint64_t cp = (cuuint64_t)(sources ? sources->src_cpad[i] : s.cin_pad);
        const void* base = sources ? (const void*)sources->src[i] : (const void*)x;
        cuuint64_t dims[4] = {cp, (cuuint64_t)s.w, (cuuint64_t)s.h, (cuuint64_t)s.n};
        cuuint64_t strides[3] = {cp, cp * s.w, cp * s.w * s.h};
        if (enc(&km.tm[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return "cuTensorMapEncodeTiled(activations) failed";
    }
    for (int b = 0; b < p.ncb; ++b) {
        km.block_x[b] = sources ? sources->block_x[b] : (uint16_t)(b * kBlock);
        km.block_src[b] = sources ? sources->block_src[b] : (uint8_t)0;
    }
    DwPwGeom g{s.n, s.h, s.w, s.oh, s.ow, s.cout_pad, pw_cout, nhwc_channels(pw_cout)};
    UmmaMixedOut mixed{};
    if (mixed_in) mixed = *mixed_in;
    int grid = sm_count * p.ctas_per_sm;
    if (grid > p.m_tiles) grid = p.m_tiles;
    const char* err = nullptr;
#define OTT_DWPW_LAUNCH(ACT, OUT)                                                                                          \
    err = p.ctas_per_sm > 1 ? launch_variant<ACT, OUT, true>(stream, grid, km, wts, p, g, ep, out, status, mixed)            \
                            : launch_variant<ACT, OUT, false>(stream, grid, km, wts, p, g, ep, out, status, mixed)
#define OTT_DWPW_ACT(OUT)                                       \
    switch (ep.pw.act_type) {                                   \
        case ACT_RELU: OTT_DWPW_LAUNCH(ACT_RELU, OUT); break;   \
        case ACT_LRELU: OTT_DWPW_LAUNCH(ACT_LRELU, OUT); break; \
        case ACT_RELU6: OTT_DWPW_LAUNCH(ACT_RELU6, OUT); break; \
        default: OTT_DWPW_LAUNCH(ACT_NONE, OUT); break;         \
    }
    if (out_dtype == DT_F32_NCHW) { OTT_DWPW_ACT(DT_F32_NCHW) } else { OTT_DWPW_ACT(DT_S8_NHWC) }
#undef OTT_DWPW_ACT
#undef OTT_DWPW_LAUNCH
    if (err) return err;
    return cudaGetLastError() == cudaSuccess ? nullptr : "dwpw_umma_kernel launch failed";
}

}  // namespace ottk
