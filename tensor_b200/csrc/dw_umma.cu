// Depthwise 3x3 int8 convolution (stride 1 or 2, pad 1) on the tensor cores, for int8 NHWC input:
// depthwise_conv2d_int8_x86_pack8_out (Tensor/DepthwiseConvKernelInt8X86Pack.cpp:19-119) with the layer's epilogue
// (Tensor/QuantizeX86.cpp:1723-1870 requantize, :851-903 dequantize) fused.
//
// The CUDA-core kernel (depthwise_tiled.cuh) needs its pixels as consecutive bytes per channel for dp4a, so with channel-
// innermost activations it spends most of its instructions on byte transposes on the way in and out. Here the layout is
// used as it lies: per 32-channel block the multiply-adds of filter tap (ky, kx) are one tcgen05.mma
//   acc[128 pixels, 32 channels] += A_tap[128 pixels, 32 channels] * diag(w[:, ky, kx])          (M 128, N 32, K 32)
// whose A operand is the TMA-loaded input tile seen through a view shifted by the tap, and whose B operand is a 32 x 32
// matrix holding the tap's weights on its diagonal. 31 of 32 products are with zeros; the tensor pipe has that much to spare
// and the sums stay exact s32. What is left for the CUDA cores is the ordinary epilogue, one accumulator row per thread.
//
// Tile: 8 x 16 output pixels (a tile row = one 8-row operand group; groups one input row (stride 2: two) apart).
// Stride 1: one TMA box per channel block brings the 10 x 18 input pixels under the tile. Stride 2: the 17 x 33 input pixels
// are fetched as two boxes that take every other column (TMA element stride 2), the columns 2*ox - 1 + {0, 2, ...} serving
// the taps kx = 0 and kx = 2 (one column further), the columns 2*ox + {0, 2, ...} the tap kx = 1; out-of-image pixels arrive
// as zeros either way. Persistent CTAs, two or three input stages, two accumulators in TMEM so that the epilogue of a tile
// overlaps the loads and MMAs of the next; warp roles and bounded waits as in dense_umma.cu.
#include <cuda.h>

#include <mutex>

#include "dw_umma.h"
#include "launch.cuh"
#include "umma_epilogue.cuh"
#include "umma_primitives.cuh"

namespace ottk {

namespace {

using namespace umma;
constexpr int kTileM = 128, kTw = 8, kTh = 16, kBlock = 32;
// Builds of the kernel: 0 = one CTA per SM, 8 epilogue warps; 1 = two CTAs per SM (narrow layers); 2 = one CTA per SM with 16
// epilogue warps and four issuing warps, for wide channel slices: a tile of 8 channel blocks is 72 MMAs, which one warp gets
// out at one per 75 cycles however many of its lanes issue (two warps reach the pipe's 40), and holds more requantize work
// than eight warps get through meanwhile.
__host__ __device__ constexpr int epi_warps_of(int build) { return build == 2 ? 16 : 8; }
__host__ __device__ constexpr int issue_warps_of(int build) { return build == 2 ? 4 : 1; }
__host__ __device__ constexpr int threads_of(int build) { return 32 * (1 + issue_warps_of(build) + epi_warps_of(build)); }
constexpr int kWideCols = 128;  // channel-slice width from which build 2 is taken
constexpr int kMaxStages = 3, kMaxAcc = 2;

// Where the channel blocks come from: one tensor map per source tensor, and per block its source and first channel.
struct DwMaps {
    CUtensorMap tm[kUmmaMaxSources];
    uint16_t block_x[kUmmaMaxGatherBlocks];
    uint8_t block_src[kUmmaMaxGatherBlocks];
};

struct DwGeom {
    int n, h, w, oh, ow;
    int cout, cpad;  // real channels, channel stride of the int8 tensors
};

template <int ACT, int OUT, int BUILD>
__global__ void __launch_bounds__(threads_of(BUILD), BUILD == 1 ? 2 : 1)
dw_umma_kernel(const __grid_constant__ DwMaps maps, const __grid_constant__ CUtensorMap tmW, const DwPlan P, const DwGeom G, const EpilogueParams ep,
               void* __restrict__ out, uint32_t* __restrict__ status) {
    constexpr int kEpiWarps = epi_warps_of(BUILD), kIssueWarps = issue_warps_of(BUILD);
    extern __shared__ uint8_t smem_raw[];
    pdl_launch_dependents();
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sW = base + P.w_off, sX = base + P.x_off;
    const uint32_t bar_w = base + P.bars, bar_full = bar_w + 8, bar_empty = bar_full + 8u * kMaxStages, bar_afull = bar_empty + 8u * kMaxStages,
                   bar_aempty = bar_afull + 8u * kMaxAcc;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + P.tmem_slot);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + P.abort_flag);
    float* sp = reinterpret_cast<float*>(base_ptr + P.params);  // scale_in, bias, scale_out: [cols] each

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // this CTA's slice of the layer's channel blocks (depthwise channels are independent, so wide layers are dealt to CTA groups)
    const int grp = blockIdx.x % P.n_groups;
    const int cb0 = grp * P.ncb;
    const int nb = P.ncb_total - cb0 < P.ncb ? P.ncb_total - cb0 : P.ncb;
    const int c_base = cb0 * kBlock;
    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmW);
        for (int cb = 0; cb < nb; ++cb) prefetch_tensormap(&maps.tm[maps.block_src[cb0 + cb]]);
        mbar_init(bar_w, 1);
        for (int i = 0; i < P.stages; ++i) {
            mbar_init(bar_full + 8u * i, 1);
            mbar_init(bar_empty + 8u * i, (uint32_t)nb);  // one commit per issuing lane
        }
        for (int i = 0; i < P.acc_bufs; ++i) {
            mbar_init(bar_afull + 8u * i, (uint32_t)nb);
            mbar_init(bar_aempty + 8u * i, kEpiWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(bar_w, (uint32_t)nb * 9u * 1024u);  // the filters do not depend on the previous kernel
        for (int i = 0; i < nb * 9; ++i) tma_load_2d(&tmW, bar_w, sW + i * 1024u, 0, (cb0 * 9 + i) * kBlock);
    }
    for (int i = threadIdx.x; i < P.cols; i += (int)blockDim.x) {
        const bool in = c_base + i < G.cpad;
        sp[i] = in ? ep.scale_in[c_base + i] : 0.f;
        sp[P.cols + i] = in ? ep.bias[c_base + i] : 0.f;
        sp[2 * P.cols + i] = in ? ep.scale_out[c_base + i] : 0.f;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"((uint32_t)P.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();  // from here on the kernel reads activations and writes outputs

    const int per_img = P.tiles_x * P.tiles_y;
    const int m_first = blockIdx.x / P.n_groups, m_step = gridDim.x / P.n_groups;
    const uint32_t acc_mask = (uint32_t)P.acc_bufs - 1u;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer ----
            uint32_t it = 0;
            bool ok = true;
            for (int m = m_first; ok && m < P.m_tiles; m += m_step, ++it) {
                const int img = m / per_img, r = m - img * per_img;
                const int y0 = (r / P.tiles_x) * kTh * P.stride - 1, x0 = (r % P.tiles_x) * kTw * P.stride - 1;
                const uint32_t st = it % P.stages, ph = (it / P.stages) & 1u;
                if (!mbar_wait(bar_empty + 8u * st, ph ^ 1u, abort_flag, status, 1u, P.wait_ns)) { ok = false; break; }
                mbar_expect_tx(bar_full + 8u * st, (uint32_t)(nb * P.sets * P.set_load_bytes));
                for (int cb = 0; cb < nb; ++cb)
                    for (int s = 0; s < P.sets; ++s)
                        tma_load_4d(&maps.tm[maps.block_src[cb0 + cb]], bar_full + 8u * st,
                                    sX + st * (uint32_t)P.stage_bytes + (uint32_t)(cb * P.block_bytes + s * P.set_bytes), (int)maps.block_x[cb0 + cb], x0 + s, y0, img);
            }
            if (!ok) {
                const unsigned long long t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 1000000ull) {}  // let bulk copies in flight land before shared memory is released
            }
        }
    } else if (warp <= kIssueWarps) {
        // lane l of issuing warp w takes channel block w + l * (issuing warps)
        const int cb = (warp - 1) + lane * kIssueWarps;
        if (cb < nb) {
            // ---- MMA issuers: lane cb issues the nine taps of channel block cb (an MMA is started by one thread; the lanes of
            // the warp execute the instruction together, so a tile costs nine issue slots however many channel blocks it has),
            // and commits its own MMAs to the barriers, whose arrival counts are the number of issuing lanes ----
            bool ok = mbar_wait(bar_w, 0, abort_flag, status, 16u, P.wait_ns);
            tc_fence_after();
            // Per tap: the filter matrix's descriptor and the offset of the shifted input view inside a block (16-byte units;
            // stride 2: the taps kx = 1 read the second column set, kx = 2 one column on). Worked out once: between two MMAs the
            // issuing thread then only adds a constant to the low word of the block's descriptor (the address field cannot carry).
            uint64_t bdesc[9];
            uint32_t aoff[9];
#pragma unroll
            for (int tap = 0; tap < 9; ++tap) {
                const int ky = tap / 3, kx = tap % 3;
                bdesc[tap] = make_smem_desc(sW + (uint32_t)(cb * 9 + tap) * 1024u, kBlock);
                const int col = P.stride == 1 ? kx : (kx >> 1);
                aoff[tap] = (uint32_t)((ky * P.set_w + col) * (kBlock >> 4)) + ((P.stride == 2 && kx == 1) ? (uint32_t)(P.set_bytes >> 4) : 0u);
            }
            const uint32_t sbo = (uint32_t)(P.stride * P.set_w * kBlock);
            uint32_t it = 0;
            for (int m = m_first; ok && m < P.m_tiles; m += m_step, ++it) {
                const uint32_t buf = it & acc_mask, use = it / (uint32_t)P.acc_bufs;
                const uint32_t st = it % P.stages, ph = (it / P.stages) & 1u;
                if (!mbar_wait(bar_aempty + 8u * buf, (use & 1u) ^ 1u, abort_flag, status, 4u, P.wait_ns)) { ok = false; break; }
                if (!mbar_wait(bar_full + 8u * st, ph, abort_flag, status, 2u, P.wait_ns)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d = tmem_base + buf * (uint32_t)P.cols + (uint32_t)(cb * kBlock);
                const uint32_t blk = sX + st * (uint32_t)P.stage_bytes + (uint32_t)(cb * P.block_bytes);
                // 8-row groups (one tile row of 8 pixels each) are `stride` input rows apart
                const uint64_t a_base = make_smem_desc(blk, kBlock, (int)sbo);
                const uint32_t a_lo = (uint32_t)a_base;
                const uint64_t a_hi = a_base & 0xFFFFFFFF00000000ull;
#pragma unroll
                for (int tap = 0; tap < 9; ++tap) umma_i8(d, a_hi | (uint64_t)(a_lo + aoff[tap]), bdesc[tap], P.idesc, tap != 0 ? 1u : 0u);
                umma_commit(bar_empty + 8u * st);
                umma_commit(bar_afull + 8u * buf);
            }
        }
    } else {
        // ---- epilogue warps ----
        const int q = warp & 3, sub = (warp - (1 + kIssueWarps)) >> 2, nsub = kEpiWarps >> 2;
        const int row = q * 32 + lane;
        const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
        const long plane = (long)G.oh * G.ow;
        const UmmaMixedOut no_side{};
        bool ok = true;
        uint32_t it = 0;
        for (int m = m_first; ok && m < P.m_tiles; m += m_step, ++it) {
            const uint32_t buf = it & acc_mask, use = it / (uint32_t)P.acc_bufs;
            if (!mbar_wait(bar_afull + 8u * buf, use & 1u, abort_flag, status, 8u, P.wait_ns)) { ok = false; break; }
            tc_fence_after();
            const int img = m / per_img, r = m - img * per_img;
            const int oy = (r / P.tiles_x) * kTh + (row >> 3), ox = (r % P.tiles_x) * kTw + (row & 7);
            store_accumulator_row<ACT, OUT>(tmem_base + buf * (uint32_t)P.cols + lane_sel, nb * kBlock, sub, nsub, oy < G.oh && ox < G.ow, img,
                                            (long)oy * G.ow + ox, plane, sp, sp + P.cols, sp + 2 * P.cols, ep.act_param0, G.cpad, G.cout, out, no_side, c_base);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_aempty + 8u * buf);
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

template <int ACT, int OUT, int BUILD>
const char* launch_variant(cudaStream_t stream, int grid, const DwMaps& tmX, const CUtensorMap& tmW, const DwPlan& p, const DwGeom& g,
                           const EpilogueParams& ep, void* out, uint32_t* status) {
    static std::mutex mu;  // several host threads may drive different GPUs through this function at once
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = dw_umma_kernel<ACT, OUT, BUILD>;
    if (dev >= 0 && dev < 64) {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set[dev]) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
                return "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed";
            attr_set[dev] = true;
        }
    }
    if (launch_overlapped(kernel, dim3(grid), dim3(threads_of(BUILD)), (size_t)p.smem_bytes, stream, tmX, tmW, p, g, ep, out, status) != cudaSuccess)
        return "dw_umma_kernel launch failed";
    return nullptr;
}

}  // namespace

bool dw_umma_plan(int channels, int stride, int smem_budget, DwPlan* plan) {
    DwPlan p{};
    if (channels < 1 || (stride != 1 && stride != 2)) return false;
    p.stride = stride;
    p.ncb_total = (channels + kBlock - 1) / kBlock;
    if (p.ncb_total > kUmmaMaxGatherBlocks) return false;
    // Blocks per CTA: two accumulators of `cols` columns must fit the 512 TMEM columns (8 blocks). Stride 2 needs 20 KB of
    // shared memory per block and stage; two blocks per CTA leave room for two CTAs per SM, which measured best on the
    // stride-2 layers of ShuffleNetV2 (219 k images/s against 216.7 k with four blocks). Wider layers are dealt to CTA groups.
    const int max_blocks = stride == 1 ? 8 : 2;
    p.n_groups = (p.ncb_total + max_blocks - 1) / max_blocks;
    p.ncb = (p.ncb_total + p.n_groups - 1) / p.n_groups;
    p.cols = p.ncb * kBlock;
    p.acc_bufs = 2;
    const int cols = p.acc_bufs * p.cols;
    p.tmem_cols = cols <= 32 ? 32 : cols <= 64 ? 64 : cols <= 128 ? 128 : cols <= 256 ? 256 : 512;
    p.idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBlock >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
    if (stride == 1) {
        p.sets = 1; p.set_w = kTw + 2; p.tile_rows = kTh + 2;
    } else {
        p.sets = 2; p.set_w = kTw + 1; p.tile_rows = 2 * kTh + 1;
    }
    p.set_load_bytes = p.set_w * p.tile_rows * kBlock;
    p.set_bytes = (p.set_load_bytes + 1023) / 1024 * 1024;
    p.block_bytes = p.sets * p.set_bytes;
    p.stage_bytes = p.ncb * p.block_bytes;
    const int fixed = 1024 /*alignment slack*/ + p.ncb * 9 * 1024 + 1024 /*barriers*/ + ((3 * p.cols * 4 + 1023) / 1024 * 1024);
    p.stages = (smem_budget - fixed) / p.stage_bytes;
    if (p.stages > kMaxStages) p.stages = kMaxStages;
    if (p.stages < 2) return false;
    // narrow layers: two CTAs per SM hide each other's latencies, if two stages each leave room for that
    const int two_cta_budget = smem_budget / 2;
    if (2 * p.tmem_cols <= 512 && fixed + 2 * p.stage_bytes <= two_cta_budget) {
        p.ctas_per_sm = 2;
        p.stages = (two_cta_budget - fixed) / p.stage_bytes;
        if (p.stages > kMaxStages) p.stages = kMaxStages;
    } else {
        p.ctas_per_sm = 1;
    }
    uint32_t off = 0;
    p.w_off = off; off += (uint32_t)p.ncb * 9u * 1024u;
    p.x_off = off; off += (uint32_t)p.stages * (uint32_t)p.stage_bytes;
    p.bars = off; off += 1024u;
    p.tmem_slot = p.bars + 8u * (1 + 2 * kMaxStages + 2 * kMaxAcc);
    p.abort_flag = p.tmem_slot + 8u;
    p.params = off; off += (uint32_t)(3 * p.cols * 4);
    p.smem_bytes = (int)off + 1024;
    // pad the request so that no more CTAs become resident than TMEM can serve (see dense_umma.cu)
    const int min_smem = smem_budget / (p.ctas_per_sm + 1) + 1;
    if (p.smem_bytes < min_smem) p.smem_bytes = min_smem;
    if (p.smem_bytes > smem_budget) return false;
    *plan = p;
    return true;
}

size_t dw_umma_weight_bytes(const DwPlan& p) { return (size_t)p.ncb_total * 9 * 1024; }

void dw_umma_pack_weights(const DwPlan& p, const int8_t* w_dw, int channels, int8_t* dst) {
    const size_t total = dw_umma_weight_bytes(p);
    for (size_t i = 0; i < total; ++i) dst[i] = 0;
    for (int ch = 0; ch < channels; ++ch) {
        const int cb = ch / kBlock, n = ch % kBlock;
        for (int tap = 0; tap < 9; ++tap) dst[((size_t)(cb * 9 + tap) * kBlock + n) * kBlock + n] = w_dw[ch * 9 + tap];
    }
}

const char* dw_umma_encode_weight_map(const DwPlan& p, const int8_t* w_dev, void* map_out) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return "cuTensorMapEncodeTiled entry point not available";
    cuuint64_t dims[2] = {(cuuint64_t)kBlock, (cuuint64_t)p.ncb_total * 9 * kBlock};
    cuuint64_t strides[1] = {(cuuint64_t)kBlock};
    cuuint32_t box[2] = {(cuuint32_t)kBlock, (cuuint32_t)kBlock};
    cuuint32_t estr[2] = {1, 1};
    return enc(reinterpret_cast<CUtensorMap*>(map_out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)w_dev, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
               ? nullptr
               : "cuTensorMapEncodeTiled(depthwise weights) failed";
}

const char* launch_dw_umma(cudaStream_t stream, int sm_count, const DwPlan& plan_in, const void* weight_map, const ConvShape& s, const int8_t* x,
                           const UmmaSources* sources, const EpilogueParams& ep, void* out, int out_dtype, uint32_t* status,
                           unsigned long long wait_limit_ns) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return "cuTensorMapEncodeTiled entry point not available";
    if (s.n == 0) return nullptr;
    if (out_dtype != DT_S8_NHWC && out_dtype != DT_F32_NCHW) return "the tensor-core depthwise kernel writes int8 NHWC or fp32 NCHW";
    DwPlan p = plan_in;
    p.wait_ns = wait_limit_ns;
    p.tiles_x = (s.ow + kTw - 1) / kTw;
    p.tiles_y = (s.oh + kTh - 1) / kTh;
    p.m_tiles = s.n * p.tiles_x * p.tiles_y;
    DwMaps km;
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
    for (int b = 0; b < p.ncb_total; ++b) {
        km.block_x[b] = sources ? sources->block_x[b] : (uint16_t)(b * kBlock);
        km.block_src[b] = sources ? sources->block_src[b] : (uint8_t)0;
    }
    DwGeom g{s.n, s.h, s.w, s.oh, s.ow, s.cout, s.cout_pad};
    int per_group = sm_count * p.ctas_per_sm / p.n_groups;  // CTAs walking over the pixel tiles, per channel group
    if (per_group < 1) per_group = 1;
    if (per_group > p.m_tiles) per_group = p.m_tiles;
    const int grid = per_group * p.n_groups;
    const CUtensorMap& tmW = *reinterpret_cast<const CUtensorMap*>(weight_map);
    const char* err = nullptr;
#define OTT_DW_LAUNCH(ACT, OUT)                                                                                  \
    err = p.ctas_per_sm > 1    ? launch_variant<ACT, OUT, 1>(stream, grid, km, tmW, p, g, ep, out, status)       \
          : p.cols >= kWideCols ? launch_variant<ACT, OUT, 2>(stream, grid, km, tmW, p, g, ep, out, status)       \
                                : launch_variant<ACT, OUT, 0>(stream, grid, km, tmW, p, g, ep, out, status)
#define OTT_DW_ACT(OUT)                                       \
    switch (ep.act_type) {                                    \
        case ACT_RELU: OTT_DW_LAUNCH(ACT_RELU, OUT); break;   \
        case ACT_LRELU: OTT_DW_LAUNCH(ACT_LRELU, OUT); break; \
        case ACT_RELU6: OTT_DW_LAUNCH(ACT_RELU6, OUT); break; \
        default: OTT_DW_LAUNCH(ACT_NONE, OUT); break;         \
    }
    if (out_dtype == DT_F32_NCHW) { OTT_DW_ACT(DT_F32_NCHW) } else { OTT_DW_ACT(DT_S8_NHWC) }
#undef OTT_DW_ACT
#undef OTT_DW_LAUNCH
    if (err) return err;
    return cudaGetLastError() == cudaSuccess ? nullptr : "dw_umma_kernel launch failed";
}

}  // namespace ottk
