// Measures what one tcgen05.mma kind::i8 (M = 128, K = 32) costs on this GPU as a function of its N, of how many warps and
// lanes issue, and of how many CTAs share an SM: the numbers the tile shapes of dense_umma.cu, dw_umma.cu and dwpw_umma.cu are
// argued from. Operands are zeros in shared memory (only the time matters); every CTA issues `reps` MMAs per issuing thread
// into its own accumulator, commits, and waits (bounded) for completion. ott_debug_mma_rate returns cycles per MMA per SM.
#include <vector>

#include "ctx.h"
#include "umma_primitives.cuh"

namespace {

using namespace ottk::umma;

struct RateResult {
    long long cycles;  // first issue to last completion, over the CTA's issuing warps
    unsigned status;
};

__global__ void __launch_bounds__(160) mma_rate_kernel(int n, int warps, int lanes, int reps, int tmem_cols, unsigned long long limit_ns, RateResult* res) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t bar[16];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ uint32_t status;
    __shared__ long long tstart[4], tend[4];
    for (int i = threadIdx.x; i < (128 + 256) * 32; i += blockDim.x) smem[i] = 0;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 16; ++i) mbar_init(smem_u32(&bar[i]), 1);
        abort_flag = 0;
        status = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    // D = s32, A = B = signed int8, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
    const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    if (warp < warps && lane < lanes) {
        const uint64_t adesc = make_smem_desc(smem_u32(smem), 32), bdesc = make_smem_desc(smem_u32(smem + 128 * 32), 32);
        const int stride = n < 32 ? 32 : n;
        const uint32_t d = tmem_base + (uint32_t)(((warp * lanes + lane) * stride) % tmem_cols);  // accumulators may alias: only time matters
        const long long t0 = clock64();
        umma_i8(d, adesc, bdesc, idesc, 0u);
#pragma unroll 8
        for (int r = 1; r < reps; ++r) umma_i8(d, adesc, bdesc, idesc, 1u);
        umma_commit(smem_u32(&bar[warp * 4 + lane]));
        mbar_wait(smem_u32(&bar[warp * 4 + lane]), 0, &abort_flag, &status, 1, limit_ns);
        const long long t1 = clock64();
        if (lane == 0) { tstart[warp] = t0; tend[warp] = t1; }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        long long a = tstart[0], b = tend[0];
        for (int w = 1; w < warps; ++w) { a = tstart[w] < a ? tstart[w] : a; b = tend[w] > b ? tend[w] : b; }
        res[blockIdx.x].cycles = b - a;
        res[blockIdx.x].status = status;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)tmem_cols) : "memory");
    }
}

}  // namespace

extern "C" int ott_debug_mma_rate(ott_ctx* ctx, int n_cols, int issuing_warps, int issuing_lanes, int ctas_per_sm, int reps, float* cycles_per_mma) {
    if (!ctx || !cycles_per_mma) return OTT_ERR_INVALID;
    if (n_cols < 16 || n_cols > 256 || n_cols % 16 || issuing_warps < 1 || issuing_warps > 4 || issuing_lanes < 1 || issuing_lanes > 4 || ctas_per_sm < 1 ||
        ctas_per_sm > 2 || reps < 8 || reps > (1 << 16))
        return ctx->fail(OTT_ERR_INVALID, "mma rate probe: N 16..256 (multiple of 16), 1..4 warps, 1..4 lanes, 1..2 CTAs per SM, 8..65536 MMAs per thread");
    cudaSetDevice(ctx->device);
    const int stride = n_cols < 32 ? 32 : n_cols;
    int cols = issuing_warps * issuing_lanes * stride;
    if (cols > 512 / ctas_per_sm) cols = 512 / ctas_per_sm;
    int tmem_cols = 32;
    while (tmem_cols < cols) tmem_cols *= 2;
    const int smem_bytes = (128 + 256) * 32 + 2048;
    const int grid = ctx->sm_count * ctas_per_sm;
    void* dev = nullptr;
    if (ctx->alloc->allocate(sizeof(RateResult) * (size_t)grid, &dev) != cudaSuccess) return ctx->fail(OTT_ERR_ALLOC, "device allocation failed");
    RateResult* res = static_cast<RateResult*>(dev);
    for (int it = 0; it < 2; ++it)  // the first run warms the instruction cache
        mma_rate_kernel<<<grid, 160, smem_bytes, ctx->stream>>>(n_cols, issuing_warps, issuing_lanes, reps, tmem_cols, ctx->wait_limit_ns, res);
    std::vector<RateResult> host((size_t)grid);
    cudaError_t e = cudaMemcpyAsync(host.data(), res, sizeof(RateResult) * (size_t)grid, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    ctx->alloc->free(dev);
    ctx->launches += 2;
    if (e != cudaSuccess) return ctx->fail(OTT_ERR_CUDA, "mma rate probe: %s", cudaGetErrorString(e));
    double sum = 0;
    unsigned st = 0;
    for (const RateResult& r : host) { sum += (double)r.cycles; st |= r.status; }
    if (st) return ctx->fail(OTT_ERR_DEVICE_WAIT, "mma rate probe: a wait ran out");
    *cycles_per_mma = (float)(sum / grid / ((double)reps * issuing_lanes * issuing_warps * ctas_per_sm));
    return OTT_OK;
}
