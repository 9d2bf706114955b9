// Host-visible plan of the fused kernel "depthwise 3x3 (stride 1 or 2, pad 1) -> 1x1 convolution": the second and third
// layer of a ShuffleNetV2 unit branch (and both layers of a stride-2 unit's left branch) in one launch, both on the tensor
// cores, the int8 tensor between them in shared memory only.
#pragma once

#include "dense_umma.h"

namespace ottk {

constexpr int kDwPwStagesMax = 4;

struct DwPwPlan {
    int stride;       // of the depthwise layer
    int ncb;          // 32-channel blocks of the depthwise layer (its stored channel count / 32, rounded up)
    int bpc;          // channel blocks per input chunk (a chunk = one TMA transaction group = one pipeline stage)
    int nchunks;      // chunks per pixel tile
    int dwcols;       // ncb * 32: accumulator columns of the depthwise stage
    int c2;           // accumulator columns of the 1x1 layer (its channel stride rounded up to 32, <= 256)
    int dw_bufs, pw_bufs, y_bufs;  // 1 or 2 of each: depthwise accumulators, 1x1 accumulators, operand tiles between the layers
    int tmem_cols;
    uint32_t idesc_dw, idesc_pw;
    int sets, set_w, tile_rows, set_load_bytes, set_bytes, block_bytes, chunk_bytes;
    int stages, ctas_per_sm;
    // shared-memory offsets from the 1 KiB-aligned base
    uint32_t w_dw, w_pw, x, y, bars, tmem_slot, abort_flag, params;
    int smem_bytes;
    // per call
    int tiles_x, tiles_y, m_tiles;
    unsigned long long wait_ns;
};

// dw_channels: stored channels of the depthwise layer (its output tensor's channel count); pw_cout: output channels of the 1x1
// layer. false: the pair does not fit one SM's shared / tensor memory.
bool dwpw_plan(int dw_channels, int stride, int pw_cout, int smem_budget, DwPwPlan* plan);

// Weight panels (host). Depthwise: as dw_umma_pack_weights ([block][tap] 32x32 diagonal matrices, 1 KiB each).
// 1x1: [c2 rows][dwcols] K-major, column k = the weight for stored depthwise channel k (zeros elsewhere).
size_t dwpw_wdw_bytes(const DwPwPlan& p);
size_t dwpw_wpw_bytes(const DwPwPlan& p);
void dwpw_pack_wdw(const DwPwPlan& p, const int8_t* w_dw /*[channels][9] in stored order*/, int channels, int8_t* dst);

struct DwPwWeights {
    alignas(128) unsigned char map_wdw[128], map_wpw[128];
};
const char* dwpw_encode_weight_maps(const DwPwPlan& p, const int8_t* wdw_dev, const int8_t* wpw_dev, DwPwWeights* out);

struct DwPwEpilogues {
    EpilogueParams dw, pw;  // per-channel arrays on the device: dw in stored channel order (dwcols entries readable up to the tensor's channel stride)
};

// s: the depthwise layer's shape (n, h, w, oh, ow, cin_pad = channel stride of x when sources == NULL; cout_pad is unused).
// sources: where the depthwise layer's channel blocks come from (NULL: block b = channels 32b.. of x). out / out_dtype /
// mixed: the 1x1 layer's output exactly as for launch_dense_umma. Returns NULL or an error text.
const char* launch_dwpw_umma(cudaStream_t stream, int sm_count, const DwPwPlan& plan, const DwPwWeights& wts, const ConvShape& s, const int8_t* x,
                             const UmmaSources* sources, int pw_cout, const DwPwEpilogues& ep, void* out, int out_dtype, uint32_t* status,
                             const UmmaMixedOut* mixed, unsigned long long wait_limit_ns);

}  // namespace ottk
