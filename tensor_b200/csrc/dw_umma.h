// Host-visible plan of the tensor-core depthwise 3x3 kernel (dw_umma.cu).
#pragma once

#include "dense_umma.h"

namespace ottk {

struct DwPlan {
    int stride;          // 1 or 2
    int ncb_total;       // 32-channel blocks of the layer
    int ncb, cols;       // blocks one CTA owns (the layer's channels are dealt to n_groups CTA groups); accumulator columns = ncb * 32
    int n_groups;
    int acc_bufs, tmem_cols;
    uint32_t idesc;
    int sets;            // input boxes per channel block: 1, or 2 (stride 2: the two column parities)
    int set_w, tile_rows;            // pixels per row / rows of one box as it lies in shared memory
    int set_load_bytes, set_bytes;   // bytes TMA writes per box; its slot (multiple of 1 KiB)
    int block_bytes, stage_bytes, stages;
    int ctas_per_sm;
    uint32_t w_off, x_off, bars, tmem_slot, abort_flag, params;  // shared-memory offsets from the 1 KiB-aligned base
    int smem_bytes;
    // per call
    int tiles_x, tiles_y, m_tiles;
    unsigned long long wait_ns;
};

bool dw_umma_plan(int channels, int stride, int smem_budget, DwPlan* plan);
size_t dw_umma_weight_bytes(const DwPlan& p);
// w_dw: int8 [channels][9] -> per (channel block, tap) a 32 x 32 K-major matrix with the tap's weights on the diagonal
void dw_umma_pack_weights(const DwPlan& p, const int8_t* w_dw, int channels, int8_t* dst);
const char* dw_umma_encode_weight_map(const DwPlan& p, const int8_t* w_dev, void* map_out);
// x: int8 NHWC [n][h][w][s.cin_pad], or (sources != NULL) channel block b = the 32 channels from block_x[b] of source tensor
// block_src[b] (channels past a source's channel stride read as zeros); out: int8 NHWC or fp32 NCHW with s.cout_pad / s.cout
// channels; rounding rule add-half-truncate only. NULL or an error text.
const char* launch_dw_umma(cudaStream_t stream, int sm_count, const DwPlan& plan, const void* weight_map, const ConvShape& s, const int8_t* x,
                           const UmmaSources* sources, const EpilogueParams& ep, void* out, int out_dtype, uint32_t* status,
                           unsigned long long wait_limit_ns);

}  // namespace ottk
