// Host-visible plan of the fused ShuffleNetV2 unit kernel: 1x1 convolution -> depthwise 3x3 (stride 1, pad 1) -> 1x1
// convolution of one branch in one launch, all three on the tensor cores, intermediates in shared memory.
#pragma once

#include "dense_umma.h"

namespace ottk {

constexpr int kUnitTw = 8, kUnitTh = 16;                 // output pixel tile (8 wide so that a tile row is one 8-row operand group)
constexpr int kUnitHaloW = kUnitTw + 2, kUnitHaloH = kUnitTh + 2;
constexpr int kUnitHaloPixels = kUnitHaloW * kUnitHaloH;  // 180: pixels of the first 1x1 layer a tile needs
constexpr int kUnitBlock = 32;                            // channels per K block everywhere in this kernel
constexpr int kUnitHaloBlockBytes = 6144;                 // one 32-channel block of a halo tile (180 x 32 B) rounded up to 256 B * 24

struct UnitPlan {
    int nkb1;      // K blocks of the first 1x1 layer (32 input channels each, possibly from several source tensors)
    int cm;        // channels between the layers (first layer's outputs = depthwise channels = second layer's inputs), padded to 32
    int c2;        // output columns of the second 1x1 layer (its channel stride: a multiple of 16)
    int epi_warps; // 8 or 16
    int ctas_per_sm;
    int tmem_cols; // power of two >= 2*cm + cm + c2
    uint32_t idesc1, idesc_dw, idesc2;
    // shared-memory offsets from the 1 KiB-aligned base
    uint32_t w1, wdw, w2, x_stage[2], y1, y2, bars, tmem_slot, abort_flag, params, total;
    int smem_bytes;
    // per call
    int tiles_x, tiles_y, m_tiles;
    unsigned long long wait_ns;
};

// cin1_blocks: K blocks of the first layer; cm_real: channels between the layers; cout2: second layer's output channels.
bool unit_plan(int cin1_blocks, int cm_real, int cout2, int smem_budget, UnitPlan* plan);

// Weight panels (host): w1 [cm][nkb1*32] K-major (rows past the real channels zero); wdw [(cm/32)*9*32 rows][32]: block
// (cb, tap) is the 32x32 diagonal matrix of the depthwise weights of channels cb*32.. at that tap; w2 [c2][cm].
void unit_pack_w1(const UnitPlan& p, const int8_t* w_korder /*[cout1][nkb1*32]*/, int cout1, int8_t* dst);
void unit_pack_wdw(const UnitPlan& p, const int8_t* w_dw /*[c][9]*/, int c, int8_t* dst);
void unit_pack_w2(const UnitPlan& p, const int8_t* w2 /*[cout2][cin2]*/, int cout2, int cin2, int8_t* dst);
size_t unit_w1_bytes(const UnitPlan& p);
size_t unit_wdw_bytes(const UnitPlan& p);
size_t unit_w2_bytes(const UnitPlan& p);

struct UnitWeights {
    alignas(128) unsigned char map_w1[128], map_wdw[128], map_w2[128];  // TMA descriptors of the three panels
};
const char* unit_encode_weight_maps(const UnitPlan& p, const int8_t* w1_dev, const int8_t* wdw_dev, const int8_t* w2_dev, UnitWeights* out);

// Epilogue parameters of the three layers: per-channel arrays on the device, padded with zeros to cm / cm / c2 entries.
struct UnitEpilogues {
    EpilogueParams e1, edw, e2;
};

// Launch. sources: where the first layer's K blocks come from (n_src int8 NHWC tensors [n][h][w][src_cpad]). out / out_dtype
// / mixed: the second layer's output exactly as for launch_dense_umma (int8 NHWC with per-channel scales, optionally fp32
// planes of chosen channels; or fp32 NCHW). Returns NULL or an error text.
const char* launch_unit_umma(cudaStream_t stream, int sm_count, const UnitPlan& plan, const UnitWeights& wts, const UmmaSources& sources, int n, int h,
                             int w, int cout2, const UnitEpilogues& ep, void* out, int out_dtype, uint32_t* status, const UmmaMixedOut* mixed,
                             unsigned long long wait_limit_ns);

}  // namespace ottk
