// Host-visible plan of the tensor-core (tcgen05) dense convolution kernel.
#pragma once

#include "kernels.h"

namespace ottk {

// Fixed per layer at create time (tiling of K and N), completed per call (tiling of the pixels).
struct UmmaPlan {
    // K: each filter tap is split into ncb channel blocks of bkc bytes (32/64/128 = the swizzle span)
    int bkc, ncb, taps, nkb, k_total;
    // N: n_tiles weight panels of bn output channels (multiple of 16, <= 256); cout_rows = n_tiles*bn
    int bn, n_tiles, cout_rows;
    int stages;      // activation tiles in flight
    int tmem_cols;   // TMEM columns allocated (acc_bufs accumulators)
    int acc_stride;  // column offset from one accumulator to the next
    int acc_bufs;    // accumulators in flight between the MMA issuer and the epilogue: 2, or 4 for narrow tiles
    uint32_t idesc;  // tcgen05 instruction descriptor
    int smem_bytes;  // dynamic shared memory of the launch
    int epi_warps;   // epilogue warps per CTA: 8 or 16
    int ctas_per_sm; // resident CTAs per SM the launch is sized for (limited by TMEM columns and shared memory)
    // per call
    int halo;        // k x k layers: one TMA box per pixel tile and channel block holds the tile plus its halo; the taps read shifted views
    int a_stage_bytes;  // bytes of one activation stage (a 128-pixel tile, or a halo tile rounded up to 1 KiB)
    int flat;                          // 1x1: activations viewed as one [pixels, channels] matrix
    int gather;                        // > 0: the K blocks come from this many int8 NHWC tensors (see UmmaSources)
    int gather_whole;                  // gathered layer whose pipeline stage holds all the K blocks of a pixel tile
    int tw, th, tiles_x, tiles_y, m_tiles;  // 128-pixel output rectangles (tw*th == 128)
    unsigned long long wait_ns;        // limit of every mbarrier wait inside the kernel
};

// Decide whether the tensor-core kernel takes this layer and how it tiles it. smem_budget = opt-in
// shared memory per block of the device. bkc_override (32/64/128) fixes the channel-block width instead of deriving it
// from cin. whole_tile_stages (1x1 layers): one pipeline stage holds all the K blocks of a pixel tile.
bool umma_plan_layer(int cin, int cout, int kh, int kw, int sh, int sw, int dh, int dw, int smem_budget, UmmaPlan* plan,
                     int bkc_override = 0, bool whole_tile_stages = false);

// A 1x1 layer whose input channels are spread over several int8 NHWC tensors (each written by one producer layer): K block
// kb of the implicit GEMM is the 32 channels starting at block_x[kb] of tensor block_src[kb]. The layer's weights are laid
// out to match (zero for channels of a block that belong to another reader).
constexpr int kUmmaMaxSources = 12, kUmmaMaxGatherBlocks = 64, kUmmaGatherBlock = 32;
struct UmmaSources {
    int n_src;
    const int8_t* src[kUmmaMaxSources];  // device, [pixels][src_cpad]
    int src_cpad[kUmmaMaxSources];       // channel stride of each tensor (multiple of 16, >= 32)
    uint16_t block_x[kUmmaMaxGatherBlocks];
    uint8_t block_src[kUmmaMaxGatherBlocks];
};

// A requantizing launch that also stores selected output channels as fp32 NCHW planes (activation(dequantize), the value an
// fp32-output layer stores): channel c when bit c of mask is set. out_f32 is a whole [n][cout][oh][ow] tensor.
struct UmmaMixedOut {
    float* out_f32;
    uint32_t mask[32];  // output channels 0..1023
    // Scattered int8 output (n_chunks > 0): the layer's output columns were laid out reader by reader, and 16-column chunk c
    // goes to dst[c] + pixel * pitch[c], straight into the input tensor of the layer that reads it (dst NULL: nobody does).
    // The fp32 planes then use plane_of_col (device array, one entry per output column) inside a tensor of f32_planes channels.
    int n_chunks;
    int f32_planes;
    const int16_t* plane_of_col;
    int8_t* dst[64];
    uint32_t pitch[64];
    unsigned long long pair_ok;  // bit c/2: chunks c and c+1 are 32 contiguous, 32-byte aligned bytes
};

// OIHW int8 -> [cout_rows][k_total] K-major panel, zero padded (host memory, dst sized cout_rows*k_total).
void umma_pack_weights(const UmmaPlan& p, const int8_t* w_oihw, int cin, int cout, int kh, int kw, int8_t* dst);

// Encode the TMA descriptor of the packed weights (128 bytes written to map_out). Returns NULL or an error text.
const char* umma_encode_weight_map(const UmmaPlan& p, const int8_t* w_dev, void* map_out);

// Launch. Returns NULL or an error text.
// sources: NULL, or where the K blocks of a plan with gather > 0 come from (x is then unused). mixed: NULL, or the fp32 side
// output of an int8 launch.
const char* launch_dense_umma(cudaStream_t stream, int sm_count, const UmmaPlan& plan, const void* weight_map,
                              const ConvShape& s, const int8_t* x, const EpilogueParams& ep, void* out, int out_dtype,
                              uint32_t* status, const UmmaSources* sources = nullptr, const UmmaMixedOut* mixed = nullptr,
                              unsigned long long wait_limit_ns = 2000000000ull);

}  // namespace ottk
