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
    int tw, th, tiles_x, tiles_y, m_tiles;  // 128-pixel output rectangles (tw*th == 128)
};

// Decide whether the tensor-core kernel takes this layer and how it tiles it. smem_budget = opt-in
// shared memory per block of the device.
bool umma_plan_layer(int cin, int cout, int kh, int kw, int sh, int sw, int dh, int dw, int smem_budget, UmmaPlan* plan);

// OIHW int8 -> [cout_rows][k_total] K-major panel, zero padded (host memory, dst sized cout_rows*k_total).
void umma_pack_weights(const UmmaPlan& p, const int8_t* w_oihw, int cin, int cout, int kh, int kw, int8_t* dst);

// Encode the TMA descriptor of the packed weights (128 bytes written to map_out). Returns NULL or an error text.
const char* umma_encode_weight_map(const UmmaPlan& p, const int8_t* w_dev, void* map_out);

// Launch. Returns NULL or an error text.
const char* launch_dense_umma(cudaStream_t stream, int sm_count, const UmmaPlan& plan, const void* weight_map,
                              const ConvShape& s, const int8_t* x, const EpilogueParams& ep, void* out, int out_dtype,
                              uint32_t* status);

}  // namespace ottk
