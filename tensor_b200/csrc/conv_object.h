// Device-side state of one quantized ConvolutionLayer (the object behind the opaque ott_conv handle).
#pragma once

#include <cstdint>
#include <vector>

#include "../../include/otter_b200.h"
#include "dense_umma.h"
#include "dw_umma.h"

struct ott_conv {
    ott_conv_desc d{};
    int kind = 0;
    bool depthwise = false;
    int cin_pad = 0, cout_pad = 0;
    int n_in_scales = 0;
    // device state, owned (allocated from the context's allocator)
    int8_t* w_dev = nullptr;
    uint32_t* w_tiled_dev = nullptr;  // depthwise only: filter rows packed for the tiled kernel
    float* scale_in_dev = nullptr;
    float* bias_dev = nullptr;
    float* scale_out_dev = nullptr;
    float* in_scales_dev = nullptr;
    int16_t* plane_map_dev = nullptr;  // optional: fp32 side output, output channel -> plane of a tensor with f32_planes channels
    int f32_planes = 0;
    // host copies for the kernels that take their parameters by value (stem kernel)
    std::vector<int8_t> w_host;
    std::vector<float> scale_in_host, bias_host, scale_out_host;
    float in_scale0 = 1.f;
    ottk::UmmaPlan plan{};
    // a layer whose input channels are gathered from several int8 tensors (ott_conv_int8_create_gathered): which K block is
    // which 32 channels of which source, and the channel count every source tensor must have
    std::vector<uint16_t> block_x;
    std::vector<uint8_t> block_src;
    std::vector<int> src_channels;
    std::vector<int8_t> w_korder;  // gathered 1x1 layer: the weights against that K order, [cout][block_x.size() * 32]
    // a depthwise layer with gathered input runs on a permuted, padded channel order (whole 16-channel groups of the sources):
    // position[c] = where logical channel c lies in that order, stored_channels = its length (also the output's channels)
    std::vector<int> position;
    int stored_channels = 0;
    int gather_group = 16;  // channels per group of that order: 16 (CUDA-core kernel) or 32 (tensor-core kernel)
    alignas(128) unsigned char weight_map[128];
    // depthwise 3x3 (stride 1 / 2, pad 1) with int8 input: the tensor-core kernel's plan, diagonal weight panel and its TMA descriptor
    bool dw_umma = false;
    ottk::DwPlan dw_plan{};
    int8_t* w_dwu_dev = nullptr;
    alignas(128) unsigned char weight_map_dw[128];
};
