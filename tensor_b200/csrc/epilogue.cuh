// Bit-exact float epilogue and prologue arithmetic shared by all convolution kernels.
//
// Every rounding step of the reference's x86 code is written out with an explicit intrinsic so that
// the compiler neither fuses nor splits anything (the library is also compiled with -fmad=false):
//   dequantize  v = fma((float)acc, scale_in, bias)      Tensor/QuantizeX86.cpp:851-903 as built with the
//                                                         reference's -Ofast -mfma flags (one FMA);
//               without bias: (float)acc * scale_in       Tensor/QuantizeX86.cpp:864-880
//   activation  ReLU / LeakyReLU / clip[0,6]              Tensor/QuantizeX86.hpp:72-106
//   requantize  q = float2int8(v * scale_out)             Tensor/QuantizeX86.cpp:1723-1870
//   float2int8  trunc(v + copysign(0.5, v)), clamp ±127   Tensor/VecIntrinsic.hpp:71-95   (rounding 0)
//               round half away from zero, clamp ±127     Tensor/QuantizeX86.cpp:18-23    (rounding 1)
//   quantize    q = float2int8(x * scale)                 Tensor/QuantizeX86.cpp:396-549
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace ottk {

enum : int { ACT_NONE = 0, ACT_RELU = 1, ACT_LRELU = 2, ACT_RELU6 = 3 };
enum : int { ROUND_ADD_HALF_TRUNC = 0, ROUND_HALF_AWAY = 1 };

// Per-layer epilogue parameters. Arrays are device pointers with one entry per (padded) output channel;
// entries of padding channels are zero so those channels come out as 0.
struct EpilogueParams {
    const float* scale_in;   // [cout_pad]
    const float* bias;       // [cout_pad] (zeros when the layer has no bias)
    const float* scale_out;  // [cout_pad] (per-tensor scale replicated); unused for fp32 output
    int has_bias;
    int act_type;
    float act_param0;
    int rounding;
};

__device__ __forceinline__ float dequant(int acc, float scale_in, float bias, int has_bias) {
    const float a = __int2float_rn(acc);
    return has_bias ? __fmaf_rn(a, scale_in, bias) : __fmul_rn(a, scale_in);
}

template <int ACT>
__device__ __forceinline__ float activate_t(float v, float p0) {
    if (ACT == ACT_RELU) return v > 0.f ? v : 0.f;
    if (ACT == ACT_LRELU) return v > 0.f ? v : __fmul_rn(v, p0);
    if (ACT == ACT_RELU6) return fminf(fmaxf(v, 0.f), 6.f);
    return v;
}

__device__ __forceinline__ float activate(float v, int act, float p0) {
    switch (act) {
        case ACT_RELU: return activate_t<ACT_RELU>(v, p0);
        case ACT_LRELU: return activate_t<ACT_LRELU>(v, p0);
        case ACT_RELU6: return activate_t<ACT_RELU6>(v, p0);
        default: return v;
    }
}

// copysign(0.5, v) as one logic instruction: (bits(v) & 0x80000000) | bits(0.5). Written as lop3 with both constants in
// registers; the compiler's own form takes two instructions per value (a logic instruction carries one immediate).
__device__ __forceinline__ float half_signed(float v) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(__float_as_uint(v)), "r"(0x80000000u), "r"(0x3F000000u));
    return __uint_as_float(r);
}

// float -> int in [-127,127], kept as int so four of them can be packed by the caller.
__device__ __forceinline__ int float2int8(float v, int rounding) {
    int i;
    if (rounding == ROUND_HALF_AWAY) {
        const float t = truncf(v);
        const float frac = __fsub_rn(v, t);  // exact
        i = __float2int_rz(t);
        if (fabsf(frac) >= 0.5f) i += (v < 0.f) ? -1 : 1;
    } else {
        const float adj = __fadd_rn(v, half_signed(v));
        i = __float2int_rz(adj);
    }
    return max(-127, min(127, i));
}

__device__ __forceinline__ int requant(int acc, float scale_in, float bias, float scale_out, const EpilogueParams& ep) {
    float v = dequant(acc, scale_in, bias, ep.has_bias);
    v = activate(v, ep.act_type, ep.act_param0);
    return float2int8(__fmul_rn(v, scale_out), ep.rounding);
}

__device__ __forceinline__ float dequant_act(int acc, float scale_in, float bias, const EpilogueParams& ep) {
    return activate(dequant(acc, scale_in, bias, ep.has_bias), ep.act_type, ep.act_param0);
}

__device__ __forceinline__ int quantize1(float x, float scale, int rounding) {
    return float2int8(__fmul_rn(x, scale), rounding);
}

// ---- fast forms used by the hot loops (same results as the functions above) ----

// two s32 -> two saturated s8 in the low half of d, upper half taken from c (cvt.pack)
__device__ __forceinline__ uint32_t pack_sat_s8x2(int hi, int lo, uint32_t c) {
    uint32_t d;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(c));
    return d;
}

// four s32 -> four saturated s8, a in byte 0
__device__ __forceinline__ uint32_t pack_sat_s8x4(int a, int b, int c, int d) {
    return pack_sat_s8x2(b, a, pack_sat_s8x2(d, c, 0));
}

// float2int8 with rounding 0, clamped below at -127 only: trunc(max(adj, -127.5)) == max(trunc(adj), -127).
// The clamp at +127 is left to pack_sat_s8x4.
__device__ __forceinline__ int f2i8_lo_clamped(float v) {
    return __float2int_rz(fmaxf(__fadd_rn(v, half_signed(v)), -127.5f));
}

// the same for v >= 0 (after ReLU / ReLU6): copysign(0.5, v) is +0.5; v == -0 truncates to 0 either way
__device__ __forceinline__ int f2i8_nonneg(float v) { return __float2int_rz(__fadd_rn(v, 0.5f)); }

// quantize 4 floats with one scale (rounding 0) and pack them, x in byte 0
__device__ __forceinline__ uint32_t quantize4_pack(float x, float y, float z, float w, float scale) {
    // the multiplies and the additions of +-0.5 as packed pairs (same IEEE operations, half the instructions)
    const float2 sc = make_float2(scale, scale);
    const float2 a = __fmul2_rn(make_float2(x, y), sc), b = __fmul2_rn(make_float2(z, w), sc);
    const float2 ra = __fadd2_rn(a, make_float2(half_signed(a.x), half_signed(a.y)));
    const float2 rb = __fadd2_rn(b, make_float2(half_signed(b.x), half_signed(b.y)));
    return pack_sat_s8x4(__float2int_rz(fmaxf(ra.x, -127.5f)), __float2int_rz(fmaxf(ra.y, -127.5f)), __float2int_rz(fmaxf(rb.x, -127.5f)),
                         __float2int_rz(fmaxf(rb.y, -127.5f)));
}

// 4x4 byte transpose: inputs are 4 words of 4 bytes; o[i] byte j = input j byte i
__device__ __forceinline__ void transpose4x4(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t o[4]) {
    const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c, d, 0x5140);
    const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c, d, 0x7362);
    o[0] = __byte_perm(t0, t1, 0x5410);
    o[1] = __byte_perm(t0, t1, 0x7632);
    o[2] = __byte_perm(t2, t3, 0x5410);
    o[3] = __byte_perm(t2, t3, 0x7632);
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)(d & 0xff) << 24);
}

}  // namespace ottk
