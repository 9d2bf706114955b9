// Epilogue building blocks shared by the tensor-core kernels that keep intermediates on the SM (unit_umma.cu, dw_umma.cu):
// requantization of 16 accumulator columns, stores into 32-byte-swizzled operand blocks in shared memory, and the output
// stage of a layer (one accumulator row = one output pixel) in the forms dense_umma.cu also writes.
#pragma once

#include "dense_umma.h"
#include "umma_primitives.cuh"

namespace ottk {

// 16 accumulators -> 16 int8 (rounding rule: add half, truncate), packed into four words
template <int ACT>
__device__ __forceinline__ void requant16(const int (&v)[16], const float* __restrict__ s_si, const float* __restrict__ s_bi,
                                          const float* __restrict__ s_so, float p0, uint32_t (&wds)[4]) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const float4 si = *reinterpret_cast<const float4*>(s_si + g * 4);
        const float4 bi = *reinterpret_cast<const float4*>(s_bi + g * 4);
        const float4 so = *reinterpret_cast<const float4*>(s_so + g * 4);
        int qv[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float2 a = make_float2(__int2float_rn(v[g * 4 + 2 * h]), __int2float_rn(v[g * 4 + 2 * h + 1]));
            const float2 t = __ffma2_rn(a, h ? make_float2(si.z, si.w) : make_float2(si.x, si.y), h ? make_float2(bi.z, bi.w) : make_float2(bi.x, bi.y));
            const float2 y = make_float2(activate_t<ACT>(t.x, p0), activate_t<ACT>(t.y, p0));
            const float2 u = __fmul2_rn(y, h ? make_float2(so.z, so.w) : make_float2(so.x, so.y));
            if (ACT == ACT_RELU || ACT == ACT_RELU6) {
                const float2 r = __fadd2_rn(u, make_float2(0.5f, 0.5f));
                qv[2 * h] = __float2int_rz(r.x);
                qv[2 * h + 1] = __float2int_rz(r.y);
            } else {
                const float2 r = __fadd2_rn(u, make_float2(half_signed(u.x), half_signed(u.y)));
                qv[2 * h] = __float2int_rz(fmaxf(r.x, -127.5f));
                qv[2 * h + 1] = __float2int_rz(fmaxf(r.y, -127.5f));
            }
        }
        wds[g] = pack_sat_s8x4(qv[0], qv[1], qv[2], qv[3]);
    }
}

// Address of 16-byte chunk `chunk` (0/1) of 32-byte row `row` of an operand block at `block` (32-byte swizzle: the chunk
// index is XORed with address bit 7, for the TMA engine, the MMA's reads and these stores alike).
__device__ __forceinline__ uint32_t swz32(uint32_t block, int row, int chunk) {
    const uint32_t a = block + (uint32_t)row * 32u + (uint32_t)chunk * 16u;
    return a ^ (((a >> 7) & 1u) << 4);
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// One accumulator row (this thread's TMEM lane = one output pixel) through a layer's output stage: fma(acc, scale_in, bias) ->
// activation -> fp32 NCHW planes, or float2int8(v * scale_out) as int8 NHWC (32-byte stores where the channel stride allows)
// with chosen channels also stored as fp32 planes (mixed). taddr = accumulator address with this warp's lane window selected;
// ncols = accumulator columns (a multiple of 32); warps sharing a lane quarter take every nsub-th 32-column chunk, starting
// at chunk sub. s_si / s_bi / s_so: the per-channel parameters of these columns in shared memory. inimg = oy * w + ox.
// c_base: the layer's channel that accumulator column 0 holds (a CTA may own a slice of the layer's channels).
template <int ACT, int OUT>
__device__ __forceinline__ void store_accumulator_row(uint32_t taddr, int ncols, int sub, int nsub, bool valid, int img, long inimg, long plane,
                                                      const float* __restrict__ s_si, const float* __restrict__ s_bi, const float* __restrict__ s_so,
                                                      float p0, int cpad, int cout, void* __restrict__ out, const UmmaMixedOut& mixed, int c_base = 0) {
    using namespace umma;
    const long pix = (long)img * plane + inimg;
    int8_t* out_s8 = reinterpret_cast<int8_t*>(out) + pix * cpad + c_base;
    float* out_f32 = nullptr;
    if (OUT == DT_F32_NCHW) out_f32 = reinterpret_cast<float*>(out) + (long)img * cout * plane + inimg;
    else if (mixed.out_f32 != nullptr)
        out_f32 = mixed.out_f32 + (long)img * (mixed.plane_of_col != nullptr ? mixed.f32_planes : cout) * plane + inimg;
    for (int c0 = sub * 32; c0 < ncols; c0 += nsub * 32) {
        int v[2][16];
        const bool two = c0 + 16 < ncols;
        __syncwarp();
        tmem_ld16(taddr + (uint32_t)c0, v[0]);
        if (two) tmem_ld16(taddr + (uint32_t)(c0 + 16), v[1]);
        tmem_wait_ld16(v[0]);
        tmem_wait_ld16(v[1]);
        if (!valid) continue;
        uint32_t wds[2][4];
        const bool have[2] = {c_base + c0 < cpad, two && c_base + c0 + 16 < cpad};
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            if (!have[half]) continue;
            const int cc = c0 + 16 * half;
            const float* si = s_si + cc;
            const float* bi = s_bi + cc;
            const float* so = s_so + cc;
            float y[16];
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const float4 s4 = *reinterpret_cast<const float4*>(si + g * 4);
                const float4 b4 = *reinterpret_cast<const float4*>(bi + g * 4);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float2 a = make_float2(__int2float_rn(v[half][g * 4 + 2 * h]), __int2float_rn(v[half][g * 4 + 2 * h + 1]));
                    const float2 t = __ffma2_rn(a, h ? make_float2(s4.z, s4.w) : make_float2(s4.x, s4.y), h ? make_float2(b4.z, b4.w) : make_float2(b4.x, b4.y));
                    y[g * 4 + 2 * h] = activate_t<ACT>(t.x, p0);
                    y[g * 4 + 2 * h + 1] = activate_t<ACT>(t.y, p0);
                }
            }
            if (OUT == DT_F32_NCHW) {
                float* o = out_f32 + (long)(c_base + cc) * plane;
                if (c_base + cc + 16 <= cout) {
#pragma unroll
                    for (int j = 0; j < 16; ++j, o += plane) *o = y[j];
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j, o += plane)
                        if (c_base + cc + j < cout) *o = y[j];
                }
                continue;
            }
            if (out_f32 != nullptr) {
                // channels that some reader wants in fp32: the planes an fp32-output layer would have written
                const int gc = c_base + cc;
                const uint32_t mk = (mixed.mask[(gc >> 5) & 31] >> (gc & 31)) & 0xFFFFu;
                if (mk != 0u) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if ((mk >> j) & 1u) {
                            const long pl = mixed.plane_of_col != nullptr ? (long)mixed.plane_of_col[gc + j] : (long)(gc + j);
                            out_f32[pl * plane] = y[j];
                        }
                }
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const float4 o4 = *reinterpret_cast<const float4*>(so + g * 4);
                int qv[4];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float2 u = __fmul2_rn(make_float2(y[g * 4 + 2 * h], y[g * 4 + 2 * h + 1]), h ? make_float2(o4.z, o4.w) : make_float2(o4.x, o4.y));
                    if (ACT == ACT_RELU || ACT == ACT_RELU6) {
                        const float2 rr = __fadd2_rn(u, make_float2(0.5f, 0.5f));
                        qv[2 * h] = __float2int_rz(rr.x);
                        qv[2 * h + 1] = __float2int_rz(rr.y);
                    } else {
                        const float2 rr = __fadd2_rn(u, make_float2(half_signed(u.x), half_signed(u.y)));
                        qv[2 * h] = __float2int_rz(fmaxf(rr.x, -127.5f));
                        qv[2 * h + 1] = __float2int_rz(fmaxf(rr.y, -127.5f));
                    }
                }
                wds[half][g] = pack_sat_s8x4(qv[0], qv[1], qv[2], qv[3]);
            }
        }
        if (OUT == DT_S8_NHWC) {
            if (have[0] && have[1] && (cpad & 31) == 0) {
                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(out_s8 + c0), "r"(wds[0][0]), "r"(wds[0][1]), "r"(wds[0][2]),
                             "r"(wds[0][3]), "r"(wds[1][0]), "r"(wds[1][1]), "r"(wds[1][2]), "r"(wds[1][3])
                             : "memory");
            } else {
                if (have[0]) *reinterpret_cast<uint4*>(out_s8 + c0) = make_uint4(wds[0][0], wds[0][1], wds[0][2], wds[0][3]);
                if (have[1]) *reinterpret_cast<uint4*>(out_s8 + c0 + 16) = make_uint4(wds[1][0], wds[1][1], wds[1][2], wds[1][3]);
            }
        }
    }
}

}  // namespace ottk
