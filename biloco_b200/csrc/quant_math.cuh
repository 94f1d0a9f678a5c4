// NVFP4 quantisation arithmetic shared by the stand-alone quantiser (act_quant.cu) and the fused linear's own
// activation prologue (slab_kernel.cuh). Every step is one IEEE fp32 operation, so a CPU restatement matches bit for bit:
//     t    = bmax / gs                      per 16-element block
//     sfD  = e4m3_rn_sat(t / D)             D = 6 or 4
//     d    = f32(sfD) * gs
//     code = e2m1_rn(x / d)                 round-to-nearest-even on {0,.5,1,1.5,2,3,4,6}, saturating; 0 if d == 0
//     mse rule: err_D = sum_{j=0..15} (x_j - value(code_j) * d)^2 in index order (separate multiply and add);
//               the block takes D = 4 iff err_4 < err_6.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace biloco {
namespace qm {

__device__ __forceinline__ uint32_t e2m1_rn(float q) {
    const float a = fabsf(q);
    uint32_t c = (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f);
    return c | ((__float_as_uint(q) >> 31) << 3);
}
__device__ __forceinline__ float e2m1_value(uint32_t code) {
    const uint32_t m = code & 7u;
    // 0, .5, 1, 1.5, 2, 3, 4, 6
    const float mag = m < 4u ? 0.5f * (float)m : (m == 4u ? 2.0f : (m == 5u ? 3.0f : (m == 6u ? 4.0f : 6.0f)));
    return (code & 8u) ? -mag : mag;
}
__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(__half(h));
}
__device__ __forceinline__ uint8_t float_to_e4m3_sat(float v) {
    return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// bf16 pair -> two floats, optionally divided by the smoothing pair and rounded back to bf16
__device__ __forceinline__ void unpack_smoothed(uint32_t w, uint32_t sm, bool smooth, float& lo, float& hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xFFFF0000u);
    if (smooth) {
        lo = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(lo, __uint_as_float(sm << 16))));
        hi = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(hi, __uint_as_float(sm & 0xFFFF0000u))));
    }
}

// One element per lane, sixteen lanes per block (lanes 0-15 and 16-31 of a warp hold one block each, all 32 lanes must
// call): the block-wide steps -- maximum, the squared errors summed in index order, packing -- go through shuffles.
// Returns in the block's first lane (lane % 16 == 0) the eight bytes of codes (element 2i in bits 0-3 of byte i) and the
// block's E4M3 scale. rule: 0 static_6, 1 static_4, 2 mse.
__device__ __forceinline__ void quant_lane16(float x, int lane, float gs, int rule, uint2& codes, uint8_t& sf) {
    const int base = lane & 16;
    float bmax = fabsf(x);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, o));
    const float t = __fdiv_rn(bmax, gs);
    uint32_t c6 = 0, c4 = 0;
    uint8_t s6 = 0, s4 = 0;
    float e6 = 0.f, e4 = 0.f;
#pragma unroll
    for (int cand = 0; cand < 2; ++cand) {
        if (cand == 0 && rule == 1) continue;
        if (cand == 1 && rule == 0) continue;
        const uint8_t sfv = float_to_e4m3_sat(__fdiv_rn(t, cand == 0 ? 6.0f : 4.0f));
        const float d = __fmul_rn(e4m3_to_float(sfv), gs);
        const uint32_t c = d > 0.f ? e2m1_rn(__fdiv_rn(x, d)) : 0u;
        float err = 0.f;
        if (rule == 2) {
            const float diff = __fsub_rn(x, __fmul_rn(e2m1_value(c), d));
            const float sq = __fmul_rn(diff, diff);
#pragma unroll
            for (int i = 0; i < 16; ++i) err = __fadd_rn(err, __shfl_sync(0xffffffffu, sq, base + i));   // index order
        }
        if (cand == 0) { c6 = c; s6 = sfv; e6 = err; } else { c4 = c; s4 = sfv; e4 = err; }
    }
    uint32_t code;
    if (rule == 0 || (rule == 2 && !(e4 < e6))) { code = c6; sf = s6; } else { code = c4; sf = s4; }
    // pack: two codes per byte, four bytes per word; the words of elements 0-7 and 8-15 end up in lanes base and base + 8
    uint32_t w = code | (__shfl_down_sync(0xffffffffu, code, 1) << 4);
    w |= (__shfl_down_sync(0xffffffffu, w, 2) << 8) | (__shfl_down_sync(0xffffffffu, w, 4) << 16) |
         (__shfl_down_sync(0xffffffffu, w, 6) << 24);
    codes = make_uint2(w, __shfl_down_sync(0xffffffffu, w, 8));
}

}  // namespace qm
}  // namespace biloco
