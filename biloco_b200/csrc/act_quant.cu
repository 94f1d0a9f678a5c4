// NVFP4 activation quantiser: bf16 [M,K] -> E2M1 codes (two per byte, element 2j in bits 0-3), E4M3 block
// scales per 16 elements in the 128x4 atom layout, one fp32 decode scale per call.
//
// Arithmetic contract (every step is a single IEEE fp32 operation, so a CPU restatement reproduces it bit
// for bit):
//     xs   = bf16_rn(x / smooth)            (only when a smoothing vector is given)
//     gs   = amax / (6 * target)            target = 448 (static_6) or 256 (static_4, mse); gs = 1 if amax == 0
//     t    = bmax / gs                      per 16-element block
//     sfD  = e4m3_rn_sat(t / D)             D = 6 or 4
//     d    = f32(sfD) * gs
//     code = e2m1_rn(xs / d)                round-to-nearest-even on {0,.5,1,1.5,2,3,4,6}, saturating; 0 if d == 0
//     mse rule: err_D = sum_{j=0..15} (xs_j - value(code_j) * d)^2 in index order (separate mul and add);
//               the block takes D = 4 iff err_4 < err_6.
// One launch: every CTA first reduces the whole activation to its maximum (redundantly: M*K*2 bytes from L2, no
// grid-wide synchronisation needed), then the CTAs share the 16-element blocks and the zero padding between them.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/biloco_b200.h"
#include "ptx.cuh"

extern "C" int biloco_internal_use_pdl();

namespace {

// Small CTAs: with programmatic dependent launch the quantiser runs on SMs that already hold a CTA of the fused kernel.
constexpr int Q_THREADS = 128;

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

// quantise one block with divisor D; returns the squared error (only when want_err)
__device__ __forceinline__ float quant_block(const float* x, float t, float D, float gs, uint8_t* sf_out, uint32_t* codes,
                                             bool want_err) {
    const uint8_t sf = float_to_e4m3_sat(__fdiv_rn(t, D));
    const float d = __fmul_rn(e4m3_to_float(sf), gs);
    *sf_out = sf;
    float err = 0.f;
    const bool live = d > 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const uint32_t c = live ? e2m1_rn(__fdiv_rn(x[j], d)) : 0u;
        codes[j] = c;
        if (want_err) {
            const float diff = __fsub_rn(x[j], __fmul_rn(e2m1_value(c), d));
            err = __fadd_rn(err, __fmul_rn(diff, diff));
        }
    }
    return err;
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

__global__ void __launch_bounds__(Q_THREADS) act_quant_kernel(const __nv_bfloat16* __restrict__ X,
                                                              const __nv_bfloat16* __restrict__ smooth,
                                                              __nv_bfloat16* __restrict__ Xs, uint8_t* __restrict__ codes,
                                                              uint8_t* __restrict__ sf, float* __restrict__ a_gscale,
                                                              float* __restrict__ alpha_out, const float* __restrict__ w_gscale,
                                                              int M, int A_rows, int K, int rule, int given_scale, float target) {
    const int kblocks = K >> 4;
    __shared__ float red[Q_THREADS / 32];
    __shared__ float gs_sh;
    // Programmatic dependent launch: the kernel that consumes these outputs may start its own preamble (weight
    // prefetch) now; this kernel reads nothing before the previous kernel of the stream has completed.
    biloco::griddep_launch_dependents();
    biloco::griddep_wait();
    // ---- tensor scale: maximum of the (smoothed) activation, every CTA for itself ----
    if (!given_scale) {
        float amax = 0.f;
        const int nvec = (M * K) >> 3, kvec = K >> 3;                    // 128-bit vectors of 8 elements
        for (int i = threadIdx.x; i < nvec; i += Q_THREADS) {
            const uint4 a = reinterpret_cast<const uint4*>(X)[i];
            uint4 c = make_uint4(0u, 0u, 0u, 0u);
            if (smooth) c = reinterpret_cast<const uint4*>(smooth)[i % kvec];
            const uint32_t w[4] = {a.x, a.y, a.z, a.w}, v[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float lo, hi;
                unpack_smoothed(w[e], v[e], smooth != nullptr, lo, hi);
                amax = fmaxf(amax, fmaxf(fabsf(lo), fabsf(hi)));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
        __syncthreads();
        if (threadIdx.x < 32) {
            float v = threadIdx.x < Q_THREADS / 32 ? red[threadIdx.x] : 0.f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
            if (threadIdx.x == 0) gs_sh = v > 0.f ? __fdiv_rn(v, 6.0f * target) : 1.0f;
        }
    } else if (threadIdx.x == 0) {
        gs_sh = a_gscale[0];
    }
    __syncthreads();
    const float gs = gs_sh;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        if (!given_scale) a_gscale[0] = gs;
        if (alpha_out && w_gscale) alpha_out[0] = __fmul_rn(w_gscale[0], gs);
    }
    // ---- zero padding: block scales of rows M .. 128-padded row count, codes of rows M .. A_rows ----
    {
        const int rows_pad = (A_rows + 127) & ~127;
        const int kgroups = kblocks >> 2;                                // the four scales of a row's k-group are adjacent
        const int npad = (rows_pad - M) * kgroups;
        for (int i = blockIdx.x * Q_THREADS + threadIdx.x; i < npad; i += gridDim.x * Q_THREADS) {
            const int row = M + i / kgroups, kg = i % kgroups;
            *reinterpret_cast<uint32_t*>(sf + ((size_t)(row >> 7) * kgroups + kg) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4) = 0u;
        }
        const int ncode = (A_rows - M) * (K >> 4);                       // 64-bit vectors of codes
        uint2* cz = reinterpret_cast<uint2*>(codes + (size_t)M * (K >> 1));
        for (int i = blockIdx.x * Q_THREADS + threadIdx.x; i < ncode; i += gridDim.x * Q_THREADS) cz[i] = make_uint2(0u, 0u);
    }
    // ---- one thread per 16-element block ----
    for (int id = blockIdx.x * Q_THREADS + threadIdx.x; id < M * kblocks; id += gridDim.x * Q_THREADS) {
    const int row = id / kblocks, kb = id - row * kblocks;
    const size_t sf_off = ((size_t)(row >> 7) * (kblocks >> 2) + (kb >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (kb & 3);
    float x[16];
    const size_t roff = (size_t)row * K;
    {   // two 128-bit loads per operand (K % 16 == 0 and 16-byte aligned bases keep them aligned)
        const uint4* px = reinterpret_cast<const uint4*>(X + roff + kb * 16);
        const uint4 a = px[0], b = px[1];
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            x[2 * e] = __uint_as_float(w[e] << 16);
            x[2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u);
        }
        if (smooth) {
            const uint4* ps = reinterpret_cast<const uint4*>(smooth + kb * 16);
            const uint4 c = ps[0], d = ps[1];
            const uint32_t v[8] = {c.x, c.y, c.z, c.w, d.x, d.y, d.z, d.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                x[2 * e] = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(x[2 * e], __uint_as_float(v[e] << 16))));
                x[2 * e + 1] = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(x[2 * e + 1], __uint_as_float(v[e] & 0xFFFF0000u))));
            }
        }
    }
    if (Xs) {
        uint32_t o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (__float_as_uint(x[2 * e]) >> 16) | (__float_as_uint(x[2 * e + 1]) & 0xFFFF0000u);
        uint4* po = reinterpret_cast<uint4*>(Xs + roff + kb * 16);
        po[0] = make_uint4(o[0], o[1], o[2], o[3]);
        po[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
    float bmax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) bmax = fmaxf(bmax, fabsf(x[j]));
    const float t = __fdiv_rn(bmax, gs);
    uint32_t c[16];
    uint8_t s;
    if (rule == BILOCO_RULE_STATIC_6) {
        quant_block(x, t, 6.0f, gs, &s, c, false);
    } else if (rule == BILOCO_RULE_STATIC_4) {
        quant_block(x, t, 4.0f, gs, &s, c, false);
    } else {
        uint32_t c4[16];
        uint8_t s4;
        const float e6 = quant_block(x, t, 6.0f, gs, &s, c, true);
        const float e4 = quant_block(x, t, 4.0f, gs, &s4, c4, true);
        if (e4 < e6) {
            s = s4;
#pragma unroll
            for (int j = 0; j < 16; ++j) c[j] = c4[j];
        }
    }
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        lo |= c[j] << (4 * j);
        hi |= c[8 + j] << (4 * j);
    }
    *reinterpret_cast<uint2*>(codes + (size_t)row * (K >> 1) + kb * 8) = make_uint2(lo, hi);
    sf[sf_off] = s;
    }
}

}  // namespace

extern "C" int biloco_b200_act_quant(const void* X_bf16, const void* smooth_bf16, void* Xs_bf16, void* A_codes, void* A_sf,
                                     float* a_gscale, float* alpha_out, const float* w_gscale, int M, int A_rows, int K,
                                     int rule, biloco_stream_t stream) {
    if (!X_bf16 || !A_codes || !A_sf || !a_gscale) return BILOCO_ERR_NULL;
    if (M < 1 || A_rows < M || A_rows > 128 || K < 64 || (K % 64) != 0) return BILOCO_ERR_SHAPE;
    const bool given_scale = (rule & BILOCO_RULE_GIVEN_SCALE) != 0;
    rule &= ~BILOCO_RULE_GIVEN_SCALE;
    if (rule != BILOCO_RULE_STATIC_6 && rule != BILOCO_RULE_STATIC_4 && rule != BILOCO_RULE_MSE) return BILOCO_ERR_MODE;
    if (((uintptr_t)A_codes & 7) || ((uintptr_t)X_bf16 & 15) || ((uintptr_t)smooth_bf16 & 15) || ((uintptr_t)Xs_bf16 & 15))
        return BILOCO_ERR_ALIGN;
    cudaStream_t s = (cudaStream_t)stream;
    const float target = rule == BILOCO_RULE_STATIC_6 ? 448.0f : 256.0f;
    int nblk = (M * (K >> 4) + Q_THREADS - 1) / Q_THREADS;
    if (nblk > 96) nblk = 96;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)nblk);
    cfg.blockDim = dim3(Q_THREADS);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = biloco_internal_use_pdl() ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, act_quant_kernel, (const __nv_bfloat16*)X_bf16, (const __nv_bfloat16*)smooth_bf16,
                           (__nv_bfloat16*)Xs_bf16, (uint8_t*)A_codes, (uint8_t*)A_sf, a_gscale, alpha_out, w_gscale, M, A_rows, K,
                           rule, given_scale ? 1 : 0, target) != cudaSuccess)
        return BILOCO_ERR_CUDA;
    return cudaGetLastError() == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}
