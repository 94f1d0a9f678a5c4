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
// grid-wide synchronisation needed), then the CTAs share the elements (one lane each, sixteen lanes per block, the
// block-wide steps through shuffles) and the zero padding between them.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/biloco_b200.h"
#include "ptx.cuh"
#include "quant_math.cuh"

extern "C" int biloco_internal_use_pdl();

namespace {

// Small CTAs: with programmatic dependent launch the quantiser runs on SMs that already hold a CTA of the fused kernel.
constexpr int Q_THREADS = 256;
constexpr int Q_MAX_CLUSTER = 8;

using biloco::qm::e2m1_rn;
using biloco::qm::e2m1_value;
using biloco::qm::e4m3_to_float;
using biloco::qm::float_to_e4m3_sat;
using biloco::qm::unpack_smoothed;

__global__ void __launch_bounds__(Q_THREADS) act_quant_kernel(const __nv_bfloat16* X, const __nv_bfloat16* smooth,
                                                              __nv_bfloat16* Xs, uint8_t* __restrict__ codes,
                                                              uint8_t* __restrict__ sf, float* __restrict__ a_gscale,
                                                              float* __restrict__ alpha_out, const float* __restrict__ w_gscale,
                                                              int M, int A_rows, int K, int rule, int given_scale, float target,
                                                              int csize, const __nv_bfloat16* __restrict__ norm_w, float eps, int n_alpha,
                                                              uint8_t* __restrict__ rec, int swiglu) {
    const int kblocks = K >> 4;
    __shared__ float red[Q_THREADS / 32];
    __shared__ float gs_sh;
    // Programmatic dependent launch: the kernel that consumes these outputs may start its own preamble (weight
    // prefetch) now; this kernel reads nothing before the previous kernel of the stream has completed.
    biloco::griddep_launch_dependents();
    biloco::griddep_wait();
    // ---- optional RMSNorm in front (per row: x * rsqrt(mean(x^2) + eps), rounded to bf16, times the bf16 weight, rounded
    //      to bf16; then the smoothing division): CTA r of the cluster takes rows r, r + csize, ..., two passes over a
    //      row (sum of squares, then normalise and store); every cluster does all rows (same values), and after the
    //      cluster barrier the rest of the kernel reads the normalised activation it has just written ----
    if (norm_w) {
        const int kvec = K >> 3;
        for (int row = csize > 1 ? (int)(blockIdx.x % (unsigned)csize) : 0; row < M; row += csize) {
            const uint4* xr = reinterpret_cast<const uint4*>(X + (size_t)row * K);
            float ss = 0.f;
            for (int i = threadIdx.x; i < kvec; i += Q_THREADS) {
                const uint4 a = xr[i];
                const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xFFFF0000u);
                    ss = fmaf(lo, lo, ss);
                    ss = fmaf(hi, hi, ss);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            __syncthreads();                                  // (red is reused from the previous row)
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
            __syncthreads();
            float tot = 0.f;
#pragma unroll
            for (int i = 0; i < Q_THREADS / 32; ++i) tot += red[i];
            const float inv = rsqrtf(tot / (float)K + eps);
            uint4* xo = reinterpret_cast<uint4*>(Xs + (size_t)row * K);
            for (int i = threadIdx.x; i < kvec; i += Q_THREADS) {
                const uint4 a = xr[i], g = reinterpret_cast<const uint4*>(norm_w)[i];
                uint4 c = make_uint4(0u, 0u, 0u, 0u);
                if (smooth) c = reinterpret_cast<const uint4*>(smooth)[i];
                const uint32_t w[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w}, sw[4] = {c.x, c.y, c.z, c.w};
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v[2] = {__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xFFFF0000u)};
                    const float gv[2] = {__uint_as_float(gw[e] << 16), __uint_as_float(gw[e] & 0xFFFF0000u)};
                    const float sv[2] = {__uint_as_float(sw[e] << 16), __uint_as_float(sw[e] & 0xFFFF0000u)};
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        v[h] = __bfloat162float(__float2bfloat16_rn(v[h] * inv));
                        v[h] = __bfloat162float(__float2bfloat16_rn(v[h] * gv[h]));
                        if (smooth) v[h] = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(v[h], sv[h])));
                    }
                    o[e] = (__float_as_uint(v[0]) >> 16) | (__float_as_uint(v[1]) & 0xFFFF0000u);
                }
                xo[i] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
        __threadfence();
        if (csize > 1) biloco::cluster_sync_all();
        else __syncthreads();
        X = Xs;                 // from here on: an already normalised and smoothed activation, nothing left to write back
        smooth = nullptr;
        Xs = nullptr;
    }
    // ---- optional gated activation in front: X is [M, 2K] = [gate | up] (the stacked output of a gate/up launch) and the
    //      activation is bf16(bf16(silu(gate)) * up), silu(g) = g / (1 + exp(-g)) in fp32 (the roundings of the separate
    //      silu and multiply kernels it replaces); then the smoothing division. Rows are shared as in the norm path ----
    if (swiglu) {
        const int kvec = K >> 3;
        for (int row = csize > 1 ? (int)(blockIdx.x % (unsigned)csize) : 0; row < M; row += csize) {
            const uint4* gr = reinterpret_cast<const uint4*>(X + (size_t)row * 2 * K);
            const uint4* ur = gr + kvec;
            uint4* xo = reinterpret_cast<uint4*>(Xs + (size_t)row * K);
            for (int i = threadIdx.x; i < kvec; i += Q_THREADS) {
                const uint4 a = gr[i], b = ur[i];
                uint4 c = make_uint4(0u, 0u, 0u, 0u);
                if (smooth) c = reinterpret_cast<const uint4*>(smooth)[i];
                const uint32_t gw[4] = {a.x, a.y, a.z, a.w}, uw[4] = {b.x, b.y, b.z, b.w}, sw[4] = {c.x, c.y, c.z, c.w};
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float gv[2] = {__uint_as_float(gw[e] << 16), __uint_as_float(gw[e] & 0xFFFF0000u)};
                    const float uv[2] = {__uint_as_float(uw[e] << 16), __uint_as_float(uw[e] & 0xFFFF0000u)};
                    const float sv[2] = {__uint_as_float(sw[e] << 16), __uint_as_float(sw[e] & 0xFFFF0000u)};
                    float v[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        v[h] = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(gv[h], __fadd_rn(1.0f, expf(-gv[h])))));
                        v[h] = __bfloat162float(__float2bfloat16_rn(__fmul_rn(v[h], uv[h])));
                        if (smooth) v[h] = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(v[h], sv[h])));
                    }
                    o[e] = (__float_as_uint(v[0]) >> 16) | (__float_as_uint(v[1]) & 0xFFFF0000u);
                }
                xo[i] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
        __threadfence();
        if (csize > 1) biloco::cluster_sync_all();
        else __syncthreads();
        X = Xs;
        smooth = nullptr;
        Xs = nullptr;
    }
    // ---- tensor scale: maximum of the (smoothed) activation. Every cluster of `csize` CTAs computes it for itself (no
    //      grid-wide synchronisation): a CTA reduces its share of the 128-bit vectors, the CTAs of the cluster exchange
    //      their maxima through distributed shared memory ----
    __shared__ float cl_red[Q_MAX_CLUSTER];
    const int crank = csize > 1 ? (int)(blockIdx.x % (unsigned)csize) : 0;
    if (!given_scale) {
        float amax = 0.f;
        const int nvec = (M * K) >> 3, kvec = K >> 3;                    // 128-bit vectors of 8 elements
#pragma unroll 4
        for (int i = crank * Q_THREADS + threadIdx.x; i < nvec; i += csize * Q_THREADS) {
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
            if (csize > 1) {       // lane r hands this CTA's maximum to CTA r of the cluster
                if (threadIdx.x < csize)
                    biloco::st_cluster_f32(biloco::map_to_cta(biloco::smem_u32(&cl_red[crank]), (uint32_t)threadIdx.x), v);
            } else if (threadIdx.x == 0) {
                cl_red[0] = v;
            }
        }
        if (csize > 1) biloco::cluster_sync_all();      // (release/acquire: the peers' values are in cl_red)
        else __syncthreads();
        if (threadIdx.x == 0) {
            float v = 0.f;
            for (int r = 0; r < csize; ++r) v = fmaxf(v, cl_red[r]);
            gs_sh = v > 0.f ? __fdiv_rn(v, 6.0f * target) : 1.0f;
        }
    } else if (threadIdx.x == 0) {
        gs_sh = a_gscale[0];
    }
    __syncthreads();
    const float gs = gs_sh;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        if (!given_scale) a_gscale[0] = gs;
        if (alpha_out && w_gscale)
            for (int i = 0; i < n_alpha; ++i) alpha_out[i] = __fmul_rn(w_gscale[i], gs);     // one per consumer of this activation
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
        // the per-k-tile record for the fused kernel, if asked for: [tile: mma_n rows x 128 B | four scale atoms]; rows M.. zero
        if (rec) {
            const int mma_n = M <= 8 ? 8 : (M <= 16 ? 16 : 32), nkt = K >> 8;
            const int rec_bytes = mma_n * 128 + 2048;
            const int tile_pad = (mma_n - M) * 8;                         // 16-byte chunks of the rows M .. mma_n-1 of one tile
            for (int i = blockIdx.x * Q_THREADS + threadIdx.x; i < nkt * tile_pad; i += gridDim.x * Q_THREADS) {
                const int kt = i / tile_pad, c = i - kt * tile_pad;
                *reinterpret_cast<uint4*>(rec + (size_t)kt * rec_bytes + M * 128 + c * 16) = make_uint4(0u, 0u, 0u, 0u);
            }
            const int sf_pad = (128 - M) * 4;                             // 4-byte groups of the rows M .. 127 of one k-tile's atoms
            for (int i = blockIdx.x * Q_THREADS + threadIdx.x; i < nkt * sf_pad; i += gridDim.x * Q_THREADS) {
                const int kt = i / sf_pad, r = i - kt * sf_pad;
                const int row = M + (r >> 2), a = r & 3;
                *reinterpret_cast<uint32_t*>(rec + (size_t)kt * rec_bytes + mma_n * 128 + a * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4) = 0u;
            }
        }
        const int ncode = (A_rows - M) * (K >> 4);                       // 64-bit vectors of codes
        uint2* cz = reinterpret_cast<uint2*>(codes + (size_t)M * (K >> 1));
        for (int i = blockIdx.x * Q_THREADS + threadIdx.x; i < ncode; i += gridDim.x * Q_THREADS) cz[i] = make_uint2(0u, 0u);
    }
    // ---- one lane per element, sixteen lanes per block: a lane's code is a handful of instructions, the block-wide
    //      steps (maximum, the squared errors summed in index order, packing) go through shuffles ----
    const int total = M * K;                                   // multiple of 64, so whole warps stay together
    for (int e0 = blockIdx.x * Q_THREADS; e0 < total; e0 += gridDim.x * Q_THREADS) {
        const int e = e0 + threadIdx.x;                        // (total % Q_THREADS may be 64: the upper half-CTA idles)
        if (e >= total) break;
        const int row = e / K, k = e - row * K;
        const int kb = k >> 4, j = k & 15;
        const int lane = threadIdx.x & 31, base = lane & 16;  // first lane of this block's group
        float x = __bfloat162float(X[e]);
        if (smooth) x = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(x, __bfloat162float(smooth[k]))));
        if (Xs) Xs[e] = __float2bfloat16_rn(x);                // (exact: x is a bf16 value)
        float bmax = fabsf(x);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, o));
        const float t = __fdiv_rn(bmax, gs);
        uint32_t code = 0;
        uint8_t sfb = 0;
        float e6 = 0.f, e4 = 0.f;
        uint32_t c6 = 0, c4 = 0;
        uint8_t s6 = 0, s4 = 0;
#pragma unroll
        for (int cand = 0; cand < 2; ++cand) {
            const float D = cand == 0 ? 6.0f : 4.0f;
            if (cand == 0 && rule == BILOCO_RULE_STATIC_4) continue;
            if (cand == 1 && rule == BILOCO_RULE_STATIC_6) continue;
            const uint8_t sfv = float_to_e4m3_sat(__fdiv_rn(t, D));
            const float d = __fmul_rn(e4m3_to_float(sfv), gs);
            const uint32_t c = d > 0.f ? e2m1_rn(__fdiv_rn(x, d)) : 0u;
            float err = 0.f;
            if (rule == BILOCO_RULE_MSE) {
                const float diff = __fsub_rn(x, __fmul_rn(e2m1_value(c), d));
                const float sq = __fmul_rn(diff, diff);
#pragma unroll
                for (int i = 0; i < 16; ++i) err = __fadd_rn(err, __shfl_sync(0xffffffffu, sq, base + i));   // index order
            }
            if (cand == 0) { c6 = c; s6 = sfv; e6 = err; } else { c4 = c; s4 = sfv; e4 = err; }
        }
        if (rule == BILOCO_RULE_STATIC_6 || (rule == BILOCO_RULE_MSE && !(e4 < e6))) { code = c6; sfb = s6; }
        else { code = c4; sfb = s4; }
        // pack: two codes per byte (element 2i in bits 0-3), four bytes per word; lanes 0 and 8 of the group store
        uint32_t w = code | (__shfl_down_sync(0xffffffffu, code, 1) << 4);
        w |= (__shfl_down_sync(0xffffffffu, w, 2) << 8) | (__shfl_down_sync(0xffffffffu, w, 4) << 16) |
             (__shfl_down_sync(0xffffffffu, w, 6) << 24);
        if ((j & 7) == 0) *reinterpret_cast<uint32_t*>(codes + (size_t)row * (K >> 1) + kb * 8 + (j >> 3) * 4) = w;
        if (j == 0)
            sf[((size_t)(row >> 7) * (kblocks >> 2) + (kb >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (kb & 3)] = sfb;
        if (rec) {      // the same codes and scale where the fused kernel's stage wants them (128-byte swizzle: chunk c of row r at c ^ (r & 7))
            const int mma_n = M <= 8 ? 8 : (M <= 16 ? 16 : 32);
            uint8_t* rk = rec + (size_t)(kb >> 4) * (mma_n * 128 + 2048);
            const int b = (kb & 15) * 8 + (j >> 3) * 4;                   // byte of the word within the tile row
            if ((j & 7) == 0) *reinterpret_cast<uint32_t*>(rk + row * 128 + (((b >> 4) ^ (row & 7)) << 4) + (b & 15)) = w;
            if (j == 0) rk[mma_n * 128 + ((kb >> 2) & 3) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (kb & 3)] = sfb;
        }
    }
}

}  // namespace

static int launch_act_quant(const void* X_bf16, const void* norm_w, float eps, const void* smooth_bf16, void* Xs_bf16, void* A_codes,
                            void* A_sf, void* A_rec, float* a_gscale, float* alpha_out, const float* w_gscale, int n_alpha, int M,
                            int A_rows, int K, int rule, biloco_stream_t stream, int swiglu = 0) {
    if (swiglu && (!Xs_bf16 || norm_w)) return BILOCO_ERR_NULL;
    if (A_rec && (M > 32 || (K % 256) != 0 || ((uintptr_t)A_rec & 15))) return BILOCO_ERR_SHAPE;
    if (!X_bf16 || !A_codes || !A_sf || !a_gscale) return BILOCO_ERR_NULL;
    if (norm_w && !Xs_bf16) return BILOCO_ERR_NULL;
    if (n_alpha < 1 || n_alpha > 16) return BILOCO_ERR_SHAPE;
    if ((uintptr_t)norm_w & 15) return BILOCO_ERR_ALIGN;
    if (M < 1 || A_rows < M || A_rows > 128 || K < 64 || (K % 64) != 0) return BILOCO_ERR_SHAPE;
    const bool given_scale = (rule & BILOCO_RULE_GIVEN_SCALE) != 0;
    rule &= ~BILOCO_RULE_GIVEN_SCALE;
    if (rule != BILOCO_RULE_STATIC_6 && rule != BILOCO_RULE_STATIC_4 && rule != BILOCO_RULE_MSE) return BILOCO_ERR_MODE;
    if (((uintptr_t)A_codes & 7) || ((uintptr_t)X_bf16 & 15) || ((uintptr_t)smooth_bf16 & 15) || ((uintptr_t)Xs_bf16 & 15))
        return BILOCO_ERR_ALIGN;
    cudaStream_t s = (cudaStream_t)stream;
    const float target = rule == BILOCO_RULE_STATIC_6 ? 448.0f : 256.0f;
    // cluster size: at most about ten 128-bit loads per thread in the maximum phase; CTAs: one element per lane up to 128 CTAs
    int csize = 1;
    while (csize < Q_MAX_CLUSTER && (M * K / 8) > csize * Q_THREADS * 10) csize *= 2;
    int nblk = (M * K + Q_THREADS - 1) / Q_THREADS;
    if (nblk > 128) nblk = 128;
    nblk = (nblk + csize - 1) / csize * csize;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)nblk);
    cfg.blockDim = dim3(Q_THREADS);
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (biloco_internal_use_pdl()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (csize > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)csize;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (cudaLaunchKernelEx(&cfg, act_quant_kernel, (const __nv_bfloat16*)X_bf16, (const __nv_bfloat16*)smooth_bf16,
                           (__nv_bfloat16*)Xs_bf16, (uint8_t*)A_codes, (uint8_t*)A_sf, a_gscale, alpha_out, w_gscale, M, A_rows, K,
                           rule, given_scale ? 1 : 0, target, csize, (const __nv_bfloat16*)norm_w, eps, n_alpha, (uint8_t*)A_rec, swiglu) != cudaSuccess)
        return BILOCO_ERR_CUDA;
    return cudaGetLastError() == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}

extern "C" int biloco_b200_act_quant(const void* X_bf16, const void* smooth_bf16, void* Xs_bf16, void* A_codes, void* A_sf,
                                     float* a_gscale, float* alpha_out, const float* w_gscale, int M, int A_rows, int K,
                                     int rule, biloco_stream_t stream) {
    return launch_act_quant(X_bf16, nullptr, 0.f, smooth_bf16, Xs_bf16, A_codes, A_sf, nullptr, a_gscale, alpha_out, w_gscale, 1, M, A_rows,
                            K, rule, stream);
}

extern "C" int biloco_b200_norm_act_quant(const void* X_bf16, const void* norm_weight_bf16, float eps, const void* smooth_bf16,
                                          void* Xn_bf16, void* A_codes, void* A_sf, void* A_rec, float* a_gscale, float* alpha_out,
                                          const float* w_gscale, int n_alpha, int M, int A_rows, int K, int rule,
                                          biloco_stream_t stream) {
    return launch_act_quant(X_bf16, norm_weight_bf16, eps, smooth_bf16, Xn_bf16, A_codes, A_sf, A_rec, a_gscale, alpha_out, w_gscale,
                            n_alpha, M, A_rows, K, rule, stream);
}

extern "C" int biloco_b200_swiglu_act_quant(const void* GU_bf16, const void* smooth_bf16, void* Xa_bf16, void* A_codes, void* A_sf,
                                            void* A_rec, float* a_gscale, float* alpha_out, const float* w_gscale, int n_alpha, int M,
                                            int A_rows, int K, int rule, biloco_stream_t stream) {
    return launch_act_quant(GU_bf16, nullptr, 0.f, smooth_bf16, Xa_bf16, A_codes, A_sf, A_rec, a_gscale, alpha_out, w_gscale, n_alpha, M,
                            A_rows, K, rule, stream, 1);
}
