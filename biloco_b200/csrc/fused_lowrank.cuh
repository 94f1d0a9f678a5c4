// CUDA-core half of the fused linear: the z stage (z = S .* (X sign(V)^T) for this CTA's slice of the ranks) and the
// expansion of z through the packed U signs. Both are written for small machine code (rolled loops, the row count
// is a template parameter) and for one memory round trip per step: every global read is issued in a single batch.
#pragma once
#include "fused_cfg.cuh"

namespace biloco {

// z stage, run by the 128 epilogue threads. CTA `cta` owns ranks [cta*R/G, (cta+1)*R/G). Per pass a tile of the
// activation (RP rows x XK k) and the sign words of up to VT_RANKS ranks are copied to shared memory with one
// batch of cp.async; then warp q accumulates rank q (and q+4): lane l owns the 32-bit sign words l, l+32, ... of
// the tile and reads the matching 32 activations as four conflict-free 128-bit shared loads.
// The sign words of the very first pass are weights, not activations: the caller copies them (z_prefetch_v) before it
// waits for the previous kernel of the stream, and passes v_preloaded = true.
template <int ROWS>
__device__ __forceinline__ void z_stage(const FusedParams& p, uint8_t* work, float* zb, int cta, int tid, bool v_preloaded) {
    constexpr int RP = ROWS < 8 ? ROWS : 8;          // rows per pass
    constexpr int XK = XT_BYTES / 2 / RP;            // k per pass
    constexpr int XW = XK / 32;                      // sign words per rank per pass
    constexpr int JN = XW / 32;                      // sign words per lane per pass
    static_assert(JN >= 1, "activation tile too small");
    const int warp = tid >> 5, lane = tid & 31;
    const int i0 = cta * p.R / p.G;
    const int i1 = (cta + 1) * p.R / p.G;
    const uint32_t xt_s = smem_u32(work);
    const uint32_t vt_s = xt_s + XT_BYTES;
    const uint32_t* vt = reinterpret_cast<const uint32_t*>(work + XT_BYTES);
    const int kbytes = p.K >> 3;

#pragma unroll 1
    for (int ic = i0; ic < i1; ic += VT_RANKS) {
        const int nr = (i1 - ic) < VT_RANKS ? (i1 - ic) : VT_RANKS;
#pragma unroll 1
        for (int mg = 0; mg < p.M; mg += RP) {       // rows beyond M inside a group repeat row M-1
            float zacc0 = 0.f, zacc1 = 0.f;          // lane mm holds row mg+mm of rank slots warp, warp+4
#pragma unroll 1
            for (int k0 = 0; k0 < p.K; k0 += XK) {
                const int kc = (p.K - k0) < XK ? (p.K - k0) : XK;     // multiple of 256
                const bool v_here = v_preloaded && ic == i0 && mg == 0 && k0 == 0;
                if (!v_here) named_bar_sync(1, EPI_THREADS);           // previous pass fully consumed
                const int nchunk = kc >> 3;                            // 16-byte chunks per activation row
#pragma unroll 1
                for (int idx = tid; idx < RP * nchunk; idx += EPI_THREADS) {
                    const int mm = idx / nchunk, c = idx - mm * nchunk;
                    const int row = (mg + mm < p.M) ? (mg + mm) : (p.M - 1);
                    const int w = c >> 2, v = c & 3;
                    cp_async16(xt_s + mm * (XK * 2) + ((((w >> 5) * 4 + v) * 32) + (w & 31)) * 16,
                               p.X + (size_t)row * p.K + k0 + c * 8);
                }
                const int vch = kc >> 7;                               // 16-byte chunks of sign bits per rank
                if (!v_here) {
#pragma unroll 1
                    for (int idx = tid; idx < nr * vch; idx += EPI_THREADS) {
                        const int q = idx / vch, c = idx - q * vch;
                        cp_async16(vt_s + q * (XK / 8) + c * 16, p.Vp + (size_t)(ic + q) * kbytes + (k0 >> 3) + c * 16);
                    }
                }
                cp_async_commit();
                cp_async_wait_all();
                if (tid == 0 && p.stamps && v_here) p.stamps[(size_t)cta * STAMP_WORDS + 8] = globaltimer_ns();
                named_bar_sync(1, EPI_THREADS);
                const int nwords = kc >> 5;
#pragma unroll
                for (int slot = 0; slot < 2; ++slot) {
                    const int rq = warp + 4 * slot;
                    if (rq < nr) {                                     // warp-uniform
#pragma unroll 1
                        for (int mm = 0; mm < RP; ++mm) {
                            float a = 0.f;
#pragma unroll 1
                            for (int j = 0; j < JN; ++j) {
                                const int w = j * 32 + lane;
                                if (w < nwords) {
                                    const uint32_t vw = vt[rq * XW + w];
                                    const uint4* xs = reinterpret_cast<const uint4*>(work + mm * (XK * 2)) + (j * 4) * 32 + lane;
#pragma unroll
                                    for (int v = 0; v < 4; ++v) {
                                        const uint4 xx = xs[v * 32];
                                        const uint32_t xw[4] = {xx.x, xx.y, xx.z, xx.w};
#pragma unroll
                                        for (int e = 0; e < 4; ++e) {
                                            a += signed_by_bit(__uint_as_float(xw[e] << 16), vw, 8 * v + 2 * e);
                                            a += signed_by_bit(__uint_as_float(xw[e] & 0xFFFF0000u), vw, 8 * v + 2 * e + 1);
                                        }
                                    }
                                }
                            }
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                            if (lane == mm) { if (slot == 0) zacc0 += a; else zacc1 += a; }
                        }
                    }
                }
            }
            if (tid == 0 && p.stamps) p.stamps[(size_t)cta * STAMP_WORDS + 9] = globaltimer_ns();
            if (lane < RP) {
                if (warp < nr) zb[(size_t)(mg + lane) * p.Rpad + ic + warp] = zacc0 * __bfloat162float(p.S[ic + warp]);
                if (warp + 4 < nr) zb[(size_t)(mg + lane) * p.Rpad + ic + warp + 4] = zacc1 * __bfloat162float(p.S[ic + warp + 4]);
            }
        }
    }
}

// Sign words of the first z pass of this CTA (ranks i0.., k = 0..XK) into the work area; no activation involved.
template <int ROWS>
__device__ __forceinline__ void z_prefetch_v(const FusedParams& p, uint8_t* work, int cta, int tid) {
    constexpr int RP = ROWS < 8 ? ROWS : 8;
    constexpr int XK = XT_BYTES / 2 / RP;
    const int i0 = cta * p.R / p.G;
    const int i1 = (cta + 1) * p.R / p.G;
    const int nr = (i1 - i0) < VT_RANKS ? (i1 - i0) : VT_RANKS;
    const int kc = p.K < XK ? p.K : XK;
    const int vch = kc >> 7;
    const uint32_t vt_s = smem_u32(work) + XT_BYTES;
#pragma unroll 1
    for (int idx = tid; idx < nr * vch; idx += EPI_THREADS) {
        const int q = idx / vch, c = idx - q * vch;
        cp_async16(vt_s + q * (XK / 8) + c * 16, p.Vp + (size_t)(i0 + q) * (p.K >> 3) + c * 16);
    }
    cp_async_commit();
}

// corr[m] += sum over rank words [w0, w1) of z[m, 32w+b] * sign(U bit b of word w of this thread's column).
// z comes from the scratch buffer in global memory and is staged ZS_WORDS words at a time in shared memory (one
// batch of coalesced 128-bit loads per chunk); uw_first holds this thread's U words of the first chunk when they
// were fetched ahead of time (use_first).
template <int ROWS>
__device__ __forceinline__ void expand_z(float (&corr)[ROWS], const float* zb, int Rpad, const int32_t* ucol, int w0, int w1,
                                         float* zs, int tid, const uint32_t* uw_first, bool use_first) {
#pragma unroll 1
    for (int c0 = w0; c0 < w1; c0 += ZS_WORDS) {
        const int cw = (w1 - c0) < ZS_WORDS ? (w1 - c0) : ZS_WORDS;
        uint32_t uwv[ZS_WORDS];
        if (use_first && c0 == w0) {
#pragma unroll
            for (int w = 0; w < ZS_WORDS; ++w) uwv[w] = uw_first[w];
        } else {
#pragma unroll
            for (int w = 0; w < ZS_WORDS; ++w) uwv[w] = (uint32_t)ucol[(w < cw) ? (c0 + w) : c0];
        }
        named_bar_sync(1, EPI_THREADS);                      // zs free again
        const int per_row = 8 * cw;
#pragma unroll 1
        for (int idx = tid; idx < ROWS * per_row; idx += EPI_THREADS) {
            const int m = idx / per_row, j = idx - m * per_row;
            const float4 zz = __ldcg(reinterpret_cast<const float4*>(zb + (size_t)m * Rpad + 32 * c0) + j);
            *reinterpret_cast<float4*>(zs + m * ZS_STRIDE + 4 * j) = zz;
        }
        named_bar_sync(1, EPI_THREADS);
#pragma unroll 1
        for (int w = 0; w < cw; ++w) {
            const uint32_t uw = uwv[0];
#pragma unroll
            for (int q = 0; q + 1 < ZS_WORDS; ++q) uwv[q] = uwv[q + 1];
#pragma unroll 1
            for (int b = 0; b < 32; b += 4) {
                const uint32_t nib = uw >> b;
                const float s0 = (nib & 1u) ? 1.f : -1.f;
                const float s1 = (nib & 2u) ? 1.f : -1.f;
                const float s2 = (nib & 4u) ? 1.f : -1.f;
                const float s3 = (nib & 8u) ? 1.f : -1.f;
                const float* zrow = zs + 32 * w + b;
#pragma unroll
                for (int m = 0; m < ROWS; ++m) {
                    const float4 zz = *reinterpret_cast<const float4*>(zrow + m * ZS_STRIDE);
                    corr[m] += (s0 * zz.x + s1 * zz.y) + (s2 * zz.z + s3 * zz.w);
                }
            }
        }
    }
}

}  // namespace biloco
