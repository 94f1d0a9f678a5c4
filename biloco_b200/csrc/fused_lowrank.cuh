// CUDA-core half of the fused linear: the z stage (z = S .* (X sign(V)^T) for this CTA's slice of the ranks) and the
// expansion of z through the packed U signs. Both are written for small machine code (rolled loops, the row count
// is a template parameter) and for one memory round trip per step: every global read is issued in a single batch.
#pragma once
#include "fused_cfg.cuh"

namespace biloco {

// z stage, run by Z_THREADS = 256 threads (the four epilogue warps and the four scale-factor warps, which have nothing
// to move until the first weights land). CTA `cta` owns ranks [cta*R/G, (cta+1)*R/G), at most VT_RANKS at a time.
// Per pass a tile of the activation (RP rows x XK k, 16-byte chunks transposed so that a warp reads consecutive
// chunks) and the sign words of the CTA's ranks are copied to shared memory with one batch of cp.async. The eight
// warps are arranged as RP rows x KW k-groups; a lane owns 32-bit sign words (32 consecutive k) of its k-group, unpacks
// the 32 activations once and adds them into one accumulator per rank under a predicate taken from the sign bit.
// Accumulators live in registers across all passes; one shuffle reduction and one shared-memory exchange at the end.
// zt = index of the calling thread among the 256.
// The sign words of the first pass are weights, not activations: z_prefetch_v copies them before the caller waits for
// the previous kernel of the stream.
constexpr int Z_THREADS = 256;

template <int RP>
__device__ __forceinline__ void z_issue_v(const FusedParams& p, uint8_t* work, int ic, int nr, int k0, int kc, int zt) {
    constexpr int XK = XT_BYTES / 2 / RP;
    const int vch = kc >> 7;                                 // 16-byte chunks of sign bits per rank
    const uint32_t vt_s = smem_u32(work) + XT_BYTES;
#pragma unroll 1
    for (int idx = zt; idx < nr * vch; idx += Z_THREADS) {
        const int q = idx / vch, c = idx - q * vch;
        cp_async16(vt_s + q * (XK / 8) + c * 16, p.Vp + (size_t)(ic + q) * (p.K >> 3) + (k0 >> 3) + c * 16);
    }
}

template <int ROWS>
__device__ __forceinline__ void z_prefetch_v(const FusedParams& p, uint8_t* work, int cta, int zt) {
    constexpr int RP = ROWS < 8 ? ROWS : 8;
    constexpr int XK = XT_BYTES / 2 / RP;
    const int i0 = cta * p.R / p.G;
    const int i1 = (cta + 1) * p.R / p.G;
    const int nr = (i1 - i0) < VT_RANKS ? (i1 - i0) : VT_RANKS;
    z_issue_v<RP>(p, work, i0, nr, 0, p.K < XK ? p.K : XK, zt);
    cp_async_commit();
}

// Adds the 32 activations xf[] into acc[q] for the ranks whose sign bit is set, and keeps their plain sum in `all`
// (sum_k s_k x_k = 2 * sum_{s_k = +1} x_k - sum_k x_k).
template <int NQ>
__device__ __forceinline__ void z_word(const float (&xf)[32], const uint32_t* vrow, int xw_stride, int nq, float (&acc)[NQ]) {
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
        if (q < nq) {                                   // warp-uniform
            const uint32_t vw = vrow[q * xw_stride];
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (vw & (1u << j)) acc[q] += xf[j];
        }
    }
}

template <int ROWS>
__device__ __forceinline__ void z_stage(const FusedParams& p, Ctrl* ctrl, uint8_t* work, float* zb, int cta, int zt, bool v_preloaded) {
    constexpr int RP = ROWS < 8 ? ROWS : 8;          // rows per pass
    constexpr int KW = 8 / RP;                       // k-groups (warps per row)
    constexpr int XK = XT_BYTES / 2 / RP;            // k per pass
    constexpr int XW = XK / 32;                      // sign words per rank per pass
    const int zw = zt >> 5, lane = zt & 31;
    const int row = zw % RP, kg = zw / RP;
    const int i0 = cta * p.R / p.G;
    const int i1 = (cta + 1) * p.R / p.G;
    const uint32_t xt_s = smem_u32(work);
    const uint32_t* vt = reinterpret_cast<const uint32_t*>(work + XT_BYTES);

#pragma unroll 1
    for (int ic = i0; ic < i1; ic += VT_RANKS) {
        const int nr = (i1 - ic) < VT_RANKS ? (i1 - ic) : VT_RANKS;
        // the coefficient this thread will need when it writes z: requested now, used after the reduction
        float s_coef = 0.f;
        if (zt < RP * VT_RANKS && (zt % VT_RANKS) < nr) s_coef = __bfloat162float(p.S[ic + (zt % VT_RANKS)]);
#pragma unroll 1
        for (int mg = 0; mg < p.M; mg += RP) {       // rows beyond M inside a group repeat row M-1
            float acc[VT_RANKS];
#pragma unroll
            for (int q = 0; q < VT_RANKS; ++q) acc[q] = 0.f;
            float all = 0.f;
#pragma unroll 1
            for (int k0 = 0; k0 < p.K; k0 += XK) {
                const int kc = (p.K - k0) < XK ? (p.K - k0) : XK;     // multiple of 256
                const bool v_here = v_preloaded && ic == i0 && mg == 0 && k0 == 0;
                if (!v_here) named_bar_sync(3, Z_THREADS);             // previous pass fully consumed
                const int nchunk = kc >> 3;                            // 16-byte chunks per activation row
#pragma unroll 1
                for (int idx = zt; idx < RP * nchunk; idx += Z_THREADS) {
                    int mm = 0, c = idx;
                    if (RP > 1) { mm = idx / nchunk; c = idx - mm * nchunk; }
                    const int r = (mg + mm < p.M) ? (mg + mm) : (p.M - 1);
                    const int w = c >> 2, v = c & 3;
                    cp_async16(xt_s + mm * (XK * 2) + ((((w >> 5) * 4 + v) * 32) + (w & 31)) * 16,
                               p.X + (size_t)r * p.K + k0 + c * 8);
                }
                if (!v_here) z_issue_v<RP>(p, work, ic, nr, k0, kc, zt);
                cp_async_commit();
                const int nwords = kc >> 5;
                // The accumulation loop runs twice over the same instructions. The first time, while the copies are
                // still in flight, it processes one word of whatever the work area holds and its result is thrown
                // away: its purpose is to pull the loop's machine code into the instruction cache (each CTA executes
                // this code once per launch, cold, and a cold instruction costs several times a warm one). The second
                // time is the real pass.
#pragma unroll 1
                for (int pass = (k0 == 0 ? 0 : 1); pass < 2; ++pass) {
                const bool dry = pass == 0;
                if (!dry) {
                    cp_async_wait_all();
                    if (zt == 0 && p.stamps && v_here) p.stamps[(size_t)cta * STAMP_WORDS + 8] = globaltimer_ns();
                    named_bar_sync(3, Z_THREADS);
                }
                const int w_end = dry ? min(nwords, kg * 32 + lane + 1) : nwords;
#pragma unroll 1
                for (int w = kg * 32 + lane; w < w_end; w += KW * 32) {
                    const uint4* xs = reinterpret_cast<const uint4*>(work + row * (XK * 2)) + ((w >> 5) * 4) * 32 + (w & 31);
                    float xf[32];
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const uint4 xx = xs[v * 32];
                        const uint32_t xw[4] = {xx.x, xx.y, xx.z, xx.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            xf[8 * v + 2 * e] = __uint_as_float(xw[e] << 16);
                            xf[8 * v + 2 * e + 1] = __uint_as_float(xw[e] & 0xFFFF0000u);
                        }
                    }
                    float s = 0.f;
#pragma unroll
                    for (int j = 0; j < 32; ++j) s += xf[j];
                    all += s;
                    z_word<VT_RANKS>(xf, vt + w, XW, nr, acc);
                }
                if (dry) {
                    all = 0.f;
#pragma unroll
                    for (int q = 0; q < VT_RANKS; ++q) acc[q] = 0.f;
                }
                }
            }
            // z[row, rank] = S * (2 * sum_plus - sum_all), summed over the lanes and the k-groups
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) all += __shfl_xor_sync(0xffffffffu, all, o);
#pragma unroll
            for (int q = 0; q < VT_RANKS; ++q) {
                float v = acc[q];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) ctrl->zred[zw][q] = 2.f * v - all;
            }
            named_bar_sync(3, Z_THREADS);
            if (zt < RP * VT_RANKS) {
                const int r = zt / VT_RANKS, q = zt - r * VT_RANKS;
                if (q < nr) {
                    float v = 0.f;
#pragma unroll
                    for (int g = 0; g < KW; ++g) v += ctrl->zred[g * RP + r][q];
                    zb[(size_t)(mg + r) * p.Rpad + ic + q] = v * s_coef;
                }
            }
            if (zt == 0 && p.stamps) p.stamps[(size_t)cta * STAMP_WORDS + 9] = globaltimer_ns();
        }
    }
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
