// CUDA-core half of the fused linear: the z stage (z = S .* (X sign(V)^T) for this CTA's slice of the ranks) and the
// expansion of z through the packed U signs. Both are written for small machine code (rolled loops, the row count
// is a template parameter) and for one memory round trip per step: every global read is issued in a single batch.
#pragma once
#include "fused_cfg.cuh"

namespace biloco {

// z stage, run by Z_THREADS = 256 threads (the four epilogue warps and the four z warps).
//
// Work is cut into items (activation row m, rank slice s): nsl slices per row, item m*nsl + s belongs to CTA
// (m*nsl + s) % G, so with G >= M every CTA reads ONE activation row (K * 2 bytes, the only read of the stage that
// depends on the previous kernel of the stream) and the sign words of its R*M/G ranks. Ranks are processed in chunks
// of what the sign-word area holds (at most ZR_MAX), k in passes of XK.
// Everything that does not depend on the previous kernel happens before the dependency wait, which is inside this
// function: the work split, the coefficients, the sign words of the first chunk (cp.async, made visible with a
// barrier). After the wait one thread requests the activation row with a single bulk copy and all threads wait on its
// mbarrier; nothing else stands between the wait and the arithmetic.
// Arithmetic: the eight warps share (run of ranks) x (block of 32 sign words) tasks, one word per lane; a lane unpacks
// the activations of its word and, for every rank of the run, adds them under predicates taken from the sign bits. One
// shuffle reduction per run of up to six ranks (z_reduce_run), per-warp partial
// sums in shared memory, one combine per chunk: z = S * (2 * sum_{sign=+1} x - sum x).
// The CUDA-core code here is bound by instruction issue, not by latency (measured: the same cycles cold and warm,
// alone or beside spinning warps), so what matters is the instruction count per element and an even spread over warps.
// zt = index of the calling thread among the 256.
constexpr int Z_THREADS = 256;
constexpr int Z_WARPS = Z_THREADS / 32;

struct ZItem { int m, ra, rb; };
__device__ __forceinline__ ZItem z_item(const FusedParams& p, int it) {
    ZItem z;
    z.m = it / p.nsl;
    const int sl = it - z.m * p.nsl;
    z.ra = sl * p.R / p.nsl;
    z.rb = (sl + 1) * p.R / p.nsl;
    return z;
}
// ranks per chunk when a pass covers kc k
__device__ __forceinline__ int z_chunk_ranks(const FusedParams& p, int kc) {
    const int c = p.vt_bytes / (kc >> 3);
    return c < ZR_MAX ? c : ZR_MAX;
}

__device__ __forceinline__ void z_issue_v(const FusedParams& p, uint8_t* work, int r0, int nr, int k0, int kc, int zt) {
    const int vch = kc >> 7;                                 // 16-byte chunks of sign bits per rank
    const uint32_t vt_s = smem_u32(work) + XT_BYTES;
#pragma unroll 1
    for (int idx = zt; idx < nr * vch; idx += Z_THREADS) {
        const int q = idx / vch, c = idx - q * vch;
        cp_async16(vt_s + q * (kc >> 3) + c * 16, p.Vp + (size_t)(r0 + q) * (p.K >> 3) + (k0 >> 3) + c * 16);
    }
}

// One 32-bit sign word (32 consecutive k) of NQ ranks: sums[q] = sum of the word's activations whose sign bit in rank
// q's word is set; plain = sum of all 32. An add under a predicate taken from the sign bit (spelled out in PTX so that
// it cannot turn into a branch or a select), two accumulators per rank, eight activations per trip of a rolled loop.
// Measured in isolation (cycles per warp and element, two warps per scheduler): this form with 8 add chains 4.0; with
// 4 chains 5.2; sign flips by XOR 7.6; multiplications by +-1 9.7. The loops are kept rolled on purpose: the kernel's
// code runs once per CTA and launch, and instruction fetch was the largest stall after barriers in the profile
// (4.1 stalled warp-cycles per issued instruction with everything unrolled).
constexpr int ZRUN = 6;                          // ranks per run of the z stage's inner loop (4.27 ranks per CTA at M = 1, r = 512, 120 CTAs: one run)
#define BILOCO_PADD(accv, vwv, bit, xv)                                                                              \
    asm("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\tand.b32 t, %1, %2;\n\tsetp.ne.u32 p, t, 0;\n\t@p add.f32 %0, %0, %3;\n\t}" \
        : "+f"(accv) : "r"(vwv), "r"(bit), "f"(xv))
template <int NQ>
__device__ __forceinline__ void z_word_n(const uint4* xs, const uint32_t* vrow, int xw_stride, int nq, float (&sums)[ZRUN], float& plain) {
    uint32_t vw[NQ];
    float a0[NQ], a1[NQ];
#pragma unroll
    for (int q = 0; q < NQ; ++q) { vw[q] = q < nq ? vrow[q * xw_stride] : 0u; a0[q] = 0.f; a1[q] = 0.f; }
    float ps = 0.f;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
        const uint4 xx = xs[c];
        const uint32_t xw[4] = {xx.x, xx.y, xx.z, xx.w};
        float xf[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            xf[2 * e] = __uint_as_float(xw[e] << 16);
            xf[2 * e + 1] = __uint_as_float(xw[e] & 0xFFFF0000u);
        }
#pragma unroll
        for (int j = 0; j < 8; j += 2)
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                BILOCO_PADD(a0[q], vw[q], 1u << j, xf[j]);
                BILOCO_PADD(a1[q], vw[q], 2u << j, xf[j + 1]);
            }
#pragma unroll
        for (int q = 0; q < NQ; ++q) vw[q] >>= 8;
        ps += ((xf[0] + xf[1]) + (xf[2] + xf[3])) + ((xf[4] + xf[5]) + (xf[6] + xf[7]));
    }
#pragma unroll
    for (int q = 0; q < ZRUN; ++q) sums[q] = q < NQ ? a0[q < NQ ? q : 0] + a1[q < NQ ? q : 0] : 0.f;
    plain = ps;
}

// The same sums for a span of e consecutive activations starting at element e0 of the pass (e even, at most 32, e0 even):
// with few ranks per CTA a lane takes K/256 elements instead of a whole sign word, so that all 256 lanes of the stage
// have work (at K = 5120 a word per lane keeps 160 lanes busy with 32 elements each; a span per lane gives 256 lanes 20
// each; at K = 2560, 80 lanes with 32 against 256 with 10). The span's sign bits come from one or two words of the rank's
// row (funnel shift); the activations are read as 32-bit pairs.
template <int NQ>
__device__ __forceinline__ void z_span_n(const uint8_t* xrow, int e0, int e, const uint32_t* vq0, int words, int nq,
                                         float (&sums)[ZRUN], float& plain) {
    uint32_t vw[NQ];
    float a0[NQ], a1[NQ];
    const int wi = e0 >> 5, sh = e0 & 31;
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
        uint32_t lo = 0u, hi = 0u;
        if (q < nq) {
            lo = vq0[q * words + wi];
            if (sh + e > 32) hi = vq0[q * words + wi + 1];     // (then wi + 1 < words: the span lies inside the pass)
        }
        vw[q] = __funnelshift_r(lo, hi, sh);
        a0[q] = 0.f;
        a1[q] = 0.f;
    }
    const uint32_t* xp = reinterpret_cast<const uint32_t*>(xrow + 2 * e0);
    float ps = 0.f;
    uint32_t m = 1u;
#pragma unroll 1
    for (int j = 0; j < e; j += 2) {
        const uint32_t xw = xp[j >> 1];
        const float x0 = __uint_as_float(xw << 16), x1 = __uint_as_float(xw & 0xFFFF0000u);
        const uint32_t m2 = m << 1;
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            BILOCO_PADD(a0[q], vw[q], m, x0);
            BILOCO_PADD(a1[q], vw[q], m2, x1);
        }
        ps += x0 + x1;
        m <<= 2;
    }
#pragma unroll
    for (int q = 0; q < ZRUN; ++q) sums[q] = q < NQ ? a0[q < NQ ? q : 0] + a1[q < NQ ? q : 0] : 0.f;
    plain = ps;
}

// Sum of v[q] over the 32 lanes for up to eight ranks at once: a lane gives away half of its values at every step
// (4 + 2 + 1 + 2 shuffles instead of 8 x 5). On return lane l holds the total of rank ((l >> 4) & 1) * 4 +
// ((l >> 3) & 1) * 2 + ((l >> 2) & 1); ranks >= ZRUN are zero.
__device__ __forceinline__ float z_reduce_run(const float (&v)[ZRUN], int lane) {
    const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4;
    float w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = i < ZRUN ? v[i < ZRUN ? i : 0] : 0.f;
    float a[4], b[2], c;
#pragma unroll
    for (int i = 0; i < 4; ++i) {        // lanes with bit 4 set keep ranks 4-7, the others ranks 0-3
        const float give = h16 ? w[i] : w[i + 4], keep = h16 ? w[i + 4] : w[i];
        a[i] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float give = h8 ? a[i] : a[i + 2], keep = h8 ? a[i + 2] : a[i];
        b[i] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
    }
    {
        const float give = h4 ? b[0] : b[1], keep = h4 ? b[1] : b[0];
        c = keep + __shfl_xor_sync(0xffffffffu, give, 4);
    }
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    return c;
}

// Contains the dependency wait (griddepcontrol.wait). Returns the validity mark of this launch's z values: the parity
// of the scratch's launch count, which is read behind the activation request so that its latency is hidden.
// Not inlined: the epilogue warps and the z warps call it from two places and share one copy of the code.
__device__ __noinline__ uint32_t z_stage(const FusedParams& p, Ctrl* ctrl, uint8_t* work, float* zb, int cta, int zt, uint32_t* seq_out) {
    const int zw = zt >> 5, lane = zt & 31;
    const int nitems = p.M * p.nsl;
    const uint32_t* vt = reinterpret_cast<const uint32_t*>(work + XT_BYTES);
    const uint32_t x_bar = smem_u32(&ctrl->x_bar);
    const int kc0 = p.K < XK ? p.K : XK;
    const int cap = z_chunk_ranks(p, kc0);
    bool waited = false;
    uint32_t x_parity = 0, seq = 0;

#pragma unroll 1
    for (int item = cta; item < nitems; item += p.G) {
        const ZItem it = z_item(p, item);
#pragma unroll 1
        for (int c0 = it.ra; c0 < it.rb;) {
            const int nrc = (it.rb - c0) < cap ? (it.rb - c0) : cap;
            // this warp's partial sums start at zero; the coefficient this thread needs at the end is requested now
            for (int q = lane; q < nrc; q += 32) ctrl->zred[zw][q] = 0.f;
            if (lane == 0) ctrl->zall[zw] = 0.f;
            float s_coef = 0.f;
            if (zt < nrc) s_coef = __bfloat162float(p.S[c0 + zt]);
#pragma unroll 1
            for (int k0 = 0; k0 < p.K; k0 += XK) {
                const int kc = (p.K - k0) < XK ? (p.K - k0) : XK;       // multiple of 256
                const int words = kc >> 5;
                if (waited) named_bar_sync(3, Z_THREADS);               // the previous pass has been consumed
                z_issue_v(p, work, c0, nrc, k0, kc, zt);
                cp_async_commit_wait_all();
                named_bar_sync(3, Z_THREADS);                           // sign words (and cleared sums) visible to all
                if (!waited) {
                    griddep_wait();             // everything below reads what earlier kernels of the stream wrote
                    fence_proxy_async_global(); // (the bulk copy below reads through the async proxy)
                    waited = true;
                    if (p.trigger == 4 && zt == 0) griddep_launch_dependents();
                    if (zt == 0 && p.stamps) p.stamps[(size_t)cta * STAMP_WORDS + 11] = globaltimer_ns();
                }
                const bool load_x = !(p.K <= XK && c0 > it.ra);         // (a single-pass row stays in place)
                if (load_x && zt == 0) {
                    mbar_arrive_expect_tx(x_bar, (uint32_t)kc * 2u);
                    bulk_load(smem_u32(work), p.X + (size_t)it.m * p.K + k0, (uint32_t)kc * 2u, x_bar);
                }
                if (zt == 0 && p.stamps && item == cta && c0 == it.ra && k0 == 0) p.stamps[(size_t)cta * STAMP_WORDS + 14] = globaltimer_ns();
                if (item == cta && c0 == it.ra && k0 == 0) seq = ld_volatile_u32(p.z_counter);
                if (load_x) {
                    wait_bar(x_bar, x_parity, ctrl, p.status, p.epoch, ST_Z, 0);       // (on failure: status set, carry on)
                    x_parity ^= 1u;
                }
                if (zt == 0 && p.stamps && item == cta && c0 == it.ra && k0 == 0) p.stamps[(size_t)cta * STAMP_WORDS + 8] = globaltimer_ns();
                if (p.trigger == 3 && zt == 0) griddep_launch_dependents();

                if (zt == 224 && p.stamps && item == cta && c0 == it.ra && k0 == 0) p.stamps[(size_t)cta * STAMP_WORDS + 2] = globaltimer_ns();
                // warp tasks = (run of up to ZRUN ranks) x (block of sign words), dealt round-robin to the eight warps: every
                // task has all its lanes busy (up to the last, partial block) whatever the number of ranks
                // (with one or two runs the words are dealt evenly to all eight warps instead: measured faster than full blocks)
                const int nruns = (nrc + ZRUN - 1) / ZRUN;
                const int e_lane = kc >> 8;                                            // elements per lane when all 256 lanes share the pass
                if (nruns <= 2 && (e_lane & 1) == 0) {
                    // few ranks: every lane takes a span of the pass (see z_span_n), all ranks of a run at once
                    const int e0 = zw * (kc >> 3) + lane * e_lane;
#pragma unroll 1
                    for (int run = 0; run < nruns; ++run) {
                        const int q0 = run * ZRUN, nq = nrc - q0;
                        float sums[ZRUN];
                        float plain = 0.f;
                        const uint32_t* vq0 = vt + (size_t)q0 * words;
                        if (nq <= 2) z_span_n<2>(work, e0, e_lane, vq0, words, nq, sums, plain);
                        else if (nq <= 4) z_span_n<4>(work, e0, e_lane, vq0, words, nq, sums, plain);
                        else if (nq == 5) z_span_n<5>(work, e0, e_lane, vq0, words, nq, sums, plain);
                        else z_span_n<6>(work, e0, e_lane, vq0, words, nq, sums, plain);
                        const float tot = z_reduce_run(sums, lane);
                        const int rl = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
                        if ((lane & 3) == 0 && rl < ZRUN && q0 + rl < nrc) ctrl->zred[zw][q0 + rl] += tot;
                        if (run == 0) {
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) plain += __shfl_xor_sync(0xffffffffu, plain, o);
                            if (lane == 0) ctrl->zall[zw] += plain;
                        }
                    }
                } else {
                    const int bs = nruns <= 2 ? (words + Z_WARPS - 1) / Z_WARPS : 32;      // sign words per block (at most 32)
                    const int nwb = (words + bs - 1) / bs;
#pragma unroll 1
                    for (int task = zw; task < nruns * nwb; task += Z_WARPS) {
                        const int run = task / nwb, wb = task - run * nwb;
                        const int q0 = run * ZRUN, nq = nrc - q0;
                        const int w = wb * bs + lane;
                        const bool active = lane < bs && w < words;
                        const uint4* xs = reinterpret_cast<const uint4*>(work) + (active ? w : 0) * 4;     // 64 bytes = 32 bf16 of word w
                        float sums[ZRUN];
#pragma unroll
                        for (int q = 0; q < ZRUN; ++q) sums[q] = 0.f;
                        float plain = 0.f;
                        if (active) {
                            const uint32_t* vrow = vt + (size_t)q0 * words + w;
                            if (nq <= 2) z_word_n<2>(xs, vrow, words, nq, sums, plain);
                            else if (nq <= 4) z_word_n<4>(xs, vrow, words, nq, sums, plain);
                            else if (nq == 5) z_word_n<5>(xs, vrow, words, nq, sums, plain);
                            else z_word_n<6>(xs, vrow, words, nq, sums, plain);
                        }
                        const float tot = z_reduce_run(sums, lane);
                        const int rl = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
                        if ((lane & 3) == 0 && rl < ZRUN && q0 + rl < nrc) ctrl->zred[zw][q0 + rl] += tot;
                        if (run == 0) {
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) plain += __shfl_xor_sync(0xffffffffu, plain, o);
                            if (lane == 0) ctrl->zall[zw] += plain;
                        }
                    }
                }
                if (zt == 0 && p.stamps && item == cta && c0 == it.ra && k0 == 0) p.stamps[(size_t)cta * STAMP_WORDS + 12] = globaltimer_ns();
            }
            named_bar_sync(3, Z_THREADS);
            if (zt < nrc) {
                float v = 0.f, a = 0.f;
#pragma unroll
                for (int g = 0; g < Z_WARPS; ++g) { v += ctrl->zred[g][zt]; a += ctrl->zall[g]; }
                // the lowest mantissa bit is the validity mark the consumers poll on (see expand_z)
                zb[(size_t)it.m * p.Rpad + c0 + zt] = __uint_as_float((__float_as_uint((2.f * v - a) * s_coef) & ~1u) | ((seq & 1u) ^ 1u));
            }
            if (zt == 0 && p.stamps) p.stamps[(size_t)cta * STAMP_WORDS + 9] = globaltimer_ns();
            named_bar_sync(3, Z_THREADS);              // the partial sums may be cleared for the next chunk
            c0 += nrc;
        }
    }
    if (!waited) {                                     // a CTA without a z item
        griddep_wait();
        if (zt == 0 && p.stamps) p.stamps[(size_t)cta * STAMP_WORDS + 11] = globaltimer_ns();
        seq = ld_volatile_u32(p.z_counter);
    }
    *seq_out = seq;
    return (seq & 1u) ^ 1u;
}

// corr[m] += sum over rank words [w0, w1) of z[m, 32w+b] * sign(U bit b of word w of this thread's column).
//
// z comes from the scratch buffer in global memory, where the z stages of all CTAs of this launch publish it, and
// there is no separate "z is complete" flag: every value is its own flag. The lowest mantissa bit of a published
// value equals `phase`, and phase flips with every launch that completes on the scratch (launch counter in the
// scratch head, bumped by the last CTA to leave), so a value left by the previous launch reads as "not yet there".
// The consumers load the values they need straight away, 128 bits at a time, and reload until all four marks match:
// one memory round trip after the last producer's store instead of three (counter, then poll, then data). The mark
// costs one unit in the last place of an fp32 z value. Ranks >= R (padding of the last rank word) are never written
// and read as zero (zb points at the first rank of the tile's column group, which has p.Rg ranks); rows >= M of the
// staging area are left as they are (their sums are never stored). Values are staged zs_words(ROWS) rank words at a
// time in shared memory.
// uw_first holds this thread's first ZS_FIRST U words when they were fetched ahead of time (use_first).
// Returns false when the poll ran out of time (status set, abort raised).
template <int ROWS>
__device__ __forceinline__ bool expand_z(float (&corr)[ROWS], const FusedParams& p, Ctrl* ctrl, const float* zb, const int32_t* ucol,
                                         int w0, int w1, float* zs, int tid, const uint32_t* uw_first, bool use_first, uint32_t phase) {
    constexpr int ZW = zs_words(ROWS);
    constexpr int ZSTR = zs_stride(ROWS);
    constexpr int NPT = (ROWS * ZW * 8 + EPI_THREADS - 1) / EPI_THREADS;     // 128-bit loads per thread per chunk
    bool good = true;
#pragma unroll 1
    for (int c0 = w0; c0 < w1 && good; c0 += ZW) {
        const int cw = (w1 - c0) < ZW ? (w1 - c0) : ZW;
        uint32_t uwv[ZW];
#pragma unroll
        for (int w = 0; w < ZW; ++w) {
            if (w < ZS_FIRST && use_first && c0 == w0) uwv[w] = uw_first[w];
            else uwv[w] = (uint32_t)ucol[(w < cw) ? (c0 + w) : c0];
        }
        const int per_row = 8 * cw;
        const int total = ROWS * per_row;
        int goff[NPT], soff[NPT];
#pragma unroll
        for (int q = 0; q < NPT; ++q) {
            const int idx = tid + q * EPI_THREADS;
            const int m = idx / per_row, j = idx - m * per_row;
            goff[q] = (idx < total && m < p.M) ? (m * p.Rpad + 32 * c0 + 4 * j) : -1;     // rows >= M: nothing to wait for
            soff[q] = m * ZSTR + 4 * j;
        }
        uint4 v[NPT];
        uint64_t t0 = 0;
#pragma unroll 1
        for (uint32_t it = 0;; ++it) {
#pragma unroll
            for (int q = 0; q < NPT; ++q)
                if (goff[q] >= 0) v[q] = ld_volatile_v4(zb + goff[q]);
            uint32_t bad = 0;
#pragma unroll
            for (int q = 0; q < NPT; ++q) {
                if (goff[q] >= 0) {
                    const int e = 32 * c0 + (soff[q] % ZSTR);           // rank of v[q].x
                    bad |= (e + 0 < p.Rg ? (v[q].x ^ phase) : 0u) | (e + 1 < p.Rg ? (v[q].y ^ phase) : 0u) |
                           (e + 2 < p.Rg ? (v[q].z ^ phase) : 0u) | (e + 3 < p.Rg ? (v[q].w ^ phase) : 0u);
                }
            }
            if (!(bad & 1u)) break;
            if ((it & 15u) == 15u) {
                if (ctrl->abort) { good = false; break; }
                const uint64_t now = globaltimer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > WAIT_BUDGET_NS) { fail(ctrl, p.status, p.epoch, ST_Z, 0); good = false; break; }
            }
        }
        if (tid == 0 && p.stamps && c0 == w0) p.stamps[(size_t)blockIdx.x * STAMP_WORDS + 15] = globaltimer_ns();
        named_bar_sync(1, EPI_THREADS);                      // zs free again (the previous chunk has been consumed)
#pragma unroll
        for (int q = 0; q < NPT; ++q) {
            if (goff[q] >= 0) {
                const int e = 32 * c0 + (soff[q] % ZSTR);
                float4 zz;
                // (the mark is cleared, so that the result does not depend on the launch count's parity)
                zz.x = e + 0 < p.Rg ? __uint_as_float(v[q].x & ~1u) : 0.f;
                zz.y = e + 1 < p.Rg ? __uint_as_float(v[q].y & ~1u) : 0.f;
                zz.z = e + 2 < p.Rg ? __uint_as_float(v[q].z & ~1u) : 0.f;
                zz.w = e + 3 < p.Rg ? __uint_as_float(v[q].w & ~1u) : 0.f;
                *reinterpret_cast<float4*>(zs + soff[q]) = zz;
            }
        }
        named_bar_sync(1, EPI_THREADS);
        if (ctrl->abort) { good = false; break; }           // uniform: written before the barrier, read after it
        // Signs as +-1.0 multipliers shared by the rows. (Adds under a predicate with a separate plain row sum, the
        // form the z stage uses, measured slower here from 4 rows up and no faster below.)
        // UNR groups of four ranks are in flight at a time: with one warp per scheduler nothing else hides the
        // shared-memory latency of the z values
        constexpr int UNR = ROWS >= 8 ? 1 : 8 / ROWS;
#pragma unroll 1
        for (int w = 0; w < cw; ++w) {
            const uint32_t uw = uwv[0];
#pragma unroll
            for (int q = 0; q + 1 < ZW; ++q) uwv[q] = uwv[q + 1];
#pragma unroll 1
            for (int b0 = 0; b0 < 32; b0 += 4 * UNR) {
                const float* zrow = zs + 32 * w + b0;
                float4 zz[UNR][ROWS];
#pragma unroll
                for (int u = 0; u < UNR; ++u)
#pragma unroll
                    for (int m = 0; m < ROWS; ++m) zz[u][m] = *reinterpret_cast<const float4*>(zrow + 4 * u + m * ZSTR);
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const uint32_t nib = uw >> (b0 + 4 * u);
                    const float s0 = (nib & 1u) ? 1.f : -1.f;
                    const float s1 = (nib & 2u) ? 1.f : -1.f;
                    const float s2 = (nib & 4u) ? 1.f : -1.f;
                    const float s3 = (nib & 8u) ? 1.f : -1.f;
#pragma unroll
                    for (int m = 0; m < ROWS; ++m)
                        corr[m] += (s0 * zz[u][m].x + s1 * zz[u][m].y) + (s2 * zz[u][m].z + s3 * zz[u][m].w);
                }
            }
        }
    }
    return good;
}

// ---------------------------------------------------------------------------------------------------------
// Expansion on the tensor cores (from LR_TC_MIN_ROWS activation rows): corr[n, m] = sum_i sign(U[i, n]) z[m, i] is a small GEMM with the tile's
// 128 columns as MMA M, the activation rows as MMA N and the ranks as K. Per chunk of 64 ranks the epilogue threads
//   * write the +-1.0 bf16 image of the chunk's U signs (thread = column; 8 table look-ups and 8 16-byte stores),
//   * poll the chunk's z values (validity mark as in expand_z) and write them as TWO bf16 operands, high part and
//     rounding remainder (z = hi + lo to 2^-17 relative), so that the products are exact and the sum is an fp32 sum,
//   * and one thread issues 4 x 2 tcgen05.mma.kind::f16 (K = 16 each) into a TMEM accumulator of its own.
// The sign image does not depend on z: it is written while z is still on its way. CUDA-core cost per column and 64
// ranks: about 60 issue slots whatever the number of rows, against 64 * rows multiply-adds.
// Operand buffers are double-buffered across chunks and segments (gchunk counts chunks since kernel start).
template <int ROWS, int MMA_N>
__device__ __forceinline__ bool expand_z_tc(const FusedParams& p, Ctrl* ctrl, uint8_t* lr, const float* zb, const int32_t* ucol, int w0, int w1,
                                            int tid, uint32_t phase, uint32_t d_tmem, int& gchunk) {
    constexpr int ZB = MMA_N * 128;                                   // bytes of one z operand (MMA_N rows x 64 bf16)
    constexpr int NPIECE = (MMA_N * 8 + EPI_THREADS - 1) / EPI_THREADS;  // 16-byte pieces (8 ranks of one row) per thread
    constexpr uint32_t idesc = make_idesc_bf16(TILE_N, MMA_N);
    const uint4* lut = reinterpret_cast<const uint4*>(lr + 2 * LR_UA_BYTES + 4 * ZB);
    const int nch = (w1 - w0 + 1) >> 1;
    bool good = true;
#pragma unroll 1
    for (int ci = 0; ci < nch; ++ci, ++gchunk) {
        const int c0 = w0 + 2 * ci;
        const int buf = gchunk & 1;
        const uint32_t uw0 = (uint32_t)ucol[c0];
        const uint32_t uw1 = (c0 + 1 < w1) ? (uint32_t)ucol[c0 + 1] : 0u;          // (a missing word meets z = 0)
        if (gchunk >= 2 && !wait_bar(smem_u32(&ctrl->lr_free[buf]), ((gchunk >> 1) - 1) & 1, ctrl, p.status, p.epoch, ST_ACC_EMPTY, 0))
            good = false;
        // sign image of this thread's column: 64 ranks = 128 bytes, 16-byte chunk c of row r at chunk c ^ (r & 7)
        {
            uint8_t* row = lr + buf * LR_UA_BYTES + (tid >> 3) * 1024 + (tid & 7) * 128;
#pragma unroll
            for (int pc = 0; pc < 8; ++pc) {
                const uint32_t byte = ((pc < 4 ? uw0 : uw1) >> (8 * (pc & 3))) & 0xFFu;
                *reinterpret_cast<uint4*>(row + ((pc ^ (tid & 7)) * 16)) = lut[byte];
            }
        }
        // z pieces: (row m, ranks 8 pc .. 8 pc + 7 of the chunk), polled until every needed value carries this launch's mark
        uint8_t* zh = lr + 2 * LR_UA_BYTES + buf * 2 * ZB;
#pragma unroll
        for (int q = 0; q < NPIECE; ++q) {
            const int idx = tid + q * EPI_THREADS;
            if (idx < MMA_N * 8) {
                const int m = idx >> 3, pc = idx & 7;
                const int e0 = 32 * c0 + 8 * pc;                              // first rank of the piece
                uint4 hi = make_uint4(0u, 0u, 0u, 0u), lo = hi;
                if (m < p.M && c0 + (pc >> 2) < w1 && e0 < p.Rg) {
                    const float* src = zb + (size_t)m * p.Rpad + e0;
                    uint4 a, b;
                    uint64_t t0 = 0;
#pragma unroll 1
                    for (uint32_t it = 0;; ++it) {
                        a = ld_volatile_v4(src);
                        b = ld_volatile_v4(src + 4);
                        uint32_t bad = 0;
                        const uint32_t v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                        for (int i = 0; i < 8; ++i) bad |= (e0 + i < p.Rg) ? (v[i] ^ phase) : 0u;
                        if (!(bad & 1u)) break;
                        if ((it & 15u) == 15u) {
                            if (ctrl->abort) { good = false; break; }
                            const uint64_t now = globaltimer_ns();
                            if (t0 == 0) t0 = now;
                            else if (now - t0 > WAIT_BUDGET_NS) { fail(ctrl, p.status, p.epoch, ST_Z, 0); good = false; break; }
                        }
                    }
                    const uint32_t v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                    uint32_t h[4], l[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float z0 = (e0 + 2 * i < p.Rg) ? __uint_as_float(v[2 * i] & ~1u) : 0.f;
                        float z1 = (e0 + 2 * i + 1 < p.Rg) ? __uint_as_float(v[2 * i + 1] & ~1u) : 0.f;
                        const __nv_bfloat16 h0 = __float2bfloat16_rn(z0), h1 = __float2bfloat16_rn(z1);
                        const __nv_bfloat16 l0 = __float2bfloat16_rn(z0 - __bfloat162float(h0));
                        const __nv_bfloat16 l1 = __float2bfloat16_rn(z1 - __bfloat162float(h1));
                        h[i] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
                        l[i] = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
                    }
                    hi = make_uint4(h[0], h[1], h[2], h[3]);
                    lo = make_uint4(l[0], l[1], l[2], l[3]);
                }
                const int off = (m >> 3) * 1024 + (m & 7) * 128 + ((pc ^ (m & 7)) * 16);
                *reinterpret_cast<uint4*>(zh + off) = hi;
                *reinterpret_cast<uint4*>(zh + ZB + off) = lo;
            }
        }
        fence_proxy_async();                                 // the operands were written with ordinary stores
        named_bar_sync(1, EPI_THREADS);
        if (ctrl->abort) { good = false; }
        if (tid == 0) {
            tc_fence_after_sync();
            const uint64_t ad = make_smem_desc(smem_u32(lr + buf * LR_UA_BYTES), 1024, 2);
            const uint64_t hd = make_smem_desc(smem_u32(zh), 1024, 2);
            const uint64_t ld = make_smem_desc(smem_u32(zh + ZB), 1024, 2);
#pragma unroll
            for (int k = 0; k < 4; ++k) {                    // 16 ranks = 32 bytes along the swizzled row: +2 in the address field
                tc_mma_bf16(d_tmem, ad + 2 * k, hd + 2 * k, idesc, (ci > 0 || k > 0) ? 1u : 0u);
                tc_mma_bf16(d_tmem, ad + 2 * k, ld + 2 * k, idesc, 1u);
            }
            tc_commit(smem_u32(&ctrl->lr_free[buf]));
            if (ci == nch - 1) tc_commit(smem_u32(&ctrl->lr_done));
        }
        if (!good) { ++gchunk; break; }
    }
    return good;
}

}  // namespace biloco
