// Row-slab schedule of the fused linear for one to four activation rows (mode 7).
//
// The other schedules cut the weight into 128-row x 256-k units and share a tile's k-range between CTAs, which costs a
// partial-sum exchange per launch. At one or two rows a launch is a dependency chain, not a stream (the weights are
// in shared memory before the activation exists), so this schedule removes every hand-off it can:
//
//  * N is split only: CTA c owns the Rt = ceil8(N / SMs) weight rows [c Rt, (c+1) Rt) for all of K. No partial sums
//    leave a CTA.
//  * A tcgen05.mma with 128 rows takes the same time (about 220 cycles, measured) whatever its N is, so the weights are
//    the N operand (up to 256 rows per instruction) and the activation is the 128-row operand. The N rows of one MMA
//    hold the SAME Rt weight rows for kg CONSECUTIVE k-tiles ("super-unit"), and the activation operand has one row per
//    (k-tile of the group, activation row): D[g' M + m, g Rt + r] is the product of activation row m over k-tile g' with
//    weight row r over k-tile g. Only the diagonal blocks g = g' are meaningful; they are summed over g in the
//    epilogue. A CTA issues 4 ceil(K / 256 / kg) MMAs in all (16 at K = N = 5120 against 80 with 128-row weight tiles).
//  * A super-unit is ONE contiguous record in global memory (biloco_b200_tile_weights_slab): the codes of its kg units
//    with the 128-byte swizzle applied (operand row g Rt + r), followed by their block scales (16 bytes per row and unit).
//    A ring of stages holds as many super-units as fit beside a second CTA on the SM; with programmatic dependent
//    launch the ring is filled while the previous kernel of the stream is still running, and the weights' scale
//    factors are moved to TMEM as soon as that kernel's CTA on this SM has returned its TMEM (a CTA takes all 512
//    columns: 256 for the accumulator, 4 sets of 64 for scale factors; the allocation waits for the predecessor).
//  * z = S .* (X sign(V)^T) is rank-sliced over the CTAs as in the other schedules (item (row m, slice s) -> CTA),
//    computed by the 256 low-rank threads from a copy of the row that every warp stages for itself with coalesced
//    16-byte loads, published in global memory with a validity mark in the lowest mantissa bit, polled by everybody.
//    The launch count whose parity is the mark lives in eight counter words to which every CTA adds its share of 2^20
//    when it leaves (fire and forget): bits 20.. of their sum change only when the last CTA has left.
//  * Whatever every CTA reads after the dependency wait is read by as few threads as possible, as whole lines, starting
//    at a line that depends on the CTA: hundreds of requests for one 128-byte line are served one after another by its
//    L2 slice (measured: 1.5 - 6 us for an activation row read in 4-byte pieces by every thread of every CTA).
//  * Expansion: work items (rank word, column) over the 256 low-rank threads, partial sums in fixed shared-memory slots,
//    fixed-order final sum: results are bit-identical from launch to launch.
//
// Warp roles (448 threads): 0-3 low-rank side, read-out and store; 4-7 GEMM side: scale factors -> TMEM, activation codes
// -> shared memory, first weight copies; 8-11 low-rank side; 12 TMEM allocation + MMA issue; 13 later weight copies.
// The row-slab kernel for activations that arrive QUANTISED (A_codes / A_sf / alpha / X), i.e. biloco_b200_fused_linear with
// BILOCO_MODE_SLAB: the headline kernel. slab_kernel.cuh holds the same schedule extended by the raw-activation prologue
// (biloco_b200_fused_linear_act) and a four-warp accumulator read-out. They are two files on purpose: every instruction of
// this kernel runs once per launch and its speed depends on how the code is laid out (instruction fetch is among its largest
// stalls); compiled from the combined source -- the prologue behind a template parameter that removes it here -- this form
// ran at 8.9 us per call where this file gives 8.4 on the same GPU (M = 1, K = N = 5120, r = 512, HBM-cold).
#pragma once
#include "fused_cfg.cuh"

namespace biloco {
namespace slabp {

constexpr int NT = 448;
constexpr int LR_THREADS = 256;
constexpr int LR_WARPS = 8;
constexpr int NSETS = 4;                 // scale-factor column sets in TMEM (64 columns each)
constexpr int SET_COL0 = 256;            // set s at 256 + 64 s: the weights' scales in columns 0..31 (eight per MMA: rows
                                         // n % 32 in the lanes, n / 32 along the columns), the activations' in 32..47
constexpr int SFA_OFF = 32;
constexpr int SLAB_TMEM_COLS = 512;      // the accumulator D[128, N <= 256] takes columns 0..255
constexpr int KG_MAX = 8;                // k-tiles per super-unit at most (activation-operand rows kg * ROWS <= 32: one TMEM lane quadrant)
constexpr int MAX_RING = 12;
constexpr int NRMAX = 8;                 // ranks per pass of the z stage
constexpr int XW_MAX = 16;               // 32-bit activation words (pairs of bf16) a thread holds per 32-element segment
constexpr int UNIT_ROW_BYTES = 144;      // 128 bytes of codes + 16 bytes of block scales per weight row and k-tile
constexpr int VT_SLAB_MAX = 16384;       // shared memory for the sign words of a CTA's ranks
constexpr int SLAB_STAMPS = 32;              // debug: 16 %globaltimer stamps per CTA followed by the same 16 as clock64

struct SlabParams {
    const uint8_t* W_slab;
    const uint8_t* A_codes;   // u8 [A_rows, K/2]
    const uint8_t* A_sf;      // 128x4 atoms
    const float* alpha;
    const __nv_bfloat16* X;
    const uint8_t* Vp;
    const int32_t* Ucol;
    const __nv_bfloat16* S;
    const __nv_bfloat16* C;
    void* Y;
    int32_t* status;
    uint32_t* z_counter;      // words [8..15]: the CTAs that leave add their shares of 2^20 here (CTA c to word 8 + c % 8):
                              // the sum's bits 20.. count the launches completed on this scratch
    float* zbuf;
    int M, N, K, R, Rw, Rpad;
    int Rt, kg, nkt, nsu, G;  // G: CTAs launched
    int Grows;                // CTAs that own weight rows (the others only compute a z slice)
    int nsl;                  // z stage: rank slices per activation row
    int ring;                 // stages in shared memory
    int stage_bytes;          // 1024-aligned
    int nbp;                  // MMA N: kg * Rt rounded up to a multiple of 16
    int atile_bytes;          // bytes of one activation tile (1024 per 8 operand rows)
    int off_ring, off_ctrl, off_us, off_work, off_accp;       // shared-memory offsets from the 1024-aligned base (the
                              // activation tiles are at offset 0, directly in front of the ring)
    int off_asf;              // activation block scales of the rows, one 16-byte entry per (k-tile, row)
    int xs_off;               // offset, inside the work area, of the staging space for the activation row (behind the sign words)
    uint32_t epoch;
    int mode;
    unsigned long long wait_ns;
    int skip_publish_cta;     // test aid: this CTA does not publish its z values (-1: none)
    int trigger;              // where the CTA lets the next kernel of the stream start: 0 after set-up, 1 once its
                              // activations are in registers and its z slice is computed, 2 once it has seen all of z,
                              // 3 after its store, 4 once its last weight record has landed
    int dbg;                  // timing experiments (wrong results): 1 no MMAs are issued, 2 the z poll does not wait
    int lut;                  // expansion by look-up table (the launcher has added the table behind the partial sums)
    int inflight;             // weight records a CTA keeps in flight while it fills its ring (0: all at once)
    unsigned long long* stamps;
};

struct SCtrl {
    uint64_t full[MAX_RING];
    uint64_t empty[MAX_RING];
    uint64_t sf_full[NSETS];
    uint64_t sf_empty[NSETS];
    uint64_t b_ready;
    uint64_t acc_full;
    uint64_t tmem_ready;      // TMEM is allocated (the allocation waits for the previous kernel's CTA on this SM)
    float zred[LR_WARPS][NRMAX + 1];
    float ztp[LR_WARPS][4];
    uint32_t tmem_base;
    uint32_t seq;             // launches completed on this scratch before this one (read once per CTA)
    volatile int abort;
    // (behind the fields of the one- and two-row kernels, whose layout stays as it was measured)
    uint64_t b_su[3];         // more than two rows: the activation codes of super-units 0..2 are in shared memory
};
static_assert(sizeof(SCtrl) <= 1024, "slab control block too large");
static_assert(LR_WARPS * (2 * NRMAX + 1) * 4 <= 1024, "the z sums of the four-row kernel live in the read-out area (at least 1024 bytes there)");

__device__ __noinline__ void sfail(SCtrl* ctrl, int32_t* status, uint32_t epoch, int code, int role) {
    ctrl->abort = 1;
    if (atomicCAS(status, 0, code) == 0) {
        status[1] = (int)blockIdx.x;
        status[2] = (int)epoch;
        status[3] = role;
    }
}

// Bounded mbarrier wait (suspending try_wait). False when the budget ran out or another role aborted.
__device__ __noinline__ bool swait(uint32_t bar, uint32_t parity, SCtrl* ctrl, const SlabParams& p, int code, int role) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 3u) == 3u) {
            if (ctrl->abort) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > p.wait_ns) { sfail(ctrl, p.status, p.epoch, code, role); return false; }
        }
    }
}

// The same by polling, for lanes of one warp that wait on different barriers.
__device__ __noinline__ bool spoll(uint32_t bar, uint32_t parity, SCtrl* ctrl, const SlabParams& p, int code, int role) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_test_wait(bar, parity)) return true;
        __nanosleep(32);
        if ((it & 63u) == 63u) {
            if (ctrl->abort) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > p.wait_ns) { sfail(ctrl, p.status, p.epoch, code, role); return false; }
        }
    }
}

__device__ __forceinline__ uint32_t ld_cg_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_add_u32(uint32_t* p, uint32_t v) {
    asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// acc += x where bit `mask` of w is set (an add under a predicate: no branch, no select)
#define BILOCO_SPADD(accv, w, mask, xv)                                                                                     \
    asm("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\tand.b32 t, %1, %2;\n\tsetp.ne.u32 p, t, 0;\n\t@p add.f32 %0, %0, %3;\n\t}" \
        : "+f"(accv) : "r"(w), "r"(mask), "f"(xv))

// Sum of v[0..7] over the 32 lanes, eight values at once: a lane gives away half of its values at every step. On
// return lane l holds the total of value ((l >> 4) & 1) * 4 + ((l >> 3) & 1) * 2 + ((l >> 2) & 1).
__device__ __forceinline__ float reduce8(const float (&v)[NRMAX], int lane) {
    const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4;
    float a[4], b[2], c;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float give = h16 ? v[i] : v[i + 4], keep = h16 ? v[i + 4] : v[i];
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

// One segment of a thread's activation span against NQ ranks: sums[q] += sum of the segment's activations whose sign bit
// in rank (r0 + q)'s row is set; plain += sum of all of them. xw holds the segment's n2 bf16 pairs; the segment starts
// at element idx of the row (bit sh of sign word wi).
// (Not inlined: it serves rows longer than 8192 elements only, and code that is never run should not sit between the
// lines that are: the kernel's instructions are fetched once per launch and instruction fetch shows in its stall profile.)
template <int NQ>
__device__ __noinline__ void zspan(const uint32_t (&xw)[XW_MAX], int n2, const uint32_t* vt, int words, int wi, int sh,
                                      int r0, int nr, float (&sums)[NRMAX], float& plain) {
    // With eight ranks the eight sums are chains enough to cover the add latency; with four, each rank gets two.
    constexpr bool TWO = NQ <= 4;
    uint32_t vw[NQ];
    float a1[TWO ? NQ : 1];
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
        uint32_t lo = 0u, hi = 0u;
        if (r0 + q < nr) {
            lo = vt[(r0 + q) * words + wi];
            if (sh + 2 * n2 > 32) hi = vt[(r0 + q) * words + wi + 1];
        }
        vw[q] = __funnelshift_r(lo, hi, sh);
        if (TWO) a1[q] = 0.f;
    }
    float ps = 0.f;
#pragma unroll
    for (int i = 0; i < XW_MAX; ++i) {
        if (i < n2) {
            const float x0 = __uint_as_float(xw[i] << 16), x1 = __uint_as_float(xw[i] & 0xFFFF0000u);
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                BILOCO_SPADD(sums[q], vw[q], 1u << (2 * i), x0);
                if (TWO) BILOCO_SPADD(a1[q], vw[q], 2u << (2 * i), x1);
                else BILOCO_SPADD(sums[q], vw[q], 2u << (2 * i), x1);
            }
            ps += x0 + x1;
        }
    }
    if (TWO) {
#pragma unroll
        for (int q = 0; q < NQ; ++q) sums[q] += a1[q];
    }
    plain += ps;
}

// The same from the staged row in shared memory, as a rolled loop. The launch runs every instruction once per CTA, so
// code size is time: straight-line code is fetched at a few cycles per instruction (measured: the unrolled span took
// 2400 cycles for 300 instructions), a loop body is fetched once.
template <int NQ>
__device__ __forceinline__ void zspan_rolled(const uint32_t* xs, int n2, const uint32_t* vt, int words, int wi, int sh,
                                             int r0, int nr, float (&sums)[NRMAX], float& plain) {
    uint32_t vw[NQ];
    float a1[NQ];
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
        uint32_t lo = 0u, hi = 0u;
        if (r0 + q < nr) {
            lo = vt[(r0 + q) * words + wi];
            if (sh + 2 * n2 > 32) hi = vt[(r0 + q) * words + wi + 1];
        }
        vw[q] = __funnelshift_r(lo, hi, sh);
        a1[q] = 0.f;
    }
    float ps = 0.f;
    uint32_t xn = xs[0];
#pragma unroll 1
    for (int i = 0; i < n2; ++i) {
        const uint32_t xc = xn;
        xn = xs[i + 1 < n2 ? i + 1 : i];              // next pair, requested before this one is used
        const float x0 = __uint_as_float(xc << 16), x1 = __uint_as_float(xc & 0xFFFF0000u);
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            BILOCO_SPADD(sums[q], vw[q], 1u, x0);
            BILOCO_SPADD(a1[q], vw[q], 2u, x1);
            vw[q] >>= 2;
        }
        ps += x0 + x1;
    }
#pragma unroll
    for (int q = 0; q < NQ; ++q) sums[q] += a1[q];
    plain += ps;
}

// Sixteen values at once (see reduce8). On return lane l holds the total of value
// ((l >> 4) & 1) * 8 + ((l >> 3) & 1) * 4 + ((l >> 2) & 1) * 2 + ((l >> 1) & 1).
__device__ __forceinline__ float reduce16(const float (&v)[2 * NRMAX], int lane) {
    const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4, h2 = lane & 2;
    float a[8], b[4], c[2], d;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float give = h16 ? v[i] : v[i + 8], keep = h16 ? v[i + 8] : v[i];
        a[i] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float give = h8 ? a[i] : a[i + 4], keep = h8 ? a[i + 4] : a[i];
        b[i] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float give = h4 ? b[i] : b[i + 2], keep = h4 ? b[i + 2] : b[i];
        c[i] = keep + __shfl_xor_sync(0xffffffffu, give, 4);
    }
    {
        const float give = h2 ? c[0] : c[1], keep = h2 ? c[1] : c[0];
        d = keep + __shfl_xor_sync(0xffffffffu, give, 2);
    }
    d += __shfl_xor_sync(0xffffffffu, d, 1);
    return d;
}

// A thread's whole span (at most 32 activations, staged in shared memory) against up to sixteen ranks in one pass: one
// chain of adds per rank (sixteen independent chains cover the add latency), the bit masks move instead of the sign words
// (one shift per pair of activations for all ranks).
__device__ __forceinline__ void zspan_rolled16(const uint32_t* xs, int n2, const uint32_t* vt, int words, int wi, int sh, int nr,
                                               float (&sums)[2 * NRMAX], float& plain) {
    uint32_t vw[2 * NRMAX];
#pragma unroll
    for (int q = 0; q < 2 * NRMAX; ++q) {
        uint32_t lo = 0u, hi = 0u;
        if (q < nr) {
            lo = vt[q * words + wi];
            if (sh + 2 * n2 > 32) hi = vt[q * words + wi + 1];
        }
        vw[q] = __funnelshift_r(lo, hi, sh);
    }
    float ps = 0.f;
    uint32_t xn = xs[0];
    uint32_t m0 = 1u;
#pragma unroll 1
    for (int i = 0; i < n2; ++i) {
        const uint32_t xc = xn;
        xn = xs[i + 1 < n2 ? i + 1 : i];
        const float x0 = __uint_as_float(xc << 16), x1 = __uint_as_float(xc & 0xFFFF0000u);
        const uint32_t m1 = m0 << 1;
#pragma unroll
        for (int q = 0; q < 2 * NRMAX; ++q) {
            BILOCO_SPADD(sums[q], vw[q], m0, x0);
            BILOCO_SPADD(sums[q], vw[q], m1, x1);
        }
        ps += x0 + x1;
        m0 <<= 2;
    }
    plain += ps;
}

// Expansion without the table (ranks or rows for which the table would not fit): per item (rank word, column) 32 adds
// under predicates taken from the word's bits. Not inlined (see zspan).
template <int ROWS>
__device__ __noinline__ void expand_padd(const float* zs, float* corrp, const uint32_t* us, int nit, int Rt, int Rw, int Rpad, int lt) {
#pragma unroll 1
    for (int id = lt; id < nit; id += LR_THREADS) {
        const int w = id / Rt, col = id - w * Rt;
        float c0[ROWS], c1[ROWS];
#pragma unroll
        for (int m = 0; m < ROWS; ++m) { c0[m] = 0.f; c1[m] = 0.f; }
        uint32_t ub = us[id];
#pragma unroll 1
        for (int b = 0; b < 32; b += 4) {
#pragma unroll
            for (int m = 0; m < ROWS; ++m) {
                const float4 zz = *reinterpret_cast<const float4*>(zs + m * Rpad + 32 * w + b);
                BILOCO_SPADD(c0[m], ub, 1u, zz.x);
                BILOCO_SPADD(c1[m], ub, 2u, zz.y);
                BILOCO_SPADD(c0[m], ub, 4u, zz.z);
                BILOCO_SPADD(c1[m], ub, 8u, zz.w);
            }
            ub >>= 4;
        }
#pragma unroll
        for (int m = 0; m < ROWS; ++m) corrp[(m * Rw + w) * Rt + col] = c0[m] + c1[m];
    }
}

// The same for four rows: the predicate of a sign bit is formed once and serves the four rows' adds (six instructions per
// bit instead of twelve). Same order of additions per row as expand_padd.
#define BILOCO_SPADD4(acc, w, mask, x0, x1, x2, x3)                                                                  \
    asm("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\tand.b32 t, %4, %5;\n\tsetp.ne.u32 p, t, 0;\n\t"                 \
        "@p add.f32 %0, %0, %6;\n\t@p add.f32 %1, %1, %7;\n\t@p add.f32 %2, %2, %8;\n\t@p add.f32 %3, %3, %9;\n\t}" \
        : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])                                                     \
        : "r"(w), "r"(mask), "f"(x0), "f"(x1), "f"(x2), "f"(x3))
__device__ __noinline__ void expand_padd4(const float* zs, float* corrp, const uint32_t* us, int nit, int Rt, int Rw, int Rpad, int lt) {
#pragma unroll 1
    for (int id = lt; id < nit; id += LR_THREADS) {
        const int w = id / Rt, col = id - w * Rt;
        float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t ub = us[id];
        const float* zw = zs + 32 * w;
#pragma unroll 1
        for (int b = 0; b < 32; b += 4) {
            const float4 z0 = *reinterpret_cast<const float4*>(zw + b);
            const float4 z1 = *reinterpret_cast<const float4*>(zw + Rpad + b);
            const float4 z2 = *reinterpret_cast<const float4*>(zw + 2 * Rpad + b);
            const float4 z3 = *reinterpret_cast<const float4*>(zw + 3 * Rpad + b);
            BILOCO_SPADD4(c0, ub, 1u, z0.x, z1.x, z2.x, z3.x);
            BILOCO_SPADD4(c1, ub, 2u, z0.y, z1.y, z2.y, z3.y);
            BILOCO_SPADD4(c0, ub, 4u, z0.z, z1.z, z2.z, z3.z);
            BILOCO_SPADD4(c1, ub, 8u, z0.w, z1.w, z2.w, z3.w);
            ub >>= 4;
        }
#pragma unroll
        for (int m = 0; m < 4; ++m) corrp[(m * Rw + w) * Rt + col] = c0[m] + c1[m];
    }
}

template <int ROWS>
__global__ void __launch_bounds__(NT, 2) slab_kernel(const __grid_constant__ SlabParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);
    SCtrl* ctrl = reinterpret_cast<SCtrl*>(sm + p.off_ctrl);
    uint8_t* atile = sm;                                                // activation tiles, directly in front of the ring
    uint32_t* us = reinterpret_cast<uint32_t*>(sm + p.off_us);          // [Rw][Rt] sign words of this CTA's columns
    uint8_t* work = sm + p.off_work;                                    // sign words of V, then z + expansion partials
    float* accp = reinterpret_cast<float*>(sm + p.off_accp);            // [kg * ROWS][nbp]: the accumulator's useful lanes

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    const int Rt = p.Rt, kg = p.kg, nsu = p.nsu, ring = p.ring;
    unsigned long long* stamps = p.stamps ? p.stamps + (size_t)cta * SLAB_STAMPS : nullptr;
    if (tid == 0 && stamps) { stamps[0] = globaltimer_ns(); stamps[16] = (unsigned long long)clock64(); }

    // ---------------- set-up ----------------
    if (tid == 0) {
#pragma unroll 1
        for (int s = 0; s < ring; ++s) {
            mbar_init(smem_u32(&ctrl->full[s]), 1);
            mbar_init(smem_u32(&ctrl->empty[s]), 1);
        }
#pragma unroll 1
        for (int q = 0; q < NSETS; ++q) {
            mbar_init(smem_u32(&ctrl->sf_full[q]), 128);
            mbar_init(smem_u32(&ctrl->sf_empty[q]), 1);
        }
        mbar_init(smem_u32(&ctrl->b_ready), 128);
        if constexpr (ROWS > 2) {
#pragma unroll 1
            for (int q = 0; q < 3; ++q) mbar_init(smem_u32(&ctrl->b_su[q]), 128);
        }
        mbar_init(smem_u32(&ctrl->acc_full), 1);
        mbar_init(smem_u32(&ctrl->tmem_ready), 1);
        ctrl->abort = 0;
        fence_mbar_init();
    }
    __syncthreads();
    if (p.trigger == 0) griddep_launch_dependents();   // the next kernel of the stream may move in and prefetch its weights
    if (tid == 0 && stamps) { stamps[1] = globaltimer_ns(); stamps[17] = (unsigned long long)clock64(); }

    const size_t su_stride = (size_t)kg * Rt * UNIT_ROW_BYTES;
    const uint8_t* wbase = p.W_slab + (size_t)cta * p.nkt * Rt * UNIT_ROW_BYTES;
    auto units_of = [&](int j) { const int left = p.nkt - j * kg; return left < kg ? left : kg; };
    auto issue_w = [&](int j) {
        const int slot = j % ring;
        const uint32_t bytes = (uint32_t)(units_of(j) * Rt * UNIT_ROW_BYTES);
        const uint32_t bar = smem_u32(&ctrl->full[slot]);
        mbar_arrive_expect_tx(bar, bytes);
        bulk_load(base + p.off_ring + slot * p.stage_bytes, wbase + (size_t)j * su_stride, bytes, bar);
    };

    const bool has_rows = cta < p.Grows;
    if (!has_rows && (warp >= FIRST_SF_WARP && warp < FIRST_Z_WARP || warp >= MMA_WARP)) {
        // a CTA without weight rows: only its low-rank threads work (z slice), the others go straight to the exit
    } else if (warp == REFILL_WARP) {
        // ================= weight copies beyond the first four (those go out from the GEMM-side warps) =================
        // The four lanes share every record (a quarter each, rounded to 16 bytes): a copy issued by one thread is served
        // piece after piece, copies of different threads overlap, and a record that is fetched after the dependency wait
        // (its stage was still occupied before) sits on the launch's critical path.
        if (lane < PRODUCERS) {
            const int first = ring < PRODUCERS ? ring : PRODUCERS;      // (records 0 .. first - 1 have gone out already)
#pragma unroll 1
            for (int j = first; j < nsu; ++j) {
                const int slot = j % ring;
                if (j >= ring && !spoll(smem_u32(&ctrl->empty[slot]), ((j / ring) - 1) & 1, ctrl, p, ST_EMPTY, warp)) break;
                const uint32_t bytes = (uint32_t)(units_of(j) * Rt * UNIT_ROW_BYTES);
                const uint32_t quarter = ((bytes >> 2) + 15u) & ~15u;
                const uint32_t off = quarter * (uint32_t)lane;
                const uint32_t bar = smem_u32(&ctrl->full[slot]);
                if (lane == 0) mbar_arrive_expect_tx(bar, bytes);
                if (off < bytes)
                    bulk_load(base + p.off_ring + slot * p.stage_bytes + off, wbase + (size_t)j * su_stride + off,
                              (bytes - off) < quarter ? (bytes - off) : quarter, bar);
            }
        }
    } else if (warp == MMA_WARP) {
        // ================= TMEM allocation, MMA issue =================
        // All 512 columns, in one allocation: it returns once the previous kernel's CTA on this SM has freed its own
        // (about a microsecond before this kernel's dependency wait returns); nobody holds columns while waiting for more.
        tmem_alloc(smem_u32(&ctrl->tmem_base), SLAB_TMEM_COLS);
        tmem_relinquish();
        tc_fence_before_sync();
        if (lane == 0) mbar_arrive(smem_u32(&ctrl->tmem_ready));
        if (lane == 0 && stamps) { stamps[10] = globaltimer_ns(); stamps[26] = (unsigned long long)clock64(); }
        const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);
        const uint32_t idesc = make_idesc_nvf4(128, p.nbp);
        // (more than two rows: the activation tiles are announced super-unit by super-unit, the first three on their own)
        bool ok = swait(smem_u32(ROWS > 2 ? &ctrl->b_su[0] : &ctrl->b_ready), 0, ctrl, p, ST_FULL, warp);
        if (lane == 0 && stamps) stamps[15] = globaltimer_ns();
        int slot = 0;                    // (j % ring and the parity of j / ring, kept by counting: no quotient by a run-time number in front of an MMA)
        uint32_t lap = 0u;
#pragma unroll 1
        for (int j = 0; ok && j < nsu; ++j) {
            const int set = j % NSETS;
            if (ROWS > 2 && j > 0 && !swait(smem_u32(j < 3 ? &ctrl->b_su[j] : &ctrl->b_ready), 0, ctrl, p, ST_FULL, warp)) break;
            if (!swait(smem_u32(&ctrl->full[slot]), lap, ctrl, p, ST_FULL, warp)) break;
            if (!swait(smem_u32(&ctrl->sf_full[set]), (j / NSETS) & 1, ctrl, p, ST_SF_FULL, warp)) break;
            tc_fence_after_sync();
            if (lane == 0) {
                const uint64_t adesc = make_smem_desc(base + j * p.atile_bytes, 1024, 2);                        // activation rows
                const uint64_t wdesc = make_smem_desc(base + p.off_ring + slot * p.stage_bytes, 1024, 2);        // weight rows (N)
                const uint32_t sf = tmem + SET_COL0 + 64u * (uint32_t)set;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (!(p.dbg & 1))
                        tc_mma_nvf4(tmem, adesc + 2 * k, wdesc + 2 * k, idesc, sf + SFA_OFF + 4 * k, sf + 8 * k, (j > 0 || k > 0) ? 1u : 0u);
                tc_commit(smem_u32(&ctrl->empty[slot]));
                tc_commit(smem_u32(&ctrl->sf_empty[set]));
                if (j == nsu - 1) tc_commit(smem_u32(&ctrl->acc_full));
            }
            __syncwarp();
            if (++slot == ring) { slot = 0; lap ^= 1u; }
        }
        if (lane == 0 && stamps) { stamps[12] = globaltimer_ns(); stamps[28] = (unsigned long long)clock64(); }
    } else if (warp >= FIRST_SF_WARP && warp < FIRST_Z_WARP) {
        // ================= GEMM side: weight copies, scale factors -> TMEM, activation codes -> shared memory =================
        const int st = tid - FIRST_SF_WARP * 32;                    // 0..127
        const int mine = warp - FIRST_SF_WARP;
        // copies issued by different warps overlap; one thread's go out one after another
        if (lane == 0 && mine < nsu && mine < ring) issue_w(mine);
        const uint32_t quad = (uint32_t)((warp & 3) * 32) << 16;
        // activation tiles start as zeros: rows without a k-tile (last super-unit) or beyond M must not contribute
        for (int i = st; i < nsu * (p.atile_bytes >> 4); i += 128) reinterpret_cast<uint4*>(atile)[i] = make_uint4(0u, 0u, 0u, 0u);
        named_bar_sync(2, 128);                                      // (another thread writes the codes into these bytes later)

        // Weights' scales of super-unit j: operand row n = g Rt + r sits in lane n % 32, column n / 32 of each MMA's eight
        // columns; a thread serves rows lane, lane + 32, ..., lane + 224 (16 bytes each in the stage: four MMAs' words).
        auto sfb_move = [&](int j, uint32_t tmem) {
            const int slot = j % ring, set = j % NSETS;
            const int rows = units_of(j) * Rt;
            const uint4* sf = reinterpret_cast<const uint4*>(sm + p.off_ring + (size_t)slot * p.stage_bytes + (size_t)rows * 128);
            uint32_t r0[16], r1[16];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int n = lane + 32 * c;
                const uint4 v = n < rows ? sf[n] : make_uint4(0u, 0u, 0u, 0u);
                r0[c] = v.x; r0[8 + c] = v.y; r1[c] = v.z; r1[8 + c] = v.w;
            }
            const uint32_t t = tmem + quad + SET_COL0 + 64u * (uint32_t)set;
            tmem_st_x16(t, r0);
            tmem_st_x16(t + 16, r1);
        };
        // Activations' scales of super-unit j: operand row n = g * M + m in lane n, first column of each MMA's four.
        const int bg = lane / ROWS, bm = lane - bg * ROWS;
        const uint4* asf = reinterpret_cast<const uint4*>(sm + p.off_asf);
        auto sfa_move = [&](int j, uint32_t tmem) {
            uint32_t ra[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) ra[i] = 0u;
            const int kt = j * kg + bg;
            if (lane < kg * ROWS && bm < p.M && kt < p.nkt) {
                const uint4 v = asf[kt * ROWS + bm];
                ra[0] = v.x; ra[4] = v.y; ra[8] = v.z; ra[12] = v.w;
            }
            tmem_st_x16(tmem + quad + SET_COL0 + 64u * (uint32_t)(j % NSETS) + SFA_OFF, ra);
        };
        const int nfirst = nsu < ring ? (nsu < NSETS ? nsu : NSETS) : (ring < NSETS ? ring : NSETS);
        bool ok = swait(smem_u32(&ctrl->tmem_ready), 0, ctrl, p, ST_FULL, warp);
        tc_fence_after_sync();
        const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);
        // before the dependency wait: the weights' scale factors of the stages filled ahead
#pragma unroll 1
        for (int j = 0; j < nfirst; ++j) {
            if (ok && !swait(smem_u32(&ctrl->full[j % ring]), 0, ctrl, p, ST_FULL, warp)) ok = false;
            if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            sfb_move(j, tmem);
        }
        tc_wait_st();
        // One and two rows: where this thread's first activation chunks go in the operand tiles, worked out here, in front of
        // the dependency wait (the quotient by kg, a run-time number, is about twenty dependent instructions: several hundred
        // cycles that would otherwise sit between the arrival of the codes and the first MMA).
        uint32_t cdst[4] = {0u, 0u, 0u, 0u};
        if constexpr (ROWS <= 2) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = st + 128 * u, c = i & 7, rest = i >> 3;
                const int m = rest % ROWS, kt = rest / ROWS;
                const int j = kt / kg, g = kt - j * kg, n = g * ROWS + m;
                cdst[u] = (uint32_t)(j * p.atile_bytes + (n >> 3) * 1024 + (n & 7) * 128 + ((c ^ (n & 7)) * 16));
            }
        }
        if (st == 0 && stamps) { stamps[13] = globaltimer_ns(); stamps[29] = (unsigned long long)clock64(); }
        griddep_wait();
        if (st == 0 && stamps) { stamps[14] = globaltimer_ns(); stamps[30] = (unsigned long long)clock64(); }
        if (ok) {
            // Every global read of this side is issued before any of them is waited for (one memory round trip in all).
            // Block scales: the four bytes of (k-tile kt, 64-k chunk a, row m) sit in atom 4 kt + a of the 128x4 layout.
            uint32_t* asf_w = reinterpret_cast<uint32_t*>(sm + p.off_asf);
            const int nsf = p.nkt * ROWS * 4;
            constexpr int NSFV = ROWS <= 2 ? 2 : 4;     // scale words and code chunks a thread requests in one batch
            constexpr int NU = ROWS <= 2 ? 4 : 8;
            uint32_t sfv[NSFV];
#pragma unroll
            for (int r = 0; r < NSFV; ++r) {
                const int i = st + 128 * r;
                sfv[r] = 0u;
                if (i < nsf) {
                    const int a = i & 3, m = (i >> 2) % ROWS, kt = (i >> 2) / ROWS;
                    if (m < p.M)
                        sfv[r] = ld_cg_u32(p.A_sf + ((size_t)(m >> 7) * (p.K >> 6) + (size_t)kt * 4 + a) * 512 + (m & 31) * 16 + ((m >> 5) & 3) * 4);
                }
            }
            // activation codes: 16-byte chunk c of row m of k-tile kt -> tile kt / kg, row n = (kt % kg) * M + m, chunk c ^ (n & 7)
            const int nchunks = p.nkt * p.M * 8;
            const int kbytes = p.K >> 1;
            // More than two rows: the tiles are announced super-unit by super-unit (the first three on their own), so that the
            // first MMAs start when a quarter of the codes has arrived; a thread signals a super-unit once its next chunk
            // lies behind it.
            const int su_chunks = kg * p.M * 8, nsig = nsu < 3 ? nsu : 3;
            int sj = 0;
#pragma unroll 1
            for (int i0 = st; i0 < nchunks || (ROWS > 2 && i0 == st); i0 += NU * 128) {      // (more rows: every thread makes the first trip)
                uint4 v[NU];
#pragma unroll
                for (int u = 0; u < NU; ++u) {
                    const int i = i0 + 128 * u;
                    if (i < nchunks) {
                        const int c = i & 7, rest = i >> 3;
                        const int m = ROWS <= 2 ? rest % ROWS : rest % p.M, kt = ROWS <= 2 ? rest / ROWS : rest / p.M;      // (one, two rows: M = ROWS)
                        v[u] = ld_cg_v4(p.A_codes + (size_t)m * kbytes + kt * 128 + c * 16);
                    }
                }
                if constexpr (ROWS > 2) {
                    if (i0 == st) {
                        // the scales were requested first: they go to shared memory and the first set to TMEM while the codes arrive
#pragma unroll
                        for (int r = 0; r < NSFV; ++r)
                            if (st + 128 * r < nsf) asf_w[st + 128 * r] = sfv[r];
                        named_bar_sync(2, 128);
                        sfa_move(0, tmem);
                        tc_wait_st();
                        tc_fence_before_sync();
                        mbar_arrive(smem_u32(&ctrl->sf_full[0]));
                    }
                }
#pragma unroll
                for (int u = 0; u < NU; ++u) {
                    const int i = i0 + 128 * u;
                    if (i < nchunks) {
                        if (ROWS <= 2 && i0 == st) {
                            *reinterpret_cast<uint4*>(atile + cdst[u]) = v[u];
                        } else {
                            const int c = i & 7, rest = i >> 3;
                            const int m = rest % p.M, kt = rest / p.M;
                            const int j = kt / kg, g = kt - j * kg, n = g * ROWS + m;
                            *reinterpret_cast<uint4*>(atile + j * p.atile_bytes + (n >> 3) * 1024 + (n & 7) * 128 + ((c ^ (n & 7)) * 16)) = v[u];
                        }
                    }
                    if constexpr (ROWS > 2) {
                        while (sj < nsig && (sj + 1) * su_chunks <= i + 128) {
                            fence_proxy_async();
                            mbar_arrive(smem_u32(&ctrl->b_su[sj]));
                            ++sj;
                        }
                    }
                }
            }
            if constexpr (ROWS > 2) {
                while (sj < nsig) {
                    fence_proxy_async();
                    mbar_arrive(smem_u32(&ctrl->b_su[sj]));
                    ++sj;
                }
            } else {
#pragma unroll
                for (int r = 0; r < NSFV; ++r)
                    if (st + 128 * r < nsf) asf_w[st + 128 * r] = sfv[r];
#pragma unroll 1
                for (int i = st + 128 * NSFV; i < nsf; i += 128) {          // (rows longer than 16384 elements)
                    const int a = i & 3, m = (i >> 2) % ROWS, kt = (i >> 2) / ROWS;
                    asf_w[i] = m < p.M ? ld_cg_u32(p.A_sf + ((size_t)(m >> 7) * (p.K >> 6) + (size_t)kt * 4 + a) * 512 + (m & 31) * 16 + ((m >> 5) & 3) * 4) : 0u;
                }
            }
            fence_proxy_async();                      // the activation tiles were written with ordinary stores
            mbar_arrive(smem_u32(&ctrl->b_ready));
            if constexpr (ROWS <= 2) named_bar_sync(2, 128);      // the scales are in shared memory
#pragma unroll 1
            for (int j = ROWS > 2 ? 1 : 0; j < nfirst; ++j) {     // (set by set: the first MMAs start while the later sets are written)
                sfa_move(j, tmem);
                tc_wait_st();
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&ctrl->sf_full[j % NSETS]));
            }
            if (st == 0 && stamps) { stamps[11] = globaltimer_ns(); stamps[27] = (unsigned long long)clock64(); }
            if (p.trigger == 4 && st == 0 && nsu <= ring) griddep_launch_dependents();
            // stages and sets that are filled again
#pragma unroll 1
            for (int j = nfirst; j < nsu; ++j) {
                const int set = j % NSETS;
                bool ready = swait(smem_u32(&ctrl->full[j % ring]), (j / ring) & 1, ctrl, p, ST_FULL, warp);
                // trigger 4: the next kernel of the stream moves in (and starts its weight burst) once this CTA's last
                // weight record has landed, i.e. after the last global read on this launch's critical path
                if (p.trigger == 4 && st == 0 && j == nsu - 1) griddep_launch_dependents();
                if (ready && j >= NSETS) ready = swait(smem_u32(&ctrl->sf_empty[set]), ((j / NSETS) - 1) & 1, ctrl, p, ST_SF_EMPTY, warp);
                if (!__all_sync(0xffffffffu, ready)) break;
                tc_fence_after_sync();
                sfb_move(j, tmem);
                sfa_move(j, tmem);
                tc_wait_st();
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&ctrl->sf_full[set]));
            }
        }
    } else {
        // ================= low-rank side (256 threads), read-out and store =================
        const int lt = warp < 4 ? tid : tid - (FIRST_Z_WARP - 4) * 32;      // 0..255
        const int lw = lt >> 5;
        const int words = p.K >> 5;                                          // sign words per rank
        uint32_t* vt = reinterpret_cast<uint32_t*>(work);
        // my z item: (row zm, ranks [ra, rb))
        const int nitems = p.M * p.nsl;
        int zm = 0, ra = 0, rb = 0;
        if (p.R > 0 && cta < nitems) {
            zm = cta / p.nsl;
            const int sl = cta - zm * p.nsl;
            ra = (int)((long long)sl * p.R / p.nsl);
            rb = (int)((long long)(sl + 1) * p.R / p.nsl);
        }
        const int nr = rb - ra;
        if (p.R > 0) {
            // sign words of my ranks (static data: before the dependency wait)
            const int vch = p.K >> 7;                                        // 16-byte chunks per rank
            const uint32_t vt_s = smem_u32(vt);
#pragma unroll 1
            for (int i = lt; i < nr * vch; i += LR_THREADS) {
                const int q = i / vch, c = i - q * vch;
                cp_async16(vt_s + (q * vch + c) * 16, p.Vp + (size_t)(ra + q) * (p.K >> 3) + c * 16);
            }
            cp_async_commit();
            // sign words of my columns, transposed to [word][column]
            const int ncol = !has_rows ? 0 : ((p.N - cta * Rt) < Rt ? (p.N - cta * Rt) : Rt);
            const int32_t* ug = p.Ucol + (size_t)cta * Rt * p.Rw;
#pragma unroll 1
            for (int i = lt; i < Rt * p.Rw; i += LR_THREADS) {
                const int col = i / p.Rw, w = i - col * p.Rw;
                us[w * Rt + col] = col < ncol ? (uint32_t)ug[i] : 0u;
            }
            cp_async_wait_all();
        }
        float s_coef[2] = {0.f, 0.f};                                        // (nr <= 2 * NRMAX: two passes at most)
        if (ROWS > 2) {                                                      // (one pass of up to sixteen ranks)
            if (lt < 2 * NRMAX && lt < nr) s_coef[0] = __bfloat162float(p.S[ra + lt]);
        } else if (lt < NRMAX) {
            if (lt < nr) s_coef[0] = __bfloat162float(p.S[ra + lt]);
            if (NRMAX + lt < nr) s_coef[1] = __bfloat162float(p.S[ra + NRMAX + lt]);
        }
        named_bar_sync(3, LR_THREADS);

        griddep_wait();            // everything below reads what earlier kernels of the stream wrote
        if (lt == 0 && stamps) { stamps[2] = globaltimer_ns(); stamps[18] = (unsigned long long)clock64(); }
        // Everything every CTA reads at this point is read by as few threads as possible: hundreds of requests for one
        // 128-byte line are served one after another by its L2 slice (measured: the launch count read by all threads
        // and the activation row read in 4-byte pieces cost 1.5 - 6 us; one reader and coalesced 16-byte loads, 0.5).
        float alpha_r = 0.f;
        if (lt < ROWS * Rt) alpha_r = __uint_as_float(ld_cg_u32(p.alpha));
        bool good = true;
        uint32_t phase = 0u;

        if (p.R > 0) {
            // ---- z stage: thread lt owns the activations [lt e, (lt + 1) e), e = K / 256 (even) ----
            const int e = p.K >> 8;
            const uint32_t* xrow = reinterpret_cast<const uint32_t*>(p.X + (size_t)zm * p.K) + ((lt * e) >> 1);
            const bool single = e <= 2 * XW_MAX;                              // the whole span fits the registers: loaded once
            uint32_t xw[XW_MAX];
            if (single && nr > 0) {
                // The warp's 32 spans are 64 e contiguous bytes of the row: fetched as 16-byte pieces (whole lines, every
                // line once per CTA), starting at a line that depends on the CTA so that the CTAs do not all ask the same
                // L2 slice at the same moment, staged in this warp's own piece of shared memory, read back span by span.
                const int nch = 4 * e;                                       // 16-byte pieces of this warp
                uint8_t* stg = work + p.xs_off + lw * (64 * e);
                const uint8_t* src = reinterpret_cast<const uint8_t*>(p.X + (size_t)zm * p.K) + (size_t)lw * 64 * e;
                const int rot = 8 * (cta % (e >> 1));
                uint4 v[3];
#pragma unroll
                for (int i = 0; i < 3; ++i) {                                // (nch <= 128: at most four rounds; the fourth below)
                    int c = lane + 32 * i + rot;
                    c = c >= nch ? c - nch : c;
                    if (lane + 32 * i < nch) v[i] = ld_cg_v4(src + c * 16);
                }
#pragma unroll
                for (int i = 0; i < 3; ++i) {
                    int c = lane + 32 * i + rot;
                    c = c >= nch ? c - nch : c;
                    if (lane + 32 * i < nch) *reinterpret_cast<uint4*>(stg + c * 16) = v[i];
                }
                if (lt == 0) {      // (behind this thread's own requests, so that it does not wait twice)
                    const uint4 c0 = ld_volatile_v4(p.z_counter + 8), c1 = ld_volatile_v4(p.z_counter + 12);
                    ctrl->seq = (((c0.x + c0.y) + (c0.z + c0.w)) + ((c1.x + c1.y) + (c1.z + c1.w))) >> 20;
                }
                if (lane + 96 < nch) {
                    int c = lane + 96 + rot;
                    c = c >= nch ? c - nch : c;
                    *reinterpret_cast<uint4*>(stg + c * 16) = ld_cg_v4(src + c * 16);
                }
                __syncwarp();
            }
            const uint32_t* mine = reinterpret_cast<const uint32_t*>(work + p.xs_off + lw * (64 * e)) + ((lane * e) >> 1);
            if (lt == 0 && !(single && nr > 0)) {
                const uint4 c0 = ld_volatile_v4(p.z_counter + 8), c1 = ld_volatile_v4(p.z_counter + 12);
                ctrl->seq = (((c0.x + c0.y) + (c0.z + c0.w)) + ((c1.x + c1.y) + (c1.z + c1.w))) >> 20;
            }
            if (lt == 0 && stamps) { stamps[3] = globaltimer_ns(); stamps[19] = (unsigned long long)clock64(); }
            if constexpr (ROWS <= 2) {
#pragma unroll 1
                for (int ps = 0; ps * NRMAX < nr; ++ps) {
                    float sums[NRMAX];
#pragma unroll
                    for (int q = 0; q < NRMAX; ++q) sums[q] = 0.f;
                    float plain = 0.f;
                    const int nq = nr - ps * NRMAX;                                  // ranks of this pass (may exceed NRMAX)
#pragma unroll 1
                    for (int s0 = 0; s0 < e; s0 += 2 * XW_MAX) {
                        const int n2 = ((e - s0) < 2 * XW_MAX ? (e - s0) : 2 * XW_MAX) >> 1;      // pairs in this segment
                        if (!single) {
#pragma unroll
                            for (int i = 0; i < XW_MAX; ++i) xw[i] = i < n2 ? ld_cg_u32(xrow + (s0 >> 1) + i) : 0u;
                        }
                        const int idx = lt * e + s0, wi = idx >> 5, sh = idx & 31;
                        if (single) {
                            if (nq <= 4) zspan_rolled<4>(mine, n2, vt, words, wi, sh, ps * NRMAX, nr, sums, plain);
                            else zspan_rolled<NRMAX>(mine, n2, vt, words, wi, sh, ps * NRMAX, nr, sums, plain);
                        } else if (nq <= 4) {
                            zspan<4>(xw, n2, vt, words, wi, sh, ps * NRMAX, nr, sums, plain);
                        } else {
                            zspan<NRMAX>(xw, n2, vt, words, wi, sh, ps * NRMAX, nr, sums, plain);
                        }
                    }
                    if (lt == 0 && stamps && ps == 0) stamps[26] = (unsigned long long)clock64();
                    const float tot = reduce8(sums, lane);
                    const int rl = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
                    if ((lane & 3) == 0) ctrl->zred[lw][rl] = tot;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) plain += __shfl_xor_sync(0xffffffffu, plain, o);
                    if (lane == 0) ctrl->zred[lw][NRMAX] = plain;
                    named_bar_sync(3, LR_THREADS);
                    if (lt == 0 && stamps && ps == 0) stamps[31] = (unsigned long long)clock64();
                    phase = (ctrl->seq & 1u) ^ 1u;
                    if (lt < NRMAX && ps * NRMAX + lt < nr) {
                        float v = 0.f, a = 0.f;
#pragma unroll
                        for (int g = 0; g < LR_WARPS; ++g) { v += ctrl->zred[g][lt]; a += ctrl->zred[g][NRMAX]; }
                        const float z = (2.f * v - a) * (ps == 0 ? s_coef[0] : s_coef[1]);
                        if (cta != p.skip_publish_cta)
                            p.zbuf[(size_t)zm * p.Rpad + ra + ps * NRMAX + lt] = __uint_as_float((__float_as_uint(z) & ~1u) | phase);
                    }
                    if ((ps + 1) * NRMAX < nr) named_bar_sync(3, LR_THREADS);      // zred is reused by the next pass
                }
            } else {
                // one pass over all ranks of the slice (at most sixteen, rows of at most 8192 elements: the launcher admits no others)
                float sums[2 * NRMAX];
#pragma unroll
                for (int q = 0; q < 2 * NRMAX; ++q) sums[q] = 0.f;
                float plain = 0.f;
                if (nr > 0) {
                    const int idx = lt * e;
                    zspan_rolled16(mine, e >> 1, vt, words, idx >> 5, idx & 31, nr, sums, plain);
                }
                if (lt == 0 && stamps) stamps[26] = (unsigned long long)clock64();
                float (*zr)[2 * NRMAX + 1] = reinterpret_cast<float (*)[2 * NRMAX + 1]>(accp);      // (the read-out area is idle until the MMAs are done)
                const float tot = reduce16(sums, lane);
                const int rl = ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
                if ((lane & 1) == 0) zr[lw][rl] = tot;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) plain += __shfl_xor_sync(0xffffffffu, plain, o);
                if (lane == 0) zr[lw][2 * NRMAX] = plain;
                named_bar_sync(3, LR_THREADS);
                if (lt == 0 && stamps) stamps[31] = (unsigned long long)clock64();
                phase = (ctrl->seq & 1u) ^ 1u;
                if (lt < 2 * NRMAX && lt < nr) {
                    float v = 0.f, a = 0.f;
#pragma unroll
                    for (int g = 0; g < LR_WARPS; ++g) { v += zr[g][lt]; a += zr[g][2 * NRMAX]; }
                    const float z = (2.f * v - a) * s_coef[0];
                    if (cta != p.skip_publish_cta)
                        p.zbuf[(size_t)zm * p.Rpad + ra + lt] = __uint_as_float((__float_as_uint(z) & ~1u) | phase);
                }
            }
            if (lt == 0 && stamps) { stamps[4] = globaltimer_ns(); stamps[20] = (unsigned long long)clock64(); }
            if (p.trigger == 1 && lt == 0) griddep_launch_dependents();

            // ---- poll z: every value is its own flag (lowest mantissa bit = this launch's mark) ----
            float* zs = reinterpret_cast<float*>(work);                         // [ROWS][Rpad] (the sign words are consumed)
            named_bar_sync(3, LR_THREADS);                                      // ... by every thread
            phase = (ctrl->seq & 1u) ^ 1u;                                      // (a CTA without ranks has not looked yet)
            const int vpr = p.Rpad >> 2;
            float zt[ROWS <= 2 ? 2 : ROWS];
#pragma unroll
            for (int m = 0; m < (ROWS <= 2 ? 2 : ROWS); ++m) zt[m] = 0.f;
            const int nvec = has_rows ? p.M * vpr : 0;                          // (a CTA without rows has no use for z)
            if constexpr (ROWS <= 2) {
#pragma unroll 1
                for (int i = lt; i < nvec && good; i += LR_THREADS) {
                    const int m = i / vpr, j = i - m * vpr;
                    const int e0 = 4 * j;
                    const float* src = p.zbuf + (size_t)m * p.Rpad + e0;
                    uint4 v;
                    uint64_t t0 = 0;
#pragma unroll 1
                    for (uint32_t it = 0;; ++it) {
                        v = ld_volatile_v4(src);
                        const uint32_t bad = (e0 + 0 < p.R ? (v.x ^ phase) : 0u) | (e0 + 1 < p.R ? (v.y ^ phase) : 0u) |
                                             (e0 + 2 < p.R ? (v.z ^ phase) : 0u) | (e0 + 3 < p.R ? (v.w ^ phase) : 0u);
                        if (!(bad & 1u) || (p.dbg & 2)) break;
                        if ((it & 15u) == 15u) {
                            if (ctrl->abort) { good = false; break; }
                            const uint64_t now = globaltimer_ns();
                            if (t0 == 0) t0 = now;
                            else if (now - t0 > p.wait_ns) { sfail(ctrl, p.status, p.epoch, ST_Z, 0); good = false; break; }
                        }
                    }
                    float4 zz;
                    zz.x = e0 + 0 < p.R ? __uint_as_float(v.x & ~1u) : 0.f;
                    zz.y = e0 + 1 < p.R ? __uint_as_float(v.y & ~1u) : 0.f;
                    zz.z = e0 + 2 < p.R ? __uint_as_float(v.z & ~1u) : 0.f;
                    zz.w = e0 + 3 < p.R ? __uint_as_float(v.w & ~1u) : 0.f;
                    *reinterpret_cast<float4*>(zs + (size_t)m * p.Rpad + e0) = zz;
                    const float t = (zz.x + zz.y) + (zz.z + zz.w);
                    if (m == 0) zt[0] += t; else zt[1] += t;
                }
            } else {
                // More rows: a thread has several vectors; two are requested before either is examined (one round trip for
                // both), and a vector is asked for again only while its marks are not this launch's.
                auto settle = [&](int i, uint4 v) {
                    const int m = i / vpr, j = i - m * vpr;
                    const int e0 = 4 * j;
                    const float* src = p.zbuf + (size_t)m * p.Rpad + e0;
                    uint64_t t0 = 0;
#pragma unroll 1
                    for (uint32_t it = 0;; ++it) {
                        const uint32_t bad = (e0 + 0 < p.R ? (v.x ^ phase) : 0u) | (e0 + 1 < p.R ? (v.y ^ phase) : 0u) |
                                             (e0 + 2 < p.R ? (v.z ^ phase) : 0u) | (e0 + 3 < p.R ? (v.w ^ phase) : 0u);
                        if (!(bad & 1u) || (p.dbg & 2)) break;
                        if ((it & 15u) == 15u) {
                            if (ctrl->abort) { good = false; break; }
                            const uint64_t now = globaltimer_ns();
                            if (t0 == 0) t0 = now;
                            else if (now - t0 > p.wait_ns) { sfail(ctrl, p.status, p.epoch, ST_Z, 0); good = false; break; }
                        }
                        v = ld_volatile_v4(src);
                    }
                    float4 zz;
                    zz.x = e0 + 0 < p.R ? __uint_as_float(v.x & ~1u) : 0.f;
                    zz.y = e0 + 1 < p.R ? __uint_as_float(v.y & ~1u) : 0.f;
                    zz.z = e0 + 2 < p.R ? __uint_as_float(v.z & ~1u) : 0.f;
                    zz.w = e0 + 3 < p.R ? __uint_as_float(v.w & ~1u) : 0.f;
                    *reinterpret_cast<float4*>(zs + (size_t)m * p.Rpad + e0) = zz;
                    const float t = (zz.x + zz.y) + (zz.z + zz.w);
#pragma unroll
                    for (int mm = 0; mm < ROWS; ++mm) zt[mm] += mm == m ? t : 0.f;
                };
#pragma unroll 1
                for (int i = lt; i < nvec && good; i += 2 * LR_THREADS) {
                    const int i2 = i + LR_THREADS;
                    const uint4 va = ld_volatile_v4(p.zbuf + (size_t)(i / vpr) * p.Rpad + 4 * (i % vpr));
                    uint4 vb = make_uint4(0u, 0u, 0u, 0u);
                    if (i2 < nvec) vb = ld_volatile_v4(p.zbuf + (size_t)(i2 / vpr) * p.Rpad + 4 * (i2 % vpr));
                    settle(i, va);
                    if (i2 < nvec && good) settle(i2, vb);
                }
            }
#pragma unroll
            for (int m = 0; m < ROWS; ++m) {
                float t = zt[m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
                if (lane == 0) ctrl->ztp[lw][m] = t;
            }
            if (lt == 0 && stamps) { stamps[5] = globaltimer_ns(); stamps[21] = (unsigned long long)clock64(); }
            named_bar_sync(3, LR_THREADS);
            if (p.trigger == 2 && lt == 0) griddep_launch_dependents();

            // ---- expansion: items (rank word w, column): sum of z over the ranks whose U bit is set ----
            float* corrp = zs + ROWS * p.Rpad;                                 // [ROWS][Rw][Rt]
            const int nit = has_rows ? p.Rw * Rt : 0;
            if (p.lut) {
                // By table: for every group of four ranks the 16 sums of its z values over the subsets of the group
                // (one thread per group: eleven adds), then a column's word is eight look-ups by nibble instead of 32
                // adds under predicates. A table line is 16 consecutive floats, so the lanes of a warp (columns of one
                // word, all nibbles) never collide on a bank.
                float* tab = corrp + ROWS * p.Rw * Rt;                         // [ROWS * Rpad / 4][16]
                const int ngr = has_rows ? ROWS * (p.Rpad >> 2) : 0;
#pragma unroll 1
                for (int gi = lt; gi < ngr; gi += LR_THREADS) {
                    const float4 z4 = *reinterpret_cast<const float4*>(zs + 4 * gi);
                    float4* t = reinterpret_cast<float4*>(tab + 16 * gi);
                    const float s01 = z4.x + z4.y, s02 = z4.x + z4.z, s12 = z4.y + z4.z, s012 = s01 + z4.z;
                    t[0] = make_float4(0.f, z4.x, z4.y, s01);
                    t[1] = make_float4(z4.z, s02, s12, s012);
                    t[2] = make_float4(z4.w, z4.x + z4.w, z4.y + z4.w, s01 + z4.w);
                    t[3] = make_float4(z4.z + z4.w, s02 + z4.w, s12 + z4.w, s012 + z4.w);
                }
                named_bar_sync(3, LR_THREADS);
#pragma unroll 1
                for (int id = lt; id < nit; id += LR_THREADS) {
                    const int w = id / Rt, col = id - w * Rt;
                    const uint32_t uw = us[id];
#pragma unroll
                    for (int m = 0; m < ROWS; ++m) {
                        const float* t = tab + (size_t)((m * p.Rw + w) * 8) * 16;
                        float c0 = 0.f, c1 = 0.f;
#pragma unroll
                        for (int i = 0; i < 8; i += 2) {
                            c0 += t[16 * i + ((uw >> (4 * i)) & 15u)];
                            c1 += t[16 * (i + 1) + ((uw >> (4 * i + 4)) & 15u)];
                        }
                        corrp[(m * p.Rw + w) * Rt + col] = c0 + c1;
                    }
                }
            } else if constexpr (ROWS <= 2) {
                expand_padd<ROWS>(zs, corrp, us, nit, Rt, p.Rw, p.Rpad, lt);
            } else {
                expand_padd4(zs, corrp, us, nit, Rt, p.Rw, p.Rpad, lt);
            }
            if (lt == 0 && stamps) { stamps[6] = globaltimer_ns(); stamps[22] = (unsigned long long)clock64(); }
        }

        // The low-rank term of this thread's output, summed in fixed order while the MMAs are still running.
        float lowrank = 0.f;
        if (p.R > 0) {
            named_bar_sync(3, LR_THREADS);                                      // the expansion's partial sums are complete
            if (has_rows && lt < ROWS * Rt) {
                const int m = lt / Rt, r = lt - m * Rt;
                const float* corrp = reinterpret_cast<const float*>(work) + ROWS * p.Rpad;
                float cs = 0.f, zt = 0.f;
                for (int w = 0; w < p.Rw; ++w) cs += corrp[(m * p.Rw + w) * Rt + r];
#pragma unroll
                for (int g = 0; g < LR_WARPS; ++g) zt += ctrl->ztp[g][m];
                lowrank = 2.f * cs - zt;
            }
        }

        // ---- accumulators: D[g' M + m, g Rt + r]; operand rows 0 .. kg M - 1 are TMEM lanes 0..15, which the two low-rank
        // warps 0 and 8 may read. They copy those lanes as they are to shared memory, half of the columns each; the
        // diagonal blocks g = g' are picked when the outputs are summed. ----
        if (has_rows && (warp == 0 || warp == FIRST_Z_WARP)) {
            if (!swait(smem_u32(&ctrl->acc_full), 0, ctrl, p, ST_ACC_FULL, warp)) good = false;
            tc_fence_after_sync();
            if (lt == 0 && stamps) { stamps[7] = globaltimer_ns(); stamps[23] = (unsigned long long)clock64(); }
            const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);
            const bool active = lane < kg * ROWS;
            const int half = (p.nbp + 63) / 64 * 32;                        // columns of the first warp (a multiple of 32)
            const int c_lo = warp == 0 ? 0 : half, c_hi = warp == 0 ? (half < p.nbp ? half : p.nbp) : p.nbp;
#pragma unroll 1
            for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
                float d[32];
                tmem_ld_x16(tmem + (uint32_t)c0, d);
                tmem_ld_x16(tmem + (uint32_t)c0 + 16, d + 16);
                tc_wait_ld();
                if (active) {
                    float4* dst = reinterpret_cast<float4*>(accp + lane * p.nbp + c0);      // (nbp and c0 are multiples of 16)
                    const int nv = (p.nbp - c0) < 32 ? (p.nbp - c0) >> 2 : 8;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (i < nv) dst[i] = make_float4(d[4 * i], d[4 * i + 1], d[4 * i + 2], d[4 * i + 3]);
                }
            }
            tc_fence_before_sync();
        }
        named_bar_sync(3, LR_THREADS);
        if (lt < ROWS * Rt) {
            const int m = lt / Rt, r = lt - m * Rt;
            const int n = cta * Rt + r;
            if (has_rows && m < p.M && n < p.N && good && ctrl->abort == 0) {
                float a = 0.f;
                for (int g = 0; g < kg; ++g) a += accp[(g * ROWS + m) * p.nbp + g * Rt + r];
                float o = alpha_r * a + lowrank;
                if (p.C) o += __bfloat162float(p.C[(size_t)m * p.N + n]);
                if (p.mode & 0x400) reinterpret_cast<float*>(p.Y)[(size_t)m * p.N + n] = o;
                else reinterpret_cast<__nv_bfloat16*>(p.Y)[(size_t)m * p.N + n] = __float2bfloat16(o);
            }
        }
        if (lt == 0 && stamps) { stamps[8] = globaltimer_ns(); stamps[24] = (unsigned long long)clock64(); }
        if (p.trigger >= 1 && lt == 0) griddep_launch_dependents();      // (at the latest here; a second call is harmless)
    }

    // ---------------- common exit ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (ctrl->abort) {
        // give copies that may still be in flight time to land before the shared memory is released
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (tid == 0) {
        // this CTA's share of 2^20: the sum over the CTAs of a launch is exactly 2^20 whatever the grid size
        if (p.R > 0) {
            const uint32_t share = (uint32_t)((((unsigned long long)(cta + 1)) << 20) / (unsigned)p.G) -
                                   (uint32_t)((((unsigned long long)cta) << 20) / (unsigned)p.G);
            red_add_u32(p.z_counter + 8 + (cta & 7), share);
        }
        if (stamps) { stamps[9] = globaltimer_ns(); stamps[25] = (unsigned long long)clock64(); }
    }
    if (warp == MMA_WARP && has_rows) {
        tc_fence_after_sync();
        tmem_dealloc(*reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base), SLAB_TMEM_COLS);
    }
}

}  // namespace slabp
}  // namespace biloco
