// Configuration, parameter block, shared-memory control block and bounded-wait helpers of the fused linear.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"
#include "schedule.h"

namespace biloco {

constexpr int TILE_N = 128;                      // weight rows per tile = MMA M
constexpr int KT = 256;                          // K elements per k-tile
constexpr int KT_BYTES = KT / 2;                 // 128 B of codes per row = one 128-byte swizzle row
constexpr int W_TILE_BYTES = TILE_N * KT_BYTES;  // 16384
constexpr int SF_TILE_BYTES = 4 * 512;           // four 128x4 atoms
constexpr int EPI_THREADS = 128;
// Warp roles: 0-3 z stage / expansion / epilogue, 4-7 weight producers, 8-11 activation producers, 12-15 scale-factor
// movers (shared memory -> TMEM), 16 MMA issue.
// Bulk copies issued by one thread complete one after the other (about 0.4 us each for anything up to 16 KB,
// measured), copies issued by different warps overlap: several producer warps are what lets one CTA pull its
// share of the weight stream at HBM speed.
constexpr int W_PRODUCERS = 4;
constexpr int A_PRODUCERS = 4;
constexpr int FIRST_W_WARP = 4;
constexpr int FIRST_A_WARP = FIRST_W_WARP + W_PRODUCERS;
constexpr int FIRST_SF_WARP = FIRST_A_WARP + A_PRODUCERS;   // 4 warps, one per 32-lane TMEM quadrant (warp id % 4)
constexpr int MMA_WARP = FIRST_SF_WARP + 4;
constexpr int NUM_THREADS = (MMA_WARP + 1) * 32;
static_assert(FIRST_SF_WARP % 4 == 0, "scale-factor warp q must own TMEM quadrant q");
constexpr int TMEM_COLS = 256;
constexpr int ACC_COL_STRIDE = 32;               // accumulator buffer b starts at column 32*b
constexpr int SF_SETS = 4;                       // scale-factor column sets, used round-robin by consecutive units
constexpr int SFA_COL = 64;                      // set q: 16 columns (4 MMAs x 4) at SFA_COL + 32*q
constexpr int SFB_COL = 80;                      // set q: 16 columns at SFB_COL + 32*q
static_assert(SFA_COL + 32 * SF_SETS <= TMEM_COLS, "scale-factor sets exceed the TMEM allocation");
constexpr int CTRL_BYTES = 1024;
constexpr int SMEM_BUDGET = 227 * 1024;
constexpr uint64_t WAIT_BUDGET_NS = 200ull * 1000 * 1000;   // 200 ms per wait

// CUDA-core work area in shared memory. During the z stage it holds a tile of the bf16 activation (XT_BYTES,
// 16-byte chunks transposed so that a warp reads consecutive chunks) and the sign words of up to VT_RANKS ranks;
// afterwards the same bytes hold the z values being expanded (ROWS x ZS_STRIDE floats).
constexpr int XT_BYTES = 16384;
constexpr int VT_RANKS = 8;
constexpr int VT_BYTES = VT_RANKS * (XT_BYTES / 2 / 8);   // one bit per k of the widest activation tile (1 row)
constexpr int WORK_BYTES = XT_BYTES + VT_BYTES;           // 24 KB
constexpr int ZS_WORDS = 4;                      // rank words (32 ranks each) of z staged at a time
constexpr int ZS_STRIDE = ZS_WORDS * 32 + 4;     // floats per staged row (+4: rows start in different banks)
constexpr int STAMP_WORDS = 16;                  // uint64 time stamps per CTA when debug stamps are on
static_assert(32 * ZS_STRIDE * 4 <= WORK_BYTES, "z staging must fit in the work area");
constexpr int RED_OFF = 8 * ZS_STRIDE * 4 + 256;   // cluster mode (rows <= 8): partial sums of the peers start here,
constexpr int RED_BYTES = WORK_BYTES - RED_OFF;    // after the z staging rows, [peer][row][128] floats

template <int MMA_N>
struct Cfg {
    static constexpr int A_TILE_BYTES = MMA_N * KT_BYTES;
    static constexpr int STAGE_BYTES = W_TILE_BYTES + A_TILE_BYTES + 2 * SF_TILE_BYTES;
    static constexpr int STAGES = (SMEM_BUDGET - 1024 - CTRL_BYTES - WORK_BYTES) / STAGE_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + CTRL_BYTES + WORK_BYTES;
    static_assert(STAGE_BYTES % 1024 == 0, "stage bases must stay 1024-byte aligned for the 128-byte swizzle");
    static_assert(STAGES >= 4 && STAGES <= 16, "stage count out of range");
};

struct FusedParams {
    const uint8_t* W_tiled;   // unit-contiguous weights (see biloco_b200_tile_weights) or null: row-major codes via TMA
    const uint8_t* W_sf;
    const uint8_t* A_sf;
    const float* alpha;
    const __nv_bfloat16* X;
    const uint8_t* Vp;
    const int32_t* Ucol;
    const __nv_bfloat16* S;
    const __nv_bfloat16* C;
    __nv_bfloat16* Y;
    int32_t* status;
    uint32_t* z_counter;      // [0] arrivals of z producers, [1] consumers that have seen it complete
    uint32_t* tile_cnt;
    float* zbuf;
    float* partials;
    int M, N, K, R, Rw, Rpad;
    int ntile, nkt, G, max_slots;
    int z_consumers;          // CTAs that wait for z in this launch (all of them, or only those that finish a tile)
    int ring;                 // pipeline stages in use (<= Cfg::STAGES). Every byte a CTA requests early is delivered
                              // ahead of its later small reads (x, z, partial sums) on the SM's inbound path, so a
                              // deep ring buys nothing for a short stream and delays the latency-critical reads
    int cluster;              // > 1: a tile belongs to a cluster of this many CTAs (partial sums through DSMEM)
    uint32_t epoch;
    int mode;
    unsigned long long* stamps;   // debug: STAMP_WORDS %globaltimer values per CTA, or null
};

struct Ctrl {   // lives in shared memory after the stages
    uint64_t full[16];
    uint64_t empty[16];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t sf_full[SF_SETS];    // scale factors of a unit are in TMEM set q (128 arrivals)
    uint64_t sf_empty[SF_SETS];   // the MMAs that read set q have completed (tcgen05.commit)
    float zred[8][VT_RANKS];      // z stage: per-warp partial sums
    uint64_t red_bar;             // cluster mode, finisher CTA: the other CTAs' partial sums are in this CTA's smem
    uint32_t tmem_base;
    volatile int abort;
};
static_assert(sizeof(Ctrl) <= CTRL_BYTES, "control block too large");

enum : int {   // status codes of waits that ran out
    ST_EMPTY = 101, ST_FULL = 102, ST_ACC_EMPTY = 103, ST_ACC_FULL = 104, ST_Z = 105, ST_TILE = 106, ST_SF_FULL = 107,
    ST_SF_EMPTY = 108, ST_CLUSTER = 109,
};

// The wait helpers are deliberately not inlined: the kernel's machine code is executed once, cold, per CTA, and
// every kilobyte of it is an instruction fetch queued behind the weight stream.

// Record the first failure and raise the CTA-wide abort flag.
__device__ __noinline__ void fail(Ctrl* ctrl, int32_t* status, uint32_t epoch, int code, int role) {
    ctrl->abort = 1;
    if (atomicCAS(status, 0, code) == 0) {
        status[1] = (int)blockIdx.x;
        status[2] = (int)epoch;
        status[3] = role;
    }
}

// Bounded mbarrier wait. Returns false when the budget ran out or another role aborted.
__device__ __noinline__ bool wait_bar(uint32_t bar, uint32_t parity, Ctrl* ctrl, int32_t* status, uint32_t epoch, int code,
                                      int role) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 31u) == 31u) {
            if (ctrl->abort) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_BUDGET_NS) { fail(ctrl, status, epoch, code, role); return false; }
        }
    }
}

// Bounded wait until *ctr >= target (acquire). One thread calls this.
__device__ __noinline__ bool wait_counter(const uint32_t* ctr, uint32_t target, Ctrl* ctrl, int32_t* status, uint32_t epoch,
                                          int code) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if ((int32_t)(ld_acquire_u32(ctr) - target) >= 0) return true;
        if ((it & 31u) == 31u) {
            if (ctrl->abort) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_BUDGET_NS) { fail(ctrl, status, epoch, code, 0); return false; }
        }
    }
}

__device__ __noinline__ bool wait_bar_cluster(uint32_t bar, uint32_t parity, Ctrl* ctrl, int32_t* status, uint32_t epoch, int code) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((it & 31u) == 31u) {
            if (ctrl->abort) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_BUDGET_NS) { fail(ctrl, status, epoch, code, 0); return false; }
        }
    }
}

// Barrier over the 128 epilogue threads followed by a uniform look at the abort flag.
__device__ __forceinline__ bool epi_sync_ok(Ctrl* ctrl) {
    named_bar_sync(1, EPI_THREADS);
    return ctrl->abort == 0;
}

__device__ __forceinline__ float signed_by_bit(float x, uint32_t word, int j) {
    return __uint_as_float(__float_as_uint(x) ^ (((~word >> j) & 1u) << 31));
}

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// One segment = a maximal run of units inside one tile. SegWalk yields the segments of the unit range [u0, u1) in
// PROCESSING order: a range that ends inside a tile has a "head" segment whose tile is finished by a later CTA, and
// it goes first, so that its partial sum is published before this CTA starts waiting for the partials of the tile
// it finishes itself. (In natural order CTA c would publish for tile t+1 only after finishing tile t, which waits
// for CTA c-1, which waits for CTA c-2, ...: a chain through every CTA of the grid.)
struct SegWalk {
    int u0, head, u1, u;
    int nkt;
    bool in_head;
    __device__ __forceinline__ SegWalk(int a, int b, int nkt_) : u0(a), u1(b), nkt(nkt_) {
        const int rem = (int)((unsigned)b % (unsigned)nkt_);
        head = (rem != 0 && b - rem > a) ? (b - rem) : b;   // == u1: no separate head segment
        in_head = head < b;
        u = in_head ? head : a;
    }
    __device__ __forceinline__ bool done() const { return !in_head && u >= head; }
    // current segment: first unit and number of units
    __device__ __forceinline__ int first() const { return u; }
    __device__ __forceinline__ int count() const {
        const int left = (in_head ? u1 : head) - u;
        const int in_tile = nkt - (int)((unsigned)u % (unsigned)nkt);
        return in_tile < left ? in_tile : left;
    }
    __device__ __forceinline__ void next() {
        if (in_head) { in_head = false; u = u0; }
        else u += count();
    }
};

// What a CTA does with one segment: the tile, its place among the tile's contributors, whether it finishes the tile,
// and the rank words [w0, w1) of the low-rank term it expands. owner_mode: the finisher expands all ranks and the
// other contributors none (their partial sums then do not wait for z); otherwise every contributor takes a share.
struct SegInfo {
    int t, nc, slot, w0, w1;
    bool complete, finisher;
};
__device__ __forceinline__ SegInfo seg_info(const FusedParams& p, int T, int cta, int u, int cnt, bool owner_mode) {
    SegInfo s;
    s.t = (int)((unsigned)u / (unsigned)p.nkt);
    s.complete = (cnt == p.nkt);
    if (p.cluster > 1) {
        s.nc = p.cluster;
        s.slot = cta - s.t * p.cluster;
        s.finisher = s.slot == p.cluster - 1;
    } else {
        const int c_first = sched_cta_of_unit(s.t * p.nkt, T, p.G);
        const int c_last = sched_cta_of_unit(s.t * p.nkt + p.nkt - 1, T, p.G);
        s.nc = c_last - c_first + 1;
        s.slot = cta - c_first;
        s.finisher = s.complete || cta == c_last;
    }
    if (owner_mode) {
        s.w0 = 0;
        s.w1 = s.finisher ? p.Rw : 0;
    } else {
        s.w0 = s.slot * p.Rw / s.nc;
        s.w1 = (s.slot + 1) * p.Rw / s.nc;
    }
    return s;
}

}  // namespace biloco
