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
// Warp roles: 0-3 z stage / expansion / epilogue; 4-7 feeders: lane 0 of each requests the weight and activation
// copies of every fourth unit, and the whole warp moves the scale factors of every unit from shared memory into its
// 32-lane TMEM quadrant; 8-11 second half of the z stage; 12 MMA issue; 13 refills.
// Bulk copies issued by one thread complete one after the other (about 0.4 us each for anything up to 16 KB,
// measured), copies issued by different warps overlap: several requesting warps are what lets one CTA pull its
// share of the weight stream at HBM speed.
constexpr int PRODUCERS = 4;
constexpr int FIRST_SF_WARP = 4;                 // 4 warps, one per 32-lane TMEM quadrant (warp id % 4)
constexpr int FIRST_Z_WARP = 8;                  // 4 warps that only take part in the z stage
constexpr int MMA_WARP = 12;
constexpr int REFILL_WARP = 13;                 // re-requests stages as they come free (lanes 0..PRODUCERS-1)
constexpr int NUM_THREADS = (REFILL_WARP + 1) * 32;
static_assert(FIRST_SF_WARP % 4 == 0, "scale-factor warp q must own TMEM quadrant q");
constexpr int TMEM_COLS = 256;
constexpr int ACC_COL_STRIDE = 32;               // accumulator buffer b starts at column 32*b
constexpr int SF_SETS = 4;                       // scale-factor column sets, used round-robin by consecutive units
constexpr int SFA_COL = 64;                      // set q: 16 columns (4 MMAs x 4) at SFA_COL + 32*q
constexpr int LR_D_COL = 192;                    // the tensor-core expansion's accumulators, 32 columns per segment parity
constexpr int SFB_COL = 80;                      // set q: 16 columns at SFB_COL + 32*q
static_assert(SFA_COL + 32 * SF_SETS <= LR_D_COL && LR_D_COL + 64 <= TMEM_COLS, "scale-factor sets exceed the TMEM allocation");
constexpr int CTRL_BYTES = 3072;
constexpr int SMEM_BUDGET = 227 * 1024;
constexpr uint64_t WAIT_BUDGET_NS = 200ull * 1000 * 1000;   // 200 ms per wait

// CUDA-core work area in shared memory. During the z stage it holds one pass of one bf16 activation row (XT_BYTES,
// 16-byte chunks transposed so that a warp reads consecutive chunks) followed by the sign words of the ranks the CTA
// computes (vt_bytes, chosen by the host: at least VT_MIN_BYTES); afterwards the same bytes hold the z values being
// expanded and, in cluster mode, the partial sums of the other CTAs of the cluster.
constexpr int XT_BYTES = 16384;
constexpr int XK = XT_BYTES / 2;                 // k per pass of the z stage
constexpr int VT_MIN_BYTES = 8192;
constexpr int VT_MAX_BYTES = 49152;
constexpr int WORK_BYTES = XT_BYTES + VT_MIN_BYTES;       // 24 KB: the smallest work area
// Tensor-core expansion (from LR_TC_MIN_ROWS rows): two 16 KB buffers for the +-1.0 bf16 image of 64 ranks of the tile's U signs
// (128 columns x 128 bytes, 128-byte swizzle), per buffer the bf16 high and low parts of the matching z values
// (MMA_N rows x 128 bytes each) and a 256-entry table byte -> eight bf16 signs.
// Measured at K = N = 5120 (us per call, CUDA-core / tensor-core expansion, r = 512): M=4 16.4 / 17.9, M=8 21.6 / 21.3,
// M=16 30.5 / 27.5, M=32 70.3 / 45.5; r = 1024, M=32: 126.5 / 80.2.
constexpr int LR_TC_MIN_ROWS = 16;
constexpr int LR_UA_BYTES = 16384;
constexpr int LR_LUT_BYTES = 4096;
__host__ __device__ constexpr int lr_bytes(int mma_n) { return 2 * LR_UA_BYTES + 4 * mma_n * 128 + LR_LUT_BYTES; }
constexpr int ZR_MAX = 64;                       // ranks per chunk of the z stage (partial sums per warp in Ctrl)
constexpr int ZS_FIRST = 4;                      // U words per segment fetched ahead of the dependency wait
// z is staged for the expansion in chunks of zs_words(ROWS) rank words (32 ranks each): ROWS x (32*words + 4) floats
// (+4: rows start in different banks), at most ZS_BYTES.
__host__ __device__ constexpr int zs_words(int rows) { return rows <= 8 ? 8 : 4; }
__host__ __device__ constexpr int zs_stride(int rows) { return zs_words(rows) * 32 + 4; }
constexpr int ZS_BYTES_SMALL = 8320;             // rows <= 8:  8 * 260 * 4
constexpr int STAMP_WORDS = 16;                  // uint64 time stamps per CTA when debug stamps are on
static_assert(32 * zs_stride(32) * 4 <= WORK_BYTES && 16 * zs_stride(16) * 4 <= WORK_BYTES, "z staging must fit in the work area");
static_assert(8 * zs_stride(8) * 4 <= ZS_BYTES_SMALL && 4 * zs_stride(4) * 4 <= ZS_BYTES_SMALL, "z staging (rows <= 8)");
constexpr int RED_OFF = ZS_BYTES_SMALL + 128;      // cluster mode (rows <= 8): partial sums of the peers start here,
constexpr int RED_BYTES = WORK_BYTES - RED_OFF;    // after the z staging rows, [peer][row][128] floats

// Launches of one or two rows: two CTAs fit on one SM (registers, shared memory and TMEM are all sized for it), so that
// with programmatic dependent launch the next kernel of the stream is resident beside this one and has its first
// weights in shared memory before this one has finished its dependent tail. More rows: one CTA per SM, deeper ring.
__host__ __device__ constexpr int ctas_per_sm(int rows) { return rows <= 2 ? 2 : 1; }
constexpr int CORESIDENT_SMEM = 113 * 1024;      // 2 x (113 KB + 1 KB reserved) = 228 KB, the SM's shared memory
template <int MMA_N>
struct Cfg {
    static constexpr int A_TILE_BYTES = MMA_N * KT_BYTES;
    static constexpr int STAGE_BYTES = W_TILE_BYTES + A_TILE_BYTES + 2 * SF_TILE_BYTES;
    static constexpr int fixed_bytes(int vt_bytes) { return 1024 + CTRL_BYTES + XT_BYTES + vt_bytes; }      // (+ lr_bytes, see the launcher)
    static constexpr int stages_alone(int vt_bytes) { return (SMEM_BUDGET - fixed_bytes(vt_bytes)) / STAGE_BYTES; }
    static constexpr int stages_shared(int vt_bytes) { return (CORESIDENT_SMEM - fixed_bytes(vt_bytes)) / STAGE_BYTES; }
    static constexpr int smem_bytes(int ring, int vt_bytes) { return ring * STAGE_BYTES + fixed_bytes(vt_bytes); }
    static constexpr int STAGES = stages_alone(VT_MIN_BYTES);          // the deepest ring
    static_assert(STAGE_BYTES % 1024 == 0, "stage bases must stay 1024-byte aligned for the 128-byte swizzle");
    static_assert(STAGES >= 4 && STAGES <= 16, "stage count out of range");
    static_assert(stages_alone(VT_MAX_BYTES + lr_bytes(MMA_N)) >= SF_SETS, "the ring must not be shorter than the scale-factor sets");
    static_assert(stages_shared(VT_MIN_BYTES) >= SF_SETS || MMA_N != 8, "the ring must not be shorter than the scale-factor sets");
};

struct FusedParams {
    const uint8_t* W_tiled;   // unit-contiguous weights (see biloco_b200_tile_weights) or null: row-major codes via TMA
    const uint8_t* W_sf;
    const uint8_t* A_sf;
    const uint8_t* A_rec;     // per k-tile [activation tile as it sits in a stage | its four scale atoms] (one copy per unit), or null
    const float* alpha;
    const __nv_bfloat16* X;
    const uint8_t* Vp;
    const int32_t* Ucol;
    const __nv_bfloat16* S;
    const __nv_bfloat16* C;
    __nv_bfloat16* Y;
    int32_t* status;
    uint32_t* z_counter;      // [0] number of launches completed on this scratch (gives the z validity bit),
                              // [1] CTAs of the current launch that have finished
    uint32_t* tile_cnt;
    float* zbuf;
    float* partials;
    uint32_t* ztc_cnt;        // tensor-core z launch (ztc_kernel.cuh): arrival counters per rank block; nullptr = not available
    size_t part_bytes;        // bytes of `partials` (the z launch keeps its partial sums there until the fused launch starts)
    // Row-parallel use (peer_reduce.cu): the thread that stores an fp32 output also stores {value, call number} into this
    // rank's slot of every peer's receive buffer, so the all-reduce's transfer starts with the tile's epilogue instead of
    // with a later launch. ar_world <= 1: off.
    uint2* const* ar_recv;    // [ar_world] device table: rank q's receive buffer as mapped here
    const uint32_t* ar_counter;   // the group's call counter (bits 20..: completed calls), advanced by the gather launch
    int ar_world, ar_rank, ar_slot;
    int M, N, K, R, Rw, Rpad;
    // Column groups: several linears that read the same activation (q/k/v, gate/up) stacked along N in one launch. Group
    // g owns the tiles [gtile[g-1], gtile[g]) (gtile[-1] = 0, unused entries INT_MAX), the ranks [g*Rg, (g+1)*Rg) of V, S
    // and z, and the decode scale alpha[g]; a column's U words cover its own group's Rg ranks (Rw words). R is the total
    // (what the z stage computes); a single linear is one group with Rg = R.
    int ngroups, Rg;
    int gtile[3];
    int ntile, nkt, G, max_slots;
    int ring;                 // pipeline stages (<= Cfg::STAGES); the shared-memory layout follows it
    int trigger;              // where the CTA lets the next kernel of the stream start: 0 after set-up, 4 after its own
                              // dependency wait, 3 once its activation row has landed, 1 after its z stage, 2 after
                              // its first expansion (an exiting CTA counts as having done so)
    int vt_bytes;             // shared memory for the z stage's sign words (VT_MIN_BYTES .. VT_MAX_BYTES)
    int lr_tc;                // expansion on the tensor cores (the launcher has added lr_bytes(MMA_N) behind the sign words)
    int nsl;                  // z stage: rank slices per activation row; work item (row m, slice s) = m*nsl + s goes to
                              // CTA (m*nsl + s) % G
    int cluster;              // > 1: a tile belongs to a cluster of this many CTAs (partial sums through DSMEM)
    uint32_t epoch;
    int mode;
    unsigned long long* stamps;   // debug: STAMP_WORDS %globaltimer values per CTA, or null
};

__device__ __forceinline__ int tile_group(const FusedParams& p, int t) {
    return (t >= p.gtile[0] ? 1 : 0) + (t >= p.gtile[1] ? 1 : 0) + (t >= p.gtile[2] ? 1 : 0);
}

struct Ctrl {   // lives in shared memory after the stages
    uint64_t full[16];
    uint64_t empty[16];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t sf_full[SF_SETS];    // scale factors of a unit are in TMEM set q (128 arrivals)
    uint64_t sf_empty[SF_SETS];   // the MMAs that read set q have completed (tcgen05.commit)
    float zred[8][ZR_MAX];        // z stage: per-warp partial sums of sum_{sign = +1} x, per rank of the chunk
    float zall[8];                // z stage: per-warp partial sums of sum x
    uint64_t red_bar;             // cluster mode, finisher CTA: the other CTAs' partial sums are in this CTA's smem
    uint64_t x_bar;               // z stage: the activation row has landed (bulk copy)
    uint64_t lr_free[2];          // tensor-core expansion: the MMAs that read operand buffer b have completed
    uint64_t lr_done;             // tensor-core expansion: the segment's last MMA has completed
    uint64_t red_free;            // cluster mode, other CTAs: the finisher's z stage is over, its work area may be written
    uint32_t tmem_base;
    volatile int abort;
    uint32_t ar_seq;          // number of the all-reduce call this launch's outputs belong to
};
static_assert(sizeof(Ctrl) <= CTRL_BYTES, "control block too large");

enum : int {   // status codes of waits that ran out
    ST_EMPTY = 101, ST_FULL = 102, ST_ACC_EMPTY = 103, ST_ACC_FULL = 104, ST_Z = 105, ST_TILE = 106, ST_SF_FULL = 107,
    ST_SF_EMPTY = 108, ST_CLUSTER = 109, ST_ACT = 110,
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
        if ((it & 3u) == 3u) {          // (a try may have been parked for up to a millisecond)
            if (ctrl->abort) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_BUDGET_NS) { fail(ctrl, status, epoch, code, role); return false; }
        }
    }
}

// Bounded mbarrier wait by polling (mbarrier.test_wait): for the lanes of the refill warp, which wait on different barriers.
__device__ __noinline__ bool poll_bar(uint32_t bar, uint32_t parity, Ctrl* ctrl, int32_t* status, uint32_t epoch, int code, int role) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_test_wait(bar, parity)) return true;
        __nanosleep(32);
        if ((it & 63u) == 63u) {
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
        if ((it & 3u) == 3u) {
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
