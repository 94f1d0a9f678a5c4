// Fused BiLoCo decode linear for sm_100a, one launch:
//
//     Y[m,n] = bf16( alpha * sum_k A[m,k] W[n,k]  +  sum_i z[m,i] sign(U[i,n])  (+ C[m,n]) ),   z = S .* (X sign(V)^T)
//
// Decode shape: M <= 32 activation rows against an N x K weight, so the kernel is a weight stream. Design:
//
//  * Operands are swapped for the tensor core: a 128-row slab of W is the MMA "A" operand (M = 128), the
//    activation rows are the MMA "B" operand (N = 8/16/32). The accumulator D[128, MMA_N] lives in TMEM with
//    TMEM lane = weight row (output column n) and TMEM column = activation row m. No 128-row zero padding of
//    the activation and only M output rows are written.
//  * Work unit = (128-row tile t, 256-wide k-tile kt): 16 KB of E2M1 codes + 2 KB of E4M3 scales. The
//    T = ntile * nkt units are split evenly over all CTAs (one per SM) as contiguous ranges in (t, kt)
//    order ("stream-K"), so every SM streams the same number of weight bytes whatever N is.
//  * Warp roles (192 threads): warps 0-3 = z stage, U expansion and epilogue (thread = TMEM lane = weight row);
//    warp 4 = TMA producer; warp 5 = TMEM allocation + MMA issue.
//  * Per stage: W codes by a 2-D TMA tile (128 rows x 128 B, 128-byte swizzle), activation codes by a 2-D TMA
//    tile (MMA_N rows x 128 B), both scale tiles by untiled bulk copies (the 128x4 atom layout is already what
//    tcgen05.cp 32x128b.warpx4 wants: 4 atoms of 512 B per k-tile). Four tcgen05.mma kind::mxf4nvf4
//    (K = 64 each) per stage.
//  * A tile whose k-range is shared by several CTAs is finished by the CTA that holds its last k-tile: the
//    others store fp32 partials (alpha*acc + their slice of the low-rank term) to scratch and bump the tile's
//    counter; the finisher adds them in slot order (deterministic), rounds and stores.
//  * Low-rank term: at entry every CTA computes a slice of the ranks of z (all M rows) on CUDA cores from the
//    bit-packed V and publishes it in scratch; an arrival counter (mode 2) tells the consumers that z is
//    complete. Counters return to zero inside the launch (the finisher of a tile clears its counter, the last
//    CTA past the z wait clears the z words), so launches on one scratch need no clearing in between and a
//    captured CUDA graph can be replayed; launches that share a scratch must not overlap. Each contributor of a tile expands z through the packed U signs for its share of the rank words
//    while its weight loads are in flight, and adds the result to the accumulators read back from TMEM.
//  * Every wait (mbarrier, counter) is bounded by a %globaltimer budget; a wait that runs out records a code in
//    the status words of the scratch, raises a CTA-wide abort flag, and the CTA leaves through the common exit
//    (TMEM freed) instead of hanging.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

#include "../../include/biloco_b200.h"
#include "ptx.cuh"
#include "schedule.h"

namespace biloco {

constexpr int TILE_N = 128;                      // weight rows per tile = MMA M
constexpr int KT = 256;                          // K elements per k-tile
constexpr int KT_BYTES = KT / 2;                 // 128 B of codes per row = one 128-byte swizzle row
constexpr int W_TILE_BYTES = TILE_N * KT_BYTES;  // 16384
constexpr int SF_TILE_BYTES = 4 * 512;           // four 128x4 atoms
constexpr int EPI_THREADS = 128;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 128;
constexpr int ACC_COL_STRIDE = 32;               // accumulator buffer b starts at column 32*b
constexpr int SFA_COL = 64;                      // 16 columns: 4 MMAs x 4
constexpr int SFB_COL = 80;                      // 16 columns
constexpr int CTRL_BYTES = 1024;
constexpr int SMEM_BUDGET = 227 * 1024;
constexpr uint64_t WAIT_BUDGET_NS = 200ull * 1000 * 1000;   // 200 ms per wait
constexpr int Z_CHUNK = 8;                       // ranks processed together in the z stage

template <int MMA_N>
struct Cfg {
    static constexpr int A_TILE_BYTES = MMA_N * KT_BYTES;
    static constexpr int STAGE_BYTES = W_TILE_BYTES + A_TILE_BYTES + 2 * SF_TILE_BYTES;
    static constexpr int STAGES = (SMEM_BUDGET - 1024 - CTRL_BYTES) / STAGE_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + CTRL_BYTES;
    static_assert(STAGE_BYTES % 1024 == 0, "stage bases must stay 1024-byte aligned for the 128-byte swizzle");
    static_assert(STAGES >= 4, "too few stages");
};

struct FusedParams {
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
    uint32_t epoch;
    int mode;
};

struct Ctrl {   // lives in shared memory after the stages
    uint64_t full[16];
    uint64_t empty[16];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    volatile int abort;
    float red[4][Z_CHUNK];
};
static_assert(sizeof(Ctrl) <= CTRL_BYTES, "control block too large");

// Record the first failure and raise the CTA-wide abort flag.
__device__ __forceinline__ void fail(Ctrl* ctrl, const FusedParams& p, int code, int role) {
    ctrl->abort = 1;
    if (atomicCAS(p.status, 0, code) == 0) {
        p.status[1] = (int)blockIdx.x;
        p.status[2] = (int)p.epoch;
        p.status[3] = role;
    }
}

// Bounded mbarrier wait. Returns false when the budget ran out or another role aborted.
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, Ctrl* ctrl, const FusedParams& p, int code, int role) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 31u) == 31u) {
            if (ctrl->abort) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_BUDGET_NS) { fail(ctrl, p, code, role); return false; }
        }
    }
}

// Bounded wait until *ctr >= target (acquire). One thread calls this.
__device__ __forceinline__ bool wait_counter(const uint32_t* ctr, uint32_t target, Ctrl* ctrl, const FusedParams& p, int code) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if ((int32_t)(ld_acquire_u32(ctr) - target) >= 0) return true;
        if ((it & 31u) == 31u) {
            if (ctrl->abort) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_BUDGET_NS) { fail(ctrl, p, code, 0); return false; }
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

template <int MMA_N>
__device__ __forceinline__ void tmem_ld_acc(uint32_t taddr, float* v) {
    if constexpr (MMA_N == 8) {
        tmem_ld_x8(taddr, v);
    } else if constexpr (MMA_N == 16) {
        tmem_ld_x16(taddr, v);
    } else {
        tmem_ld_x16(taddr, v);
        tmem_ld_x16(taddr + 16, v + 16);
    }
}

// Segments (maximal runs of units inside one tile) of the unit range [u0, u1), in PROCESSING order.
// A range that ends inside a tile has a "head" segment whose tile is finished by a later CTA. It goes first:
// its partial sum is then published before this CTA starts waiting for the partials of the tile it finishes
// itself. (In natural order CTA c would publish for tile t+1 only after finishing tile t, which waits for CTA
// c-1, which waits for CTA c-2, ...: a chain through every CTA of the grid.)
// f(u_start, count) returns false to stop.
template <class F>
__device__ __forceinline__ void for_each_segment(long long u0, long long u1, int nkt, F&& f) {
    const long long rem = u1 % nkt;
    const long long head = (rem != 0 && u1 - rem > u0) ? (u1 - rem) : u1;   // == u1: no separate head segment
    if (head < u1 && !f(head, (int)(u1 - head))) return;
    for (long long u = u0; u < head;) {
        const long long left = head - u;
        const int in_tile = nkt - (int)(u % nkt);
        const int cnt = (int)(in_tile < left ? in_tile : left);
        if (!f(u, cnt)) return;
        u += cnt;
    }
}

enum : int {   // status codes of waits that ran out
    ST_EMPTY = 101, ST_FULL = 102, ST_ACC_EMPTY = 103, ST_ACC_FULL = 104, ST_Z = 105, ST_TILE = 106,
};

template <int MMA_N>
__global__ void __launch_bounds__(NUM_THREADS, 1)
fused_linear_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA, const FusedParams p) {
    using C = Cfg<MMA_N>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t stage0 = (raw + 1023u) & ~1023u;                 // shared-window address of stage 0
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem_raw + (stage0 - raw) + C::STAGES * C::STAGE_BYTES);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int cta = blockIdx.x;

    const long long T = (long long)p.ntile * p.nkt;
    const long long u0 = sched_first_unit(cta, T, p.G);
    const long long u1 = sched_first_unit(cta + 1, T, p.G);

    // ---------------- set-up ----------------
    if (tid == 128) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->full[s]), 1);
            mbar_init(smem_u32(&ctrl->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&ctrl->acc_full[b]), 1);
            mbar_init(smem_u32(&ctrl->acc_empty[b]), EPI_THREADS);
        }
        ctrl->abort = 0;
        fence_mbar_init();
        prefetch_tmap(&tmW);
        prefetch_tmap(&tmA);
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(&ctrl->tmem_base), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = ctrl->tmem_base;

    if (warp == 4) {
        // ================= TMA producer =================
        if (lane == 0) {
            int i = 0;
            for_each_segment(u0, u1, p.nkt, [&](long long us, int cnt) {
                for (long long u = us; u < us + cnt; ++u, ++i) {
                    const int s = i % C::STAGES;
                    const int use = i / C::STAGES;
                    if (use > 0 && !wait_bar(smem_u32(&ctrl->empty[s]), (use - 1) & 1, ctrl, p, ST_EMPTY, 4)) return false;
                    const int t = (int)(u / p.nkt);
                    const int kt = (int)(u % p.nkt);
                    const uint32_t sbase = stage0 + s * C::STAGE_BYTES;
                    const uint32_t bar = smem_u32(&ctrl->full[s]);
                    mbar_arrive_expect_tx(bar, C::STAGE_BYTES);
                    tma_load_2d(sbase, &tmW, kt * KT_BYTES, t * TILE_N, bar);
                    tma_load_2d(sbase + W_TILE_BYTES, &tmA, kt * KT_BYTES, 0, bar);
                    bulk_load(sbase + W_TILE_BYTES + C::A_TILE_BYTES,
                              p.W_sf + ((size_t)t * (p.K >> 6) + (size_t)kt * 4) * 512, SF_TILE_BYTES, bar);
                    bulk_load(sbase + W_TILE_BYTES + C::A_TILE_BYTES + SF_TILE_BYTES,
                              p.A_sf + (size_t)kt * 4 * 512, SF_TILE_BYTES, bar);
                }
                return true;
            });
        }
    } else if (warp == 5) {
        // ================= MMA issue =================
        constexpr uint32_t idesc = make_idesc_nvf4(TILE_N, MMA_N);
        int i = 0, seg = 0;
        for_each_segment(u0, u1, p.nkt, [&](long long, int cnt) {
            const int buf = seg & 1;
            if (seg >= 2 && !wait_bar(smem_u32(&ctrl->acc_empty[buf]), ((seg >> 1) - 1) & 1, ctrl, p, ST_ACC_EMPTY, 5)) return false;
            tc_fence_after_sync();
            for (int j = 0; j < cnt; ++j, ++i) {
                const int s = i % C::STAGES;
                if (!wait_bar(smem_u32(&ctrl->full[s]), (i / C::STAGES) & 1, ctrl, p, ST_FULL, 5)) return false;
                tc_fence_after_sync();
                if (lane == 0) {
                    const uint32_t sbase = stage0 + s * C::STAGE_BYTES;
                    const uint32_t wsf = sbase + W_TILE_BYTES + C::A_TILE_BYTES;
                    const uint32_t asf = wsf + SF_TILE_BYTES;
#pragma unroll
                    for (int a = 0; a < 4; ++a) {
                        tc_cp_32x128b_warpx4(tmem + SFA_COL + 4 * a, make_smem_desc(wsf + 512 * a, 128, 0));
                        tc_cp_32x128b_warpx4(tmem + SFB_COL + 4 * a, make_smem_desc(asf + 512 * a, 128, 0));
                    }
                    const uint64_t wdesc = make_smem_desc(sbase, 1024, 2);
                    const uint64_t adesc = make_smem_desc(sbase + W_TILE_BYTES, 1024, 2);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        // 64 K-elements = 32 B further along the swizzled row: +2 in the (address >> 4) field
                        tc_mma_nvf4(tmem + buf * ACC_COL_STRIDE, wdesc + 2 * k, adesc + 2 * k, idesc,
                                    tmem + SFA_COL + 4 * k, tmem + SFB_COL + 4 * k, (j > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&ctrl->empty[s]));
                    if (j == cnt - 1) tc_commit(smem_u32(&ctrl->acc_full[buf]));
                }
                __syncwarp();
            }
            ++seg;
            return true;
        });
    } else {
        // ================= z stage, expansion, epilogue (128 threads) =================
        const int Rpad = p.Rpad;
        float* zb = p.zbuf + (size_t)(p.epoch & 1u) * 32 * Rpad;
        if (p.R > 0) {
            const int i0 = (int)((long long)cta * p.R / p.G);
            const int i1 = (int)((long long)(cta + 1) * p.R / p.G);
            const int kbytes = p.K >> 3;
            for (int ic = i0; ic < i1; ic += Z_CHUNK) {
                const int nr = (i1 - ic) < Z_CHUNK ? (i1 - ic) : Z_CHUNK;
                for (int m = 0; m < p.M; ++m) {
                    float acc[Z_CHUNK];
#pragma unroll
                    for (int q = 0; q < Z_CHUNK; ++q) acc[q] = 0.f;
                    const __nv_bfloat16* xrow = p.X + (size_t)m * p.K;
                    for (int kb = tid; kb < kbytes; kb += EPI_THREADS) {
                        const uint4 xp = *reinterpret_cast<const uint4*>(xrow + kb * 8);
                        const uint32_t xw[4] = {xp.x, xp.y, xp.z, xp.w};
                        float xf[8];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            xf[2 * e] = __uint_as_float(xw[e] << 16);
                            xf[2 * e + 1] = __uint_as_float(xw[e] & 0xFFFF0000u);
                        }
#pragma unroll
                        for (int q = 0; q < Z_CHUNK; ++q) {
                            if (q < nr) {
                                const uint32_t vb = p.Vp[(size_t)(ic + q) * kbytes + kb];
#pragma unroll
                                for (int j = 0; j < 8; ++j) acc[q] += signed_by_bit(xf[j], vb, j);
                            }
                        }
                    }
#pragma unroll
                    for (int q = 0; q < Z_CHUNK; ++q) {
                        float v = acc[q];
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                        if (lane == 0) ctrl->red[warp][q] = v;
                    }
                    named_bar_sync(1, EPI_THREADS);
                    if (tid < nr) {
                        const float v = (ctrl->red[0][tid] + ctrl->red[1][tid]) + (ctrl->red[2][tid] + ctrl->red[3][tid]);
                        zb[(size_t)m * Rpad + ic + tid] = v * __bfloat162float(p.S[ic + tid]);
                    }
                    named_bar_sync(1, EPI_THREADS);
                }
            }
            __threadfence();
            named_bar_sync(1, EPI_THREADS);
            if (tid == 0) red_release_add_u32(p.z_counter, 1u);
        }

        bool z_ready = false;
        const float alpha = p.alpha[0];
        int seg = 0;
        for_each_segment(u0, u1, p.nkt, [&](long long u, int cnt) {
            const int t = (int)(u / p.nkt);
            const int buf = seg & 1;
            const bool complete = (cnt == p.nkt);
            const int c_first = sched_cta_of_unit((long long)t * p.nkt, T, p.G);
            const int c_last = sched_cta_of_unit((long long)t * p.nkt + p.nkt - 1, T, p.G);
            const int nc = c_last - c_first + 1;
            const int slot = cta - c_first;
            const int n = t * TILE_N + tid;
            const bool valid = n < p.N;

            float corr[MMA_N];
#pragma unroll
            for (int m = 0; m < MMA_N; ++m) corr[m] = 0.f;
            if (p.R > 0) {
                if (!z_ready) {
                    if (tid == 0 && wait_counter(p.z_counter, (uint32_t)p.G, ctrl, p, ST_Z)) {
                        // the last CTA to get here clears both words for the next launch on this scratch
                        if (atomicAdd(p.z_counter + 1, 1u) == (uint32_t)p.G - 1u) {
                            p.z_counter[0] = 0u;
                            p.z_counter[1] = 0u;
                        }
                    }
                    if (!epi_sync_ok(ctrl)) return false;
                    z_ready = true;
                }
                const int w0 = (int)((long long)slot * p.Rw / nc);
                const int w1 = (int)((long long)(slot + 1) * p.Rw / nc);
                const int32_t* ucol = p.Ucol + (size_t)(valid ? n : 0) * p.Rw;
                for (int w = w0; w < w1; ++w) {
                    const uint32_t uw = valid ? (uint32_t)ucol[w] : 0u;
#pragma unroll (MMA_N <= 8 ? 8 : 2)
                    for (int b = 0; b < 32; b += 4) {
                        const float s0 = ((uw >> b) & 1u) ? 1.f : -1.f;
                        const float s1 = ((uw >> (b + 1)) & 1u) ? 1.f : -1.f;
                        const float s2 = ((uw >> (b + 2)) & 1u) ? 1.f : -1.f;
                        const float s3 = ((uw >> (b + 3)) & 1u) ? 1.f : -1.f;
#pragma unroll
                        for (int m = 0; m < MMA_N; ++m) {
                            if (m < p.M) {
                                const float4 zz = __ldcg(reinterpret_cast<const float4*>(zb + (size_t)m * Rpad + 32 * w + b));
                                corr[m] += (s0 * zz.x + s1 * zz.y) + (s2 * zz.z + s3 * zz.w);
                            }
                        }
                    }
                }
            }

            // accumulators of this segment
            wait_bar(smem_u32(&ctrl->acc_full[buf]), (seg >> 1) & 1, ctrl, p, ST_ACC_FULL, warp);
            if (!epi_sync_ok(ctrl)) return false;
            tc_fence_after_sync();
            float acc[MMA_N];
            tmem_ld_acc<MMA_N>(tmem + ((uint32_t)(warp * 32) << 16) + buf * ACC_COL_STRIDE, acc);
            tc_wait_ld();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&ctrl->acc_empty[buf]));

            float v[MMA_N];
#pragma unroll
            for (int m = 0; m < MMA_N; ++m) v[m] = alpha * acc[m] + corr[m];

            if (!complete && cta != c_last) {
                // contributor: publish the fp32 partial
                float* P = p.partials + ((size_t)t * p.max_slots + slot) * MMA_N * TILE_N;
#pragma unroll
                for (int m = 0; m < MMA_N; ++m)
                    if (m < p.M) P[m * TILE_N + tid] = v[m];
                __threadfence();
                named_bar_sync(1, EPI_THREADS);
                if (tid == 0) red_release_add_u32(p.tile_cnt + t, 1u);
            } else {
                if (!complete) {
                    // finisher: wait for the nc-1 partials of this call, add them in slot order
                    if (tid == 0 && wait_counter(p.tile_cnt + t, (uint32_t)(nc - 1), ctrl, p, ST_TILE))
                        p.tile_cnt[t] = 0u;      // only this CTA reads it; ready for the next launch
                    if (!epi_sync_ok(ctrl)) return false;
                    for (int sl = 0; sl < nc - 1; ++sl) {
                        const float* P = p.partials + ((size_t)t * p.max_slots + sl) * MMA_N * TILE_N;
#pragma unroll
                        for (int m = 0; m < MMA_N; ++m)
                            if (m < p.M) v[m] += __ldcg(P + m * TILE_N + tid);
                    }
                }
                if (valid) {
#pragma unroll
                    for (int m = 0; m < MMA_N; ++m) {
                        if (m < p.M) {
                            float o = v[m];
                            if (p.C) o += __bfloat162float(p.C[(size_t)m * p.N + n]);
                            p.Y[(size_t)m * p.N + n] = __float2bfloat16(o);
                        }
                    }
                }
            }
            ++seg;
            return true;
        });
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
    if (warp == 5) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// -----------------------------------------------------------------------------------------------------------
// Host side
// -----------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)f;
    });
    return fn;
}

struct MapKey {
    const void* ptr; int rows, kbytes, box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && kbytes == o.kbytes && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.kbytes << 20) ^ ((size_t)k.box_rows << 40);
    }
};

// u8 [rows, kbytes] row-major, box = box_rows x 128 B, 128-byte swizzle. Cached: encoding costs microseconds.
static int get_tensor_map(const void* ptr, int rows, int kbytes, int box_rows, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{ptr, rows, kbytes, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return BILOCO_OK; }
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return BILOCO_ERR_CUDA;
    const cuuint64_t gdim[2] = {(cuuint64_t)kbytes, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)kbytes};
    const cuuint32_t box[2] = {(cuuint32_t)KT_BYTES, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return BILOCO_ERR_CUDA;
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return BILOCO_OK;
}

static int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cached[dev] = n;
    }
    return cached[dev];
}

static int mma_n_for(int M) { return M <= 8 ? 8 : (M <= 16 ? 16 : 32); }

struct ScratchLayout {
    size_t off_zcnt, off_tilecnt, off_z, off_part, total;
    int ntile, nkt, G, max_slots, Rw, Rpad, mma_n;
};

static bool make_layout(int M, int N, int K, int R, int num_sms, ScratchLayout* L) {
    if (M < 1 || M > 32 || N < 8 || (N % 8) || K < KT || (K % KT) || R < 0 || num_sms < 1) return false;
    L->mma_n = mma_n_for(M);
    L->ntile = (N + TILE_N - 1) / TILE_N;
    L->nkt = K / KT;
    const long long T = (long long)L->ntile * L->nkt;
    L->G = (int)(T < num_sms ? T : num_sms);
    L->max_slots = sched_max_slots(L->ntile, L->nkt, L->G);
    L->Rw = (R + 31) / 32;
    L->Rpad = L->Rw * 32;
    size_t off = 64;                                     // 16 status words
    L->off_zcnt = off; off += 64;
    L->off_tilecnt = off; off += ((size_t)L->ntile * 4 + 127) / 128 * 128;
    L->off_z = off; off += (size_t)2 * 32 * L->Rpad * sizeof(float);
    L->off_part = off; off += (size_t)L->ntile * L->max_slots * L->mma_n * TILE_N * sizeof(float);
    L->total = (off + 255) / 256 * 256;
    return true;
}

template <int MMA_N>
static int launch(const CUtensorMap& tmW, const CUtensorMap& tmA, const FusedParams& p, cudaStream_t stream) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(fused_linear_kernel<MMA_N>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<MMA_N>::SMEM_BYTES) !=
            cudaSuccess)
            return BILOCO_ERR_CUDA;
        attr_set[dev] = true;
    }
    fused_linear_kernel<MMA_N><<<p.G, NUM_THREADS, Cfg<MMA_N>::SMEM_BYTES, stream>>>(tmW, tmA, p);
    return cudaGetLastError() == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}

}  // namespace biloco

using namespace biloco;

extern "C" size_t biloco_b200_scratch_bytes(int M, int N, int K, int R, int num_sms) {
    if (num_sms == 0) num_sms = device_sm_count();
    ScratchLayout L;
    if (!make_layout(M, N, K, R, num_sms, &L)) return 0;
    return L.total;
}

extern "C" size_t biloco_b200_scratch_head_bytes(int M, int N, int K, int R, int num_sms) {
    if (num_sms == 0) num_sms = device_sm_count();
    ScratchLayout L;
    if (!make_layout(M, N, K, R, num_sms, &L)) return 0;
    return L.off_z;
}

extern "C" int biloco_b200_schedule_info(int M, int N, int K, int R, int num_sms, int* out6) {
    if (!out6) return BILOCO_ERR_NULL;
    if (num_sms == 0) num_sms = device_sm_count();
    ScratchLayout L;
    if (!make_layout(M, N, K, R, num_sms, &L)) return BILOCO_ERR_SHAPE;
    out6[0] = L.ntile; out6[1] = L.nkt; out6[2] = L.G; out6[3] = L.max_slots; out6[4] = L.mma_n;
    out6[5] = L.mma_n == 8 ? Cfg<8>::STAGES : (L.mma_n == 16 ? Cfg<16>::STAGES : Cfg<32>::STAGES);
    return BILOCO_OK;
}

extern "C" int biloco_b200_fused_linear(const void* W_codes, const void* W_sf, const float* alpha, const void* A_codes,
                                        const void* A_sf, const void* X_bf16, const void* V_packed, const int32_t* U_col32,
                                        const void* S_bf16, const void* C_bf16, void* Y_bf16, void* scratch,
                                        size_t scratch_bytes, int M, int A_rows, int N, int K, int R, int mode, int epoch,
                                        biloco_stream_t stream) {
    if (!W_codes || !W_sf || !alpha || !A_codes || !A_sf || !Y_bf16 || !scratch) return BILOCO_ERR_NULL;
    if (R > 0 && (!X_bf16 || !V_packed || !U_col32 || !S_bf16)) return BILOCO_ERR_NULL;
    if (mode != BILOCO_MODE_COUNTER) return BILOCO_ERR_MODE;
    if (epoch < 1) return BILOCO_ERR_EPOCH;
    if (A_rows < M || A_rows > 128) return BILOCO_ERR_SHAPE;
    const int sms = device_sm_count();
    if (sms < 1) return BILOCO_ERR_CUDA;
    ScratchLayout L;
    if (!make_layout(M, N, K, R, sms, &L)) return BILOCO_ERR_SHAPE;
    if (scratch_bytes < L.total) return BILOCO_ERR_SCRATCH;
    if (((uintptr_t)W_codes & 15) || ((uintptr_t)A_codes & 15) || ((uintptr_t)W_sf & 15) || ((uintptr_t)A_sf & 15) ||
        ((uintptr_t)X_bf16 & 15) || ((uintptr_t)scratch & 255) || ((uintptr_t)U_col32 & 3))
        return BILOCO_ERR_ALIGN;

    CUtensorMap tmW, tmA;
    int rc = get_tensor_map(W_codes, N, K / 2, TILE_N, &tmW);
    if (rc != BILOCO_OK) return rc;
    rc = get_tensor_map(A_codes, A_rows, K / 2, L.mma_n, &tmA);
    if (rc != BILOCO_OK) return rc;

    uint8_t* sc = (uint8_t*)scratch;
    FusedParams p;
    p.W_sf = (const uint8_t*)W_sf;
    p.A_sf = (const uint8_t*)A_sf;
    p.alpha = alpha;
    p.X = (const __nv_bfloat16*)X_bf16;
    p.Vp = (const uint8_t*)V_packed;
    p.Ucol = U_col32;
    p.S = (const __nv_bfloat16*)S_bf16;
    p.C = (const __nv_bfloat16*)C_bf16;
    p.Y = (__nv_bfloat16*)Y_bf16;
    p.status = (int32_t*)sc;
    p.z_counter = (uint32_t*)(sc + L.off_zcnt);
    p.tile_cnt = (uint32_t*)(sc + L.off_tilecnt);
    p.zbuf = (float*)(sc + L.off_z);
    p.partials = (float*)(sc + L.off_part);
    p.M = M; p.N = N; p.K = K; p.R = R; p.Rw = L.Rw; p.Rpad = L.Rpad;
    p.ntile = L.ntile; p.nkt = L.nkt; p.G = L.G; p.max_slots = L.max_slots;
    p.epoch = (uint32_t)epoch;
    p.mode = mode;

    cudaStream_t s = (cudaStream_t)stream;
    switch (L.mma_n) {
        case 8: return launch<8>(tmW, tmA, p, s);
        case 16: return launch<16>(tmW, tmA, p, s);
        default: return launch<32>(tmW, tmA, p, s);
    }
}

extern "C" int biloco_b200_read_status(const void* scratch, int32_t* out16, biloco_stream_t stream) {
    if (!scratch || !out16) return BILOCO_ERR_NULL;
    if (cudaMemcpyAsync(out16, scratch, 16 * sizeof(int32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream) != cudaSuccess)
        return BILOCO_ERR_CUDA;
    return cudaStreamSynchronize((cudaStream_t)stream) == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}
