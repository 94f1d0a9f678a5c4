// z stage on the tensor cores, as a launch of its own in front of the fused linear (used from ZTC_MIN_ROWS activation rows).
//
//     z[m, i] = S_i * sum_k sign(V[i, k]) x[m, k]            (reference: z workers, csrc/biloco_side.cuh:135-430,
//                                                              csrc/biloco_branch_lut.cuh:101-177 phase Z)
// is a small GEMM: 128 ranks as MMA M, the activation rows as MMA N (8 / 16 / 32), K as K. The products are exact (bf16 x
// times +-1.0) and the accumulator is fp32, so this is the same sum as the CUDA-core stage up to the order of the additions.
// On the CUDA cores the stage costs M * R * K predicated adds (12 M warp instructions at M = 32, r = 512, K = 5120: most of
// the launch); here it is R / 128 * K / 16 MMAs of 128 x N x 16, spread over the SMs by splitting K:
//   * CTA (rb, ks) takes rank block rb (128 ranks) and the 64-element chunks [ks nch / nks, (ks + 1) nch / nks) of K. Per chunk:
//     the +-1.0 bf16 image of the chunk's V signs (128 rows x 128 bytes, 256-entry byte table, 128-byte swizzle) and the chunk
//     of X (N rows x 128 bytes) go to shared memory (two buffers), one thread issues four tcgen05.mma.kind::f16.
//     The sign image does not depend on x: the first chunks are built before the dependency wait.
//   * The CTA's partial sums [N][128] go to global memory; a counter per rank block (monotonic: launch l ends at (l + 1) nks)
//     tells when all nks partials of the block are there; then every CTA of the block adds an nks-th of the block's outputs
//     over the partials IN ks ORDER (deterministic), scales by S and stores z with the validity mark the consumers poll on.
//   * The fused linear that follows (programmatic dependent launch) runs without z items of its own.
// Every wait is bounded; a wait that ran out is recorded in the status words of the scratch (code ST_Z).
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include "fused_cfg.cuh"
#include "ptx.cuh"

namespace biloco {
namespace ztc {

constexpr int ZT = 256;                    // threads
constexpr int A_BYTES = 128 * 128;         // sign image of one chunk: 128 ranks x 64 bf16
constexpr int ZTC_TMEM_COLS = 32;
constexpr int NBUF = 4;                    // operand buffers: a CTA's chunks are staged up to four at a time (one barrier, the MMAs back to back)
constexpr int ZTC_MIN_ROWS = 16;           // activation rows from which the launcher uses this kernel by default

struct ZtcParams {
    const uint8_t* Vp;            // [R][K/8] sign bits (set = +1)
    const __nv_bfloat16* X;       // [M][K]
    const __nv_bfloat16* S;       // [R]
    float* zbuf;                  // [M][Rpad], values carry the validity mark in their lowest mantissa bit
    float* part;                  // [nrb * nks][N][128] partial sums
    uint32_t* cnt;                // [nrb] arrivals (monotonic)
    const uint32_t* z_counter;    // [0] launches completed on this scratch
    int32_t* status;
    unsigned long long wait_ns;
    int M, K, R, Rpad, nrb, nks;
    uint32_t epoch;
};

__device__ __forceinline__ void zfail(int32_t* status, uint32_t epoch, int role) {
    if (atomicCAS(status, 0, (int)ST_Z) == 0) {
        status[1] = (int)blockIdx.x;
        status[2] = (int)epoch;
        status[3] = role;
    }
}

__device__ __forceinline__ bool zwait(uint32_t bar, uint32_t parity, const ZtcParams& p, int role) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 3u) == 3u) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > p.wait_ns) { zfail(p.status, p.epoch, role); return false; }
        }
    }
}

template <int NB>
__global__ void __launch_bounds__(ZT) ztc_kernel(const __grid_constant__ ZtcParams p) {
    extern __shared__ uint8_t ztc_raw[];
    const uint32_t raw = smem_u32(ztc_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = ztc_raw + (base - raw);
    constexpr int B_BYTES = NB * 128;
    uint8_t* Abuf = sm;                                  // [NBUF][A_BYTES]
    uint8_t* Bbuf = sm + NBUF * A_BYTES;                 // [NBUF][B_BYTES] (1024-aligned: B_BYTES is 1024, 2048 or 4096)
    uint4* lut = reinterpret_cast<uint4*>(sm + NBUF * A_BYTES + NBUF * B_BYTES);     // [256] byte of sign bits -> eight bf16 +-1.0
    __shared__ __align__(8) uint64_t bar_free[NBUF];
    __shared__ __align__(8) uint64_t bar_done;
    __shared__ uint32_t tmem_base_s;
    __shared__ int ok_s;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rb = blockIdx.x / p.nks, ks = blockIdx.x - rb * p.nks;
    const int nch = p.K >> 6;
    const int c0 = (int)((long long)ks * nch / p.nks), c1 = (int)((long long)(ks + 1) * nch / p.nks);
    const int kbytes = p.K >> 3;

    if (tid == 0) {
        for (int b = 0; b < NBUF; ++b) mbar_init(smem_u32(&bar_free[b]), 1);
        mbar_init(smem_u32(&bar_done), 1);
        fence_mbar_init();
        ok_s = 1;
    }
    {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            w[i] = (((tid >> (2 * i)) & 1) ? 0x3F80u : 0xBF80u) | ((((tid >> (2 * i + 1)) & 1) ? 0x3F80u : 0xBF80u) << 16);
        lut[tid] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_base_s), ZTC_TMEM_COLS);
        tmem_relinquish();
        tc_fence_before_sync();
    }
    __syncthreads();
    griddep_launch_dependents();               // the fused linear may move in and prefetch its weights
    tc_fence_after_sync();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&tmem_base_s);
    constexpr uint32_t idesc = make_idesc_bf16(128, NB);

    // sign image of chunk c into buffer b: thread = (rank r = tid & 127, half h = tid >> 7): four bytes of V -> four 16-byte pieces
    auto build_a = [&](int c, int b) {
        const int r = tid & 127, h = tid >> 7;
        const int rank = rb * 128 + r;
        uint32_t bits = 0u;
        if (rank < p.R) bits = *reinterpret_cast<const uint32_t*>(p.Vp + (size_t)rank * kbytes + c * 8 + h * 4);
        uint8_t* row = Abuf + b * A_BYTES + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int pc = h * 4 + i;
            *reinterpret_cast<uint4*>(row + ((pc ^ (r & 7)) * 16)) = rank < p.R ? lut[(bits >> (8 * i)) & 0xFFu] : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    bool ok = true;
    // the sign images of the first round of chunks do not depend on this call's activation
#pragma unroll 1
    for (int i = 0; i < NBUF && c0 + i < c1; ++i) build_a(c0 + i, i);
    griddep_wait();                            // X comes from the previous kernel of the stream
    const uint32_t seq = ld_volatile_u32(p.z_counter);
#pragma unroll 1
    for (int r0 = c0; r0 < c1; r0 += NBUF) {
        const int nr = (c1 - r0) < NBUF ? (c1 - r0) : NBUF;
        const int round = (r0 - c0) / NBUF;
        // the round's pieces of X: all requested before any is used (one memory round trip per round)
        uint4 xv[NBUF];
        const int m = tid >> 3, pc = tid & 7;
#pragma unroll
        for (int i = 0; i < NBUF; ++i) {
            xv[i] = make_uint4(0u, 0u, 0u, 0u);
            if (i < nr && tid < NB * 8 && m < p.M) xv[i] = *reinterpret_cast<const uint4*>(p.X + (size_t)m * p.K + (r0 + i) * 64 + pc * 8);
        }
        if (round > 0) {
#pragma unroll 1
            for (int i = 0; i < nr; ++i) {
                if (ok && !zwait(smem_u32(&bar_free[i]), (uint32_t)((round - 1) & 1), p, 1)) ok = false;
            }
            tc_fence_after_sync();
#pragma unroll 1
            for (int i = 0; i < nr; ++i) build_a(r0 + i, i);
        }
        if (tid < NB * 8) {
#pragma unroll
            for (int i = 0; i < NBUF; ++i)
                if (i < nr) *reinterpret_cast<uint4*>(Bbuf + i * B_BYTES + (m >> 3) * 1024 + (m & 7) * 128 + ((pc ^ (m & 7)) * 16)) = xv[i];
        }
        fence_proxy_async();                   // operands written with ordinary stores
        if (!ok) ok_s = 0;
        __syncthreads();
        if (!ok_s) break;
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll 1
            for (int i = 0; i < nr; ++i) {
                const uint64_t ad = make_smem_desc(smem_u32(Abuf + i * A_BYTES), 1024, 2);
                const uint64_t bd = make_smem_desc(smem_u32(Bbuf + i * B_BYTES), 1024, 2);
#pragma unroll
                for (int k = 0; k < 4; ++k) tc_mma_bf16(tmem, ad + 2 * k, bd + 2 * k, idesc, (r0 + i > c0 || k > 0) ? 1u : 0u);
                tc_commit(smem_u32(&bar_free[i]));
            }
            if (r0 + nr == c1) tc_commit(smem_u32(&bar_done));
        }
    }
    ok = ok_s != 0;
    if (ok && c0 < c1 && !zwait(smem_u32(&bar_done), 0, p, 2)) ok = false;
    tc_fence_after_sync();
    // partial sums: lane = rank, NB columns = activation rows
    float* mypart = p.part + (size_t)blockIdx.x * NB * 128;
    if (warp < 4 && ok) {
        float d[NB];
        if (c0 < c1) {
            const uint32_t t = tmem + ((uint32_t)(warp * 32) << 16);
            if (NB == 8) tmem_ld_x8(t, d);
            else {
#pragma unroll
                for (int j = 0; j < NB / 16; ++j) tmem_ld_x16(t + 16 * j, d + 16 * j);
            }
            tc_wait_ld();
        } else {
#pragma unroll
            for (int j = 0; j < NB; ++j) d[j] = 0.f;
        }
#pragma unroll
        for (int m = 0; m < NB; ++m)
            if (m < p.M) mypart[m * 128 + warp * 32 + lane] = d[m];
    }
    tc_fence_before_sync();
    __threadfence();
    if (!ok) ok_s = 0;
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, ZTC_TMEM_COLS);
    }
    // arrival, then wait for the block's other CTAs (a failed CTA arrives too, so that nobody waits for it in vain; its
    // status word tells the host that the result is void)
    const uint32_t target = (seq + 1u) * (uint32_t)p.nks;
    if (tid == 0) {
        red_release_add_u32(p.cnt + rb, 1u);
        uint64_t t0 = 0;
        for (uint32_t it = 0;; ++it) {
            if ((int32_t)(ld_acquire_u32(p.cnt + rb) - target) >= 0) break;
            if ((it & 15u) == 15u) {
                const uint64_t now = globaltimer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > p.wait_ns) { zfail(p.status, p.epoch, 3); ok_s = 0; break; }
            }
        }
    }
    __syncthreads();
    if (!ok_s) return;
    // this CTA's share of the block's outputs: elements e = m * 128 + r, added over the partials in ks order
    const int E = p.M * 128;
    const int e0 = (int)((long long)ks * E / p.nks), e1 = (int)((long long)(ks + 1) * E / p.nks);
    const uint32_t mark = (seq & 1u) ^ 1u;
    const float* pb = p.part + (size_t)rb * p.nks * NB * 128;
    for (int e = e0 + tid; e < e1; e += ZT) {
        const int m = e >> 7, r = e & 127;
        const int rank = rb * 128 + r;
        float t = 0.f;
        int j = 0;
        for (; j + 8 <= p.nks; j += 8) {
            float x[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) x[q] = __ldcg(pb + (size_t)(j + q) * NB * 128 + e);
#pragma unroll
            for (int q = 0; q < 8; ++q) t = __fadd_rn(t, x[q]);
        }
        for (; j < p.nks; ++j) t = __fadd_rn(t, __ldcg(pb + (size_t)j * NB * 128 + e));
        if (rank < p.R) {
            const float z = __fmul_rn(t, __bfloat162float(p.S[rank]));
            p.zbuf[(size_t)m * p.Rpad + rank] = __uint_as_float((__float_as_uint(z) & ~1u) | mark);
        }
    }
}

}  // namespace ztc
}  // namespace biloco
