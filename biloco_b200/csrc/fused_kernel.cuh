// The fused linear kernel. Template parameters: MMA_N = tensor-core N (activation rows per MMA: 8/16/32),
// ROWS = activation rows carried by the CUDA-core half (M rounded up to 1/2/4/8/16/32; rows beyond M repeat row M-1
// and are never stored).
#pragma once
#include "fused_cfg.cuh"
#include "fused_lowrank.cuh"

namespace biloco {

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

template <int MMA_N, int ROWS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
fused_linear_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
                    const __grid_constant__ FusedParams p) {
    static_assert(ROWS <= MMA_N, "the tensor-core tile must cover the rows");
    using C = Cfg<MMA_N>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t stage0 = (raw + 1023u) & ~1023u;                 // shared-window address of stage 0
    uint8_t* after_stages = smem_raw + (stage0 - raw) + C::STAGES * C::STAGE_BYTES;
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(after_stages);
    uint8_t* work = after_stages + CTRL_BYTES;                       // WORK_BYTES, 1024-byte aligned

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int cta = blockIdx.x;

    const int T = p.ntile * p.nkt;
    const int u0 = sched_first_unit(cta, T, p.G);
    const int u1 = sched_first_unit(cta + 1, T, p.G);

    // ---------------- set-up ----------------
    if (tid == 128) {
#pragma unroll 1
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->full[s]), 1);
            mbar_init(smem_u32(&ctrl->empty[s]), 1);
        }
#pragma unroll 1
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
    if (tid == 0 && p.stamps) p.stamps[(size_t)cta * STAMP_WORDS + 0] = globaltimer_ns();

    if (warp == 4) {
        // ================= TMA producer =================
        // wait until the epilogue threads have issued their first small loads (U words, V bits, x): those requests
        // then sit ahead of the ~100 KB per SM of weight traffic issued next
        asm volatile("bar.sync 2, %0;" ::"r"(EPI_THREADS + 32) : "memory");
        if (lane == 0) {
            int i = 0;
            bool ok = true;
#pragma unroll 1
            for (SegWalk sw(u0, u1, p.nkt); ok && !sw.done(); sw.next()) {
                const int us = sw.first();
                const int cnt = sw.count();
                int t = (int)((unsigned)us / (unsigned)p.nkt);
                int kt = us - t * p.nkt;
#pragma unroll 1
                for (int u = us; u < us + cnt; ++u, ++i, ++kt) {
                    const int s = i % C::STAGES;
                    const int use = i / C::STAGES;
                    if (use > 0 && !wait_bar(smem_u32(&ctrl->empty[s]), (use - 1) & 1, ctrl, p.status, p.epoch, ST_EMPTY, 4)) {
                        ok = false;
                        break;
                    }
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
            }
        }
    } else if (warp == 5) {
        // ================= MMA issue =================
        constexpr uint32_t idesc = make_idesc_nvf4(TILE_N, MMA_N);
        int i = 0, seg = 0;
        bool ok = true;
#pragma unroll 1
        for (SegWalk sw(u0, u1, p.nkt); ok && !sw.done(); sw.next(), ++seg) {
            const int cnt = sw.count();
            const int buf = seg & 1;
            if (seg >= 2 && !wait_bar(smem_u32(&ctrl->acc_empty[buf]), ((seg >> 1) - 1) & 1, ctrl, p.status, p.epoch, ST_ACC_EMPTY, 5))
                break;
            tc_fence_after_sync();
#pragma unroll 1
            for (int j = 0; j < cnt; ++j, ++i) {
                const int s = i % C::STAGES;
                if (!wait_bar(smem_u32(&ctrl->full[s]), (i / C::STAGES) & 1, ctrl, p.status, p.epoch, ST_FULL, 5)) { ok = false; break; }
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
                    if (p.stamps) p.stamps[(size_t)cta * STAMP_WORDS + 7] = globaltimer_ns();   // latest stage landed
                }
                __syncwarp();
            }
        }
    } else {
        // ================= z stage, expansion, epilogue (128 threads) =================
        float* zb = p.zbuf + (size_t)(p.epoch & 1u) * 32 * p.Rpad;
        float* zs = reinterpret_cast<float*>(work);
        bool signal_pending = true;

        // U words of the first chunk of the first two segments: requested before anything else, so that they do
        // not queue behind the weight stream later
        uint32_t uw_first[2][ZS_WORDS];
#pragma unroll
        for (int g = 0; g < 2; ++g)
#pragma unroll
            for (int w = 0; w < ZS_WORDS; ++w) uw_first[g][w] = 0u;
        if (p.R > 0) {
            SegWalk sw(u0, u1, p.nkt);
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                if (!sw.done()) {
                    const int t = (int)((unsigned)sw.first() / (unsigned)p.nkt);
                    const int c_first = sched_cta_of_unit(t * p.nkt, T, p.G);
                    const int nc = sched_cta_of_unit(t * p.nkt + p.nkt - 1, T, p.G) - c_first + 1;
                    const int w0 = (cta - c_first) * p.Rw / nc;
                    const int w1 = (cta - c_first + 1) * p.Rw / nc;
                    const int n = t * TILE_N + tid;
                    const int32_t* ucol = p.Ucol + (size_t)(n < p.N ? n : 0) * p.Rw;
#pragma unroll
                    for (int w = 0; w < ZS_WORDS; ++w) uw_first[g][w] = (uint32_t)ucol[(w0 + w < w1) ? (w0 + w) : (w0 < w1 ? w0 : 0)];
                    sw.next();
                }
            }

            z_stage<ROWS>(p, work, zb, cta, tid, signal_pending);
            if (signal_pending) {   // this CTA had no ranks to compute
                asm volatile("bar.arrive 2, %0;" ::"r"(EPI_THREADS + 32) : "memory");
                signal_pending = false;
            }
            named_bar_sync(1, EPI_THREADS);    // orders every z store before thread 0's (cumulative) release
            if (tid == 0) {
                red_release_add_u32(p.z_counter, 1u);
                if (p.stamps) p.stamps[(size_t)cta * STAMP_WORDS + 1] = globaltimer_ns();
            }
        }
        if (signal_pending) asm volatile("bar.arrive 2, %0;" ::"r"(EPI_THREADS + 32) : "memory");

        bool z_ready = false;
        const float alpha = p.alpha[0];
        int seg = 0;
#pragma unroll 1
        for (SegWalk sw(u0, u1, p.nkt); !sw.done(); sw.next(), ++seg) {
            const int u = sw.first();
            const int cnt = sw.count();
            const int t = (int)((unsigned)u / (unsigned)p.nkt);
            const int buf = seg & 1;
            const bool complete = (cnt == p.nkt);
            const int c_first = sched_cta_of_unit(t * p.nkt, T, p.G);
            const int c_last = sched_cta_of_unit(t * p.nkt + p.nkt - 1, T, p.G);
            const int nc = c_last - c_first + 1;
            const int slot = cta - c_first;
            const int n = t * TILE_N + tid;
            const bool valid = n < p.N;

            float corr[ROWS];
#pragma unroll
            for (int m = 0; m < ROWS; ++m) corr[m] = 0.f;
            if (p.R > 0) {
                if (!z_ready) {
                    if (tid == 0 && wait_counter(p.z_counter, (uint32_t)p.G, ctrl, p.status, p.epoch, ST_Z)) {
                        // the last CTA to get here clears both words for the next launch on this scratch
                        if (atomicAdd(p.z_counter + 1, 1u) == (uint32_t)p.G - 1u) {
                            p.z_counter[0] = 0u;
                            p.z_counter[1] = 0u;
                        }
                    }
                    if (!epi_sync_ok(ctrl)) break;
                    z_ready = true;
                    if (tid == 0 && p.stamps) p.stamps[(size_t)cta * STAMP_WORDS + 2] = globaltimer_ns();
                }
                const int w0 = slot * p.Rw / nc;
                const int w1 = (slot + 1) * p.Rw / nc;
                const int32_t* ucol = p.Ucol + (size_t)(valid ? n : 0) * p.Rw;
                uint32_t uw_sel[ZS_WORDS];
#pragma unroll
                for (int w = 0; w < ZS_WORDS; ++w) uw_sel[w] = (seg & 1) ? uw_first[1][w] : uw_first[0][w];
                expand_z<ROWS>(corr, zb, p.Rpad, ucol, w0, w1, zs, tid, uw_sel, seg < 2);
                if (tid == 0 && p.stamps && seg == 0) p.stamps[(size_t)cta * STAMP_WORDS + 3] = globaltimer_ns();
            }

            // accumulators of this segment
            wait_bar(smem_u32(&ctrl->acc_full[buf]), (seg >> 1) & 1, ctrl, p.status, p.epoch, ST_ACC_FULL, warp);
            if (!epi_sync_ok(ctrl)) break;
            tc_fence_after_sync();
            if (tid == 0 && p.stamps && seg == 0) p.stamps[(size_t)cta * STAMP_WORDS + 4] = globaltimer_ns();
            float acc[MMA_N];
            tmem_ld_acc<MMA_N>(tmem + ((uint32_t)(warp * 32) << 16) + buf * ACC_COL_STRIDE, acc);
            tc_wait_ld();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&ctrl->acc_empty[buf]));

            float v[ROWS];
#pragma unroll
            for (int m = 0; m < ROWS; ++m) v[m] = alpha * acc[m] + corr[m];

            if (!complete && cta != c_last) {
                // contributor: publish the fp32 partial
                float* P = p.partials + ((size_t)t * p.max_slots + slot) * MMA_N * TILE_N;
#pragma unroll
                for (int m = 0; m < ROWS; ++m) P[m * TILE_N + tid] = v[m];
                named_bar_sync(1, EPI_THREADS);     // orders all partial stores before thread 0's (cumulative) release
                if (tid == 0) red_release_add_u32(p.tile_cnt + t, 1u);
            } else {
                if (!complete) {
                    // finisher: wait for the nc-1 partials of this launch, add them in slot order
                    if (tid == 0 && wait_counter(p.tile_cnt + t, (uint32_t)(nc - 1), ctrl, p.status, p.epoch, ST_TILE))
                        p.tile_cnt[t] = 0u;      // only this CTA reads it; ready for the next launch
                    if (!epi_sync_ok(ctrl)) break;
#pragma unroll 1
                    for (int sl = 0; sl < nc - 1; ++sl) {
                        const float* P = p.partials + ((size_t)t * p.max_slots + sl) * MMA_N * TILE_N;
                        float pv[ROWS];
#pragma unroll
                        for (int m = 0; m < ROWS; ++m) pv[m] = __ldcg(P + m * TILE_N + tid);
#pragma unroll
                        for (int m = 0; m < ROWS; ++m) v[m] += pv[m];
                    }
                }
                if (valid) {
#pragma unroll
                    for (int m = 0; m < ROWS; ++m) {
                        if (m < p.M) {
                            float o = v[m];
                            if (p.C) o += __bfloat162float(p.C[(size_t)m * p.N + n]);
                            p.Y[(size_t)m * p.N + n] = __float2bfloat16(o);
                        }
                    }
                }
            }
            if (tid == 0 && p.stamps) p.stamps[(size_t)cta * STAMP_WORDS + 5 + (seg > 0 ? 1 : 0)] = globaltimer_ns();
        }
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

}  // namespace biloco
