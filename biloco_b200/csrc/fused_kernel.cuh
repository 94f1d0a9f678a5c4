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

// Row-parallel use: this rank's fp32 output element `idx`, with the number of the all-reduce call it belongs to, into this
// rank's slot of every peer's receive buffer (one aligned 8-byte store each: value and flag travel together; the gather
// launch of peer_reduce.cu polls for them).
__device__ __forceinline__ void ar_push(const FusedParams& p, uint32_t seq, int idx, float v) {
    const size_t off = (size_t)(seq & 1u) * p.ar_world * p.ar_slot + (size_t)p.ar_rank * p.ar_slot + idx;
    const uint32_t bits = __float_as_uint(v);
    for (int q = 0; q < p.ar_world; ++q) {
        if (q == p.ar_rank) continue;
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p.ar_recv[q] + off), "r"(bits), "r"(seq) : "memory");
    }
}

// PUSH: the epilogue also stores its fp32 outputs into the peers' receive buffers (row-parallel use). An instantiation of its
// own: compiled into the one kernel behind a run-time switch, the push cost every launch that does not use it (M = 32,
// K = N = 5120, r = 512: 32.3 us per call with the switch, 29.7 without the code).
template <int MMA_N, int ROWS, bool PUSH = false>
__global__ void __launch_bounds__(NUM_THREADS, ctas_per_sm(ROWS))
fused_linear_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
                    const __grid_constant__ FusedParams p) {
    static_assert(ROWS <= MMA_N, "the tensor-core tile must cover the rows");
    using C = Cfg<MMA_N>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t stage0 = (raw + 1023u) & ~1023u;                 // shared-window address of stage 0
    const int ring = p.ring;                                        // stages in use; the host sized the allocation for it
    uint8_t* after_stages = smem_raw + (stage0 - raw) + ring * C::STAGE_BYTES;
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(after_stages);
    uint8_t* work = after_stages + CTRL_BYTES;                       // WORK_BYTES, 1024-byte aligned

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int cta = blockIdx.x;

    const int T = p.ntile * p.nkt;
    int u0, u1;
    if (p.cluster > 1) {      // CTA r of the cluster that owns tile t takes k-tiles [r*nkt/c, (r+1)*nkt/c)
        const int t = cta / p.cluster, r = cta - t * p.cluster;
        u0 = t * p.nkt + r * p.nkt / p.cluster;
        u1 = t * p.nkt + (r + 1) * p.nkt / p.cluster;
    } else {
        u0 = sched_first_unit(cta, T, p.G);
        u1 = sched_first_unit(cta + 1, T, p.G);
    }

    uint32_t seq = 0;         // (thread 0) launches completed on this scratch before this one

    // ---------------- set-up ----------------
    if (tid == 0 && p.stamps) {
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        p.stamps[(size_t)cta * STAMP_WORDS + 10] = globaltimer_ns();
        p.stamps[(size_t)cta * STAMP_WORDS + 1] = clock64();
        p.stamps[(size_t)cta * STAMP_WORDS + 7] = smid;
    }
    if (tid == FIRST_SF_WARP * 32) {
#pragma unroll 1
        for (int s = 0; s < ring; ++s) {
            mbar_init(smem_u32(&ctrl->full[s]), 1);     // the stage's producer; the copies complete the byte count
            mbar_init(smem_u32(&ctrl->empty[s]), 1);
        }
#pragma unroll 1
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&ctrl->acc_full[b]), 1);
            mbar_init(smem_u32(&ctrl->acc_empty[b]), EPI_THREADS);
        }
        for (int q = 0; q < SF_SETS; ++q) {
            mbar_init(smem_u32(&ctrl->sf_full[q]), 128);
            mbar_init(smem_u32(&ctrl->sf_empty[q]), 1);
        }
        mbar_init(smem_u32(&ctrl->red_bar), p.cluster > 1 ? (uint32_t)(p.cluster - 1) : 1u);
        mbar_init(smem_u32(&ctrl->red_free), 1);
        mbar_init(smem_u32(&ctrl->x_bar), 1);
        mbar_init(smem_u32(&ctrl->lr_free[0]), 1);
        mbar_init(smem_u32(&ctrl->lr_free[1]), 1);
        mbar_init(smem_u32(&ctrl->lr_done), 1);
        ctrl->abort = 0;
        fence_mbar_init();
        prefetch_tmap(&tmW);
        prefetch_tmap(&tmA);
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&ctrl->tmem_base), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (p.cluster > 1) cluster_sync_all();   // every CTA's barriers exist before a peer may arrive on them
    const uint32_t tmem = ctrl->tmem_base;
    if (p.trigger == 0) griddep_launch_dependents();   // the next kernel of the stream may start its set-up and weight prefetch
    if (tid == 0 && p.stamps) p.stamps[(size_t)cta * STAMP_WORDS + 0] = globaltimer_ns();

    // copy requests of unit i (in processing order) into stage i % ring
    const int nunits = u1 - u0;
    const int head = SegWalk(u0, u1, p.nkt).head;     // units [head, u1) are processed first, then [u0, head)
    const int nhead = u1 - head;
    auto issue_w = [&](int i) {
        const int u = i < nhead ? head + i : u0 + (i - nhead);
        const uint32_t sbase = stage0 + (i % ring) * C::STAGE_BYTES;
        const uint32_t bar = smem_u32(&ctrl->full[i % ring]);
        mbar_arrive_expect_tx(bar, W_TILE_BYTES + C::A_TILE_BYTES + 2 * SF_TILE_BYTES);
        if (p.W_tiled) {
            // one contiguous 18 KB record per unit: pre-swizzled codes followed by the scale atoms
            bulk_load(sbase, p.W_tiled + (size_t)u * (W_TILE_BYTES + SF_TILE_BYTES), W_TILE_BYTES + SF_TILE_BYTES, bar);
        } else {
            const int t = (int)((unsigned)u / (unsigned)p.nkt), kt = u - t * p.nkt;
            tma_load_2d(sbase, &tmW, kt * KT_BYTES, t * TILE_N, bar);
            bulk_load(sbase + W_TILE_BYTES, p.W_sf + ((size_t)t * (p.K >> 6) + (size_t)kt * 4) * 512, SF_TILE_BYTES, bar);
        }
    };
    auto issue_a = [&](int i) {
        const int u = i < nhead ? head + i : u0 + (i - nhead);
        const int kt = (int)((unsigned)u % (unsigned)p.nkt);
        const uint32_t sbase = stage0 + (i % ring) * C::STAGE_BYTES;
        const uint32_t bar = smem_u32(&ctrl->full[i % ring]);
        if (p.A_rec) {      // one copy: the tile (already swizzled) and its scale atoms, laid out by the activation quantiser
            bulk_load(sbase + W_TILE_BYTES + SF_TILE_BYTES, p.A_rec + (size_t)kt * (C::A_TILE_BYTES + SF_TILE_BYTES),
                      C::A_TILE_BYTES + SF_TILE_BYTES, bar);
        } else {
            tma_load_2d(sbase + W_TILE_BYTES + SF_TILE_BYTES, &tmA, kt * KT_BYTES, 0, bar);
            bulk_load(sbase + W_TILE_BYTES + SF_TILE_BYTES + C::A_TILE_BYTES, p.A_sf + (size_t)kt * 4 * 512, SF_TILE_BYTES, bar);
        }
    };
    if (warp >= FIRST_Z_WARP && warp < MMA_WARP) {
        // ================= z warps: second half of the z stage =================
        if (p.R > 0) {
            const int zt = EPI_THREADS + (tid - FIRST_Z_WARP * 32);
            uint32_t seq_unused;
            z_stage(p, ctrl, work, p.zbuf, cta, zt, &seq_unused);     // (contains the dependency wait)
            named_bar_sync(3, Z_THREADS);      // the work area is free for the expansion
        }
    } else if (warp >= FIRST_SF_WARP && warp < FIRST_Z_WARP) {
        // ================= feeders: copy requests + scale-factor moves =================
        // Lane 0 of feeder j requests the copies of units j, j+PRODUCERS, ... (in processing order). Weights do not
        // depend on the previous kernel of the stream: the first ring of weight records is requested at once, before
        // the dependency wait; activations are what that kernel produced and follow the wait. Later units are
        // requested by the refill warp, as their stages come free.
        const int mine = warp - FIRST_SF_WARP;
        if (lane == 0) {
#pragma unroll 1
            for (int i = mine; i < nunits && i < ring; i += PRODUCERS) issue_w(i);
            griddep_wait();
            fence_proxy_async_global();       // the activation was written by ordinary stores of the previous kernel
#pragma unroll 1
            for (int i = mine; i < nunits && i < ring; i += PRODUCERS) issue_a(i);
        }
        __syncwarp();

        // The block-scaled MMA reads its scale factors from TMEM, lane l of every 32-lane quadrant holding rows
        // l, l+32, l+64, l+96 of the 128x4 atom in four consecutive columns. tcgen05.cp can place an atom there, but
        // eight of them per unit occupy the tensor pipe longer than the unit's four MMAs (measured); here warp q
        // writes quadrant q from registers instead: per unit 8 x 128-bit shared loads and 2 x tcgen05.st per thread.
        const uint32_t quad = (uint32_t)((warp & 3) * 32) << 16;
        // (Leaving the TMEM stores of unit i in flight while waiting for unit i+1, and signalling unit i only then, was
        // measured slower: 37.0 against 34.3 us on 8192 x 28672.)
#pragma unroll 1
        for (int i = 0; i < nunits; ++i) {
            const int s = i % ring;
            const int q = i % SF_SETS;
            bool ready = wait_bar(smem_u32(&ctrl->full[s]), (i / ring) & 1, ctrl, p.status, p.epoch, ST_FULL, warp);
            if (ready && i >= SF_SETS)
                ready = wait_bar(smem_u32(&ctrl->sf_empty[q]), ((i / SF_SETS) - 1) & 1, ctrl, p.status, p.epoch, ST_SF_EMPTY, warp);
            if (!__all_sync(0xffffffffu, ready)) break;     // warp-uniform: the TMEM stores are warp-wide
            tc_fence_after_sync();
            const uint8_t* stage = smem_raw + (stage0 - raw) + s * C::STAGE_BYTES;
            const uint4* wsf = reinterpret_cast<const uint4*>(stage + W_TILE_BYTES) + lane;
            const uint4* asf = reinterpret_cast<const uint4*>(stage + W_TILE_BYTES + SF_TILE_BYTES + C::A_TILE_BYTES) + lane;
            uint32_t ra[16], rb[16];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const uint4 x = wsf[a * 32], y = asf[a * 32];       // atom a, row `lane`: 16 bytes = 4 columns
                ra[4 * a] = x.x; ra[4 * a + 1] = x.y; ra[4 * a + 2] = x.z; ra[4 * a + 3] = x.w;
                rb[4 * a] = y.x; rb[4 * a + 1] = y.y; rb[4 * a + 2] = y.z; rb[4 * a + 3] = y.w;
            }
            tmem_st_x16(tmem + quad + 32u * q + SFA_COL, ra);
            tmem_st_x16(tmem + quad + 32u * q + SFB_COL, rb);
            tc_wait_st();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&ctrl->sf_full[q]));
        }
    } else if (warp == REFILL_WARP) {
        // ================= refills =================
        // Lane j < PRODUCERS re-requests stage (i % ring) for units i = ring + j, ring + j + PRODUCERS, ... as soon as the
        // MMAs of the unit that held the stage have completed. A warp of its own: a thread is held up while its copy
        // request is accepted (about 0.4 us measured), which must not sit inside the scale-factor loop of the feeders
        // (measured there: 0.9 us per unit and CTA, 3.0 TB/s on 8192 x 28672 instead of 4.6).
        if (lane < PRODUCERS) {
            griddep_wait();
            fence_proxy_async_global();
#pragma unroll 1
            for (int i = ring + lane; i < nunits; i += PRODUCERS) {
                if (!poll_bar(smem_u32(&ctrl->empty[i % ring]), ((i / ring) - 1) & 1, ctrl, p.status, p.epoch, ST_EMPTY, warp)) break;
                issue_w(i);
                issue_a(i);
            }
        }
    } else if (warp == MMA_WARP) {
        // ================= MMA issue =================
        constexpr uint32_t idesc = make_idesc_nvf4(TILE_N, MMA_N);
        int i = 0, seg = 0;
        bool ok = true;
#pragma unroll 1
        for (SegWalk sw(u0, u1, p.nkt); ok && !sw.done(); sw.next(), ++seg) {
            const int cnt = sw.count();
            const int buf = seg & 1;
            if (seg >= 2 && !wait_bar(smem_u32(&ctrl->acc_empty[buf]), ((seg >> 1) - 1) & 1, ctrl, p.status, p.epoch, ST_ACC_EMPTY, MMA_WARP))
                break;
            tc_fence_after_sync();
#pragma unroll 1
            for (int j = 0; j < cnt; ++j, ++i) {
                const int s = i % ring;
                if (!wait_bar(smem_u32(&ctrl->full[s]), (i / ring) & 1, ctrl, p.status, p.epoch, ST_FULL, MMA_WARP)) { ok = false; break; }
                if (!wait_bar(smem_u32(&ctrl->sf_full[i % SF_SETS]), (i / SF_SETS) & 1, ctrl, p.status, p.epoch, ST_SF_FULL, MMA_WARP)) { ok = false; break; }
                tc_fence_after_sync();
                if (lane == 0) {
                    const uint32_t sbase = stage0 + s * C::STAGE_BYTES;
                    const uint32_t sfset = 32u * (uint32_t)(i % SF_SETS);
                    const uint64_t wdesc = make_smem_desc(sbase, 1024, 2);
                    const uint64_t adesc = make_smem_desc(sbase + W_TILE_BYTES + SF_TILE_BYTES, 1024, 2);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        // 64 K-elements = 32 B further along the swizzled row: +2 in the (address >> 4) field
                        tc_mma_nvf4(tmem + buf * ACC_COL_STRIDE, wdesc + 2 * k, adesc + 2 * k, idesc,
                                    tmem + sfset + SFA_COL + 4 * k, tmem + sfset + SFB_COL + 4 * k, (j > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&ctrl->empty[s]));
                    tc_commit(smem_u32(&ctrl->sf_empty[i % SF_SETS]));
                    if (j == cnt - 1) tc_commit(smem_u32(&ctrl->acc_full[buf]));
                }
                __syncwarp();
            }
        }
    } else {
        // ================= z stage, expansion, epilogue (128 threads) =================
        float* zs = reinterpret_cast<float*>(work);
        const bool owner_mode = (p.mode & 0xff) == 4;
        // tensor-core expansion: operand buffers behind the sign words; table byte -> eight +-1.0 bf16 (bit set = +1)
        uint8_t* lr = work + XT_BYTES + p.vt_bytes;
        int gchunk = 0, lrseg = 0;
        if constexpr (ROWS >= LR_TC_MIN_ROWS) {
            if (p.lr_tc) {
                uint4* lut = reinterpret_cast<uint4*>(lr + 2 * LR_UA_BYTES + 4 * MMA_N * 128);
#pragma unroll
                for (int e = tid; e < 256; e += EPI_THREADS) {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        w[i] = (((e >> (2 * i)) & 1) ? 0x3F80u : 0xBF80u) | ((((e >> (2 * i + 1)) & 1) ? 0x3F80u : 0xBF80u) << 16);
                    lut[e] = make_uint4(w[0], w[1], w[2], w[3]);
                }
                // (made visible to the other epilogue threads by the barriers of the z stage)
            }
        }

        // U words of the first two segments' first ranks: requested before anything else, so that they do not queue
        // behind the weight stream later
        uint32_t uw_first[2][ZS_FIRST];
#pragma unroll
        for (int g = 0; g < 2; ++g)
#pragma unroll
            for (int w = 0; w < ZS_FIRST; ++w) uw_first[g][w] = 0u;
        uint32_t phase = 0;
        if (p.R > 0) {
            SegWalk sw(u0, u1, p.nkt);
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                if (!sw.done()) {
                    const SegInfo si = seg_info(p, T, cta, sw.first(), sw.count(), owner_mode);
                    const int n = si.t * TILE_N + tid;
                    const int32_t* ucol = p.Ucol + (size_t)(n < p.N ? n : 0) * p.Rw;
#pragma unroll
                    for (int w = 0; w < ZS_FIRST; ++w)
                        uw_first[g][w] = (uint32_t)ucol[(si.w0 + w < si.w1) ? (si.w0 + w) : (si.w0 < si.w1 ? si.w0 : 0)];
                    sw.next();
                }
            }

            // (contains the dependency wait; also reads the number of launches completed on this scratch so far: its
            // parity is the validity mark of this launch's z values)
            phase = z_stage(p, ctrl, work, p.zbuf, cta, tid, &seq);
            named_bar_sync(3, Z_THREADS);      // the work area is free for the expansion
        }
        if (p.trigger == 1 && tid == 0) griddep_launch_dependents();
        griddep_wait();            // (again, for the R == 0 path; a second wait returns at once)
        if (PUSH && tid == 0) ctrl->ar_seq = (ld_volatile_u32(p.ar_counter) >> 20) + 1u;      // (read by the storing threads behind a barrier)
        // Cluster mode: the other CTAs of the cluster deposit their partial sums in this (the finishing) CTA's work
        // area, which its z stage has been using until now: tell them it is free.
        if (p.cluster > 1 && (cta % p.cluster) == p.cluster - 1 && tid < p.cluster - 1)
            mbar_arrive_remote_release(map_to_cta(smem_u32(&ctrl->red_free), (uint32_t)tid));

        int seg = 0;
#pragma unroll 1
        for (SegWalk sw(u0, u1, p.nkt); !sw.done(); sw.next(), ++seg) {
            const SegInfo si = seg_info(p, T, cta, sw.first(), sw.count(), owner_mode);
            const int t = si.t, nc = si.nc, slot = si.slot;
            const int buf = seg & 1;
            const bool complete = si.complete;
            const int n = t * TILE_N + tid;
            const bool valid = n < p.N;
            const int grp = tile_group(p, t);
            const float alpha = p.alpha[grp];       // (requested here, needed after the expansion)
            const float* zbg = p.zbuf + grp * p.Rg;

            float corr[ROWS];
#pragma unroll
            for (int m = 0; m < ROWS; ++m) corr[m] = 0.f;
            // every contributor of a tile expands its share of the ranks (mode 4: the finisher expands them all)
            if (p.R > 0 && si.w0 < si.w1) {
                const int32_t* ucol = p.Ucol + (size_t)(valid ? n : 0) * p.Rw;
                uint32_t uw_sel[ZS_FIRST];
#pragma unroll
                for (int w = 0; w < ZS_FIRST; ++w) uw_sel[w] = (seg & 1) ? uw_first[1][w] : uw_first[0][w];
                bool on_tc = false;
                if constexpr (ROWS >= LR_TC_MIN_ROWS) on_tc = p.lr_tc != 0;
                if (on_tc) {
                    if constexpr (ROWS >= LR_TC_MIN_ROWS) {
                        const uint32_t d2 = tmem + LR_D_COL + 32u * (uint32_t)(lrseg & 1);
                        if (!expand_z_tc<ROWS, MMA_N>(p, ctrl, lr, zbg, ucol, si.w0, si.w1, tid, phase, d2, gchunk)) break;
                        // the segment's sums: wait for its last MMA, read the accumulator (lane = this thread's column)
                        if (!wait_bar(smem_u32(&ctrl->lr_done), lrseg & 1, ctrl, p.status, p.epoch, ST_ACC_FULL, warp)) break;
                        tc_fence_after_sync();
                        float c2[MMA_N];
                        tmem_ld_acc<MMA_N>(d2 + ((uint32_t)(warp * 32) << 16), c2);
                        tc_wait_ld();
                        tc_fence_before_sync();
#pragma unroll
                        for (int m = 0; m < ROWS; ++m) corr[m] = c2[m];
                        ++lrseg;
                    }
                } else if (!expand_z<ROWS>(corr, p, ctrl, zbg, ucol, si.w0, si.w1, zs, tid, uw_sel, seg < 2, phase)) {
                    break;
                }
                if (tid == 0 && p.stamps && seg == 0) p.stamps[(size_t)cta * STAMP_WORDS + 3] = globaltimer_ns();
            }
            if (p.trigger == 2 && tid == 0 && seg == 0) griddep_launch_dependents();

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

            if (p.cluster > 1) {
                // ---- cluster mode: partial sums travel through the finisher's shared memory ----
                const uint32_t red0 = smem_u32(work + RED_OFF);
                if (!si.finisher) {
                    wait_bar_cluster(smem_u32(&ctrl->red_free), 0, ctrl, p.status, p.epoch, ST_CLUSTER);
                    if (!epi_sync_ok(ctrl)) break;
                    const uint32_t dst = map_to_cta(red0 + (uint32_t)((slot * ROWS) * TILE_N + tid) * 4u, (uint32_t)(p.cluster - 1));
#pragma unroll
                    for (int m = 0; m < ROWS; ++m) st_cluster_f32(dst + (uint32_t)(m * TILE_N) * 4u, v[m]);
                    named_bar_sync(1, EPI_THREADS);     // all 128 stores precede thread 0's (cumulative) release
                    if (tid == 0) mbar_arrive_remote_release(map_to_cta(smem_u32(&ctrl->red_bar), (uint32_t)(p.cluster - 1)));
                } else {
                    wait_bar_cluster(smem_u32(&ctrl->red_bar), 0, ctrl, p.status, p.epoch, ST_CLUSTER);
                    if (!epi_sync_ok(ctrl)) break;
                    const float* red = reinterpret_cast<const float*>(work + RED_OFF);
#pragma unroll 1
                    for (int sl = 0; sl < nc - 1; ++sl)
#pragma unroll
                        for (int m = 0; m < ROWS; ++m) v[m] += red[(sl * ROWS + m) * TILE_N + tid];
                    if (valid) {
#pragma unroll
                        for (int m = 0; m < ROWS; ++m) {
                            if (m < p.M) {
                                float o = v[m];
                                if (p.C) o += __bfloat162float(p.C[(size_t)m * p.N + n]);
                                if (p.mode & 0x400) {
                                    reinterpret_cast<float*>(p.Y)[(size_t)m * p.N + n] = o;
                                    if constexpr (PUSH) ar_push(p, ctrl->ar_seq, m * p.N + n, o);
                                } else p.Y[(size_t)m * p.N + n] = __float2bfloat16(o);
                            }
                        }
                    }
                }
            } else if (!si.finisher) {
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
                            if (p.mode & 0x400) {
                                reinterpret_cast<float*>(p.Y)[(size_t)m * p.N + n] = o;
                                if constexpr (PUSH) ar_push(p, ctrl->ar_seq, m * p.N + n, o);
                            } else p.Y[(size_t)m * p.N + n] = __float2bfloat16(o);
                        }
                    }
                }
            }
            if (tid == 0 && p.stamps && seg == 0) p.stamps[(size_t)cta * STAMP_WORDS + 5] = globaltimer_ns();
        }
    }

    // ---------------- common exit ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0 && p.stamps) { p.stamps[(size_t)cta * STAMP_WORDS + 13] = globaltimer_ns(); p.stamps[(size_t)cta * STAMP_WORDS + 6] = clock64(); }
    if (ctrl->abort) {
        // give copies that may still be in flight time to land before the shared memory is released
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    // The last CTA to get here advances the scratch's launch count, which flips the validity mark of z for the next
    // launch (whose reads of the count follow the completion of this grid).
    if (tid == 0 && p.R > 0) {
        if (atomicAdd(p.z_counter + 1, 1u) == (uint32_t)p.G - 1u) {
            p.z_counter[1] = 0u;
            p.z_counter[0] = seq + 1u;
        }
    }
    // cluster mode: no CTA leaves while a peer could still write into its shared memory (also on the failure path:
    // every CTA gets here because every wait is bounded)
    if (p.cluster > 1) cluster_sync_all();
    if (warp == MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

}  // namespace biloco
