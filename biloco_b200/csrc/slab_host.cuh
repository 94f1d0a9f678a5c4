// Host side of the row-slab schedule (mode 7): geometry, the weight re-layout kernel and the launcher.
// Included by fused_linear.cu (one translation unit: the launch options are shared).
#pragma once
#include "slab_kernel.cuh"
#include "slab_plain_kernel.cuh"

namespace biloco {
namespace slab {

struct Geo {
    int Rt, kg, nkt, nsu, G;        // rows per CTA, k-tiles per super-unit, k-tiles, super-units per CTA, CTAs with rows
    int grid;                       // CTAs launched: one per SM, the ones beyond G only take part in the z stage
    int nbp;                        // MMA N: kg * Rt rounded up to a multiple of 16
    int nsl, nr;                    // z stage: rank slices per activation row, most ranks of a slice
    int rows;                       // 1, 2 or 4 (template parameter; three rows run as four)
    int stage_bytes, ring, atile_bytes, lut;
    int off_ring, off_ctrl, off_us, off_work, off_accp, off_asf, xs_off, smem_bytes;
};

// Weight layout: depends on N, K and the SM count only (not on M), so one re-laid copy serves every M the schedule takes.
static bool slab_layout(int N, int K, int num_sms, Geo* g) {
    if (N < 8 || (N % 8) || K < 512 || (K % 512) || num_sms < 1) return false;      // (K / 256 must be even: a thread's span is pairs)
    int rt = (N + num_sms - 1) / num_sms;
    rt = (rt + 7) / 8 * 8;
    if (rt > 128) return false;
    g->Rt = rt;
    g->G = (N + rt - 1) / rt;
    g->nkt = K / KT;
    // as many k-tiles per MMA as its 256 operand rows take (at most KG_MAX), then evened out over the super-units
    int kmax = 256 / rt;
    if (kmax > KG_MAX) kmax = KG_MAX;
    if (kmax > g->nkt) kmax = g->nkt;
    g->nsu = (g->nkt + kmax - 1) / kmax;
    g->kg = (g->nkt + g->nsu - 1) / g->nsu;
    g->nbp = (g->kg * rt + 15) / 16 * 16;
    g->stage_bytes = (g->kg * rt * UNIT_ROW_BYTES + 1023) / 1024 * 1024;
    return true;
}

static bool slab_geometry(int M, int N, int K, int R, int num_sms, bool coresident, Geo* g, bool raw = false) {
    // (the raw-activation form exists for one and two rows)
    if (M < 1 || M > (raw ? 2 : 4) || R < 0) return false;
    if (!slab_layout(N, K, num_sms, g)) return false;
    g->rows = M <= 2 ? M : 4;
    if (g->kg * g->rows > 32) return false;                                        // (operand rows: one TMEM lane quadrant)
    // One CTA per SM, always: with exactly as many CTAs as SMs every SM hosts one CTA of this launch beside one of the
    // next, and none hosts two of the same launch (which would take turns on the SM's tensor memory).
    g->grid = (R > 0 && g->G < num_sms) ? num_sms : g->G;
    g->nsl = g->grid / M > 1 ? g->grid / M : 1;
    g->nr = R > 0 ? (R + g->nsl - 1) / g->nsl : 0;
    if (g->nr > 2 * NRMAX) return false;
    // (more than two rows: the z stage is one pass over a staged row, the activation's scales one batch of requests)
    if (g->rows > 2 && K / 256 > 2 * XW_MAX) return false;
    const int Rw = (R + 31) / 32, Rpad = Rw * 32;
    const int vt = g->nr * (K / 8);
    if (vt > VT_SLAB_MAX) return false;
    // work area: during the z stage the sign words of the CTA's ranks and a staged copy of the activation row (rows of
    // up to 8192 elements; longer rows are read span by span without staging); afterwards z and the expansion's
    // partial sums
    g->xs_off = (vt + 15) / 16 * 16;
    // (raw-activation form: all M rows of the activation are formed and staged there, whatever K and R are)
    const int zwork = raw ? g->xs_off + M * 2 * K : (R > 0 ? g->xs_off + (K / 256 <= 2 * XW_MAX ? 2 * K : 0) : 0);
    // expansion by table (16 sums per group of four ranks: 16 bytes per rank and row): always where the table is small, and
    // up to 16 KB (two rows at r = 512, four at r = 256) where it costs no stage of the weight ring
    const int work_plain = g->rows * Rpad * 4 + g->rows * Rw * g->Rt * 4, table = g->rows * Rpad * 16;
    g->atile_bytes = (g->kg * g->rows + 7) / 8 * 1024;
    const int atiles = g->nsu * g->atile_bytes;
    // (more than two rows: the read-out area also holds the z stage's per-warp sums, 8 x 17 floats, while it is idle)
    const int us = (Rw * g->Rt * 4 + 15) / 16 * 16;
    const int accp = (g->rows > 2 && g->kg * g->rows * g->nbp * 4 < 1024) ? 1024 : g->kg * g->rows * g->nbp * 4;
    const int asf = g->nkt * g->rows * 16;
    const int budget = (coresident ? CORESIDENT_SMEM : SMEM_BUDGET) - 1024;       // (alignment slack)
    auto ring_for = [&](int work_bytes, int* fixed_out) {
        int w = work_bytes < zwork ? zwork : work_bytes;
        w = (w + 15) / 16 * 16;
        const int fixed = atiles + 1024 + us + w + accp + asf;
        int r = (budget - fixed) / g->stage_bytes;
        if (r > MAX_RING) r = MAX_RING;
        if (r > g->nsu) r = g->nsu;
        *fixed_out = w;
        return r;
    };
    int work = 0, work_t = 0;
    int ring = ring_for(work_plain, &work);
    g->lut = 0;
    if (R > 0 && table <= 16384) {
        const int ring_t = ring_for(work_plain + table, &work_t);
        if (table <= 8192 || ring_t == ring) { g->lut = 1; ring = ring_t; work = work_t; }
    }
    if (ring < 1 || (ring < 2 && g->nsu >= 2)) return false;
    g->ring = ring;
    g->off_ring = atiles;
    g->off_ctrl = g->off_ring + ring * g->stage_bytes;
    g->off_us = g->off_ctrl + 1024;
    g->off_work = g->off_us + us;
    g->off_accp = g->off_work + work;
    g->off_asf = g->off_accp + accp;
    int total = g->off_asf + asf;
    // The tensor core reads 128 rows x 128 bytes from an activation tile's base and nbp rows x 128 bytes from a stage's
    // base, whatever lies there: both windows must stay inside the allocation.
    const int a_end = (g->nsu - 1) * g->atile_bytes + 16384;
    const int w_end = g->off_ring + (ring - 1) * g->stage_bytes + g->nbp * 128;
    if (total < a_end) total = a_end;
    if (total < w_end) total = w_end;
    g->smem_bytes = total + 1024;
    return g->smem_bytes <= (coresident ? CORESIDENT_SMEM : SMEM_BUDGET);
}

// One block per (CTA slab c, k-tile kt): the unit's codes go to MMA row g Rt + r of its super-unit with the 128-byte
// swizzle applied (16-byte chunk ch at chunk ch ^ (r & 7)), its block scales (four 32-bit words per row, one per 64-k
// chunk) behind the codes of all units of the super-unit.
__global__ void tile_weights_slab_kernel(const uint8_t* __restrict__ W, const uint8_t* __restrict__ W_sf, uint8_t* __restrict__ out,
                                         int N, int K, int Rt, int kg, int nkt) {
    const int c = blockIdx.x / nkt, kt = blockIdx.x - c * nkt;
    const int j = kt / kg, g = kt - j * kg;
    const int nu = (nkt - j * kg) < kg ? (nkt - j * kg) : kg;
    uint8_t* su = out + ((size_t)c * nkt + (size_t)j * kg) * Rt * UNIT_ROW_BYTES;
    for (int i = threadIdx.x; i < Rt * 8; i += blockDim.x) {
        const int r = i >> 3, ch = i & 7;
        const int n = c * Rt + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (n < N) v = *reinterpret_cast<const uint4*>(W + (size_t)n * (K >> 1) + kt * KT_BYTES + ch * 16);
        *reinterpret_cast<uint4*>(su + (size_t)(g * Rt + r) * 128 + ((ch ^ (r & 7)) * 16)) = v;
    }
    for (int i = threadIdx.x; i < Rt * 4; i += blockDim.x) {
        const int r = i >> 2, a = i & 3;
        const int n = c * Rt + r;
        uint32_t v = 0u;
        if (n < N)
            v = *reinterpret_cast<const uint32_t*>(W_sf + ((size_t)(n >> 7) * (K >> 6) + (size_t)kt * 4 + a) * 512 + (n & 31) * 16 + ((n >> 5) & 3) * 4);
        *reinterpret_cast<uint32_t*>(su + (size_t)nu * Rt * 128 + (size_t)(g * Rt + r) * 16 + a * 4) = v;
    }
}

template <int ROWS, bool RAW>
static int slab_launch_rows(const SlabParams& p, const Geo& g, bool pdl, cudaStream_t stream) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(slab_kernel<ROWS, RAW>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET) != cudaSuccess)
            return BILOCO_ERR_CUDA;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)g.grid);
    cfg.blockDim = dim3(NT);
    cfg.dynamicSmemBytes = (size_t)g.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, slab_kernel<ROWS, RAW>, p);
    return e == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}

// The same for the plain form (slab_plain_kernel.cuh: activations quantised by the caller).
template <int ROWS>
static int slabp_launch_rows(const slabp::SlabParams& p, const Geo& g, bool pdl, cudaStream_t stream) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(slabp::slab_kernel<ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET) != cudaSuccess)
            return BILOCO_ERR_CUDA;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)g.grid);
    cfg.blockDim = dim3(slabp::NT);
    cfg.dynamicSmemBytes = (size_t)g.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, slabp::slab_kernel<ROWS>, p);
    return e == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}

}  // namespace slab
}  // namespace biloco
