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
//    order ("stream-K", schedule.h), so every SM streams the same number of weight bytes whatever N is.
//  * Warp roles (448 threads): warps 0-3 = z stage, U expansion and epilogue (thread = TMEM lane = weight row);
//    warps 4-7 = feeders (first copy requests; scale factors from shared memory into TMEM with tcgen05.st, one
//    32-lane quadrant each); warps 8-11 = second half of the z stage; warp 12 = TMEM allocation + MMA issue;
//    warp 13 = refills (re-requests stages as they come free).
//  * Per stage: one contiguous 18 KB record (codes already swizzled + the four 512 B scale atoms) by a bulk copy, or
//    from row-major weights a 2-D TMA tile (128 rows x 128 B, 128-byte swizzle) + a bulk copy of the atoms; the
//    activation tile likewise. Four tcgen05.mma kind::mxf4nvf4 (K = 64 each) per stage.
//  * A tile whose k-range is shared by several CTAs is finished by the CTA that holds its last k-tile: the
//    others store fp32 partials (alpha*acc + their slice of the low-rank term) to scratch and bump the tile's
//    counter; the finisher adds them in slot order (deterministic), rounds and stores.
//  * Low-rank term: at entry every CTA computes a slice of the ranks of z (all M rows) on CUDA cores from the
//    bit-packed V and publishes it in scratch. There is no completion flag: each published value carries a
//    validity mark in its lowest mantissa bit that flips from launch to launch, and the consumers poll the
//    values themselves. Each contributor of a tile expands z through the packed U signs for its share of the
//    rank words and adds the result to the accumulators read back from TMEM.
//    Tile counters return to zero inside the launch and the last CTA to leave advances the scratch's launch
//    count, so launches on one scratch need no clearing in between and a captured CUDA graph can be replayed;
//    launches that share a scratch must not overlap.
//  * Every wait (mbarrier, counter) is bounded by a %globaltimer budget; a wait that runs out records a code in
//    the status words of the scratch, raises a CTA-wide abort flag, and the CTA leaves through the common exit
//    (TMEM freed) instead of hanging.
//  * The machine code is kept small on purpose (rolled loops, non-inlined wait helpers, one instantiation per
//    row count): each CTA runs it once, cold, and instruction fetches queue behind the weight stream.
//
// Device code: fused_cfg.cuh (configuration, waits), fused_lowrank.cuh (z stage, expansion), fused_kernel.cuh.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

#include "../../include/biloco_b200.h"
#include "fused_kernel.cuh"
#include "ztc_kernel.cuh"

namespace biloco {

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

static int g_ring = 0;                           // pipeline stages: 0 = chosen per kernel, else clamped to what fits
static int g_use_pdl = 1;                        // launch with programmatic stream serialization

static unsigned long long* g_stamps = nullptr;   // debug time-stamp buffer for subsequent launches (or null)
static size_t g_stamps_bytes = 0;
static size_t g_stamps_seq = 0;
static int g_lr_tc = 1;                          // expansion on the tensor cores where the kernel supports it
static int g_ztc = -1;                           // z stage as a tensor-core launch of its own: -1 from ZTC_MIN_ROWS rows, 0 never, n > 0 from n rows
static int g_trigger = -1;                        // < 0: chosen per launch (see launch())
static unsigned long long g_wait_ns = WAIT_BUDGET_NS;   // budget of a device-side wait (row-slab schedule)
static int g_inflight = 0;                        // row-slab schedule: weight records in flight while the ring fills (0: all)
static bool slab_coresident() { return g_use_pdl != 0; }      // (two launches side by side on an SM: half of its shared memory each)
static int g_dbg = 0;                             // row-slab schedule: timing experiments (see SlabParams::dbg)
static int g_skip_publish = -1;                   // test aid: this CTA of a row-slab launch keeps its z values to itself

// Streams on which an operand re-layout (tile_weights, tile_weights_slab, pack_u_col32) was the last thing this library
// enqueued. The fused kernels read their static operands BEFORE griddepcontrol.wait when they are launched with
// programmatic stream serialization (that is the point: the weight prefetch overlaps the previous kernel), so a fused
// launch that directly follows the kernel which WRITES such an operand must not start early: the first fused launch on
// such a stream goes out as a plain launch.
extern "C" unsigned long long biloco_internal_wait_ns() { return g_wait_ns; }
static std::mutex g_fresh_mu;
static std::unordered_map<cudaStream_t, int> g_fresh_streams;
extern "C" void biloco_internal_mark_relayout(cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(g_fresh_mu);
    g_fresh_streams[stream] = 1;
}
static bool consume_relayout_mark(cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(g_fresh_mu);
    auto it = g_fresh_streams.find(stream);
    if (it == g_fresh_streams.end()) return false;
    g_fresh_streams.erase(it);
    return true;
}

static int mma_n_for(int M) { return M <= 8 ? 8 : (M <= 16 ? 16 : 32); }

struct ScratchLayout {
    size_t off_zcnt, off_tilecnt, off_z, off_arec, off_ztc, off_part, part_bytes, total;
    int ntile, nkt, G, max_slots, Rw, Rpad, mma_n;
};

static bool make_layout(int M, int N, int K, int R, int num_sms, ScratchLayout* L) {
    if (M < 1 || M > 32 || N < 8 || (N % 8) || K < KT || (K % KT) || R < 0 || num_sms < 1) return false;
    L->mma_n = mma_n_for(M);
    L->ntile = (N + TILE_N - 1) / TILE_N;
    L->nkt = K / KT;
    const long long T = (long long)L->ntile * L->nkt;
    L->G = (int)(T < num_sms ? T : num_sms);
    if (!sched_fits_32bit(L->ntile, L->nkt, L->G) || (long long)R * (L->G + 1) >= (1ll << 31)) return false;
    L->max_slots = sched_max_slots(L->ntile, L->nkt, L->G);
    L->Rw = (R + 31) / 32;
    L->Rpad = L->Rw * 32;
    size_t off = 64;                                     // 16 status words
    L->off_zcnt = off; off += 64;
    L->off_tilecnt = off; off += ((size_t)L->ntile * 4 + 127) / 128 * 128;
    L->off_z = off; off += (size_t)2 * 32 * L->Rpad * sizeof(float);
    // raw-activation form of the row-slab schedule: one 16-byte record per 16-element block of the activation (M <= 2)
    L->off_arec = off; off += (M <= 2 && K % 512 == 0) ? (size_t)M * K : 0;
    L->off_ztc = off; off = (off + 64 + 255) / 256 * 256;      // arrival counters of the tensor-core z launch (16 rank blocks)
    {
        // split-K partial sums of the fused kernel; the tensor-core z launch parks its own partial sums there first
        size_t part = (size_t)L->ntile * L->max_slots * L->mma_n * TILE_N * sizeof(float);
        const int nrb = (R + 127) / 128;
        if (M >= ztc::ZTC_MIN_ROWS && nrb >= 1 && nrb <= 16 && nrb <= num_sms) {      // (fewer rows: the z launch is optional and used only if it fits)
            int nks = num_sms / nrb;
            if (nks > K / 64) nks = K / 64;
            const size_t zp = (size_t)nrb * nks * L->mma_n * 128 * sizeof(float);
            if (zp > part) part = zp;
        }
        L->off_part = off; off += part;
        L->part_bytes = part;
    }
    L->total = (off + 255) / 256 * 256;
    return true;
}

// Re-layout of the weights into the order the kernel streams them: record u = (tile t, k-tile kt) holds the 128 x 128 B
// block of codes with the 128-byte swizzle already applied (16-byte chunk c of row r stored at chunk c ^ (r & 7)),
// followed by the four 512-byte scale atoms of that block. Rows beyond N are zero.
__global__ void tile_weights_kernel(const uint8_t* __restrict__ W, const uint8_t* __restrict__ W_sf, uint8_t* __restrict__ out,
                                    int N, int K, int nkt) {
    const int u = blockIdx.x;
    const int t = u / nkt, kt = u - t * nkt;
    uint8_t* rec = out + (size_t)u * (W_TILE_BYTES + SF_TILE_BYTES);
    for (int i = threadIdx.x; i < W_TILE_BYTES / 16; i += blockDim.x) {
        const int r = i >> 3, c = i & 7;
        const int n = t * TILE_N + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (n < N) v = *reinterpret_cast<const uint4*>(W + (size_t)n * (K >> 1) + kt * KT_BYTES + c * 16);
        *reinterpret_cast<uint4*>(rec + r * 128 + ((c ^ (r & 7)) * 16)) = v;
    }
    const uint8_t* sf = W_sf + ((size_t)t * (K >> 6) + (size_t)kt * 4) * 512;
    for (int i = threadIdx.x; i < SF_TILE_BYTES / 16; i += blockDim.x)
        *reinterpret_cast<uint4*>(rec + W_TILE_BYTES + i * 16) = *reinterpret_cast<const uint4*>(sf + i * 16);
}

// Cluster mode: tile t is owned by a cluster of c CTAs that split its k-tiles; c = as many as fit on the device
// (ntile * c <= SMs), at most 8, at most one per k-tile. 0 when the shape does not suit the mode: fewer than two
// CTAs per tile, more than 8 rows (the peers' partial sums must fit the finisher's work area), or a grid that would
// leave more than a third of the SMs idle.
static int max_active_clusters(int rows, int cluster);

// on_device: also ask the driver how many such clusters the current device holds at once (needs a CUDA context); the
// host-only form (an SM count given by the caller) cannot know and assumes they all fit.
static int cluster_size_for(int M, int ntile, int nkt, int num_sms, bool on_device) {
    if (M > 8) return 0;
    int c = num_sms / ntile;
    if (c > 8) c = 8;
    if (c > nkt) c = nkt;
    const int rows = M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8));
    while (c >= 2 && (c - 1) * rows * TILE_N * 4 > RED_BYTES) --c;     // the peers' partial sums must fit beside the staged z
    if (on_device)
        while (c >= 2 && max_active_clusters(rows, c) < ntile) --c;    // every cluster of the launch must be resident at once
    if (c < 2) return 0;
    if (ntile * c * 3 < num_sms * 2) return 0;
    return c;
}

// Clusters of `cluster` CTAs of the kernel for `rows` activation rows that the current device holds at the same time
// (CTAs with the shared memory the launcher gives them: half an SM for rows <= 2, a whole SM above). Every CTA of a
// launch must be resident at once (the z exchange), so a cluster schedule needs at least one cluster slot per tile;
// the number depends on how the device's SMs are grouped, which only the driver knows. 0 when the query fails.
template <int MMA_N, int ROWS>
static int query_active_clusters(int cluster) {
    if (cudaFuncSetAttribute(fused_linear_kernel<MMA_N, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET) != cudaSuccess)
        return 0;
    if (cluster > 8 && cudaFuncSetAttribute(fused_linear_kernel<MMA_N, ROWS>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
        return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)cluster);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = ctas_per_sm(ROWS) == 2 ? (size_t)CORESIDENT_SMEM : (size_t)SMEM_BUDGET;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, fused_linear_kernel<MMA_N, ROWS>, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

static int max_active_clusters(int rows, int cluster) {
    static int cache[64][6][9];           // [device][row class][cluster size], 0 = not asked yet, -1 = query failed
    int dev = 0;
    if (cluster < 2 || cluster > 8 || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    const int rc = rows <= 1 ? 0 : (rows <= 2 ? 1 : (rows <= 4 ? 2 : (rows <= 8 ? 3 : (rows <= 16 ? 4 : 5))));
    int& c = cache[dev][rc][cluster];
    if (c == 0) {
        int n = 0;
        switch (rc) {
            case 0: n = query_active_clusters<8, 1>(cluster); break;
            case 1: n = query_active_clusters<8, 2>(cluster); break;
            case 2: n = query_active_clusters<8, 4>(cluster); break;
            case 3: n = query_active_clusters<8, 8>(cluster); break;
            case 4: n = query_active_clusters<16, 16>(cluster); break;
            default: n = query_active_clusters<32, 32>(cluster); break;
        }
        // The cluster query credits one CTA per SM also for rows <= 2, whose CTAs are built so that two share an SM
        // (launch bounds, 113 KB of shared memory). Twice the count is relied on only if the occupancy query for a
        // single CTA of that size confirms that two are resident per SM.
        if (n > 0 && rc <= 1) {
            int per_sm = 0;
            const cudaError_t e = rc == 0
                ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_linear_kernel<8, 1>, NUM_THREADS, (size_t)CORESIDENT_SMEM)
                : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_linear_kernel<8, 2>, NUM_THREADS, (size_t)CORESIDENT_SMEM);
            if (e == cudaSuccess && per_sm >= 2) n *= 2;
            else cudaGetLastError();
        }
        c = n > 0 ? n : -1;
    }
    return c > 0 ? c : 0;
}

static int rows_for(int M) { return M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : (M <= 8 ? 8 : (M <= 16 ? 16 : 32)))); }

template <int MMA_N, int ROWS>
static int launch(const CUtensorMap& tmW, const CUtensorMap& tmA, const FusedParams& p_in, cudaStream_t stream) {
    using C = Cfg<MMA_N>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(fused_linear_kernel<MMA_N, ROWS, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 SMEM_BUDGET) != cudaSuccess ||
            cudaFuncSetAttribute(fused_linear_kernel<MMA_N, ROWS, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 SMEM_BUDGET) != cudaSuccess)
            return BILOCO_ERR_CUDA;
        // (clusters of more than eight CTAs: query_active_clusters allows them for the plain instantiation)
        if (cudaFuncSetAttribute(fused_linear_kernel<MMA_N, ROWS, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
            cudaGetLastError();
        attr_set[dev] = true;
    }
    // z stage geometry: nsl rank slices per activation row, and shared memory for the sign words of one slice
    FusedParams p = p_in;
    p.nsl = p.G / p.M > 1 ? p.G / p.M : 1;
    int vt = VT_MIN_BYTES;
    if (p.R > 0) {
        const int ranks = (p.R + p.nsl - 1) / p.nsl;
        const int kc = p.K < XK ? p.K : XK;
        vt = (ranks * (kc / 8) + 1023) & ~1023;
        if (vt < VT_MIN_BYTES) vt = VT_MIN_BYTES;
        if (vt > VT_MAX_BYTES) vt = VT_MAX_BYTES;
    }
    p.vt_bytes = vt;
    // z on the tensor cores as a launch of its own in front of this one (ztc_kernel.cuh): the fused kernel then has no z items
    int dev_sms = 0;
    cudaDeviceGetAttribute(&dev_sms, cudaDevAttrMultiProcessorCount, dev);
    const int ztc_from = g_ztc < 0 ? ztc::ZTC_MIN_ROWS : g_ztc;
    bool use_ztc = ztc_from > 0 && p.M >= ztc_from && p.R > 0 && p.ztc_cnt != nullptr && dev_sms > 0;
    int z_nrb = 0, z_nks = 0;
    if (use_ztc) {
        z_nrb = (p.R + 127) / 128;
        if (z_nrb > 16 || z_nrb > dev_sms) use_ztc = false;
        else {
            z_nks = dev_sms / z_nrb;
            if (z_nks > p.K / 64) z_nks = p.K / 64;
            if ((size_t)z_nrb * z_nks * MMA_N * 128 * sizeof(float) > p.part_bytes) use_ztc = false;
        }
    }
    if (use_ztc) p.nsl = 0;
    // expansion on the tensor cores from 16 rows up (below that the CUDA-core form is as fast); its operand buffers sit
    // behind the sign words
    p.lr_tc = (ROWS >= LR_TC_MIN_ROWS && p.R > 0 && g_lr_tc) ? 1 : 0;
    const int extra = p.lr_tc ? lr_bytes(MMA_N) : 0;
    // where a CTA lets the next launch of the stream start (measured at K = N = 5120: once the activation row has
    // landed for the cluster schedule, straight after set-up otherwise)
    p.trigger = g_trigger >= 0 ? g_trigger : (p.cluster > 1 ? 3 : 0);
    // Ring depth decides how many CTAs share an SM: with the short ring the next launch of the stream moves in beside
    // this one (only useful when launches overlap, i.e. with programmatic dependent launch).
    int ring = C::stages_alone(vt + extra);
    if (g_ring) ring = g_ring < ring ? g_ring : ring;
    else if (ctas_per_sm(ROWS) == 2 && g_use_pdl && C::stages_shared(vt + extra) >= SF_SETS) ring = C::stages_shared(vt + extra);
    if (ring < SF_SETS) ring = SF_SETS;
    p.ring = ring;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.G);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = (size_t)C::smem_bytes(ring, vt + extra);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    // Every CTA of the grid must be resident at the same time (the z exchange). A cluster launch whose CTAs each take a
    // whole SM and together nearly all SMs (48 clusters of 3 on 148 SMs, say) only fits when the clusters pack perfectly;
    // started early, beside the last CTAs of a predecessor with another cluster shape, the first clusters were placed
    // where the rest no longer fitted and the launch sat until its waits ran out (seen with q/k/v stacked at M = 8 behind
    // a 7-CTA-cluster launch). Such launches start on an empty device: no programmatic early start for them.
    const bool tight_clusters = p.cluster > 1 && ctas_per_sm(ROWS) == 1 && p.G * 20 > dev_sms * 17;
    bool after_relayout = consume_relayout_mark(stream);
    if (use_ztc) {
        ztc::ZtcParams z;
        z.Vp = p.Vp; z.X = p.X; z.S = p.S; z.zbuf = p.zbuf; z.part = p.partials; z.cnt = p.ztc_cnt; z.z_counter = p.z_counter;
        z.status = p.status; z.wait_ns = WAIT_BUDGET_NS; z.M = p.M; z.K = p.K; z.R = p.R; z.Rpad = p.Rpad; z.nrb = z_nrb; z.nks = z_nks;
        z.epoch = p.epoch;
        cudaLaunchConfig_t zc = {};
        zc.gridDim = dim3((unsigned)(z_nrb * z_nks));
        zc.blockDim = dim3(ztc::ZT);
        zc.dynamicSmemBytes = (size_t)(1024 + ztc::NBUF * (ztc::A_BYTES + MMA_N * 128) + 4096);
        static bool zattr[64] = {false};
        if (dev >= 0 && dev < 64 && !zattr[dev]) {
            if (cudaFuncSetAttribute(ztc::ztc_kernel<MMA_N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess)
                return BILOCO_ERR_CUDA;
            zattr[dev] = true;
        }
        zc.stream = stream;
        cudaLaunchAttribute za[1];
        int nz = 0;
        if (g_use_pdl && !after_relayout) {
            za[nz].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            za[nz].val.programmaticStreamSerializationAllowed = 1;
            ++nz;
        }
        zc.attrs = za;
        zc.numAttrs = nz;
        if (cudaLaunchKernelEx(&zc, ztc::ztc_kernel<MMA_N>, z) != cudaSuccess) return BILOCO_ERR_CUDA;
        after_relayout = false;      // (the z launch stands between the re-layout and this one)
    }
    if (g_use_pdl && !tight_clusters && !after_relayout) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (p.cluster > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)p.cluster;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    // (the instantiation whose epilogue pushes to the peers only where a group of more than one rank is given)
    const cudaError_t e = p.ar_world > 1 ? cudaLaunchKernelEx(&cfg, fused_linear_kernel<MMA_N, ROWS, true>, tmW, tmA, p)
                                         : cudaLaunchKernelEx(&cfg, fused_linear_kernel<MMA_N, ROWS, false>, tmW, tmA, p);
    return e == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}

}  // namespace biloco

#include "slab_host.cuh"

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
    return L.off_part;      // status words, counters and the z hand-off area (whose validity marks are relative to the counters)
}

extern "C" int biloco_b200_max_active_clusters(int M, int cluster) {
    if (M < 1 || M > 32) return 0;
    return max_active_clusters(rows_for(M), cluster);
}

extern "C" int biloco_b200_mode_supported(int M, int N, int K, int R, int mode, int num_sms) {
    const bool on_device = num_sms == 0;
    if (num_sms == 0) num_sms = device_sm_count();
    ScratchLayout L;
    if (!make_layout(M, N, K, R, num_sms, &L)) return 0;
    if (mode == BILOCO_MODE_COUNTER || mode == BILOCO_MODE_OWNER) return 1;
    if (mode == BILOCO_MODE_CLUSTER) return cluster_size_for(M, L.ntile, L.nkt, num_sms, on_device) >= 2 ? 1 : 0;
    if (mode == BILOCO_MODE_SLAB) {
        slab::Geo g;
        return slab::slab_geometry(M, N, K, R, num_sms, slab_coresident(), &g) ? 1 : 0;
    }
    return 0;
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

extern "C" size_t biloco_b200_tiled_bytes(int N, int K) {
    if (N < 1 || K < KT || (K % KT)) return 0;
    return (size_t)((N + TILE_N - 1) / TILE_N) * (K / KT) * (W_TILE_BYTES + SF_TILE_BYTES);
}

extern "C" int biloco_b200_tile_weights(const void* W_codes, const void* W_sf, void* W_tiled, int N, int K, biloco_stream_t stream) {
    if (!W_codes || !W_sf || !W_tiled) return BILOCO_ERR_NULL;
    if (N < 1 || K < KT || (K % KT)) return BILOCO_ERR_SHAPE;
    if (((uintptr_t)W_tiled & 15) || ((uintptr_t)W_codes & 15) || ((uintptr_t)W_sf & 15) || ((uintptr_t)W_tiled & 15)) return BILOCO_ERR_ALIGN;
    const int nkt = K / KT;
    const long long units = (long long)((N + TILE_N - 1) / TILE_N) * nkt;
    if (units > 0x7fffffffll) return BILOCO_ERR_LIMIT;
    tile_weights_kernel<<<(unsigned)units, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)W_codes, (const uint8_t*)W_sf,
                                                                            (uint8_t*)W_tiled, N, K, nkt);
    biloco_internal_mark_relayout((cudaStream_t)stream);
    return cudaGetLastError() == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}

// Raw-activation arguments of the row-slab schedule (the kernel quantises the activation itself).
struct SlabAct {
    const void* Xraw; const void* norm_w; const void* smooth; const float* w_gscale; float* act_out; float eps; int rule; int swiglu;
};

static int slab_launch(const void* W_slab, const float* alpha, const void* A_codes, const void* A_sf, const void* X_bf16,
                       const void* V_packed, const int32_t* U_col32, const void* S_bf16, const void* C_bf16, void* Y, void* scratch,
                       const ScratchLayout& L, int M, int N, int K, int R, int mode, int epoch, int sms, const SlabAct* act,
                       cudaStream_t stream) {
    slab::Geo g;
    if (!slab::slab_geometry(M, N, K, R, sms, slab_coresident(), &g, act != nullptr)) return BILOCO_ERR_SHAPE;
    if (!W_slab) return BILOCO_ERR_NULL;
    if ((uintptr_t)W_slab & 15) return BILOCO_ERR_ALIGN;
    uint8_t* sc = (uint8_t*)scratch;
    // the fields both forms of the kernel share (two parameter structs: see slab_plain_kernel.cuh)
    auto fill = [&](auto& q, int stamp_words) {
        q.W_slab = (const uint8_t*)W_slab;
        q.A_codes = (const uint8_t*)A_codes;
        q.A_sf = (const uint8_t*)A_sf;
        q.alpha = alpha;
        q.X = (const __nv_bfloat16*)X_bf16;
        q.Vp = (const uint8_t*)V_packed;
        q.Ucol = U_col32;
        q.S = (const __nv_bfloat16*)S_bf16;
        q.C = (const __nv_bfloat16*)C_bf16;
        q.Y = Y;
        q.status = (int32_t*)sc;
        q.z_counter = (uint32_t*)(sc + L.off_zcnt);
        q.zbuf = (float*)(sc + L.off_z);
        q.M = M; q.N = N; q.K = K; q.R = R; q.Rw = L.Rw; q.Rpad = L.Rpad;
        q.Rt = g.Rt; q.kg = g.kg; q.nkt = g.nkt; q.nsu = g.nsu; q.G = g.grid; q.Grows = g.G;
        q.nsl = g.nsl;
        q.ring = g_ring > 0 && g_ring < g.ring ? g_ring : g.ring;
        q.stage_bytes = g.stage_bytes;
        // (a shorter ring keeps the offsets computed for the full one: the stages simply stay unused)
        q.nbp = g.nbp; q.atile_bytes = g.atile_bytes;
        q.off_ring = g.off_ring; q.off_ctrl = g.off_ctrl; q.off_us = g.off_us; q.off_work = g.off_work; q.off_accp = g.off_accp;
        q.xs_off = g.xs_off; q.off_asf = g.off_asf;
        q.epoch = (uint32_t)epoch;
        q.mode = mode;
        q.wait_ns = g_wait_ns;
        q.skip_publish_cta = g_skip_publish;
        q.trigger = g_trigger >= 0 ? g_trigger : 1;      // (measured: 8.3 us per call at K = N = 5120 against 8.4 with 0)
        q.inflight = g_inflight;
        q.lut = g.lut;
        q.dbg = g_dbg;
        q.stamps = nullptr;
        if (g_stamps && g_stamps_bytes >= (size_t)g.grid * stamp_words * 8) {
            const size_t per = (size_t)g.grid * stamp_words, slots = g_stamps_bytes / (per * 8);
            q.stamps = g_stamps + (g_stamps_seq++ % slots) * per;
        }
    };
    const bool pdl = g_use_pdl != 0 && !consume_relayout_mark(stream);
    if (!act) {
        slabp::SlabParams q;
        fill(q, slabp::SLAB_STAMPS);
        return M <= 1 ? slab::slabp_launch_rows<1>(q, g, pdl, stream)
                      : (M == 2 ? slab::slabp_launch_rows<2>(q, g, pdl, stream) : slab::slabp_launch_rows<4>(q, g, pdl, stream));
    }
    slab::SlabParams q;
    fill(q, slab::SLAB_STAMPS);
    q.act_rec = (unsigned long long*)(sc + L.off_arec);
    q.Xraw = (const __nv_bfloat16*)act->Xraw;
    q.norm_w = (const __nv_bfloat16*)act->norm_w;
    q.smooth = (const __nv_bfloat16*)act->smooth;
    q.w_gscale = act->w_gscale;
    q.act_out = act->act_out;
    q.eps = act->eps; q.act_rule = act->rule; q.act_swiglu = act->swiglu;
    // (the raw form's MMAs start ~6 us after the dependency wait: released at set-up, the next launch moves in as soon as the
    // previous one has left and its weight burst is over before this launch fetches its late record; released after the
    // z stage, as the plain form does, the burst lands on that fetch. Measured end to end: 13.85 against 14.56 us per layer.)
    if (g_trigger < 0) q.trigger = 0;
    return M <= 1 ? slab::slab_launch_rows<1, true>(q, g, pdl, stream) : slab::slab_launch_rows<2, true>(q, g, pdl, stream);
}

// Row-parallel use: where the epilogue pushes its fp32 outputs (peer_reduce.cu's receive buffers).
struct ArPush {
    void* const* recv_ptrs_dev; const int* status; int world, rank, slot_elems;
};

static int fused_linear_impl(const void* W_codes, const void* W_sf, const void* W_tiled, const float* alpha, const void* A_codes,
                             const void* A_sf, const void* A_rec, const void* X_bf16, const void* V_packed, const int32_t* U_col32,
                             const void* S_bf16, const void* C_bf16, void* Y_bf16, void* scratch,
                             size_t scratch_bytes, int M, int A_rows, int N, int K, int R, int mode, int epoch,
                             biloco_stream_t stream, int n_groups = 1, const int* group_rows = nullptr, const ArPush* ar = nullptr) {
    if ((uintptr_t)A_rec & 15) return BILOCO_ERR_ALIGN;
    // column groups: R ranks per group, group g covers group_rows[g] output columns (whole 128-column tiles)
    int gtile[3] = {0x7fffffff, 0x7fffffff, 0x7fffffff};
    const int Rg = R;
    if (n_groups != 1) {
        if (n_groups < 1 || n_groups > 4 || !group_rows || R < 32 || (R % 32)) return BILOCO_ERR_SHAPE;
        long long rows = 0;
        for (int g = 0; g < n_groups; ++g) {
            if (group_rows[g] < TILE_N || (group_rows[g] % TILE_N)) return BILOCO_ERR_SHAPE;
            rows += group_rows[g];
            if (g < n_groups - 1) gtile[g] = (int)(rows / TILE_N);
        }
        if (rows != N) return BILOCO_ERR_SHAPE;
        if ((long long)R * n_groups > 0x7fffffff) return BILOCO_ERR_LIMIT;
        R *= n_groups;
    }
    if ((!W_tiled && (!W_codes || !W_sf)) || !alpha || !A_codes || !A_sf || !Y_bf16 || !scratch) return BILOCO_ERR_NULL;
    if (R > 0 && (!X_bf16 || !V_packed || !U_col32 || !S_bf16)) return BILOCO_ERR_NULL;
    if ((mode & 0xff) != BILOCO_MODE_COUNTER && (mode & 0xff) != BILOCO_MODE_OWNER && (mode & 0xff) != BILOCO_MODE_CLUSTER &&
        (mode & 0xff) != BILOCO_MODE_SLAB)
        return BILOCO_ERR_MODE;
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

    if ((mode & 0xff) == BILOCO_MODE_SLAB) {
        // row slabs: W_tiled is the copy made by biloco_b200_tile_weights_slab (required), one column group
        if (n_groups != 1) return BILOCO_ERR_SHAPE;
        return slab_launch(W_tiled, alpha, A_codes, A_sf, X_bf16, V_packed, U_col32, S_bf16, C_bf16, Y_bf16, scratch, L, M, N, K, R,
                           mode, epoch, sms, nullptr, (cudaStream_t)stream);
    }

    CUtensorMap tmW, tmA;
    int rc = get_tensor_map(A_codes, A_rows, K / 2, L.mma_n, &tmA);
    if (rc != BILOCO_OK) return rc;
    if (W_tiled) tmW = tmA;     // not used by the kernel on the tiled path
    else rc = get_tensor_map(W_codes, N, K / 2, TILE_N, &tmW);
    if (rc != BILOCO_OK) return rc;

    uint8_t* sc = (uint8_t*)scratch;
    FusedParams p;
    p.W_tiled = (const uint8_t*)W_tiled;
    p.W_sf = (const uint8_t*)W_sf;
    p.A_sf = (const uint8_t*)A_sf;
    p.A_rec = (const uint8_t*)A_rec;
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
    p.ztc_cnt = (uint32_t*)(sc + L.off_ztc);
    p.part_bytes = L.part_bytes;
    p.ar_recv = nullptr; p.ar_counter = nullptr; p.ar_world = 0; p.ar_rank = 0; p.ar_slot = 0;
    if (ar) {
        if (!(mode & 0x400) || (mode & 0xff) == BILOCO_MODE_SLAB) return BILOCO_ERR_MODE;      // fp32 partial sums of the tile kernels only
        if (!ar->recv_ptrs_dev || !ar->status) return BILOCO_ERR_NULL;
        if (ar->world < 2 || ar->world > 16 || ar->rank < 0 || ar->rank >= ar->world || (long long)M * N > ar->slot_elems) return BILOCO_ERR_SHAPE;
        if (((uintptr_t)ar->recv_ptrs_dev & 7) || ((uintptr_t)ar->status & 3)) return BILOCO_ERR_ALIGN;
        p.ar_recv = (uint2* const*)ar->recv_ptrs_dev;
        p.ar_counter = (const uint32_t*)ar->status + 8;
        p.ar_world = ar->world; p.ar_rank = ar->rank; p.ar_slot = ar->slot_elems;
    }
    p.M = M; p.N = N; p.K = K; p.R = R; p.Rw = (Rg + 31) / 32; p.Rpad = L.Rpad;
    p.ngroups = n_groups; p.Rg = Rg;
    for (int g = 0; g < 3; ++g) p.gtile[g] = gtile[g];
    p.ntile = L.ntile; p.nkt = L.nkt; p.G = L.G; p.max_slots = L.max_slots;
    p.epoch = (uint32_t)epoch;
    p.mode = mode;
    p.cluster = 0;
    p.ring = g_ring;
    if ((mode & 0xff) == BILOCO_MODE_CLUSTER) {
        p.cluster = cluster_size_for(M, L.ntile, L.nkt, sms, true);
        if (p.cluster < 2) return BILOCO_ERR_SHAPE;
        p.G = L.ntile * p.cluster;
    }
    p.stamps = nullptr;
    if (g_stamps && g_stamps_bytes >= (size_t)p.G * STAMP_WORDS * 8) {     // consecutive launches rotate through the buffer
        const size_t per = (size_t)p.G * STAMP_WORDS, slots = g_stamps_bytes / (per * 8);
        p.stamps = g_stamps + (g_stamps_seq++ % slots) * per;
    }

    cudaStream_t s = (cudaStream_t)stream;
    switch (rows_for(M)) {
        case 1: return launch<8, 1>(tmW, tmA, p, s);
        case 2: return launch<8, 2>(tmW, tmA, p, s);
        case 4: return launch<8, 4>(tmW, tmA, p, s);
        case 8: return launch<8, 8>(tmW, tmA, p, s);
        case 16: return launch<16, 16>(tmW, tmA, p, s);
        default: return launch<32, 32>(tmW, tmA, p, s);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Entry point for callers that may not allocate device memory (see include/biloco_b200.h). Its scratch is the
// file-scope array below: every GPU that loads this library holds BILOCO_NOALLOC_SCRATCH_BYTES for it until exit.
// In host code the array's name is only a stand-in; the device address comes from cudaGetSymbolAddress.
// ---------------------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_noalloc_scratch[BILOCO_NOALLOC_SCRATCH_BYTES];
static void* g_noalloc_ptr[64] = {nullptr};                 // per device, filled by the first call on that device


extern "C" int biloco_b200_fused_linear(const void* W_codes, const void* W_sf, const void* W_tiled, const float* alpha, const void* A_codes,
                                        const void* A_sf, const void* X_bf16, const void* V_packed, const int32_t* U_col32,
                                        const void* S_bf16, const void* C_bf16, void* Y_bf16, void* scratch,
                                        size_t scratch_bytes, int M, int A_rows, int N, int K, int R, int mode, int epoch,
                                        biloco_stream_t stream) {
    return fused_linear_impl(W_codes, W_sf, W_tiled, alpha, A_codes, A_sf, nullptr, X_bf16, V_packed, U_col32, S_bf16, C_bf16, Y_bf16,
                             scratch, scratch_bytes, M, A_rows, N, K, R, mode, epoch, stream);
}

extern "C" int biloco_b200_fused_linear_act_supported(int M, int N, int K, int R, int num_sms) {
    if (num_sms <= 0) num_sms = device_sm_count();
    if (num_sms < 1 || M < 1 || M > 2) return 0;
    ScratchLayout L;
    if (!make_layout(M, N, K, R, num_sms, &L)) return 0;
    slab::Geo g;
    return slab::slab_geometry(M, N, K, R, num_sms, slab_coresident(), &g, true) ? 1 : 0;
}

extern "C" int biloco_b200_fused_linear_act(const void* W_slab, const float* w_gscale, const void* X_raw_bf16, const void* norm_weight_bf16,
                                            float eps, const void* smooth_bf16, int swiglu, int rule, const void* V_packed,
                                            const int32_t* U_col32, const void* S_bf16, const void* C_bf16, void* Y, float* act_out,
                                            void* scratch, size_t scratch_bytes, int M, int N, int K, int R, int flags, int epoch,
                                            biloco_stream_t stream) {
    if (!W_slab || !w_gscale || !X_raw_bf16 || !Y || !scratch) return BILOCO_ERR_NULL;
    if (R > 0 && (!V_packed || !U_col32 || !S_bf16)) return BILOCO_ERR_NULL;
    if (rule != BILOCO_RULE_STATIC_6 && rule != BILOCO_RULE_STATIC_4 && rule != BILOCO_RULE_MSE) return BILOCO_ERR_MODE;
    if (swiglu && norm_weight_bf16) return BILOCO_ERR_MODE;
    if (flags & ~0x400) return BILOCO_ERR_MODE;
    if (epoch < 1) return BILOCO_ERR_EPOCH;
    if (M < 1 || M > 2) return BILOCO_ERR_SHAPE;
    const int sms = device_sm_count();
    if (sms < 1) return BILOCO_ERR_CUDA;
    ScratchLayout L;
    if (!make_layout(M, N, K, R, sms, &L)) return BILOCO_ERR_SHAPE;
    if (scratch_bytes < L.total) return BILOCO_ERR_SCRATCH;
    if (((uintptr_t)X_raw_bf16 & 15) || ((uintptr_t)norm_weight_bf16 & 15) || ((uintptr_t)smooth_bf16 & 15) ||
        ((uintptr_t)scratch & 255) || ((uintptr_t)U_col32 & 3) || ((uintptr_t)w_gscale & 3) || ((uintptr_t)act_out & 3))
        return BILOCO_ERR_ALIGN;
    SlabAct act = {X_raw_bf16, norm_weight_bf16, smooth_bf16, w_gscale, act_out, eps, rule, swiglu ? 1 : 0};
    return slab_launch(W_slab, nullptr, nullptr, nullptr, nullptr, V_packed, U_col32, S_bf16, C_bf16, Y, scratch, L, M, N, K, R,
                       BILOCO_MODE_SLAB | (flags & 0x400), epoch, sms, &act, (cudaStream_t)stream);
}

extern "C" int biloco_b200_fused_linear_rec(const void* W_codes, const void* W_sf, const void* W_tiled, const float* alpha,
                                            const void* A_codes, const void* A_sf, const void* A_rec, const void* X_bf16,
                                            const void* V_packed, const int32_t* U_col32, const void* S_bf16, const void* C_bf16,
                                            void* Y_bf16, void* scratch, size_t scratch_bytes, int M, int A_rows, int N, int K,
                                            int R, int mode, int epoch, biloco_stream_t stream) {
    return fused_linear_impl(W_codes, W_sf, W_tiled, alpha, A_codes, A_sf, A_rec, X_bf16, V_packed, U_col32, S_bf16, C_bf16, Y_bf16,
                             scratch, scratch_bytes, M, A_rows, N, K, R, mode, epoch, stream);
}

extern "C" int biloco_b200_fused_linear_push(const void* W_codes, const void* W_sf, const void* W_tiled, const float* alpha,
                                             const void* A_codes, const void* A_sf, const void* A_rec, const void* X_bf16,
                                             const void* V_packed, const int32_t* U_col32, const void* S_bf16, const void* C_bf16,
                                             void* Y_f32, void* scratch, size_t scratch_bytes, int M, int A_rows, int N, int K,
                                             int R, int mode, int epoch, void* const* recv_ptrs_dev, const int* ar_status, int world,
                                             int rank, int slot_elems, biloco_stream_t stream) {
    const ArPush ar = {recv_ptrs_dev, ar_status, world, rank, slot_elems};
    return fused_linear_impl(W_codes, W_sf, W_tiled, alpha, A_codes, A_sf, A_rec, X_bf16, V_packed, U_col32, S_bf16, C_bf16, Y_f32,
                             scratch, scratch_bytes, M, A_rows, N, K, R, mode, epoch, stream, 1, nullptr, &ar);
}

extern "C" int biloco_b200_fused_linear_grouped(const void* W_codes, const void* W_sf, const void* W_tiled, const float* alpha,
                                                const void* A_codes, const void* A_sf, const void* A_rec, const void* X_bf16,
                                                const void* V_packed, const int32_t* U_col32, const void* S_bf16,
                                                const void* C_bf16, void* Y_bf16, void* scratch, size_t scratch_bytes, int M,
                                                int A_rows, int N, int K, int R, int n_groups, const int* group_rows, int mode,
                                                int epoch, biloco_stream_t stream) {
    if (n_groups < 1 || !group_rows) return BILOCO_ERR_NULL;
    if (n_groups == 1 && group_rows[0] != N) return BILOCO_ERR_SHAPE;
    return fused_linear_impl(W_codes, W_sf, W_tiled, alpha, A_codes, A_sf, A_rec, X_bf16, V_packed, U_col32, S_bf16, C_bf16, Y_bf16,
                             scratch, scratch_bytes, M, A_rows, N, K, R, mode, epoch, stream, n_groups, group_rows);
}

extern "C" size_t biloco_b200_act_rec_bytes(int M, int K) {
    if (M < 1 || M > 32 || K < KT || (K % KT)) return 0;
    const int mma_n = M <= 8 ? 8 : (M <= 16 ? 16 : 32);
    return (size_t)(K / KT) * (size_t)(mma_n * KT_BYTES + SF_TILE_BYTES);
}

extern "C" int biloco_b200_fused_linear_noalloc(const void* W_codes, const void* W_sf, const void* W_tiled, const float* alpha,
                                                const void* A_codes, const void* A_sf, const void* X_bf16,
                                                const void* V_packed, const int32_t* U_col32, const void* S_bf16,
                                                const void* C_bf16, void* Y_bf16, int M, int A_rows, int N, int K, int R,
                                                int mode, biloco_stream_t stream) {
    if ((!W_tiled && (!W_codes || !W_sf)) || !alpha || !A_codes || !A_sf || !Y_bf16) return BILOCO_ERR_NULL;
    if (R > 0 && (!X_bf16 || !V_packed || !U_col32 || !S_bf16)) return BILOCO_ERR_NULL;
    if ((mode & 0xff) != BILOCO_MODE_COUNTER && (mode & 0xff) != BILOCO_MODE_OWNER) return BILOCO_ERR_MODE;
    if (A_rows < M || A_rows > 128) return BILOCO_ERR_SHAPE;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BILOCO_ERR_CUDA;
    const int sms = device_sm_count();
    if (sms < 1) return BILOCO_ERR_CUDA;
    ScratchLayout L;
    if (!make_layout(M, N, K, R, sms, &L)) return BILOCO_ERR_SHAPE;
    if (L.total > (size_t)BILOCO_NOALLOC_SCRATCH_BYTES) return BILOCO_ERR_LIMIT;     // beyond the built-in scratch
    if (((uintptr_t)W_tiled & 15) || ((uintptr_t)W_codes & 15) || ((uintptr_t)A_codes & 15) || ((uintptr_t)W_sf & 15) ||
        ((uintptr_t)A_sf & 15) || ((uintptr_t)X_bf16 & 15) || ((uintptr_t)U_col32 & 3))
        return BILOCO_ERR_ALIGN;
    cudaStream_t s = (cudaStream_t)stream;

    // set-up, once per device with that device current: the array's device address
    if (!g_noalloc_ptr[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || !ptr) return BILOCO_ERR_CUDA;
        g_noalloc_ptr[dev] = ptr;
    }
    uint8_t* sc = (uint8_t*)g_noalloc_ptr[dev];

    // The array keeps what the last call left, possibly from another problem shape or from a call whose wait gave up:
    // status words, launch count, tile counters and the z area all restart from zero on every call (the z values'
    // validity marks are relative to the launch count).
    const size_t clear = L.off_part;
    if (cudaMemsetAsync(sc, 0, clear, s) != cudaSuccess) return BILOCO_ERR_CUDA;

    // tensor maps are encoded on the stack for every call (the cache of the allocating entry point grows on the heap)
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return BILOCO_ERR_CUDA;
    auto encode = [&](const void* ptr, int rows, int box_rows, CUtensorMap* out) -> bool {
        const cuuint64_t gdim[2] = {(cuuint64_t)(K / 2), (cuuint64_t)rows};
        const cuuint64_t gstride[1] = {(cuuint64_t)(K / 2)};
        const cuuint32_t box[2] = {(cuuint32_t)KT_BYTES, (cuuint32_t)box_rows};
        const cuuint32_t estr[2] = {1, 1};
        return enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    CUtensorMap tmW, tmA;
    if (!encode(A_codes, A_rows, L.mma_n, &tmA)) return BILOCO_ERR_CUDA;
    if (W_tiled) tmW = tmA;
    else if (!encode(W_codes, N, TILE_N, &tmW)) return BILOCO_ERR_CUDA;

    FusedParams p;
    p.W_tiled = (const uint8_t*)W_tiled;
    p.W_sf = (const uint8_t*)W_sf;
    p.A_sf = (const uint8_t*)A_sf;
    p.A_rec = nullptr;
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
    p.ztc_cnt = (uint32_t*)(sc + L.off_ztc);
    p.part_bytes = L.part_bytes;
    p.ar_recv = nullptr; p.ar_counter = nullptr; p.ar_world = 0; p.ar_rank = 0; p.ar_slot = 0;
    p.M = M; p.N = N; p.K = K; p.R = R; p.Rw = L.Rw; p.Rpad = L.Rpad;
    p.ngroups = 1; p.Rg = R;
    for (int g = 0; g < 3; ++g) p.gtile[g] = 0x7fffffff;
    p.ntile = L.ntile; p.nkt = L.nkt; p.G = L.G; p.max_slots = L.max_slots;
    p.epoch = 1u;
    p.mode = mode;
    p.cluster = 0;
    p.ring = g_ring;
    p.stamps = nullptr;
    switch (rows_for(M)) {
        case 1: return launch<8, 1>(tmW, tmA, p, s);
        case 2: return launch<8, 2>(tmW, tmA, p, s);
        case 4: return launch<8, 4>(tmW, tmA, p, s);
        case 8: return launch<8, 8>(tmW, tmA, p, s);
        case 16: return launch<16, 16>(tmW, tmA, p, s);
        default: return launch<32, 32>(tmW, tmA, p, s);
    }
}

extern "C" int biloco_b200_noalloc_status(int32_t* out16, biloco_stream_t stream) {
    int dev = 0;
    if (!out16) return BILOCO_ERR_NULL;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || !g_noalloc_ptr[dev]) return BILOCO_ERR_CUDA;
    return biloco_b200_read_status(g_noalloc_ptr[dev], out16, stream);
}

// (shared with the activation quantiser's launcher; not part of the public interface)
extern "C" int biloco_internal_use_pdl() { return g_use_pdl; }

extern "C" int biloco_b200_set_option(int option, int value) {
    if (option == BILOCO_OPT_PDL) { g_use_pdl = value ? 1 : 0; return BILOCO_OK; }
    if (option == BILOCO_OPT_TRIGGER) { g_trigger = value; return BILOCO_OK; }
    if (option == BILOCO_OPT_LR_TC) { g_lr_tc = value ? 1 : 0; return BILOCO_OK; }
    if (option == BILOCO_OPT_ZTC) { g_ztc = value; return BILOCO_OK; }
    if (option == BILOCO_OPT_RING) { g_ring = value <= 0 ? 0 : value; return BILOCO_OK; }
    if (option == BILOCO_OPT_WAIT_BUDGET_US) {
        g_wait_ns = value <= 0 ? WAIT_BUDGET_NS : (unsigned long long)value * 1000ull;
        return BILOCO_OK;
    }
    if (option == BILOCO_OPT_SKIP_PUBLISH) { g_skip_publish = value; return BILOCO_OK; }
    if (option == 9) { g_dbg = value; return BILOCO_OK; }      // (timing experiments; results are wrong while set)
    if (option == BILOCO_OPT_INFLIGHT) { g_inflight = value < 0 ? 0 : value; return BILOCO_OK; }
    return BILOCO_ERR_MODE;
}

extern "C" int biloco_b200_debug_stamps(void* device_buf, size_t bytes) {
    g_stamps = (unsigned long long*)device_buf;
    g_stamps_bytes = device_buf ? bytes : 0;
    g_stamps_seq = 0;
    return BILOCO_OK;
}

extern "C" size_t biloco_b200_slab_bytes(int N, int K, int num_sms) {
    if (num_sms == 0) num_sms = device_sm_count();
    slab::Geo g;
    if (!slab::slab_layout(N, K, num_sms, &g)) return 0;
    return (size_t)g.G * g.nkt * g.Rt * slab::UNIT_ROW_BYTES;
}

extern "C" int biloco_b200_slab_info(int M, int N, int K, int R, int num_sms, int* out8) {
    if (!out8) return BILOCO_ERR_NULL;
    if (num_sms == 0) num_sms = device_sm_count();
    slab::Geo g;
    if (!slab::slab_geometry(M, N, K, R, num_sms, slab_coresident(), &g)) return BILOCO_ERR_SHAPE;
    out8[0] = g.Rt; out8[1] = g.kg; out8[2] = g.nkt; out8[3] = g.nsu; out8[4] = g.grid; out8[5] = g.ring; out8[6] = g.smem_bytes;
    out8[7] = g.nr;
    return BILOCO_OK;
}

extern "C" int biloco_b200_tile_weights_slab(const void* W_codes, const void* W_sf, void* W_slab, int N, int K, int num_sms,
                                             biloco_stream_t stream) {
    if (!W_codes || !W_sf || !W_slab) return BILOCO_ERR_NULL;
    if (num_sms == 0) num_sms = device_sm_count();
    slab::Geo g;
    if (!slab::slab_layout(N, K, num_sms, &g)) return BILOCO_ERR_SHAPE;
    if (((uintptr_t)W_slab & 15) || ((uintptr_t)W_codes & 15) || ((uintptr_t)W_sf & 15)) return BILOCO_ERR_ALIGN;
    slab::tile_weights_slab_kernel<<<(unsigned)(g.G * g.nkt), 128, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)W_codes, (const uint8_t*)W_sf, (uint8_t*)W_slab, N, K, g.Rt, g.kg, g.nkt);
    biloco_internal_mark_relayout((cudaStream_t)stream);
    return cudaGetLastError() == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}

extern "C" int biloco_b200_read_status(const void* scratch, int32_t* out16, biloco_stream_t stream) {
    if (!scratch || !out16) return BILOCO_ERR_NULL;
    if (cudaMemcpyAsync(out16, scratch, 16 * sizeof(int32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream) != cudaSuccess)
        return BILOCO_ERR_CUDA;
    return cudaStreamSynchronize((cudaStream_t)stream) == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}
