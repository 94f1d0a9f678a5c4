// Greedy sign peeling  W ~ sum_i alpha_i u_i v_i^T  (u_i, v_i in {+-1}) on the GPU: the decomposition that produces the
// packed operands of the fused linear (reference: biloco/peel.py:14-42, binary_peel).
//
// The reference runs, per atom, 2 T matrix-vector products with the m x n fp32 residual, one more for the coefficient and
// a rank-one update: 2 T + 1 reads and one read + write of the residual, each its own library kernel. Here one PASS over
// the residual does a whole alternation  u = sgn(R v),  t = R^T u :
//   * a CTA owns a band of rows; it brings a few rows at a time into shared memory, each warp forms the dot product of
//     one row with v (signs applied by flipping the sign bit: exact), the row's sign u_r is known at once, and every
//     thread adds  u_r R[r][c]  for its own columns c from the rows in shared memory (fixed order: deterministic);
//   * the rank-one update of the PREVIOUS atom,  R <- R - alpha u' v'^T,  is applied while the rows are loaded in the
//     first pass of the next atom and written back from there (no separate update pass);
//   * the column sums of the CTAs are added in CTA order by a small second kernel, which also takes the signs of v, and,
//     after the last alternation, the coefficient  alpha = u^T R v / (m n)  from per-CTA partial sums of a dots-only pass.
// Per atom: T + 1 reads of the residual and one write, against the reference's 2 T + 2 reads and one write. HBM/L2-bound
// fp32 streaming; nothing here is GEMM-shaped (the operands are vectors).
//
// Arithmetic: fp32, one fused multiply-add free: products with +-1 are sign flips, sums are plain fp32 additions in a
// fixed order (per lane in column order, shuffle tree, warps / CTAs in index order). The reference's cuBLAS products add in
// an unspecified order, so signs of near-zero sums, and with them later atoms, can differ from a given cuBLAS run just as two
// cuBLAS versions differ from each other; on inputs whose sums are exact in fp32 the results are identical.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/biloco_b200.h"
#include "ptx.cuh"

namespace {

constexpr int PT = 512;                 // threads per CTA
constexpr int PW = PT / 32;
constexpr int PEEL_SMEM = 200 * 1024;   // two stages of rows + the sign bytes of v and of the previous atom's v
constexpr int MAXC = 28;                // columns per thread: n <= PT * MAXC = 14336
constexpr unsigned long long PEEL_WAIT_NS = 2000000000ull;      // bound of a wait for a row copy (2 s)

__device__ __forceinline__ float flipb(float x, uint32_t signbyte) {      // x * s, s = -1 iff signbyte = 0x80: exact
    return __uint_as_float(__float_as_uint(x) ^ (signbyte << 24));
}
__device__ __forceinline__ float flip(float x, float s) {
    return __uint_as_float(__float_as_uint(x) ^ (__float_as_uint(s) & 0x80000000u));
}
__device__ __forceinline__ float sgn1(float x) { return x < 0.f ? -1.0f : 1.0f; }      // sign with sgn(0) = +1 (NaN -> +1)

struct PeelArgs {
    float* R;                 // [m][n] residual, updated in place when `deflate`
    const float* v;           // [n] current right signs (+-1)
    float* u;                 // [m] left signs: written (passes with column sums), read (coefficient pass)
    const float* u_prev;      // [m] previous atom's signs and coefficient (deflate)
    const float* v_prev;      // [n]
    const float* alpha_prev;  // [1]
    float* colpart;           // [G][n] per-CTA column sums
    float* apart;             // [G] per-CTA partial sums of u^T R v (coefficient pass)
    int* err;                 // [1] set when a bounded wait ran out
    int m, n, rb;             // rb: rows per stage (a power of two, <= PW)
    int deflate;              // apply R <- R - alpha_prev u_prev v_prev^T to the staged rows and store them back
    int dots_only;            // coefficient pass: u is read, no column sums
};

__device__ __forceinline__ bool peel_wait(uint32_t bar, uint32_t parity, int* err) {
    if (biloco::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = biloco::globaltimer_ns();
    while (!biloco::mbar_try_wait(bar, parity)) {
        if (biloco::globaltimer_ns() - t0 > PEEL_WAIT_NS) { *err = 1; return false; }
    }
    return true;
}

// One pass over the residual (see the file header). grid = G CTAs, CTA c owns rows [c m / G, (c + 1) m / G). Rows travel
// between global and shared memory as bulk copies (one per row, two stages in flight); the warps only touch shared memory.
template <int RB>
__global__ void __launch_bounds__(PT, 1) peel_pass_kernel(PeelArgs a) {
    extern __shared__ __align__(128) uint8_t smraw[];
    const int n = a.n, nv = n >> 2;
    constexpr int rb = RB;
    float* stage0 = reinterpret_cast<float*>(smraw);                    // [2][rb][n]
    uint8_t* vs = smraw + (size_t)2 * rb * n * 4;                       // [n] sign bytes of v (0x80 = negative)
    uint8_t* vp = vs + n;                                               // [n] sign bytes of v_prev
    __shared__ __align__(8) uint64_t full[2];
    __shared__ float dseg[PW];                                          // partial dot products of the warps
    __shared__ float us[PW];                                            // signs of the stage's rows
    __shared__ float aus[PW];                                           // alpha * u_prev of the stage's rows
    __shared__ int bad;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gridDim.x, c = blockIdx.x;
    const int r0 = (int)((long long)c * a.m / G), r1 = (int)((long long)(c + 1) * a.m / G);
    const int nch = (r1 - r0 + rb - 1) / rb;
    const uint32_t row_bytes = (uint32_t)n * 4u;
    if (tid == 0) {
        biloco::mbar_init(biloco::smem_u32(&full[0]), 1);
        biloco::mbar_init(biloco::smem_u32(&full[1]), 1);
        biloco::fence_mbar_init();
        bad = 0;
    }
    __syncthreads();
    constexpr int wpr = PW / RB;                   // warps per row
    const int myrow = warp / wpr, myseg = warp - myrow * wpr;
    const int v0i = (int)((long long)myseg * nv / wpr), v1i = (int)((long long)(myseg + 1) * nv / wpr);
    // Chunk k into stage k % 2: lane 0 of EVERY warp copies the piece of a row that its warp will read (a thread's bulk
    // copies are served one after another, copies of different threads overlap); thread 0 announces the byte count.
    auto issue = [&](int k) {
        const int st = k & 1, rbeg = r0 + k * rb;
        const int nr = (r1 - rbeg) < rb ? (r1 - rbeg) : rb;
        const uint32_t bar = biloco::smem_u32(&full[st]);
        if (tid == 0) biloco::mbar_arrive_expect_tx(bar, row_bytes * (uint32_t)nr);
        if (lane == 0 && myrow < nr && v1i > v0i)
            biloco::bulk_load(biloco::smem_u32(stage0 + ((size_t)st * rb + myrow) * n + 4 * (size_t)v0i),
                              a.R + (size_t)(rbeg + myrow) * n + 4 * (size_t)v0i, (uint32_t)(v1i - v0i) * 16u, bar);
    };
    if (nch > 0) issue(0);
    if (nch > 1) issue(1);
    for (int i = tid; i < n; i += PT) {
        vs[i] = (uint8_t)((__float_as_uint(a.v[i]) >> 24) & 0x80u);
        if (a.deflate) vp[i] = (uint8_t)((__float_as_uint(a.v_prev[i]) >> 24) & 0x80u);
    }
    const float alpha = a.deflate ? a.alpha_prev[0] : 0.f;
    float col[MAXC];
#pragma unroll
    for (int k = 0; k < MAXC; ++k) col[k] = 0.f;
    float asum = 0.f;
    __syncthreads();
    for (int k = 0; k < nch; ++k) {
        const int st = k & 1, rbeg = r0 + k * rb;
        const int nr = (r1 - rbeg) < rb ? (r1 - rbeg) : rb;
        if (!peel_wait(biloco::smem_u32(&full[st]), (uint32_t)((k >> 1) & 1), a.err)) bad = 1;
        if (a.deflate && tid < nr) aus[tid] = __fmul_rn(alpha, a.u_prev[rbeg + tid]);
        __syncthreads();
        if (bad) break;
        float* rows = stage0 + (size_t)st * rb * n;
        // ---- the warp's segment of its row: the previous atom's update (in shared memory), the partial dot product ----
        float d = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;      // (four chains: x, y, z, w lanes of the vectors; combined below in a fixed order)
        if (myrow < nr) {
            float4* s4 = reinterpret_cast<float4*>(rows + (size_t)myrow * n);
            const float au = a.deflate ? aus[myrow] : 0.f;
#pragma unroll 4
            for (int i = v0i + lane; i < v1i; i += 32) {
                float4 x = s4[i];
                const uint32_t sv = reinterpret_cast<const uint32_t*>(vs)[i];
                if (a.deflate) {
                    const uint32_t pv = reinterpret_cast<const uint32_t*>(vp)[i];
                    x.x = __fsub_rn(x.x, flipb(au, pv & 0xffu)); x.y = __fsub_rn(x.y, flipb(au, (pv >> 8) & 0xffu));
                    x.z = __fsub_rn(x.z, flipb(au, (pv >> 16) & 0xffu)); x.w = __fsub_rn(x.w, flipb(au, pv >> 24));
                    s4[i] = x;
                }
                d = __fadd_rn(d, flipb(x.x, sv & 0xffu)); d1 = __fadd_rn(d1, flipb(x.y, (sv >> 8) & 0xffu));
                d2 = __fadd_rn(d2, flipb(x.z, (sv >> 16) & 0xffu)); d3 = __fadd_rn(d3, flipb(x.w, sv >> 24));
            }
        }
        d = __fadd_rn(__fadd_rn(d, d1), __fadd_rn(d2, d3));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) d = __fadd_rn(d, __shfl_xor_sync(0xffffffffu, d, o));
        if (lane == 0) dseg[warp] = d;
        if (a.deflate) biloco::fence_proxy_async();      // the updated rows go back to global memory as bulk copies
        __syncthreads();
        if (tid < nr) {                                  // the row's dot product: its segments in order
            float t = 0.f;
            for (int j = 0; j < wpr; ++j) t = __fadd_rn(t, dseg[tid * wpr + j]);
            if (a.dots_only) {
                dseg[tid * wpr] = flip(t, a.u[rbeg + tid]);
            } else {
                const float s1 = sgn1(t);
                us[tid] = s1;
                a.u[rbeg + tid] = s1;
            }
        }
        if (a.deflate && tid == 0) {
            for (int q = 0; q < nr; ++q)
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(a.R + (size_t)(rbeg + q) * n),
                             "r"(biloco::smem_u32(rows + (size_t)q * n)), "r"(row_bytes) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        __syncthreads();
        if (a.dots_only) {
            if (tid == 0)
                for (int q = 0; q < nr; ++q) asum = __fadd_rn(asum, dseg[q * wpr]);
        } else {
            // column sums of the stage, rows in order
            float usr[RB];
#pragma unroll
            for (int q = 0; q < RB; ++q) usr[q] = us[q];
#pragma unroll
            for (int kk = 0; kk < MAXC; ++kk) {
                if (kk * PT >= n) break;                       // (uniform: the columns beyond n belong to nobody)
                const int cc = tid + kk * PT;
                if (cc < n) {
                    float t = col[kk];
#pragma unroll
                    for (int q = 0; q < RB; ++q)
                        if (q < nr) t = __fadd_rn(t, flip(rows[(size_t)q * n + cc], usr[q]));
                    col[kk] = t;
                }
            }
        }
        // the stage is free once everybody has read it (and the copies out of it have read it): refill it
        if (a.deflate && tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncthreads();
        if (k + 2 < nch) issue(k + 2);
    }
    if (a.deflate && tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    if (bad) {      // copies may still be in flight towards the stages: let them land before the shared memory is released
        const uint64_t t0 = biloco::globaltimer_ns();
        while (biloco::globaltimer_ns() - t0 < 2000000ull) { }
        return;
    }
    if (a.dots_only) {
        if (tid == 0) a.apart[c] = asum;
    } else {
#pragma unroll
        for (int kk = 0; kk < MAXC; ++kk) {
            const int cc = tid + kk * PT;
            if (cc < n) a.colpart[(size_t)c * n + cc] = col[kk];
        }
    }
}

// v[c] = sgn(sum over the CTAs of their column sums); optionally stored as column `atom` of V [n][r] too. A block takes 32
// columns; its eight warps each add an eighth of the CTAs' values (in CTA order, sixteen loads in flight), and the eight
// sums are added in warp order: a fixed order, with an eighth of the serial latency.
__global__ void __launch_bounds__(256) peel_colsign_kernel(const float* __restrict__ colpart, float* __restrict__ v, float* __restrict__ Vout,
                                                           int n, int G, int r, int atom) {
    __shared__ float part[8][32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    const int g0 = (int)((long long)w * G / 8), g1 = (int)((long long)(w + 1) * G / 8);
    float t = 0.f;
    if (c < n) {
        int g = g0;
        for (; g + 16 <= g1; g += 16) {
            float x[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = __ldcg(colpart + (size_t)(g + i) * n + c);
#pragma unroll
            for (int i = 0; i < 16; ++i) t = __fadd_rn(t, x[i]);
        }
        for (; g < g1; ++g) t = __fadd_rn(t, __ldcg(colpart + (size_t)g * n + c));
    }
    part[w][lane] = t;
    __syncthreads();
    if (w == 0 && c < n) {
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) tot = __fadd_rn(tot, part[i][lane]);
        const float s = sgn1(tot);
        v[c] = s;
        if (Vout) Vout[(size_t)c * r + atom] = s;
    }
}

// alpha = (sum of the CTAs' partial sums, in order) / (m n); also S[atom], and u as column `atom` of U [m][r].
__global__ void peel_alpha_kernel(const float* __restrict__ apart, int G, float scale, float* __restrict__ alpha, float* __restrict__ S,
                                  const float* __restrict__ u, float* __restrict__ Uout, int m, int r, int atom) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        float t = 0.f;
        for (int g = 0; g < G; ++g) t = __fadd_rn(t, apart[g]);
        const float al = __fdiv_rn(t, scale);
        alpha[0] = al;
        S[atom] = al;
    }
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < m; i += gridDim.x * blockDim.x) Uout[(size_t)i * r + atom] = u[i];
}

__global__ void peel_sign_copy_kernel(const float* __restrict__ src, float* __restrict__ dst, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = sgn1(src[i]);
}

// rows per stage: the largest power of two (at most PW) such that two stages and the two sign vectors fit
static int peel_rows_per_stage(int n) {
    const long long room = (long long)PEEL_SMEM - 2ll * n;
    int rb = 0;
    for (int t = 1; t <= PW; t *= 2)
        if (2ll * t * n * 4 <= room) rb = t;
    return rb;
}

static void launch_pass(const PeelArgs& a, int G, size_t smem, cudaStream_t stream) {
    switch (a.rb) {
        case 1: peel_pass_kernel<1><<<G, PT, smem, stream>>>(a); break;
        case 2: peel_pass_kernel<2><<<G, PT, smem, stream>>>(a); break;
        case 4: peel_pass_kernel<4><<<G, PT, smem, stream>>>(a); break;
        case 8: peel_pass_kernel<8><<<G, PT, smem, stream>>>(a); break;
        default: peel_pass_kernel<16><<<G, PT, smem, stream>>>(a); break;
    }
}

}  // namespace

extern "C" size_t biloco_b200_peel_scratch_bytes(int m, int n, int num_sms) {
    if (num_sms <= 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 0;
        if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    }
    if (m < 1 || n < 4 || (n % 4) || n > PT * MAXC || peel_rows_per_stage(n) < 1) return 0;
    const int G = m < num_sms ? m : num_sms;
    // column sums [G][n], coefficient partial sums [G], u, u_prev [m], v, v_prev [n], alpha [4] (alpha, error flag)
    return ((size_t)G * n + G + 2 * (size_t)m + 2 * (size_t)n + 4) * sizeof(float) + 256;
}

extern "C" int biloco_b200_binary_peel(float* R, const float* v_init, float* U, float* V, float* S, void* scratch, size_t scratch_bytes,
                                       int m, int n, int r, int T, biloco_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!R || !v_init || !U || !V || !S || !scratch) return BILOCO_ERR_NULL;
    if (m < 1 || n < 4 || (n % 4) || n > PT * MAXC || r < 1 || T < 1) return BILOCO_ERR_SHAPE;
    const int rb = peel_rows_per_stage(n);
    if (rb < 1) return BILOCO_ERR_SHAPE;
    if (((uintptr_t)R & 15) || ((uintptr_t)v_init & 15) || ((uintptr_t)scratch & 15)) return BILOCO_ERR_ALIGN;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return BILOCO_ERR_CUDA;
    const size_t need = biloco_b200_peel_scratch_bytes(m, n, sms);
    if (need == 0) return BILOCO_ERR_SHAPE;
    if (scratch_bytes < need) return BILOCO_ERR_SCRATCH;
    const int G = m < sms ? m : sms;
    const size_t smem = (size_t)2 * rb * n * sizeof(float) + 2 * (size_t)n;
    static bool attr_set[64] = {false};
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(peel_pass_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PEEL_SMEM + 1024) != cudaSuccess ||
            cudaFuncSetAttribute(peel_pass_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PEEL_SMEM + 1024) != cudaSuccess ||
            cudaFuncSetAttribute(peel_pass_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, PEEL_SMEM + 1024) != cudaSuccess ||
            cudaFuncSetAttribute(peel_pass_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, PEEL_SMEM + 1024) != cudaSuccess ||
            cudaFuncSetAttribute(peel_pass_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, PEEL_SMEM + 1024) != cudaSuccess)
            return BILOCO_ERR_CUDA;
        attr_set[dev] = true;
    }
    // scratch carve-up (every piece a multiple of 16 bytes from a 16-byte aligned base)
    float* base = (float*)scratch;
    auto up4 = [](size_t x) { return (x + 3) / 4 * 4; };
    float* colpart = base;                  base += up4((size_t)G * n);
    float* apart = base;                    base += up4((size_t)G);
    float* u_cur = base;                    base += up4((size_t)m);
    float* u_prev = base;                   base += up4((size_t)m);
    float* v_cur = base;                    base += up4((size_t)n);
    float* v_prev = base;                   base += up4((size_t)n);
    float* alpha = base;

    PeelArgs a;
    a.R = R; a.colpart = colpart; a.apart = apart; a.m = m; a.n = n; a.rb = rb;
    a.err = (int*)(alpha + 1);
    cudaMemsetAsync(alpha, 0, 16, stream);
    a.alpha_prev = alpha;
    const int cb = 256, cg = (n + cb - 1) / cb;
    for (int atom = 0; atom < r; ++atom) {
        // (the atom's vectors alternate between the two buffers, so that the previous atom's stay readable for the update)
        float* u = (atom & 1) ? u_prev : u_cur;
        float* up = (atom & 1) ? u_cur : u_prev;
        float* v = (atom & 1) ? v_prev : v_cur;
        float* vpv = (atom & 1) ? v_cur : v_prev;
        peel_sign_copy_kernel<<<cg, cb, 0, stream>>>(v_init + (size_t)atom * n, v, n);
        for (int t = 0; t < T; ++t) {
            a.v = v; a.u = u; a.u_prev = up; a.v_prev = vpv;
            a.deflate = (t == 0 && atom > 0) ? 1 : 0;
            a.dots_only = 0;
            launch_pass(a, G, smem, stream);
            peel_colsign_kernel<<<(n + 31) / 32, 256, 0, stream>>>(colpart, v, t == T - 1 ? V : nullptr, n, G, r, atom);
        }
        a.v = v; a.u = u; a.deflate = 0; a.dots_only = 1;
        launch_pass(a, G, smem, stream);
        peel_alpha_kernel<<<(m + 255) / 256 < 64 ? (m + 255) / 256 : 64, 256, 0, stream>>>(apart, G, (float)m * (float)n, alpha, S, u, U, m, r,
                                                                                             atom);
    }
    // the last atom's update (the passes above apply an update at the start of the NEXT atom)
    {
        const int atom = r;      // parity of the buffers as if another atom followed
        a.u = (atom & 1) ? u_prev : u_cur;                 // (scratch: overwritten, not used)
        a.u_prev = (atom & 1) ? u_cur : u_prev;
        a.v_prev = (atom & 1) ? v_cur : v_prev;
        a.v = a.v_prev;
        a.deflate = 1; a.dots_only = 0;
        launch_pass(a, G, smem, stream);
    }
    if (cudaGetLastError() != cudaSuccess) return BILOCO_ERR_CUDA;
    // the decomposition is an offline step: wait for it and report a wait that ran out on the device
    int h_err = 0;
    if (cudaMemcpyAsync(&h_err, a.err, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return BILOCO_ERR_CUDA;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return BILOCO_ERR_CUDA;
    return h_err ? BILOCO_ERR_WAIT : BILOCO_OK;
}
