// One decode step of attention for M <= 32 sequences, the step between the stacked q/k/v launch and the output
// projection: optional per-head RMS norm of q and k, rotary embedding at the current position, the new key and value
// written into the cache, and attention of every query head over the cache up to that position. One launch replaces the
// few dozen element-wise kernels a framework issues for these steps (each a launch of a few microseconds on a vector of
// a few thousand elements). Not part of the fused linear; a piece of the decode step around it.
//
// Arithmetic (mirrors the composition in plain tensor operations, so that the two can be compared closely):
//     norm:   x * rsqrt(mean(x^2) + eps) in fp32, rounded to bf16, times the bf16 weight, rounded to bf16
//     rotary: halves (x1, x2) of the head: (x1*cos - x2*sin, x2*cos + x1*sin), separate fp32 multiplies and adds, rounded to bf16
//     scores: fp32 dot products of bf16 q and k, times 1/sqrt(D); softmax and the weighted sum of v in fp32; output bf16
// Grid = (query heads, sequences); a CTA computes the new key of its KV head for itself (the first query head of the
// group also stores it), so no CTA reads cache entries written in this launch.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/biloco_b200.h"
#include "ptx.cuh"

extern "C" int biloco_internal_use_pdl();

namespace {

constexpr int AT_THREADS = 256;
constexpr int AT_WARPS = AT_THREADS / 32;

struct AttnParams {
    const __nv_bfloat16* qkv;       // [M, (H + 2*KVH) * D]: q heads, then k heads, then v heads
    const __nv_bfloat16* q_norm;    // [D] or null
    const __nv_bfloat16* k_norm;    // [D] or null
    const float* cos;               // [max_len, D/2]
    const float* sin;
    const long long* pos;           // device scalar: the position being written
    __nv_bfloat16* k_cache;         // [M, KVH, max_len, D]
    __nv_bfloat16* v_cache;
    __nv_bfloat16* out;             // [M, H * D]
    int M, H, KVH, max_len;
    float eps, scale;
};

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// one head vector (D elements in shared memory, one warp): optional norm, then rotary at (cs, sn)
template <int D>
__device__ __forceinline__ void norm_rope(float* x, const __nv_bfloat16* w, float eps, const float* cs, const float* sn, int lane) {
    if (w) {
        float ss = 0.f;
#pragma unroll
        for (int i = lane; i < D; i += 32) ss = fmaf(x[i], x[i], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
        for (int i = lane; i < D; i += 32) x[i] = bf16r(__fmul_rn(bf16r(__fmul_rn(x[i], inv)), __bfloat162float(w[i])));
        __syncwarp();
    }
#pragma unroll
    for (int i = lane; i < D / 2; i += 32) {
        const float x1 = x[i], x2 = x[i + D / 2], c = cs[i], s = sn[i];
        x[i] = bf16r(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)));
        x[i + D / 2] = bf16r(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s)));
    }
    __syncwarp();
}

template <int D>
__global__ void __launch_bounds__(AT_THREADS) decode_attention_kernel(AttnParams p) {
    constexpr int EPL = D / 32;                      // elements per lane
    __shared__ float q_s[D], k_s[D], v_s[D];
    __shared__ float w_m[AT_WARPS], w_l[AT_WARPS], w_acc[AT_WARPS][D];
    const int h = blockIdx.x, m = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int group = p.H / p.KVH, g = h / group;
    biloco::griddep_launch_dependents();             // the next kernel of the stream may start its preamble
    biloco::griddep_wait();                          // q/k/v come from the previous kernel
    const long long pos_ll = p.pos[0];
    if (pos_ll < 0 || pos_ll >= p.max_len) return;   // (nothing sensible to do; uniform over the grid)
    const int pos = (int)pos_ll;
    const __nv_bfloat16* row = p.qkv + (size_t)m * (p.H + 2 * p.KVH) * D;
    if (tid < D) {
        q_s[tid] = __bfloat162float(row[h * D + tid]);
        k_s[tid] = __bfloat162float(row[(p.H + g) * D + tid]);
        v_s[tid] = __bfloat162float(row[(p.H + p.KVH + g) * D + tid]);
    }
    __syncthreads();
    const float* cs = p.cos + (size_t)pos * (D / 2);
    const float* sn = p.sin + (size_t)pos * (D / 2);
    if (warp == 0) norm_rope<D>(q_s, p.q_norm, p.eps, cs, sn, lane);
    if (warp == 1) norm_rope<D>(k_s, p.k_norm, p.eps, cs, sn, lane);
    __syncthreads();
    const size_t cache_row = ((size_t)m * p.KVH + g) * p.max_len;
    if (h % group == 0 && tid < D) {
        p.k_cache[(cache_row + pos) * D + tid] = __float2bfloat16_rn(k_s[tid]);      // (exact: bf16 values)
        p.v_cache[(cache_row + pos) * D + tid] = __float2bfloat16_rn(v_s[tid]);
    }
    // this lane's slice of the query (elements lane*EPL ..), pre-multiplied by nothing: scores are scaled afterwards
    float q[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) q[e] = q_s[lane * EPL + e];
    float mx = -INFINITY, l = 0.f, acc[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
    constexpr int UNR = 4;                           // positions in flight per warp
    for (int p0 = warp * UNR; p0 <= pos; p0 += AT_WARPS * UNR) {
        float kv[UNR][EPL], vv[UNR][EPL], sc[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int pp = p0 + u;
            if (pp < pos) {
                const __nv_bfloat16* kr = p.k_cache + (cache_row + pp) * D + lane * EPL;
                const __nv_bfloat16* vr = p.v_cache + (cache_row + pp) * D + lane * EPL;
                if constexpr (EPL == 4) {
                    const uint2 a = *reinterpret_cast<const uint2*>(kr), b = *reinterpret_cast<const uint2*>(vr);
                    kv[u][0] = __uint_as_float(a.x << 16); kv[u][1] = __uint_as_float(a.x & 0xFFFF0000u);
                    kv[u][2] = __uint_as_float(a.y << 16); kv[u][3] = __uint_as_float(a.y & 0xFFFF0000u);
                    vv[u][0] = __uint_as_float(b.x << 16); vv[u][1] = __uint_as_float(b.x & 0xFFFF0000u);
                    vv[u][2] = __uint_as_float(b.y << 16); vv[u][3] = __uint_as_float(b.y & 0xFFFF0000u);
                } else {
                    const uint32_t a = *reinterpret_cast<const uint32_t*>(kr), b = *reinterpret_cast<const uint32_t*>(vr);
                    kv[u][0] = __uint_as_float(a << 16); kv[u][1] = __uint_as_float(a & 0xFFFF0000u);
                    vv[u][0] = __uint_as_float(b << 16); vv[u][1] = __uint_as_float(b & 0xFFFF0000u);
                }
            } else {
#pragma unroll
                for (int e = 0; e < EPL; ++e) {      // the position being written (or beyond it: masked below)
                    kv[u][e] = k_s[lane * EPL + e];
                    vv[u][e] = v_s[lane * EPL + e];
                }
            }
            float d = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) d = fmaf(q[e], kv[u][e], d);
            sc[u] = d;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < UNR; ++u) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            if (p0 + u > pos) continue;              // (warp-uniform)
            const float s = sc[u] * p.scale;
            const float nm = fmaxf(mx, s);
            const float corr = __expf(mx - nm), w = __expf(s - nm);
            l = l * corr + w;
#pragma unroll
            for (int e = 0; e < EPL; ++e) acc[e] = acc[e] * corr + w * vv[u][e];
            mx = nm;
        }
    }
    if (lane == 0) { w_m[warp] = mx; w_l[warp] = l; }
#pragma unroll
    for (int e = 0; e < EPL; ++e) w_acc[warp][lane * EPL + e] = acc[e];
    __syncthreads();
    if (tid < D) {
        float gm = -INFINITY;
#pragma unroll
        for (int w = 0; w < AT_WARPS; ++w) gm = fmaxf(gm, w_m[w]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < AT_WARPS; ++w) {
            const float f = w_m[w] == -INFINITY ? 0.f : __expf(w_m[w] - gm);
            num += f * w_acc[w][tid];
            den += f * w_l[w];
        }
        p.out[((size_t)m * p.H + h) * D + tid] = __float2bfloat16_rn(num / den);
    }
}

}  // namespace

extern "C" int biloco_b200_decode_attention(const void* qkv_bf16, const void* q_norm_bf16, const void* k_norm_bf16, float eps,
                                            const float* cos_table, const float* sin_table, const long long* pos_dev,
                                            void* k_cache_bf16, void* v_cache_bf16, void* out_bf16, int M, int H, int KVH, int D,
                                            int max_len, biloco_stream_t stream) {
    if (!qkv_bf16 || !cos_table || !sin_table || !pos_dev || !k_cache_bf16 || !v_cache_bf16 || !out_bf16) return BILOCO_ERR_NULL;
    if (M < 1 || M > 65535 || H < 1 || KVH < 1 || (H % KVH) != 0 || (D != 64 && D != 128) || max_len < 1) return BILOCO_ERR_SHAPE;
    if (((uintptr_t)qkv_bf16 & 7) || ((uintptr_t)k_cache_bf16 & 7) || ((uintptr_t)v_cache_bf16 & 7)) return BILOCO_ERR_ALIGN;
    AttnParams p;
    p.qkv = (const __nv_bfloat16*)qkv_bf16;
    p.q_norm = (const __nv_bfloat16*)q_norm_bf16;
    p.k_norm = (const __nv_bfloat16*)k_norm_bf16;
    p.cos = cos_table; p.sin = sin_table; p.pos = pos_dev;
    p.k_cache = (__nv_bfloat16*)k_cache_bf16; p.v_cache = (__nv_bfloat16*)v_cache_bf16; p.out = (__nv_bfloat16*)out_bf16;
    p.M = M; p.H = H; p.KVH = KVH; p.max_len = max_len;
    p.eps = eps;
    p.scale = 1.0f / sqrtf((float)D);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)H, (unsigned)M);
    cfg.blockDim = dim3(AT_THREADS);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (biloco_internal_use_pdl()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    const cudaError_t e = D == 128 ? cudaLaunchKernelEx(&cfg, decode_attention_kernel<128>, p)
                                   : cudaLaunchKernelEx(&cfg, decode_attention_kernel<64>, p);
    return e == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}
