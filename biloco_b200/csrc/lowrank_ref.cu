// Unfused low-rank term on CUDA cores (the device-side comparator of the fused kernel) and the U re-layout.
//   binary_z:      z[m,i] = S[i] * sum_k sign(V[i,k]) X[m,k]     fp32
//   binary_expand: Y[m,n] = bf16( sum_i z[m,i] sign(U[i,n]) )
//   pack_u_col32:  U_packed [R,N/8] -> int32 [N, ceil(R/32)]
// Signs are bit-packed LSB-first, bit set = +1.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/biloco_b200.h"

namespace {

constexpr int Z_THREADS = 128;
constexpr int Z_RANKS = 4;  // ranks per CTA

// x with its sign flipped where the bit is 0
__device__ __forceinline__ float signed_by_bit(float x, uint32_t word, int j) {
    const uint32_t flip = ((~word >> j) & 1u) << 31;
    return __uint_as_float(__float_as_uint(x) ^ flip);
}

// grid (ceil(R / Z_RANKS), M). Thread t walks the 32-bit sign words t, t+128, ... of its ranks; each word
// covers 32 consecutive k, whose activations arrive as four 128-bit loads.
__global__ void __launch_bounds__(Z_THREADS) binary_z_kernel(const __nv_bfloat16* __restrict__ X,
                                                             const uint8_t* __restrict__ Vp,
                                                             const __nv_bfloat16* __restrict__ S,
                                                             float* __restrict__ z, int K, int R) {
    const int m = blockIdx.y;
    const int i0 = blockIdx.x * Z_RANKS;
    const int tid = threadIdx.x;
    const int kbytes = K >> 3;
    const int nwords = (K & 31) ? 0 : (K >> 5);  // word path needs 4-byte aligned sign rows; otherwise go bytewise
    float acc[Z_RANKS];
#pragma unroll
    for (int q = 0; q < Z_RANKS; ++q) acc[q] = 0.f;

    const __nv_bfloat16* xrow = X + (size_t)m * K;
    for (int w = tid; w < nwords; w += Z_THREADS) {
        float xf[32];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const uint4 p = *reinterpret_cast<const uint4*>(xrow + w * 32 + v * 8);
            const uint32_t u[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                xf[v * 8 + 2 * e] = __uint_as_float(u[e] << 16);
                xf[v * 8 + 2 * e + 1] = __uint_as_float(u[e] & 0xFFFF0000u);
            }
        }
#pragma unroll
        for (int q = 0; q < Z_RANKS; ++q) {
            if (i0 + q < R) {
                const uint32_t word = *reinterpret_cast<const uint32_t*>(Vp + (size_t)(i0 + q) * kbytes + w * 4);
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[q] += signed_by_bit(xf[j], word, j);
            }
        }
    }
    for (int b = nwords * 4 + tid; b < kbytes; b += Z_THREADS) {  // K % 32 != 0: one byte (8 k) at a time
#pragma unroll
        for (int q = 0; q < Z_RANKS; ++q) {
            if (i0 + q < R) {
                const uint32_t word = Vp[(size_t)(i0 + q) * kbytes + b];
                for (int j = 0; j < 8; ++j) acc[q] += signed_by_bit(__bfloat162float(xrow[b * 8 + j]), word, j);
            }
        }
    }

    __shared__ float part[Z_RANKS][Z_THREADS / 32];
#pragma unroll
    for (int q = 0; q < Z_RANKS; ++q) {
        float v = acc[q];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((tid & 31) == 0) part[q][tid >> 5] = v;
    }
    __syncthreads();
    if (tid < Z_RANKS && i0 + tid < R) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < Z_THREADS / 32; ++w) v += part[tid][w];
        z[(size_t)m * R + i0 + tid] = v * __bfloat162float(S[i0 + tid]);
    }
}

constexpr int E_THREADS = 128;

// grid (ceil(N/128), M); thread = output column. The z row sits in shared memory; every rank costs one
// (L1-resident) byte load and one add.
__global__ void __launch_bounds__(E_THREADS) binary_expand_kernel(const float* __restrict__ z,
                                                                  const uint8_t* __restrict__ Up,
                                                                  __nv_bfloat16* __restrict__ Y, int N, int R) {
    extern __shared__ float zs[];
    const int m = blockIdx.y;
    const int n = blockIdx.x * E_THREADS + threadIdx.x;
    for (int i = threadIdx.x; i < R; i += E_THREADS) zs[i] = z[(size_t)m * R + i];
    __syncthreads();
    if (n >= N) return;
    const int nb = N >> 3;
    const uint8_t* col = Up + (n >> 3);
    const int bit = n & 7;
    float acc = 0.f;
    for (int i = 0; i < R; ++i) {
        const uint32_t b = col[(size_t)i * nb];
        acc += signed_by_bit(zs[i], b, bit);
    }
    Y[(size_t)m * N + n] = __float2bfloat16(acc);
}

// One thread per (column n, word w).
__global__ void pack_u_col32_kernel(const uint8_t* __restrict__ Up, int32_t* __restrict__ out, int N, int R, int words) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N * words) return;
    const int n = idx / words, w = idx % words;
    const int nb = N >> 3;
    uint32_t v = 0;
    for (int b = 0; b < 32; ++b) {
        const int i = w * 32 + b;
        if (i < R) v |= (uint32_t)((Up[(size_t)i * nb + (n >> 3)] >> (n & 7)) & 1u) << b;
    }
    out[idx] = (int32_t)v;
}

}  // namespace

extern "C" int biloco_b200_binary_z(const void* X_bf16, const void* V_packed, const void* S_bf16, float* z, int M,
                                    int K, int R, biloco_stream_t stream) {
    if (!X_bf16 || !V_packed || !S_bf16 || !z) return BILOCO_ERR_NULL;
    if (M < 1 || R < 1 || K < 8 || (K % 8) != 0) return BILOCO_ERR_SHAPE;
    if (((uintptr_t)X_bf16 & 15) || ((uintptr_t)V_packed & 3)) return BILOCO_ERR_ALIGN;
    dim3 grid((R + Z_RANKS - 1) / Z_RANKS, M);
    binary_z_kernel<<<grid, Z_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)X_bf16, (const uint8_t*)V_packed,
                                                                   (const __nv_bfloat16*)S_bf16, z, K, R);
    return cudaGetLastError() == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}

extern "C" int biloco_b200_binary_expand(const float* z, const void* U_packed, void* Y_bf16, int M, int N, int R,
                                         biloco_stream_t stream) {
    if (!z || !U_packed || !Y_bf16) return BILOCO_ERR_NULL;
    if (M < 1 || R < 1 || N < 8 || (N % 8) != 0 || R > 8192) return BILOCO_ERR_SHAPE;
    dim3 grid((N + E_THREADS - 1) / E_THREADS, M);
    binary_expand_kernel<<<grid, E_THREADS, R * sizeof(float), (cudaStream_t)stream>>>(z, (const uint8_t*)U_packed,
                                                                                        (__nv_bfloat16*)Y_bf16, N, R);
    return cudaGetLastError() == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}

extern "C" void biloco_internal_mark_relayout(cudaStream_t stream);      // (fused_linear.cu: the next fused launch on this stream starts plain)

extern "C" int biloco_b200_pack_u_col32(const void* U_packed, int32_t* U_col32, int N, int R, biloco_stream_t stream) {
    if (!U_packed || !U_col32) return BILOCO_ERR_NULL;
    if (R < 1 || N < 8 || (N % 8) != 0) return BILOCO_ERR_SHAPE;
    const int words = (R + 31) / 32;
    const long long total = (long long)N * words;
    pack_u_col32_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)U_packed, U_col32,
                                                                                           N, R, words);
    biloco_internal_mark_relayout((cudaStream_t)stream);
    return cudaGetLastError() == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}
