// CUDA-core NVFP4 GEMM: D[m,n] = bf16(alpha * sum_k A[m,k] W[n,k] + C[m,n]). One warp per output element,
// lanes stride over 16-element blocks. It exists to cross-check the tensor-core kernel on the device at
// sizes where the CPU oracle is slow; it is not a fast path.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/biloco_b200.h"

namespace {

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(__half(h));
}
__device__ __forceinline__ float e2m1_value(uint32_t code) {
    const uint32_t m = code & 7u;
    const float mag = m < 4u ? 0.5f * (float)m : (m == 4u ? 2.0f : (m == 5u ? 3.0f : (m == 6u ? 4.0f : 6.0f)));
    return (code & 8u) ? -mag : mag;
}
__device__ __forceinline__ size_t sf_offset(int row, int kb, int kblocks) {
    return ((size_t)(row >> 7) * ((kblocks + 3) >> 2) + (kb >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (kb & 3);
}

constexpr int WARPS = 4;

__global__ void __launch_bounds__(WARPS * 32) fp4_gemm_simt_kernel(const uint8_t* __restrict__ A, const uint8_t* __restrict__ A_sf,
                                                                    const uint8_t* __restrict__ W, const uint8_t* __restrict__ W_sf,
                                                                    const float* __restrict__ alpha,
                                                                    const __nv_bfloat16* __restrict__ C,
                                                                    __nv_bfloat16* __restrict__ D, int N, int K) {
    const int n = blockIdx.x * WARPS + (threadIdx.x >> 5);
    const int m = blockIdx.y;
    const int lane = threadIdx.x & 31;
    if (n >= N) return;
    const int kblocks = K >> 4;
    float acc = 0.f;
    for (int kb = lane; kb < kblocks; kb += 32) {
        const uint2 a = *reinterpret_cast<const uint2*>(A + (size_t)m * (K >> 1) + kb * 8);
        const uint2 w = *reinterpret_cast<const uint2*>(W + (size_t)n * (K >> 1) + kb * 8);
        const float sa = e4m3_to_float(A_sf[sf_offset(m, kb, kblocks)]);
        const float sw = e4m3_to_float(W_sf[sf_offset(n, kb, kblocks)]);
        float dot = 0.f;   // exact: products are multiples of 1/4 bounded by 36, 16 terms
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            dot += e2m1_value(a.x >> (4 * j)) * e2m1_value(w.x >> (4 * j));
            dot += e2m1_value(a.y >> (4 * j)) * e2m1_value(w.y >> (4 * j));
        }
        acc += dot * (sa * sw);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
        float v = alpha[0] * acc;
        if (C) v += __bfloat162float(C[(size_t)m * N + n]);
        D[(size_t)m * N + n] = __float2bfloat16(v);
    }
}

}  // namespace

extern "C" int biloco_b200_fp4_gemm_simt(const void* A_codes, const void* A_sf, const void* W_codes, const void* W_sf,
                                         const float* alpha, const void* C_bf16, void* D_bf16, int M, int N, int K,
                                         biloco_stream_t stream) {
    if (!A_codes || !A_sf || !W_codes || !W_sf || !alpha || !D_bf16) return BILOCO_ERR_NULL;
    if (M < 1 || M > 128 || N < 1 || K < 16 || (K % 16) != 0) return BILOCO_ERR_SHAPE;
    if (((uintptr_t)A_codes & 7) || ((uintptr_t)W_codes & 7)) return BILOCO_ERR_ALIGN;
    dim3 grid((N + WARPS - 1) / WARPS, M);
    fp4_gemm_simt_kernel<<<grid, WARPS * 32, 0, (cudaStream_t)stream>>>((const uint8_t*)A_codes, (const uint8_t*)A_sf,
                                                                        (const uint8_t*)W_codes, (const uint8_t*)W_sf, alpha,
                                                                        (const __nv_bfloat16*)C_bf16, (__nv_bfloat16*)D_bf16, N, K);
    return cudaGetLastError() == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}
