// One-launch all-reduce of the row-parallel linears' fp32 partial outputs over peer memory (NVLink / NVSwitch, plain
// stores and loads), one process per GPU. No counterpart in the reference (it has no distributed code); it takes the place
// of ncclAllReduce + the cast to bf16 behind a K-sharded fused linear, where the message is M x N fp32 = 32 KB .. 1 MB and
// the collective's cost is latency, not bandwidth.
//
// Protocol (one traversal of the link, no fence, no separate flag):
//   * every rank owns a receive buffer  [2 sets][world senders][slot_elems]  of 8-byte words, mapped by all peers
//     (cudaIpc: biloco_b200_peer_buffer_create / _open);
//   * the calls of a group are numbered by a counter that lives in each rank's own buffer and that the kernel itself
//     advances (every CTA adds its share of 2^20 when it leaves; bits 20.. count the completed calls), so a captured CUDA
//     graph can be replayed; the ranks issue the group's calls in the same order, so their counters agree. Call `seq`
//     (1 .. 4096, cyclic) uses set seq % 2: rank r stores, for every element i of its
//     partial, the word {value bits, seq} into slot [set][r][i] of every peer -- an aligned 8-byte store is one
//     transaction, so the value and its flag arrive together;
//   * then it polls its own buffer: element i of sender p is there once the word's flag equals seq (the previous use of
//     the set, call seq - 2, left seq - 2), adds the world's values IN RANK ORDER (its own from the local partial), adds
//     the optional bf16 residual and rounds once. Every rank forms the same sum bit for bit.
//   * A rank can only be one call ahead of a peer (it needs the peer's words of the current call to finish it), and one
//     call ahead writes the other set: two sets are enough.
// Every poll is bounded by a time budget; when it runs out the kernel records it in `status` and returns (the output of
// that call is then undefined, the context stays usable).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/biloco_b200.h"
#include "ptx.cuh"

extern "C" int biloco_internal_use_pdl();
extern "C" unsigned long long biloco_internal_wait_ns();

namespace {

constexpr int AR_THREADS = 256;
constexpr int AR_MAX_WORLD = 16;

struct ArArgs {
    const float* partial;
    const __nv_bfloat16* residual;
    void* out;
    uint2* const* recv;       // [world] (device memory): rank p's receive buffer as mapped here (entry `rank`: the local one)
    int* status;              // local: [0..3] error words, [8] the call counter
    unsigned long long wait_ns;
    int world, rank, count, slot_elems;
    int out_f32;
    int pushed;               // the producer of `partial` has stored this rank's words into the peers' buffers already
};

__global__ void __launch_bounds__(AR_THREADS) peer_allreduce_kernel(ArArgs a) {
    biloco::griddep_launch_dependents();
    biloco::griddep_wait();                         // the partial sums come from the previous kernel of the stream
    uint32_t* counter = reinterpret_cast<uint32_t*>(a.status) + 8;
    const uint32_t seq = (biloco::ld_volatile_u32(counter) >> 20) + 1u;
    const int set = (int)(seq & 1u);
    const size_t set_off = (size_t)set * a.world * a.slot_elems;
    const int stride = gridDim.x * AR_THREADS;
    // push (unless the fused linear's epilogue has done it: biloco_b200_fused_linear_push)
    for (int i = blockIdx.x * AR_THREADS + threadIdx.x; i < a.count && !a.pushed; i += stride) {
        const uint32_t bits = __float_as_uint(a.partial[i]);
        for (int p = 0; p < a.world; ++p) {
            if (p == a.rank) continue;
            uint2* dst = a.recv[p] + set_off + (size_t)a.rank * a.slot_elems + i;
            asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(bits), "r"(seq) : "memory");
        }
    }
    // gather: the peers' words of an element are requested together (one local round trip per attempt, not one per peer),
    // re-requested only where the flag is not there yet, and added in rank order once all have arrived
    const uint2* mine = a.recv[a.rank] + set_off;
    bool ok = true;
    for (int i = blockIdx.x * AR_THREADS + threadIdx.x; i < a.count && ok; i += stride) {
        uint32_t val[AR_MAX_WORLD];
        uint32_t need = 0u;
#pragma unroll
        for (int q = 0; q < AR_MAX_WORLD; ++q) {
            val[q] = 0u;
            if (q < a.world && q != a.rank) need |= 1u << q;
        }
        uint64_t t0 = 0;
        for (uint32_t it = 0; need; ++it) {
            uint32_t f[AR_MAX_WORLD];
#pragma unroll
            for (int q = 0; q < AR_MAX_WORLD; ++q) {
                f[q] = 0u;
                if (need & (1u << q)) {
                    const uint2* src = mine + (size_t)q * a.slot_elems + i;
                    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(val[q]), "=r"(f[q]) : "l"(src) : "memory");
                }
            }
#pragma unroll
            for (int q = 0; q < AR_MAX_WORLD; ++q)
                if ((need & (1u << q)) && f[q] == seq) need &= ~(1u << q);
            if (need && (it & 63u) == 63u) {
                const uint64_t now = biloco::globaltimer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > a.wait_ns) { ok = false; break; }
            }
        }
        if (!ok) {
            if (atomicCAS(a.status, 0, 1) == 0) { a.status[1] = i; a.status[2] = (int)seq; a.status[3] = a.rank; }
            break;
        }
        float sum = 0.f;
        const float own = a.partial[i];
#pragma unroll
        for (int q = 0; q < AR_MAX_WORLD; ++q)
            if (q < a.world) sum = __fadd_rn(sum, q == a.rank ? own : __uint_as_float(val[q]));
        if (a.residual) sum = __fadd_rn(sum, __bfloat162float(a.residual[i]));
        if (a.out_f32) reinterpret_cast<float*>(a.out)[i] = sum;
        else reinterpret_cast<__nv_bfloat16*>(a.out)[i] = __float2bfloat16_rn(sum);
    }
    // this CTA's share of 2^20 (the shares of a launch add up to exactly 2^20 whatever the grid size), also after a failure
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t c = blockIdx.x, G = gridDim.x;
        const uint32_t share = (uint32_t)((((unsigned long long)(c + 1)) << 20) / G) - (uint32_t)((((unsigned long long)c) << 20) / G);
        asm volatile("red.global.add.u32 [%0], %1;" ::"l"(counter), "r"(share) : "memory");
    }
}

}  // namespace

extern "C" size_t biloco_b200_peer_buffer_bytes(int world, int slot_elems) {
    if (world < 1 || world > AR_MAX_WORLD || slot_elems < 1) return 0;
    return (size_t)2 * world * slot_elems * sizeof(uint2);
}

extern "C" int biloco_b200_peer_buffer_create(size_t bytes, void** ptr, void* handle64) {
    if (!ptr || !handle64 || bytes == 0) return BILOCO_ERR_NULL;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return BILOCO_ERR_CUDA;
    if (cudaMemset(p, 0, bytes) != cudaSuccess) { cudaFree(p); return BILOCO_ERR_CUDA; }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaFree(p); return BILOCO_ERR_CUDA; }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    memcpy(handle64, &h, 64);
    *ptr = p;
    return BILOCO_OK;
}

extern "C" int biloco_b200_peer_buffer_open(const void* handle64, void** ptr) {
    if (!handle64 || !ptr) return BILOCO_ERR_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return BILOCO_ERR_CUDA;
    *ptr = p;
    return BILOCO_OK;
}

extern "C" int biloco_b200_peer_buffer_close(void* ptr) {
    if (!ptr) return BILOCO_ERR_NULL;
    return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}

extern "C" int biloco_b200_peer_buffer_destroy(void* ptr) {
    if (!ptr) return BILOCO_ERR_NULL;
    return cudaFree(ptr) == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}

extern "C" int biloco_b200_peer_allreduce(const float* partial, const void* residual_bf16, void* out, void* const* recv_ptrs_dev,
                                          int* status, int world, int rank, int count, int slot_elems, int flags,
                                          biloco_stream_t stream) {
    if (!partial || !out || !recv_ptrs_dev || !status) return BILOCO_ERR_NULL;
    if (world < 1 || world > AR_MAX_WORLD || rank < 0 || rank >= world || count < 1 || count > slot_elems) return BILOCO_ERR_SHAPE;
    if (flags & ~(BILOCO_OUT_FP32 | BILOCO_AR_PUSHED)) return BILOCO_ERR_MODE;
    if (((uintptr_t)partial & 3) || ((uintptr_t)recv_ptrs_dev & 7) || ((uintptr_t)status & 3)) return BILOCO_ERR_ALIGN;
    ArArgs a;
    a.partial = partial;
    a.residual = (const __nv_bfloat16*)residual_bf16;
    a.out = out;
    a.recv = (uint2* const*)recv_ptrs_dev;
    a.status = status;
    a.wait_ns = biloco_internal_wait_ns();
    a.world = world; a.rank = rank; a.count = count; a.slot_elems = slot_elems;
    a.out_f32 = (flags & BILOCO_OUT_FP32) ? 1 : 0;
    a.pushed = (flags & BILOCO_AR_PUSHED) ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    int blocks = (count + AR_THREADS - 1) / AR_THREADS;
    if (blocks > 1184) blocks = 1184;                  // (eight CTAs per SM on 148 SMs; larger messages stride)
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(AR_THREADS);
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
    return cudaLaunchKernelEx(&cfg, peer_allreduce_kernel, a) == cudaSuccess ? BILOCO_OK : BILOCO_ERR_CUDA;
}
