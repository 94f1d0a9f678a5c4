// Stream-K work split of the fused linear: T = ntile * nkt units in (tile, k-tile) order are cut into G
// contiguous ranges, CTA c owning [floor(c*T/G), floor((c+1)*T/G)). Shared by host and device code.
// All arithmetic is 32-bit (64-bit division is a long software routine on the GPU, and this code is inlined in
// a kernel whose instruction footprint matters): the host checks (T + 1) * (G + 1) < 2^31 before launching.
#pragma once

#if defined(__CUDACC__)
#define BILOCO_HD __host__ __device__ inline
#else
#define BILOCO_HD inline
#endif

namespace biloco {

// first unit of CTA c (c may equal G: one past the last unit)
BILOCO_HD int sched_first_unit(int c, int T, int G) { return (int)((unsigned)c * (unsigned)T / (unsigned)G); }

// the CTA whose range contains unit u: the largest c with floor(c*T/G) <= u
BILOCO_HD int sched_cta_of_unit(int u, int T, int G) { return (int)(((unsigned)(u + 1) * (unsigned)G - 1u) / (unsigned)T); }

BILOCO_HD bool sched_fits_32bit(int ntile, int nkt, int G) {
    return ((long long)ntile * nkt + 1) * ((long long)G + 1) < (1ll << 31);
}

// Largest number of partial-sum slots any tile needs = max over tiles of (#contributing CTAs - 1), at least 1.
BILOCO_HD int sched_max_slots(int ntile, int nkt, int G) {
    const int T = ntile * nkt;
    int best = 1;
    for (int t = 0; t < ntile; ++t) {
        const int c0 = sched_cta_of_unit(t * nkt, T, G);
        const int c1 = sched_cta_of_unit(t * nkt + nkt - 1, T, G);
        if (c1 - c0 > best) best = c1 - c0;
    }
    return best;
}

}  // namespace biloco
