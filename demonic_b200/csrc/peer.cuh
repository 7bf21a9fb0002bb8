// peer.cuh -- output exchange fused into the GEMV kernel for the row-sharded path.
//
// Instead of a separate all-gather after the kernel, every CTA of the GEMV pushes the
// contiguous run of rows it computed into all `world` replicas of y with plain st.global
// to peer-mapped memory over NVLink (loads never cross the link, no multicast is
// involved).  The CTA that sees every other CTA finished then publishes this rank's epoch
// number in each peer's flag word (release, system scope) and waits -- with a bound --
// until all peers have published theirs, so completion of the kernel on a GPU means the
// whole replicated y has landed there.
//
// y is double-buffered by epoch parity: a rank can be at most one exchange ahead of
// a peer (it cannot finish epoch e+1 before the peer has signalled e+1), so writes of
// epoch e+1 never touch the buffer a slower peer's consumers of epoch e still read.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dmc {

constexpr int kMaxPeers = 8;

struct PeerOut {
    float *y[kMaxPeers];         // base of each rank's double-buffered y (2 * stride floats)
    unsigned *flags[kMaxPeers];  // each rank's flag array, one word per sender
    unsigned *epoch;             // local: number of completed exchanges
    unsigned *counter;           // local: CTA arrival counter, zero between kernels
    int *err;                    // local error word (pinned host memory)
    long long stride;            // floats per y buffer
    int world, rank;
    int debug;                   // measurement only: 1 = skip the push, 2 = skip the flag wait
};

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Epoch this kernel is producing (uniform over the grid: the word only changes in
// peer_finish of the last CTA, after every CTA has passed its arrival).
__device__ __forceinline__ unsigned peer_epoch(const PeerOut *p) { return __ldcg(p->epoch) + 1u; }

// During the kernel every CTA stores its outputs into this rank's own replica (ordinary
// local stores); the exchange happens once, in peer_finish.
__device__ __forceinline__ void peer_store(const PeerOut *p, unsigned e, long long idx, float v) {
    p->y[p->rank][(long long)(e & 1u) * p->stride + idx] = v;
}

// Called by every thread of a CTA once all its warps have stored their rows (after a
// __syncthreads): the CTA copies its own contiguous run y[first, first+count) of this rank's
// replica into every peer's replica.  Every CTA pushes its own rows as soon as it has them, so
// the NVLink traffic overlaps the CTAs that are still streaming weights.
template <int THREADS>
__device__ __forceinline__ void peer_push(const PeerOut *p, unsigned e, long long first, long long count) {
    if (p->world <= 1 || (p->debug & 1)) return;
    const long long base = (long long)(e & 1u) * p->stride + first;
    const float *src = p->y[p->rank] + base;
    bool wrote = false;
    for (long long i = threadIdx.x; i < count; i += THREADS) {
        const float v = __ldcg(src + i);
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
            if (r < p->world && r != p->rank) p->y[r][base + i] = v;
        wrote = true;
    }
    if (wrote) __threadfence_system();  // the remote stores are performed before this CTA reports in
}

// Called by every thread of every CTA after peer_push.  The CTA that arrives last publishes the
// epoch in the peers' flag words and waits, bounded, for theirs.
template <int THREADS>
__device__ __forceinline__ void peer_finish(const PeerOut *p, unsigned e, int *s_last) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned total = gridDim.x * gridDim.y * gridDim.z;
        *s_last = (atomicAdd(p->counter, 1u) == total - 1u);
    }
    __syncthreads();
    if (!*s_last) return;
    __threadfence_system();
    const int t = threadIdx.x;
    __syncthreads();
    if (t < p->world) st_release_sys(p->flags[t] + p->rank, e);  // tell rank t that our slice has landed
    if (t < p->world && !(p->debug & 2)) {
        const unsigned *mine = p->flags[p->rank] + t;
        const long long t0 = clock64();
        // epochs only grow; a wrapped comparison keeps this right after 2^32 exchanges
        while ((int)(ld_acquire_sys(mine) - e) < 0) {
            if (clock64() - t0 > (1LL << 31)) {  // ~1 s: give up instead of hanging
                *(volatile int *)p->err = 3;
                break;
            }
        }
    }
    __syncthreads();
    if (t == 0) {
        *p->counter = 0u;
        *p->epoch = e;
        __threadfence();
    }
}

}  // namespace dmc
