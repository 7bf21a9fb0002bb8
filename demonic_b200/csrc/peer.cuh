// peer.cuh -- output exchange fused into the GEMV kernel for the row-sharded path.
//
// Instead of a separate all-gather after the kernel, the GEMV's last CTA (the one that
// sees every other CTA finished) pushes this rank's y slice into all `world` replicas
// with plain st.global to peer-mapped memory over NVLink (loads never cross the link,
// no multicast is involved), publishes this rank's epoch number in each peer's flag
// word (release, system scope) and then waits -- with a bound -- until all peers have
// published theirs, so completion of the kernel on a GPU means the whole replicated y
// has landed there.
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

// Called by every thread of every CTA after its last peer_store.  The CTA that arrives last
// pushes this rank's finished slice y[yoff, yoff+count) to every peer with coalesced stores
// (remote traffic as full 128-byte lines instead of one 4-byte packet per row), publishes the
// epoch in the peers' flag words and waits, bounded, for theirs.
template <int THREADS>
__device__ __forceinline__ void peer_finish(const PeerOut *p, unsigned e, long long yoff, long long count,
                                            int *s_last) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned total = gridDim.x * gridDim.y * gridDim.z;
        *s_last = (atomicAdd(p->counter, 1u) == total - 1u);
    }
    __syncthreads();
    if (!*s_last) return;
    __threadfence();
    const int t = threadIdx.x;
    const long long base = (long long)(e & 1u) * p->stride + yoff;
    const float *src = p->y[p->rank] + base;
    if (p->world > 1 && !(p->debug & 1)) {
        const bool vec = ((base | count) & 3) == 0;  // every replica has the same offset, so one test serves all
        for (int r = 0; r < p->world; ++r) {
            if (r == p->rank) continue;
            float *dst = p->y[r] + base;
            if (vec) {
                const float4 *s4 = reinterpret_cast<const float4 *>(src);
                float4 *d4 = reinterpret_cast<float4 *>(dst);
                for (long long i = t; i < count / 4; i += THREADS) d4[i] = __ldcg(s4 + i);
            } else {
                for (long long i = t; i < count; i += THREADS) dst[i] = __ldcg(src + i);
            }
        }
        __threadfence_system();  // each writer: its remote stores are visible before the flag below
    }
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
