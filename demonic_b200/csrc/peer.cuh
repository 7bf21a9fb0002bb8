// peer.cuh -- output exchange fused into the GEMV kernel for the row-sharded path.
//
// Instead of a separate all-gather after the kernel, the GEMV stores every output element
// into all `world` replicas of y as soon as it is computed, with plain st.global to
// peer-mapped memory over NVLink (loads never cross the link, no multicast is involved).  The CTA that sees every other CTA finished then publishes this rank's epoch
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
    int mode;                    // 1: last CTA exchanges flags; 2: every CTA adds to the peers' arrival counters;
                                 // 3: tagged elements, validated by peer_gather_kernel
    unsigned long long *ty[kMaxPeers];  // mode 3: each rank's tagged replica, 2 * stride {f32 value, u32 epoch} pairs
    float *yplain;               // mode 3: local plain y the gather kernel fills
};

// mode 2: every rank contributes exactly kPeerQuantum units per exchange to each arrival counter,
// spread over its CTAs, so the counter of a finished exchange e reads e * world * kPeerQuantum
// whatever the grids were.
constexpr unsigned kPeerQuantum = 1u << 16;

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
// Mode 3 counts differently: the word holds the exchanges completed before the current batch of
// launches (it is advanced once per batch, by peer_batch_end_kernel) and `j` is the position of this
// exchange in the batch, so a kernel that does not wait for its predecessor still knows its epoch.
__device__ __forceinline__ unsigned peer_epoch(const PeerOut *p, int j) {
    return __ldcg(p->epoch) + 1u + (p->mode == 3 ? (unsigned)j : 0u);
}

// Each finished output element goes straight into every rank's replica: one local store and
// world-1 remote stores, issued by the lane that holds the row's sum while the rest of the grid
// is still streaming weights.  No fence here: the writers release at GPU scope (fence + arrival
// counter in peer_finish) and the last CTA's system-scope fence and release are cumulative over
// everything ordered before them.  (A system-scope fence per writer thread was measured at
// ~15 us per kernel on B200.)
__device__ __forceinline__ void peer_store(const PeerOut *p, unsigned e, long long idx, float v) {
    const long long off = (long long)(e & 1u) * p->stride + idx;
    if (p->mode == 3) {
        // the element carries its epoch: the reader needs no flag and the writer no fence (an aligned
        // 8-byte store is single-copy atomic, also across NVLink)
        const unsigned long long pr = ((unsigned long long)e << 32) | (unsigned long long)__float_as_uint(v);
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
            if (r < p->world && !((p->debug & 1) && r != p->rank)) p->ty[r][off] = pr;
        return;
    }
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
        if (r < p->world && !((p->debug & 1) && r != p->rank)) p->y[r][off] = v;
}

__device__ __forceinline__ void red_add_sys(unsigned *p, unsigned v) {
    asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// mode 2, head of the kernel (after the dependency wait): exchange e may only start writing once
// exchange e-1 has landed here in full -- the buffer it writes is the one exchange e-2 used, and a
// GEMV that consumes the previous y needs it anyway.  Thread 0 polls, the CTA follows.  Bounded.
__device__ __forceinline__ void peer_begin(const PeerOut *p, unsigned e) {
    if (p->mode != 2 || (p->debug & 2)) return;
    if (threadIdx.x == 0) {
        const unsigned target = (e - 1u) * (unsigned)p->world * kPeerQuantum;
        const unsigned *mine = p->flags[p->rank];
        const long long t0 = clock64();
        while ((int)(ld_acquire_sys(mine) - target) < 0) {
            if (clock64() - t0 > (1LL << 31)) {  // ~1 s: give up instead of hanging
                *(volatile int *)p->err = 4;
                break;
            }
        }
    }
    __syncthreads();
}

// mode 2, tail: one thread per CTA makes the CTA's stores visible everywhere and adds the CTA's share
// to every rank's arrival counter (remote reductions, nothing waits for them); the CTA that leaves
// last advances the local epoch word.  Nobody waits here for the peers: the next exchange's
// peer_begin, or peer_wait_kernel, does.
template <int THREADS>
__device__ __forceinline__ void peer_finish_counted(const PeerOut *p, unsigned e) {
    __syncthreads();
    if (threadIdx.x != 0) return;
    __threadfence_system();
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    const unsigned cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    const unsigned share = (unsigned)(((unsigned long long)kPeerQuantum * (cta + 1u)) / total -
                                      ((unsigned long long)kPeerQuantum * cta) / total);
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
        if (r < p->world) red_add_sys(p->flags[r], share);
    if (atomicAdd(p->counter, 1u) == total - 1u) {
        *p->counter = 0u;
        *p->epoch = e;
        __threadfence();
    }
}

// Called by every thread of every CTA after its last peer_store.  The CTA that arrives last publishes the
// epoch in the peers' flag words and waits, bounded, for theirs.
template <int THREADS>
__device__ __forceinline__ void peer_finish(const PeerOut *p, unsigned e, int *s_last) {
    if ((p->debug & 16) || p->mode == 3) return;  // mode 3: nothing to do here, the elements speak for themselves
    if (p->mode == 2) {
        peer_finish_counted<THREADS>(p, e);
        return;
    }
    // only the lanes that stored outputs (lane 0 of each warp) have anything to order
    if ((threadIdx.x & 31) == 0) __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned total = gridDim.x * gridDim.y * gridDim.z;
        *s_last = (atomicAdd(p->counter, 1u) == total - 1u);
    }
    __syncthreads();
    if (!*s_last) return;
    __threadfence();  // acquire side of the arrival counter; the release below is at system scope
    const int t = threadIdx.x;
    __syncthreads();
    if (t < p->world && !(p->debug & 32)) st_release_sys(p->flags[t] + p->rank, e);  // tell rank t that our slice has landed
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
