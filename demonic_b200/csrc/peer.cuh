// peer.cuh -- output exchange fused into the GEMV kernel for the row-sharded path.
//
// Instead of a separate all-gather after the kernel, the GEMV stores every finished row sum
// into all `world` replicas of y as soon as it is computed, with plain st.global to
// peer-mapped memory over NVLink (loads never cross the link, no multicast is involved).
// Every element travels as an 8-byte {f32 value, u32 epoch} pair: the epoch names the
// exchange that wrote it, so the writers need no fence, no flag and no arrival counter -- an
// aligned 8-byte store is single-copy atomic, also across NVLink.  A small gather kernel
// (shard.cu) running beside the GEMV re-reads the local replica, with a bound, until every
// pair carries the current epoch, and writes the plain f32 y.
//
// The replica is double-buffered by epoch parity, so the stores of exchange e + 1 never touch
// the pairs a slower rank's gather of exchange e is still reading.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dmc {

constexpr int kMaxPeers = 8;

struct PeerOut {
    unsigned long long *ty[kMaxPeers];  // each rank's tagged replica: 2 * stride {value, epoch} pairs
    float *yplain;                      // local plain y the gather kernel fills (2 * stride floats)
    unsigned *epoch;                    // local: exchanges completed before the current batch of launches
    int *err;                           // local error word (pinned host memory)
    long long stride;                   // elements per buffer
    long long wait_cycles;              // bound of the gather kernel's wait, in clock64 cycles
    int world, rank;
};

// Epoch of the exchange a kernel produces: the epoch word holds the exchanges completed before
// the current batch of launches (advanced once per batch by peer_batch_end_kernel, before any
// kernel of the next batch can start) and `j` is the position of this exchange in the batch, so a
// kernel that does not wait for its predecessor still knows its epoch.
__device__ __forceinline__ unsigned peer_epoch(const PeerOut *p, int j) {
    return __ldcg(p->epoch) + 1u + (unsigned)j;
}

// One local and world - 1 remote stores, issued by the lane that holds the row's sum while the
// rest of the grid is still streaming weights.
__device__ __forceinline__ void peer_store(const PeerOut *p, unsigned e, long long idx, float v) {
    const long long off = (long long)(e & 1u) * p->stride + idx;
    const unsigned long long pr = ((unsigned long long)e << 32) | (unsigned long long)__float_as_uint(v);
    // replicas are visited starting from the own rank, so that at any moment the ranks' stores are
    // spread over all replicas instead of converging on one
#pragma unroll
    for (int i = 0; i < kMaxPeers; ++i) {
        if (i < p->world) {
            int r = p->rank + i;
            if (r >= p->world) r -= p->world;
            p->ty[r][off] = pr;
        }
    }
}

}  // namespace dmc
