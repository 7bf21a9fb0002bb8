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
// the pairs a slower rank's gather of exchange e is still reading.  Exchange e + 2 reuses the
// buffer of exchange e: before its first store a GEMV checks (bounded) that the gather of exchange
// e has completed on EVERY rank -- each gather, when its last CTA is done, publishes its epoch into
// a small array in every rank's memory, in epoch order.  With that guard the GEMVs of a batch of
// independent exchanges need not wait for one another: exchange e + 1 streams its weights while the
// stores of exchange e are still crossing NVLink.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dmc {

constexpr int kMaxPeers = 8;
// CTA slots a sharded GEMV that would fill the device leaves free, for the kernel that checks the
// arrivals of the exchange beside it (one CTA of that kernel fits the room one GEMV CTA leaves).
constexpr int kGatherCtas = 4;

struct PeerOut {
    unsigned long long *ty[kMaxPeers];  // each rank's tagged replica: 2 * stride {value, epoch} pairs
    float *yplain;                      // local plain y the gather kernel fills (2 * stride floats)
    unsigned *gdone[kMaxPeers];         // gdone[q][s] (in rank q's memory): last epoch whose gather completed on rank s
    unsigned *gcount;                   // local: four CTA arrival counters of the gather kernel, indexed by epoch & 3
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

// Before the first store of exchange e: the buffer it writes last held exchange e - 2, whose arrival
// check must have completed on every rank.  One thread reads the local copy of the published epochs
// (eight words, two 16-byte asynchronous copies issued together by peer_guard_load so that they are in flight beside
// the loads that stage x; one word at a time they would put `world` L2 round trips in front of every
// CTA's first row) and peer_guard_ok looks at them afterwards.  Normally all are there long before:
// that gather finished a whole GEMV ago.  Otherwise peer_wait_buffer_free polls, bounded.
__device__ __forceinline__ void peer_guard_load(const PeerOut *p, unsigned *smem_words) {
    static_assert(kMaxPeers == 8, "two 16-byte copies cover the published epochs");
    const unsigned *mine = p->gdone[p->rank];  // 16-byte aligned by the layout dmc_cuda_shard_init builds
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_words);
    // asynchronous copies through L2 into shared memory: nothing is held in registers meanwhile
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(mine) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16u), "l"(mine + 4) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
}

__device__ __forceinline__ bool peer_guard_ok(const PeerOut *p, unsigned e, const unsigned *smem_words) {
    asm volatile("cp.async.wait_all;" ::: "memory");
    bool ok = true;
#pragma unroll
    for (int s = 0; s < kMaxPeers; ++s)
        if (s < p->world && (int)(*(volatile const unsigned *)(smem_words + s) - (e - 2u)) < 0) ok = false;
    return ok;
}

static __device__ __noinline__ void peer_wait_buffer_free(const PeerOut *p, unsigned e) {
    if (e < 3u) return;
    const unsigned need = e - 2u;
    const unsigned *mine = p->gdone[p->rank];
    const long long t0 = clock64();
    for (int s = 0; s < p->world; ++s) {
        while ((int)(*(volatile const unsigned *)(mine + s) - need) < 0) {
            if (clock64() - t0 > p->wait_cycles) {  // give up instead of hanging: the host reads the error word
                *(volatile int *)p->err = 7;
                return;
            }
            __nanosleep(100);
        }
    }
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
