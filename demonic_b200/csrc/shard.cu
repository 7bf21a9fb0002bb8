// shard.cu -- row-sharded GEMV across the GPUs of one box, one process per GPU.
//
// y = W.x with W[n][k] split by rows: rank r of `world` owns rows
// [n*r/world, n*(r+1)/world) -- a contiguous block uploaded once to its own HBM --
// runs the single-GPU kernel on it, and the f32 output slices are exchanged so every
// rank ends with the whole y.  The reference has no multi-GPU code at all
// (collectives are reserved words that error, compiler/src/interp.rs:7431-7446);
// this is the one exchange the path needs.  K is never split across ranks: that
// would need a reduction of partial sums (more bytes, a second rounding order).
//
// Between GPUs with peer access the exchange is fused into the GEMV kernel (peer.cuh).
// Otherwise, or on request, ncclAllGather (ragged splits: one ncclBroadcast per rank in a
// group) follows the kernel on the context's stream.  NCCL is opened with dlopen so the
// library loads on hosts without it; an already-loaded copy (e.g. the one PyTorch
// bundles) is reused rather than loading a second one beside it.
#include <dlfcn.h>

#include <algorithm>
#include <cstring>

#include "peer.cuh"
#include "runtime.h"

namespace dmc {
namespace {

typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0, ncclFloat32 = 7, ncclUint8 = 1 };

struct NcclApi {
    void *lib = nullptr;
    int (*GetUniqueId)(ncclUniqueId *) = nullptr;
    int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*Broadcast)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
};

struct Shard {
    bool ready = false;
    int rank = 0, world = 1;
    ncclComm_t comm = nullptr;
    // one allocation, shared with the peers through CUDA IPC:
    //   [2 * max_n floats: plain y, double-buffered by epoch] [tail: the epoch word] [2 * max_n tagged pairs]
    char *region = nullptr;
    float *y = nullptr;
    int64_t max_n = 0;
    void *peer_base[kMaxPeers] = {};  // peers' regions as mapped here (own entry = region)
    PeerOut *d_peer = nullptr;        // device copy of the exchange descriptor
    unsigned *d_epoch = nullptr;
    bool fused_ok = false;            // peer mappings are in place on EVERY rank (agreed at init)
    bool last_fused = false;          // which buffer holds the latest result
};
constexpr size_t kTailBytes = 256;

// [y: 2 * max_n floats][tail: epoch word][tagged y: 2 * max_n pairs]
size_t region_bytes(int64_t max_n) { return (size_t)2 * max_n * sizeof(float) + kTailBytes + (size_t)2 * max_n * 8; }

NcclApi g_nccl;
Shard g_shard;

int load_nccl() {
    if (g_nccl.lib) return DMC_CUDA_OK;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // reuse a copy the process already has
    if (!h) {
        const char *env = getenv("DMC_NCCL_LIB");
        if (env) h = dlopen(env, RTLD_NOW | RTLD_LOCAL);
    }
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!h) return fail(DMC_CUDA_ERR_NCCL, "NCCL is not available: %s", dlerror());
#define SYM(field, name)                                                                          \
    *(void **)(&g_nccl.field) = dlsym(h, name);                                                   \
    if (!g_nccl.field) return fail(DMC_CUDA_ERR_NCCL, "NCCL symbol %s is missing", name);
    SYM(GetUniqueId, "ncclGetUniqueId")
    SYM(CommInitRank, "ncclCommInitRank")
    SYM(CommDestroy, "ncclCommDestroy")
    SYM(AllGather, "ncclAllGather")
    SYM(Broadcast, "ncclBroadcast")
    SYM(GroupStart, "ncclGroupStart")
    SYM(GroupEnd, "ncclGroupEnd")
    SYM(GetErrorString, "ncclGetErrorString")
#undef SYM
    g_nccl.lib = h;
    return DMC_CUDA_OK;
}

#define DMC_NCCL_TRY(expr)                                                                        \
    do {                                                                                          \
        int r__ = (expr);                                                                         \
        if (r__ != ncclSuccess)                                                                   \
            return fail(DMC_CUDA_ERR_NCCL, "%s failed: %s", #expr, g_nccl.GetErrorString(r__));  \
    } while (0)

// Whether a sharded GEMV uses the exchange fused into the kernel.  Every argument has the same value
// on every rank (`fused_ok` is the AND over all ranks, agreed in shard_init), so every rank takes the
// same path; n < world (some slices empty) keeps the fused path too, the empty ranks just store nothing.
bool fused_path_chosen(int world, bool fused_ok, int shard_fused, int64_t k, int64_t n) {
    const bool want = shard_fused < 0 ? world >= 2 : shard_fused != 0;
    return want && fused_ok && k > 0 && n > 0;
}

void shard_range(int64_t n, int rank, int world, int64_t *r0, int64_t *r1) {
    *r0 = n * rank / world;
    *r1 = n * (rank + 1) / world;
}

// The replicated y arrives as {value, epoch} pairs written by every rank's GEMV.  This kernel
// does not wait for the local GEMV to complete (whose completion includes the acknowledgement of its
// remote stores): it runs beside it, and re-reads each pair (bounded) until it carries the epoch of
// this exchange, then writes the plain y of that epoch's parity.  j: position of the exchange in the
// current batch of launches; n: rows of the whole y.
//
// Shape: a few CTAs that fit exactly into the CTA slots the sharded GEMV leaves free for them
// (kGatherCtas slots: a GEMV CTA is 256 threads x 128 registers, a gather CTA 512 threads x <= 64), so
// that the gather really is resident beside the GEMV and -- when exchanges overlap -- does not sit in
// slots the next GEMV needs.  A warp owns chunks of 256 consecutive 16-byte pieces (4 KiB).  Pieces that
// are neighbours in y are produced by neighbouring warps of the GEMV at about the same time, so one lane
// per chunk watches the chunk's last piece (re-reading it every ~100 ns), and only when those have
// arrived are the others read, eight per lane with the loads issued together, usually all there:
// hundreds of times fewer polling reads than one per piece, which matters because they compete with the
// weight stream for L2 for as long as the GEMVs run.
constexpr int kGatherThreads = 512, kGatherChunk = 256;
int gather_ctas(int64_t n) {
    const int64_t per_cta = (int64_t)(kGatherThreads / 32) * kGatherChunk;  // pieces one CTA covers in one pass
    return (int)std::max<int64_t>(1, std::min<int64_t>(kGatherCtas, (n / 2 + per_cta - 1) / per_cta));
}

__global__ void __launch_bounds__(kGatherThreads, 2) peer_gather_kernel(const PeerOut *p, int n, int j, float *dst_override) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // the epoch word was advanced before any kernel of this batch could start (peer_batch_end_kernel)
    const unsigned e = *(volatile const unsigned *)p->epoch + 1u + (unsigned)j;
    const unsigned long long *src = p->ty[p->rank] + (size_t)(e & 1u) * p->stride;
    float *dst = dst_override ? dst_override : p->yplain + (size_t)(e & 1u) * p->stride;
    const int pairs2 = n / 2;  // 16-byte pieces
    const long long limit = p->wait_cycles;
    __shared__ int s_failed;
    if (threadIdx.x == 0) s_failed = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * kGatherThreads + threadIdx.x) >> 5, warps = gridDim.x * (kGatherThreads / 32);
    const long long t0 = clock64();
    auto load_piece = [&](int i, unsigned &a0, unsigned &a1, unsigned &b0, unsigned &b1) {
        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(b0), "=r"(b1) : "l"(src + 2 * (size_t)i) : "memory");
    };
    // lane l watches the last piece of this warp's l-th chunk (a timeout is reported by the loop below)
    for (int c0 = (warp + lane * warps) * kGatherChunk; c0 < pairs2; c0 += 32 * warps * kGatherChunk) {
        const int watched = min(c0 + kGatherChunk, pairs2) - 1;
        for (;;) {
            unsigned a0, a1, b0, b1;
            load_piece(watched, a0, a1, b0, b1);
            if ((a1 == e && b1 == e) || clock64() - t0 > limit) break;
            __nanosleep(100);
        }
    }
    __syncwarp();
    for (int c0 = warp * kGatherChunk; c0 < pairs2; c0 += warps * kGatherChunk) {
        constexpr int P = kGatherChunk / 32;
        unsigned a0[P], a1[P], b0[P], b1[P];
        unsigned missing = 0u;
#pragma unroll
        for (int t = 0; t < P; ++t)
            if (c0 + t * 32 + lane < pairs2) missing |= 1u << t;
        // every round re-reads all of the lane's missing pieces at once: one L2 round trip per round,
        // not one per piece
        while (missing) {
#pragma unroll
            for (int t = 0; t < P; ++t)
                if (missing >> t & 1u) load_piece(c0 + t * 32 + lane, a0[t], a1[t], b0[t], b1[t]);
#pragma unroll
            for (int t = 0; t < P; ++t) {
                if ((missing >> t & 1u) && a1[t] == e && b1[t] == e) {
                    *reinterpret_cast<float2 *>(dst + 2 * (size_t)(c0 + t * 32 + lane)) = make_float2(__uint_as_float(a0[t]), __uint_as_float(b0[t]));
                    missing &= ~(1u << t);
                }
            }
            if (!missing) break;
            if (clock64() - t0 > limit) {  // give up instead of hanging: the host reads the error word
                *(volatile int *)p->err = 6;
                s_failed = 1;
                break;
            }
            __nanosleep(100);
        }
    }
    if ((n & 1) && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long v;
        const long long t0 = clock64();
        for (;;) {
            asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(src + (n - 1)) : "memory");
            if ((unsigned)(v >> 32) == e) break;
            if (clock64() - t0 > limit) {
                *(volatile int *)p->err = 6;
                s_failed = 1;
                break;
            }
            __nanosleep(100);
        }
        dst[n - 1] = __uint_as_float((unsigned)v);
    }
    // The CTA that finishes last tells every rank that this rank has read exchange e completely (its
    // replica buffer may be reused by exchange e + 2).  Publications go out in epoch order, so a
    // published value e means "every exchange up to e".  A gather that gave up publishes nothing.
    __threadfence();
    __syncthreads();
    if (threadIdx.x != 0) return;
    unsigned *cnt = p->gcount + (e & 3u);
    const unsigned arrived = atomicAdd(cnt, 1u);
    if (s_failed) atomicOr(p->gcount + 4, 1u << (e & 3u));
    if (arrived != gridDim.x - 1u) return;
    *cnt = 0u;
    const unsigned failed = atomicAnd(p->gcount + 4, ~(1u << (e & 3u))) & (1u << (e & 3u));
    __threadfence();
    if (failed) return;
    const unsigned *own = p->gdone[p->rank] + p->rank;
    const long long t1 = clock64();
    while (*(volatile const unsigned *)own != e - 1u) {  // the previous exchange's publication first
        if (clock64() - t1 > limit) {
            *(volatile int *)p->err = 8;
            return;
        }
        __nanosleep(100);
    }
    for (int i = 0; i < kMaxPeers; ++i) {
        if (i < p->world) {
            int r = p->rank + 1 + i;  // own word last: the next local gather's publication waits on it
            if (r >= p->world) r -= p->world;
            *(volatile unsigned *)(p->gdone[r] + p->rank) = e;
        }
    }
}

// Closes a batch of `count` exchanges.  Waits for everything before it, then advances the
// epoch word -- before any kernel of the next batch can start, since those launch only after the
// launch_dependents below.
__global__ void peer_batch_end_kernel(const PeerOut *p, int count) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) {
        *(volatile unsigned *)p->epoch = *(volatile unsigned *)p->epoch + (unsigned)count;
        __threadfence();
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// j: position of this call in a batch of back-to-back sharded GEMVs; end_batch: it is the last one.
// dst: where the whole y goes on this rank (device, n floats); null = the library's own y buffers.
int shard_gemv_on(const void *dW_shard, const float *dx, int64_t k, int64_t n, int wdtype, cudaStream_t s,
                  int j = 0, bool end_batch = true, float *dst = nullptr) {
    Shard &sh = g_shard;
    if (!sh.ready) return fail(DMC_CUDA_ERR_BAD_ARG, "shard_gemv: dmc_cuda_shard_init has not been called");
    if (n > sh.max_n) return fail(DMC_CUDA_ERR_UNSUPPORTED, "shard_gemv: n=%lld beyond the max_n=%lld given to shard_init",
                                  (long long)n, (long long)sh.max_n);
    int64_t r0, r1;
    shard_range(n, sh.rank, sh.world, &r0, &r1);
    // Measured on B200 (65536x8192): the fused exchange is ahead of ncclAllGather from 2 ranks up
    // (89.5 vs 95.4 us at 2, 26.0 vs 42.5 us at 8).  The choice uses only facts that are the same on
    // every rank -- a rank that took the other path would leave its peers waiting for it.
    if (fused_path_chosen(sh.world, sh.fused_ok, tuning().shard_fused, k, n)) {
        // one kernel: GEMV whose epilogue stores into every replica; the gather kernel beside it
        // validates the arrivals.  A rank whose slice is empty still runs the gather and the batch
        // end, so its epoch stays in step with its peers.
        Context &c = ctx();
        int rc = DMC_CUDA_OK;
        if (r1 > r0) {
            c.peer = sh.d_peer;
            c.peer_yoff = r0;
            c.peer_j = j;
            rc = launch_gemv(dW_shard, dx, sh.y + r0, 1, k, r1 - r0, 1, 0, 0, DMC_LAYOUT_NK, wdtype, -1, s);
            c.peer = nullptr;
            c.peer_yoff = 0;
            c.peer_j = 0;
        }
        sh.last_fused = true;
        if (rc == DMC_CUDA_OK) {
            const PeerOut *pp = sh.d_peer;
            int rows = (int)n, jj = j;
            void *params[] = {&pp, &rows, &jj, &dst};
            const int ctas = gather_ctas(n);
            // the gather never waits for its predecessor; what it writes is recorded so that a consumer of y does
            rc = launch_ex((const void *)peer_gather_kernel, dim3(ctas), dim3(kGatherThreads), 0, s, params,
                           c.nowait_inflight ? kLaunchOverlap : kLaunchTracked);
            if (dst) c.inflight_writes.push_back(AddrRange{(uintptr_t)dst, (uintptr_t)dst + (size_t)n * 4});
            else c.inflight_writes.push_back(AddrRange{(uintptr_t)sh.y, (uintptr_t)sh.y + (size_t)2 * sh.max_n * 4});
            if (rc == DMC_CUDA_OK && end_batch) {
                int count = j + 1;
                void *params2[] = {&pp, &count};
                rc = launch_ex((const void *)peer_batch_end_kernel, dim3(1), dim3(32), 0, s, params2, kLaunchTracked);
            }
        }
        return rc;
    }
    sh.last_fused = false;
    int rc = launch_gemv(dW_shard, dx, sh.y + r0, 1, k, r1 - r0, 1, 0, 0, DMC_LAYOUT_NK, wdtype, -1, s);
    if (rc) return rc;
    if (sh.world == 1) return DMC_CUDA_OK;
    ctx().untracked_inflight = true;  // the collective below writes y outside the launch planner's view
    struct CopyOut {  // the NCCL exchange fills the library's own y; a caller's destination gets a copy
        float *dst, *src; int64_t n; cudaStream_t s;
        ~CopyOut() { if (dst) cudaMemcpyAsync(dst, src, (size_t)n * 4, cudaMemcpyDeviceToDevice, s); }
    } copy_out{dst, sh.y, n, s};
    if (n % sh.world == 0) {
        DMC_NCCL_TRY(g_nccl.AllGather(sh.y + r0, sh.y, (size_t)(n / sh.world), ncclFloat32, sh.comm, s));
    } else {  // ragged: every rank broadcasts its slice
        DMC_NCCL_TRY(g_nccl.GroupStart());
        for (int r = 0; r < sh.world; ++r) {
            int64_t a, b;
            shard_range(n, r, sh.world, &a, &b);
            if (b > a) {
                int e = g_nccl.Broadcast(sh.y + a, sh.y + a, (size_t)(b - a), ncclFloat32, r, sh.comm, s);
                if (e != ncclSuccess) {
                    g_nccl.GroupEnd();
                    return fail(DMC_CUDA_ERR_NCCL, "ncclBroadcast failed: %s", g_nccl.GetErrorString(e));
                }
            }
        }
        DMC_NCCL_TRY(g_nccl.GroupEnd());
    }
    return DMC_CUDA_OK;
}

}  // namespace

int shard_gemv_to_host(const void *dW_shard, const float *dx, int64_t k, int64_t n, int wdtype, float *h_dst,
                       cudaStream_t stream) {
    Shard &sh = g_shard;
    if (sh.ready && n <= sh.max_n && fused_path_chosen(sh.world, sh.fused_ok, tuning().shard_fused, k, n))
        return shard_gemv_on(dW_shard, dx, k, n, wdtype, stream, 0, true, h_dst);
    int rc = shard_gemv_on(dW_shard, dx, k, n, wdtype, stream);
    if (rc) return rc;
    DMC_CUDA_TRY(cudaMemcpyAsync(h_dst, sh.y, (size_t)n * 4, cudaMemcpyDeviceToHost, stream));
    ctx().done_is_last = false;
    return DMC_CUDA_OK;
}

}  // namespace dmc

using namespace dmc;

extern "C" void dmc_cuda_shard_range(int64_t n, int rank, int world, int64_t *r0, int64_t *r1) {
    if (world < 1) world = 1;
    shard_range(n, rank, world, r0, r1);
}

extern "C" int dmc_cuda_shard_unique_id(uint8_t *out128) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    int rc = load_nccl();
    if (rc) return rc;
    ncclUniqueId id;
    DMC_NCCL_TRY(g_nccl.GetUniqueId(&id));
    memcpy(out128, id.internal, 128);
    return DMC_CUDA_OK;
}

namespace dmc {
namespace {

void shard_release(Shard &sh) {
    for (int r = 0; r < sh.world && r < kMaxPeers; ++r)
        if (r != sh.rank && sh.peer_base[r]) cudaIpcCloseMemHandle(sh.peer_base[r]);
    if (sh.comm) g_nccl.CommDestroy(sh.comm);
    if (sh.d_peer) cudaFree(sh.d_peer);
    if (sh.region) cudaFree(sh.region);
    sh = Shard();
}

int shard_init_locked(int rank, int world, const uint8_t *id128, int64_t max_n) {
    Shard &sh = g_shard;
    sh.rank = rank;
    sh.world = world;
    if (world > 1 || inject_failure("nccl_init")) {
        if (inject_failure("nccl_init")) return fail(DMC_CUDA_ERR_NCCL, "ncclCommInitRank failed: injected");
        if (!id128) return fail(DMC_CUDA_ERR_BAD_ARG, "shard_init: world > 1 needs the 128-byte NCCL id");
        int rc = load_nccl();
        if (rc) return rc;
        ncclUniqueId id;
        memcpy(id.internal, id128, 128);
        DMC_NCCL_TRY(g_nccl.CommInitRank(&sh.comm, world, id, rank));
    }
    max_n = (max_n + 3) & ~(int64_t)3;  // keeps both halves of every double buffer 16-byte aligned
    const size_t bytes = region_bytes(max_n);
    DMC_CUDA_TRY(dmc_malloc((void **)&sh.region, bytes));
    DMC_CUDA_TRY(cudaMemset(sh.region, 0, bytes));
    sh.y = reinterpret_cast<float *>(sh.region);
    sh.max_n = max_n;
    sh.peer_base[rank] = sh.region;
    bool mine_ok = world <= kMaxPeers && !inject_failure("ipc_open");
    cudaStream_t s = ctx().stream;
    if (world > 1) {
        // exchange the IPC handle of the region through the communicator itself
        cudaIpcMemHandle_t mine, all[kMaxPeers];
        char *d_h = nullptr;
        if (mine_ok) {
            DMC_CUDA_TRY(cudaIpcGetMemHandle(&mine, sh.region));
            DMC_CUDA_TRY(dmc_malloc((void **)&d_h, sizeof(mine) * world));
            DMC_CUDA_TRY(cudaMemcpy(d_h + sizeof(mine) * rank, &mine, sizeof(mine), cudaMemcpyHostToDevice));
            DMC_NCCL_TRY(g_nccl.AllGather(d_h + sizeof(mine) * rank, d_h, sizeof(mine), ncclUint8, sh.comm, s));
            DMC_CUDA_TRY(cudaStreamSynchronize(s));
            DMC_CUDA_TRY(cudaMemcpy(all, d_h, sizeof(mine) * world, cudaMemcpyDeviceToHost));
            cudaFree(d_h);
            for (int r = 0; r < world; ++r) {
                if (r == rank) continue;
                cudaError_t e = cudaIpcOpenMemHandle(&sh.peer_base[r], all[r], cudaIpcMemLazyEnablePeerAccess);
                if (e != cudaSuccess) {  // no peer access between these GPUs: keep the NCCL exchange
                    cudaGetLastError();
                    sh.peer_base[r] = nullptr;
                    mine_ok = false;
                    break;
                }
            }
        }
        // Every rank must take the same path in every later call: the fused exchange is used only
        // if the mappings are in place on all of them (one byte per rank, gathered; AND).
        unsigned char *d_ok = nullptr, ok_all[kMaxPeers + 56] = {};
        const size_t slots = (size_t)std::max(world, 1);
        DMC_CUDA_TRY(dmc_malloc((void **)&d_ok, slots));
        const unsigned char ok_byte = mine_ok ? 1 : 0;
        DMC_CUDA_TRY(cudaMemcpy(d_ok + rank, &ok_byte, 1, cudaMemcpyHostToDevice));
        DMC_NCCL_TRY(g_nccl.AllGather(d_ok + rank, d_ok, 1, ncclUint8, sh.comm, s));
        DMC_CUDA_TRY(cudaStreamSynchronize(s));
        DMC_CUDA_TRY(cudaMemcpy(ok_all, d_ok, std::min(slots, sizeof(ok_all)), cudaMemcpyDeviceToHost));
        cudaFree(d_ok);
        sh.fused_ok = world <= kMaxPeers;
        for (int r = 0; r < world && r < (int)sizeof(ok_all); ++r) sh.fused_ok = sh.fused_ok && ok_all[r] != 0;
    } else {
        sh.fused_ok = mine_ok;
    }
    if (sh.fused_ok) {
        PeerOut po = {};
        for (int r = 0; r < world; ++r)
            po.ty[r] = reinterpret_cast<unsigned long long *>(static_cast<char *>(sh.peer_base[r]) +
                                                              (size_t)2 * max_n * sizeof(float) + kTailBytes);
        po.yplain = sh.y;
        // tail of the region: [0] the epoch word, [8..12] the gather's arrival counters + failure mask,
        // [16..24) the published epochs of every rank's gather (written by the peers)
        for (int r = 0; r < world; ++r)
            po.gdone[r] = reinterpret_cast<unsigned *>(static_cast<char *>(sh.peer_base[r]) + (size_t)2 * max_n * sizeof(float)) + 16;
        po.epoch = reinterpret_cast<unsigned *>(sh.region + (size_t)2 * max_n * sizeof(float));
        po.gcount = po.epoch + 8;
        po.err = ctx().err_word;
        po.stride = max_n;
        // bound of the gather kernel's wait for its peers: "wait_limit_us", by default about a second
        const long long us = tuning().wait_limit_us > 0 ? tuning().wait_limit_us : 1000000;
        po.wait_cycles = us * (long long)(ctx().clock_khz / 1000);
        po.world = world;
        po.rank = rank;
        sh.d_epoch = po.epoch;
        DMC_CUDA_TRY(dmc_malloc((void **)&sh.d_peer, sizeof(PeerOut)));
        DMC_CUDA_TRY(cudaMemcpy(sh.d_peer, &po, sizeof(po), cudaMemcpyHostToDevice));
    }
    if (world > 1) {  // nobody may store into a peer before that peer has zeroed its region
        DMC_NCCL_TRY(g_nccl.AllGather(sh.y + rank, sh.y, 1, ncclFloat32, sh.comm, s));
        DMC_CUDA_TRY(cudaStreamSynchronize(s));
        DMC_CUDA_TRY(cudaMemset(sh.y, 0, (size_t)world * sizeof(float)));
    }
    stream_drained();
    sh.ready = true;
    return DMC_CUDA_OK;
}

}  // namespace
}  // namespace dmc

extern "C" int dmc_cuda_shard_init(int rank, int world, const uint8_t *id128, int64_t max_n) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    if (world < 1 || rank < 0 || rank >= world || max_n < 1)
        return fail(DMC_CUDA_ERR_BAD_ARG, "shard_init: bad rank %d / world %d / max_n %lld", rank, world, (long long)max_n);
    int rc = ensure_init();
    if (rc) return rc;
    if (g_shard.ready) return fail(DMC_CUDA_ERR_BAD_ARG, "shard_init: already initialised");
    rc = shard_init_locked(rank, world, id128, max_n);
    if (rc) shard_release(g_shard);  // nothing half-built stays behind a failed init
    return rc;
}

// 1 when sharded GEMVs of this size would use the exchange fused into the kernel, 0 for the NCCL exchange.
extern "C" int dmc_cuda_shard_uses_fused(int64_t k, int64_t n) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (!g_shard.ready) return 0;
    return fused_path_chosen(g_shard.world, g_shard.fused_ok, tuning().shard_fused, k, n) ? 1 : 0;
}

// The same decision from explicit facts (pure; no device): lets a host check that every rank would agree.
extern "C" int dmc_cuda_shard_path(int world, int peer_access_everywhere, int shard_fused, int64_t k, int64_t n) {
    return fused_path_chosen(world, peer_access_everywhere != 0, shard_fused, k, n) ? 1 : 0;
}

extern "C" void dmc_cuda_shard_shutdown(void) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    Shard &sh = g_shard;
    if (!sh.ready) return;
    if (ctx().ready) cudaStreamSynchronize(ctx().stream);
    stream_drained();
    shard_release(sh);
}

extern "C" float *dmc_cuda_shard_output(void) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    Shard &sh = g_shard;
    if (!sh.ready) return nullptr;
    if (!sh.last_fused) return sh.y;
    // the fused exchange alternates between two buffers; after a synchronisation the epoch word counts the
    // completed exchanges, so its parity names the current one
    unsigned e = 0;
    cudaStreamSynchronize(ctx().stream);
    cudaMemcpy(&e, sh.d_epoch, sizeof(e), cudaMemcpyDeviceToHost);
    return sh.y + (size_t)(e & 1u) * sh.max_n;
}

// Self-test of the bounded waits: run the gather for an exchange that no GEMV writes.  Every thread of
// it re-reads its pair until the configured limit ("wait_limit_us" at shard_init) runs out, records the
// error word and returns; the host then reports DMC_CUDA_ERR_TIMEOUT like any other failed call.
// Nothing faults or hangs, the context stays usable (clear the error and carry on).
extern "C" int dmc_cuda_shard_probe_timeout(int64_t n) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    Shard &sh = g_shard;
    if (!sh.ready || !sh.fused_ok || n < 1 || n > sh.max_n)
        return fail(DMC_CUDA_ERR_BAD_ARG, "shard_probe_timeout: needs dmc_cuda_shard_init with the fused exchange and 1 <= n <= max_n");
    const PeerOut *pp = sh.d_peer;
    int rows = (int)n, far = 1 << 20;  // an epoch a million exchanges ahead: nobody has written it
    float *none = nullptr;
    void *params[] = {&pp, &rows, &far, &none};
    const int ctas = gather_ctas(n);
    int rc = launch_ex((const void *)peer_gather_kernel, dim3(ctas), dim3(kGatherThreads), 0, ctx().stream, params);
    if (rc) return rc;
    DMC_CUDA_TRY(cudaStreamSynchronize(ctx().stream));
    stream_drained();
    return check_device_error();
}

extern "C" float *dmc_cuda_shard_output_previous(void) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    Shard &sh = g_shard;
    if (!sh.ready) return nullptr;
    cudaStreamSynchronize(ctx().stream);
    if (!sh.last_fused) return sh.y;
    unsigned e = 0;
    cudaMemcpy(&e, sh.d_epoch, sizeof(e), cudaMemcpyDeviceToHost);
    return sh.y + (size_t)((e + 1u) & 1u) * sh.max_n;
}

extern "C" int dmc_cuda_shard_gemv(const void *dW_shard, const float *dx, int64_t k, int64_t n, int wdtype) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    return shard_gemv_on(dW_shard, dx, k, n, wdtype, ctx().stream);
}

extern "C" int dmc_cuda_shard_gemv_batch(const void *const *dW_shards, int count, const float *dx, float *const *dy_out,
                                         int64_t k, int64_t n, int wdtype) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    if (!dW_shards || count < 1) return fail(DMC_CUDA_ERR_BAD_ARG, "shard_gemv_batch: needs count >= 1 weight shards");
    for (int i = 0; i < count; ++i) {
        int rc = shard_gemv_on(dW_shards[i], dx, k, n, wdtype, ctx().stream, i, i == count - 1, dy_out ? dy_out[i] : nullptr);
        if (rc) return rc;
    }
    return DMC_CUDA_OK;
}

extern "C" double dmc_cuda_bench_shard(const void *const *dW_shards, int copies, const float *dx, int64_t k,
                                       int64_t n, int wdtype, int steps, int warmup, int use_graph) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return -1.0;
    if (!g_shard.ready || copies < 1 || steps < 1 || warmup < 0) {
        fail(DMC_CUDA_ERR_BAD_ARG, "bench_shard: needs shard_init, copies >= 1, steps >= 1");
        return -1.0;
    }
    Context &c = ctx();
    cudaStream_t s = c.stream;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    double us = -1.0;
    auto one_step = [&]() -> int {
        for (int i = 0; i < copies; ++i) {
            int rc = shard_gemv_on(dW_shards[i], dx, k, n, wdtype, s, i, i == copies - 1);
            if (rc) return rc;
        }
        return DMC_CUDA_OK;
    };
    auto body = [&]() -> int {
        int rc = one_step();  // eager: sizes scratch, lets NCCL set up its channels
        if (rc) return rc;
        DMC_CUDA_TRY(cudaStreamSynchronize(s));
        stream_drained();
        DMC_CUDA_TRY(cudaEventCreate(&e0));
        DMC_CUDA_TRY(cudaEventCreate(&e1));
        int64_t per_step = 0;
        if (use_graph) {
            const int64_t before = c.launches;
            DMC_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
            rc = one_step();
            cudaError_t ce = cudaStreamEndCapture(s, &graph);
            stream_drained();
            if (rc) return rc;
            DMC_CUDA_TRY(ce);
            per_step = c.launches - before;
            DMC_CUDA_TRY(cudaGraphInstantiate(&exec, graph, 0));
        }
        auto run_step = [&]() -> int {
            if (!use_graph) return one_step();
            DMC_CUDA_TRY(cudaGraphLaunch(exec, s));
            c.launches += per_step;
            return DMC_CUDA_OK;
        };
        for (int i = 0; i < warmup; ++i)
            if ((rc = run_step())) return rc;
        DMC_CUDA_TRY(cudaStreamSynchronize(s));
        DMC_CUDA_TRY(cudaEventRecord(e0, s));
        for (int i = 0; i < steps; ++i)
            if ((rc = run_step())) return rc;
        DMC_CUDA_TRY(cudaEventRecord(e1, s));
        DMC_CUDA_TRY(cudaStreamSynchronize(s));
        float ms = 0.0f;
        DMC_CUDA_TRY(cudaEventElapsedTime(&ms, e0, e1));
        us = (double)ms * 1000.0 / steps;
        return DMC_CUDA_OK;
    };
    body();
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    return dmc::status() ? -1.0 : us;
}
