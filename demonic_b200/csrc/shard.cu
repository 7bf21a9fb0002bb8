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
// Exchange mode 0: ncclAllGather (ragged splits: one ncclBroadcast per rank in a
// group) on the context's stream.  NCCL is opened with dlopen so the library loads
// on hosts without it; an already-loaded copy (e.g. the one PyTorch bundles) is
// reused rather than loading a second one beside it.
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
    //   [2 * max_n floats: y, double-buffered by epoch] [kMaxPeers flag words] [epoch] [CTA counter]
    char *region = nullptr;
    float *y = nullptr;
    int64_t max_n = 0;
    void *peer_base[kMaxPeers] = {};  // peers' regions as mapped here (own entry = region)
    PeerOut *d_peer = nullptr;        // device copy of the exchange descriptor
    unsigned *d_epoch = nullptr;
    int peer_mode = 3;  // 3: tagged elements + gather kernel (default); 2: counted arrivals; 1: flag exchange by the last CTA
    bool fused_ok = false;            // peer mappings are in place
    bool last_fused = false;          // which buffer holds the latest result
};
constexpr size_t kTailBytes = 256;

// [y: 2 * max_n floats][tail: flags, epoch, counters][tagged y: 2 * max_n pairs]
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

void shard_range(int64_t n, int rank, int world, int64_t *r0, int64_t *r1) {
    *r0 = n * rank / world;
    *r1 = n * (rank + 1) / world;
}

// Local GEMV into y[r0, r1) then the exchange, all on `s`.
// Closes an exchange for consumers that are not themselves a sharded GEMV: returns once every rank's
// share of the current epoch has been counted here.  One thread.
__global__ void peer_wait_kernel(const PeerOut *p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x != 0 || (p->debug & 2)) return;
    const unsigned e = __ldcg(p->epoch);
    const unsigned target = e * (unsigned)p->world * kPeerQuantum;
    const unsigned *mine = p->flags[p->rank];
    const long long t0 = clock64();
    while ((int)(ld_acquire_sys(mine) - target) < 0) {
        if (clock64() - t0 > (1LL << 31)) {
            *(volatile int *)p->err = 5;
            break;
        }
    }
}

// mode 3: the replicated y arrives as {value, epoch} pairs written by every rank's GEMV.  This kernel
// does not wait for the local GEMV to complete (whose completion includes the acknowledgement of its
// remote stores): it runs beside it, and re-reads each pair (bounded) until it carries the epoch of
// this exchange, then writes the plain y of that epoch's parity.  j: position of the exchange in the
// current batch of launches; n: rows of the whole y.
__global__ void __launch_bounds__(256) peer_gather_kernel(const PeerOut *p, int n, int j) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // the epoch word was advanced before any kernel of this batch could start (peer_batch_end_kernel)
    const unsigned e = *(volatile const unsigned *)p->epoch + 1u + (unsigned)j;
    const unsigned long long *src = p->ty[p->rank] + (size_t)(e & 1u) * p->stride;
    float *dst = p->yplain + (size_t)(e & 1u) * p->stride;
    const int pairs2 = n / 2;  // 16-byte pieces
    const bool skip = (p->debug & 2) != 0;
    const int first = blockIdx.x * blockDim.x;
    // While the GEMVs are still streaming, one thread per CTA watches one piece at a relaxed pace, so
    // that the 32K threads of this grid do not load L2 for the whole duration of the GEMV.
    if (threadIdx.x == 0 && first < pairs2 && !skip) {
        const long long t0 = clock64();
        for (;;) {
            unsigned a0, a1, b0, b1;
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(b0), "=r"(b1) : "l"(src + 2 * (size_t)first) : "memory");
            if (a1 == e && b1 == e) break;
            if (clock64() - t0 > (1LL << 31)) break;  // the loop below reports it
            __nanosleep(200);
        }
    }
    __syncthreads();
    for (int i = first + threadIdx.x; i < pairs2; i += gridDim.x * blockDim.x) {
        unsigned a0, a1, b0, b1;
        const long long t0 = clock64();
        for (;;) {
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(b0), "=r"(b1) : "l"(src + 2 * (size_t)i) : "memory");
            if ((a1 == e && b1 == e) || skip) break;
            if (clock64() - t0 > (1LL << 31)) {  // ~1 s: give up instead of hanging
                *(volatile int *)p->err = 6;
                break;
            }
            __nanosleep(100);
        }
        *reinterpret_cast<float2 *>(dst + 2 * (size_t)i) = make_float2(__uint_as_float(a0), __uint_as_float(b0));
    }
    if ((n & 1) && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long v;
        const long long t0 = clock64();
        for (;;) {
            asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(src + (n - 1)) : "memory");
            if ((unsigned)(v >> 32) == e || skip) break;
            if (clock64() - t0 > (1LL << 31)) {
                *(volatile int *)p->err = 6;
                break;
            }
            __nanosleep(100);
        }
        dst[n - 1] = __uint_as_float((unsigned)v);
    }
}

// mode 3: closes a batch of `count` exchanges.  Waits for everything before it, then advances the
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
int shard_gemv_on(const void *dW_shard, const float *dx, int64_t k, int64_t n, int wdtype, cudaStream_t s,
                  int j = 0, bool end_batch = true) {
    Shard &sh = g_shard;
    if (!sh.ready) return fail(DMC_CUDA_ERR_BAD_ARG, "shard_gemv: dmc_cuda_shard_init has not been called");
    if (n > sh.max_n) return fail(DMC_CUDA_ERR_UNSUPPORTED, "shard_gemv: n=%lld beyond the max_n=%lld given to shard_init",
                                  (long long)n, (long long)sh.max_n);
    int64_t r0, r1;
    shard_range(n, sh.rank, sh.world, &r0, &r1);
    // Measured on B200 (65536x8192): the fused exchange is ahead of ncclAllGather from 2 ranks up
    // (89.5 vs 95.4 us at 2, 26.0 vs 42.5 us at 8).
    const bool want_fused = tuning().shard_fused < 0 ? sh.world >= 2 : tuning().shard_fused != 0;
    if (want_fused && sh.fused_ok && r1 > r0 && k > 0) {
        // one kernel: GEMV whose epilogue stores into every replica and closes with the flag exchange
        Context &c = ctx();
        c.peer = sh.d_peer;
        c.peer_yoff = r0;
        c.peer_j = j;
        const int mode = sh.peer_mode;
        int rc = launch_gemv(dW_shard, dx, sh.y + r0, 1, k, r1 - r0, 1, 0, 0, DMC_LAYOUT_NK, wdtype, -1, s);
        c.peer = nullptr;
        c.peer_yoff = 0;
        c.peer_j = 0;
        sh.last_fused = true;
        if (rc == DMC_CUDA_OK && mode == 3) {
            const PeerOut *pp = sh.d_peer;
            int rows = (int)n, jj = j;
            void *params[] = {&pp, &rows, &jj};
            const int ctas = (int)std::max<int64_t>(1, std::min<int64_t>(128, (n / 2 + 255) / 256));  // one 16-byte piece per thread up to 64K rows
            rc = launch_ex((const void *)peer_gather_kernel, dim3(ctas), dim3(256), 0, s, params);
            if (rc == DMC_CUDA_OK && end_batch) {
                int count = j + 1;
                void *params2[] = {&pp, &count};
                rc = launch_ex((const void *)peer_batch_end_kernel, dim3(1), dim3(32), 0, s, params2);
            }
        }
        if (rc == DMC_CUDA_OK && mode == 2 && end_batch) {
            const PeerOut *pp = sh.d_peer;
            void *params[] = {&pp};
            rc = launch_ex((const void *)peer_wait_kernel, dim3(1), dim3(32), 0, s, params);
        }
        return rc;
    }
    sh.last_fused = false;
    int rc = launch_gemv(dW_shard, dx, sh.y + r0, 1, k, r1 - r0, 1, 0, 0, DMC_LAYOUT_NK, wdtype, -1, s);
    if (rc) return rc;
    if (sh.world == 1) return DMC_CUDA_OK;
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

extern "C" int dmc_cuda_shard_init(int rank, int world, const uint8_t *id128, int64_t max_n) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    if (world < 1 || rank < 0 || rank >= world || max_n < 1)
        return fail(DMC_CUDA_ERR_BAD_ARG, "shard_init: bad rank %d / world %d / max_n %lld", rank, world, (long long)max_n);
    int rc = ensure_init();
    if (rc) return rc;
    Shard &sh = g_shard;
    if (sh.ready) return fail(DMC_CUDA_ERR_BAD_ARG, "shard_init: already initialised");
    if (world > 1) {
        if (!id128) return fail(DMC_CUDA_ERR_BAD_ARG, "shard_init: world > 1 needs the 128-byte NCCL id");
        rc = load_nccl();
        if (rc) return rc;
        ncclUniqueId id;
        memcpy(id.internal, id128, 128);
        DMC_NCCL_TRY(g_nccl.CommInitRank(&sh.comm, world, id, rank));
    }
    max_n = (max_n + 3) & ~(int64_t)3;  // keeps both halves of every double buffer 16-byte aligned
    const size_t bytes = region_bytes(max_n);
    DMC_CUDA_TRY(cudaMalloc((void **)&sh.region, bytes));
    DMC_CUDA_TRY(cudaMemset(sh.region, 0, bytes));
    sh.y = reinterpret_cast<float *>(sh.region);
    sh.max_n = max_n;
    sh.rank = rank;
    sh.world = world;
    sh.peer_base[rank] = sh.region;
    sh.fused_ok = world <= kMaxPeers;
    if (world > 1 && sh.fused_ok) {
        // exchange the IPC handle of the region through the communicator itself
        cudaIpcMemHandle_t mine, all[kMaxPeers];
        DMC_CUDA_TRY(cudaIpcGetMemHandle(&mine, sh.region));
        char *d_h = nullptr;
        DMC_CUDA_TRY(cudaMalloc((void **)&d_h, sizeof(mine) * world));
        DMC_CUDA_TRY(cudaMemcpy(d_h + sizeof(mine) * rank, &mine, sizeof(mine), cudaMemcpyHostToDevice));
        cudaStream_t s = ctx().stream;
        DMC_NCCL_TRY(g_nccl.AllGather(d_h + sizeof(mine) * rank, d_h, sizeof(mine), ncclUint8, sh.comm, s));
        DMC_CUDA_TRY(cudaStreamSynchronize(s));
        DMC_CUDA_TRY(cudaMemcpy(all, d_h, sizeof(mine) * world, cudaMemcpyDeviceToHost));
        cudaFree(d_h);
        for (int r = 0; r < world; ++r) {
            if (r == rank) continue;
            cudaError_t e = cudaIpcOpenMemHandle(&sh.peer_base[r], all[r], cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {  // no peer access between these GPUs: keep the NCCL exchange
                cudaGetLastError();
                sh.fused_ok = false;
                break;
            }
        }
    }
    if (sh.fused_ok) {
        PeerOut po = {};
        for (int r = 0; r < world; ++r) {
            char *base = static_cast<char *>(sh.peer_base[r]);
            po.y[r] = reinterpret_cast<float *>(base);
            po.flags[r] = reinterpret_cast<unsigned *>(base + (size_t)2 * max_n * sizeof(float));
            po.ty[r] = reinterpret_cast<unsigned long long *>(base + (size_t)2 * max_n * sizeof(float) + kTailBytes);
        }
        po.yplain = sh.y;
        unsigned *tail = reinterpret_cast<unsigned *>(sh.region + (size_t)2 * max_n * sizeof(float));
        po.epoch = tail + kMaxPeers;
        po.counter = tail + kMaxPeers + 1;
        po.err = ctx().err_word;
        po.stride = max_n;
        po.world = world;
        po.rank = rank;
        po.debug = tuning().shard_debug;
        // the two fused protocols keep different state in the flag words: the choice is made once, here
        {
            const int want = tuning().shard_exchange;
            po.mode = sh.peer_mode = (want >= 1 && want <= 3) ? want : 3;
        }
        sh.d_epoch = po.epoch;
        DMC_CUDA_TRY(cudaMalloc((void **)&sh.d_peer, sizeof(PeerOut)));
        DMC_CUDA_TRY(cudaMemcpy(sh.d_peer, &po, sizeof(po), cudaMemcpyHostToDevice));
    }
    if (world > 1) {  // nobody may store into a peer before that peer has zeroed its flags
        DMC_NCCL_TRY(g_nccl.AllGather(sh.y + rank, sh.y, 1, ncclFloat32, sh.comm, ctx().stream));
        DMC_CUDA_TRY(cudaStreamSynchronize(ctx().stream));
        DMC_CUDA_TRY(cudaMemset(sh.y, 0, (size_t)world * sizeof(float)));
    }
    sh.ready = true;
    return DMC_CUDA_OK;
}

extern "C" void dmc_cuda_shard_shutdown(void) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    Shard &sh = g_shard;
    if (!sh.ready) return;
    if (ctx().ready) cudaStreamSynchronize(ctx().stream);
    for (int r = 0; r < sh.world && r < kMaxPeers; ++r)
        if (r != sh.rank && sh.peer_base[r]) cudaIpcCloseMemHandle(sh.peer_base[r]);
    if (sh.comm) g_nccl.CommDestroy(sh.comm);
    if (sh.d_peer) cudaFree(sh.d_peer);
    if (sh.region) cudaFree(sh.region);
    sh = Shard();
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

extern "C" int dmc_cuda_shard_gemv(const void *dW_shard, const float *dx, int64_t k, int64_t n, int wdtype) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    return shard_gemv_on(dW_shard, dx, k, n, wdtype, ctx().stream);
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
        // with the counted exchange every GEMV begins by waiting for the previous exchange to have landed,
        // so only the last one of the step needs the separate closing wait
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
        DMC_CUDA_TRY(cudaEventCreate(&e0));
        DMC_CUDA_TRY(cudaEventCreate(&e1));
        int64_t per_step = 0;
        if (use_graph) {
            const int64_t before = c.launches;
            DMC_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
            rc = one_step();
            cudaError_t ce = cudaStreamEndCapture(s, &graph);
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
