// runtime.h -- internal interface between the translation units of libdmc_cuda.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/dmc_cuda.h"

namespace dmc {

struct FpKey {
    uint64_t h1, h2, bytes;
    uint64_t shape = 0;  // (k << 32 | n) when the device copy is stored transposed, else 0
    bool operator==(const FpKey &o) const {
        return h1 == o.h1 && h2 == o.h2 && bytes == o.bytes && shape == o.shape;
    }
};
struct FpKeyHash {
    size_t operator()(const FpKey &k) const {
        return (size_t)(k.h1 ^ (k.h2 * 0x9e3779b97f4a7c15ULL) ^ k.bytes ^ (k.shape * 0xff51afd7ed558ccdULL));
    }
};

struct RegisteredRange {
    uintptr_t host;
    size_t bytes;
    void *dev;
    int wdtype;
    int64_t k = 0, n = 0;  // shape when the range is one [k, n] matrix stored k-contiguous on the device, else 0
};

struct AddrRange {
    uintptr_t lo, hi;
};

struct PendingReadback {
    const float *src;  // pinned staging
    float *dst;        // caller's `out`
    size_t elems;
    bool on_device;    // y still sits in the device buffer (same offset): the flush brings it to `src`
};

struct Context {
    int device = -1;
    bool ready = false;
    cudaStream_t stream = nullptr;
    int sm_count = 148;
    int clock_khz = 1900000;  // SM clock, converts the wait limit to clock64 cycles
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;  // per-call kernel timing (DMC_CUDA_TIME)

    // activation / output staging: pinned host mirrors of device buffers, bump-allocated
    // while deferred calls are outstanding (reference: compiler/src/gpu.rs:201-219)
    char *h_x = nullptr, *h_y = nullptr;
    char *d_x = nullptr, *d_y = nullptr;
    size_t x_cap = 0, y_cap = 0, x_off = 0, y_off = 0;
    std::vector<PendingReadback> pending;

    // split-K scratch
    float *partial = nullptr;
    size_t partial_cap = 0;  // bytes
    unsigned *counters = nullptr;
    size_t counters_cap = 0;  // elements

    // transient f32 operand upload buffer (dmc_matmul_f32_gpu)
    char *d_tmpw = nullptr;
    size_t tmpw_cap = 0;
    // (hi, lo) bf16 split of f32 activations for the tensor-core GEMM
    char *d_tmpx = nullptr;
    size_t tmpx_cap = 0;

    // resident weights
    std::unordered_map<FpKey, void *, FpKeyHash> by_fingerprint;
    // What the last call with a weight at a given host address resolved to.  A hit lets a call launch
    // first and take the content fingerprint while the GPU runs; the fingerprint is still compared on
    // every call, and a call whose weight turned out to have changed is repeated the slow way.
    struct Guess {
        size_t bytes;
        FpKey key;
        void *dev;
        int layout;
    };
    std::unordered_map<uintptr_t, Guess> by_address;
    std::vector<RegisteredRange> registered;
    int64_t resident_bytes = 0;

    // error word written by kernels whose bounded waits run out (pinned, device-visible)
    int *err_word = nullptr;
    // Completion word of the host-pointer calls (pinned): the kernel that delivers a call's y writes the
    // call's sequence number here last.  done_is_last: nothing has been put on the stream since.
    unsigned *done_word = nullptr;
    unsigned done_seq = 0;
    bool done_is_last = false;
    unsigned *deliver_count = nullptr;  // device: arrival counter of the delivering kernel's CTAs

    // set by the sharded path around a launch: the NK kernel then stores y into every rank's replica
    const void *peer = nullptr;  // device pointer to a PeerOut
    long long peer_yoff = 0;
    int peer_j = 0;

    // Ranges the launches since the stream was last known to be drained read and write; decides which
    // GEMVs may skip their dependency wait (gemv_launch.cu).
    std::vector<AddrRange> inflight_reads, inflight_writes;
    bool nowait_inflight = false;     // a kernel that skipped its wait has been launched since
    bool untracked_inflight = false;  // so has a kernel whose ranges were not recorded

    // set by the decode step around a launch: elementwise prologue of the NK kernel's x staging
    int pro = 0;
    const float *pro_add = nullptr, *pro_g = nullptr;
    float *pro_hout = nullptr;
    float pro_eps = 0.0f;
    unsigned long long *amax = nullptr;  // arg-max epilogue of the NK kernel (GemvArgs::amax)

    // pinned staging ring of the weight ingest, allocated on first use
    unsigned char *ingest_ring = nullptr;

    int64_t launches = 0;
};

// tuning knobs (dmc_cuda_set_param)
struct Tuning {
    int pdl = 1;            // programmatic dependent launch on the GEMV kernels
    int kn_ctas_per_sm = 0; // 0 = per-variant default
    int kn_ksplit = 0;      // 0 = derive from kn_ctas_per_sm
    int nk_ctas_per_sm = 0; // 0 = per-variant default
    int nk_even_rounds = 1; // row kernel, more row groups than warps: 1 = fewer CTAs with equal shares when few warps would own an extra group, 2 = always, 0 = always all CTA slots
    int tma_ring_kb = 0;    // shared-memory ring per CTA (0 = 96 KiB)
    int tma_stage_kb = 0;   // target stage size (0 = 32 KiB)
    int tma_ctas_per_sm = 0;
    int store_nk = 1;       // keep resident [k,n] weights k-contiguous on the device
    int nk_default = -1;    // NK variant used when the caller passes -1 (-1 = library choice)
    int tc_ksplit = 0;      // tcgen05 GEMM: K splits (0 = derive from the tile count)
    int tc_smem_kb = 0;     // tcgen05 GEMM: shared-memory ring budget per CTA
    int tc_min_m = 0;       // activation rows from which `@` goes to the tensor cores (0 = library default)
    int zero_copy_y = 1;    // host-pointer entry points with host_io_kernels = 0: kernels store y directly into pinned host memory
    int decode_fused = 1;   // decode step: fuse the companions into the GEMVs / attention (0 = one kernel per op)
    int shard_fused = -1;   // sharded GEMV: 1 = peer stores fused into the kernel, 0 = NCCL all-gather, -1 = by world size
    int shard_overlap = 1;  // sharded GEMVs of one batch overlap (0 = each waits for the previous exchange's gather)
    int overlap_independent = 1;  // GEMVs that touch nothing a running kernel touches skip their dependency wait
    int wait_limit_us = 0;  // bound of the device-side waits on another rank, microseconds (0 = about one second)
    int timing = 0;         // per-call phase timing printed to stderr (also DMC_CUDA_TIME=1)
    int spin_sync = 0;      // host-pointer entry points poll the stream instead of blocking on it
    int host_io_kernels = 1; // host-pointer entry points move x and y (up to 64 KiB each) with kernels, not the copy engines
};

Context &ctx();
Tuning &tuning();
std::mutex &ctx_mutex();

// Record a sticky error (first one wins) and return its code.
int fail(int code, const char *fmt, ...);
int status();
#define DMC_CUDA_TRY(expr)                                                                   \
    do {                                                                                     \
        cudaError_t e__ = (expr);                                                            \
        if (e__ != cudaSuccess)                                                              \
            return ::dmc::fail(e__ == cudaErrorMemoryAllocation ? DMC_CUDA_ERR_OOM           \
                                                                : DMC_CUDA_ERR_CUDA,         \
                               "%s failed: %s", #expr, cudaGetErrorString(e__));             \
    } while (0)

int ensure_init();  // lazy dmc_cuda_init on the current device; returns status
// Turn a code left in the pinned error word by a kernel whose bounded wait ran out into the sticky
// DMC_CUDA_ERR_TIMEOUT; returns the status.
int check_device_error();

// Launch one GEMV (all pointers on the device).  batch slices at strides ls/rs elements.
int launch_gemv(const void *dW, const float *dx, float *dy, int64_t m, int64_t k, int64_t n,
                int64_t batch, int64_t ls, int64_t rs, int layout, int wdtype, int variant,
                cudaStream_t stream);


// One kernel launch with the library's launch attributes (programmatic dependent launch).
//   kLaunchUntracked  the kernel waits for its predecessors; what it reads and writes is not recorded
//   kLaunchTracked    it waits; the caller has recorded its ranges in the context
//   kLaunchOverlap    it skips its dependency wait (the caller checked that it conflicts with nothing in flight)
enum { kLaunchUntracked = 0, kLaunchTracked = 1, kLaunchOverlap = 2 };
constexpr size_t kMaxTrackedRanges = 1024;
int launch_ex(const void *fn, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, void **params,
              int mode = kLaunchUntracked);
// The context's stream has been synchronised (or is about to run a fully serialising operation):
// forget the recorded ranges.
void stream_drained();
// cudaMalloc / cudaMallocHost through one door, so that a test can make them fail on the host
// (environment variable DMC_CUDA_INJECT, see dmc_cuda.cu).
cudaError_t dmc_malloc(void **p, size_t bytes);
cudaError_t dmc_malloc_host(void **p, size_t bytes);
// True when DMC_CUDA_INJECT names `what` (comma-separated list).
bool inject_failure(const char *what);
// x of a host-pointer call from its pinned mirror to the device, and y from the device to its pinned
// mirror followed by the call's sequence number in Context::done_word (gemv_launch.cu).
int launch_stage_x(const float *h_src, float *d_dst, size_t elems, cudaStream_t stream);
int launch_deliver(const float *d_src, float *h_dst, size_t elems, cudaStream_t stream);
// Sharded GEMV (shard.cu) whose whole y ends up in `h_dst`, pinned host memory the device can write: with
// the fused exchange the kernel that checks the arrivals writes it there itself; otherwise one copy follows.
int shard_gemv_to_host(const void *dW_shard, const float *dx, int64_t k, int64_t n, int wdtype, float *h_dst,
                       cudaStream_t stream);
// Grow the context's split-K scratch (partials in bytes, arrival counters in elements).
int ensure_scratch(size_t partial_bytes, size_t ncounters);

// Time line of a chain of GEMVs (gemv_launch.cu).
int timeline_nk(const void *const *dWs, int count, const float *dx, float *dy, int64_t k, int64_t n, int dependent,
                unsigned long long *stamps_out, int64_t stamps_cap_words, cudaStream_t s);

// tcgen05 GEMM: Y[m][n] = X @ W' with W [n][k] bf16 (k contiguous) and X bf16 or f32.
bool gemm_tc_eligible(int64_t m, int64_t k, int64_t n, const void *dW, const void *dX);
int launch_gemm_tc(const void *dW, const void *dXbf16, float *dY, int64_t m, int64_t k, int64_t n, int pair,
                   cudaStream_t stream);
int launch_gemm_tc_f32x(const void *dW, const float *dX, float *dY, int64_t m, int64_t k, int64_t n,
                        cudaStream_t stream);

// True when a vectorised NK kernel takes an [n, k] weight of this shape (alignment of
// freshly allocated device buffers assumed).
bool nk_fast_eligible(int64_t k, int64_t n, int wdtype);

// dst[cols][rows] = src[rows][cols] for 2- or 4-byte elements, on `stream`.
int launch_transpose(const void *src, void *dst, int64_t rows, int64_t cols, int elem_bytes, cudaStream_t stream);

}  // namespace dmc
