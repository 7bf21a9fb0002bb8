// dmc_cuda.cu -- context, resident-weight registry, staging and the C ABI of
// libdmc_cuda.so (declared in include/dmc_cuda.h).  The structure answers the
// reference's Metal runtime (compiler/src/gpu.rs:186-325, 476-660): weights
// stay on the device keyed by content, the small activation and output vectors
// cross per call through reused staging, deferred calls queue on one stream.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <algorithm>

#include "runtime.h"

namespace dmc {

namespace {
Context g_ctx;
Tuning g_tuning;
std::mutex g_mutex;
int g_status = DMC_CUDA_OK;
char g_msg[512] = "";
}  // namespace

Context &ctx() { return g_ctx; }
Tuning &tuning() { return g_tuning; }
std::mutex &ctx_mutex() { return g_mutex; }
int status() { return g_status; }

int fail(int code, const char *fmt, ...) {
    if (g_status == DMC_CUDA_OK) {
        g_status = code;
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(g_msg, sizeof(g_msg), fmt, ap);
        va_end(ap);
        if (getenv("DMC_CUDA_DEBUG")) fprintf(stderr, "[dmc_cuda] error %d: %s\n", code, g_msg);
    }
    return code;
}

// Host-side failure injection for tests: DMC_CUDA_INJECT is a comma-separated list of the calls
// that should report failure without being made ("malloc", "malloc_host", "nccl_init", "ipc_open",
// "stream").  Nothing on the device is touched by an injected failure.
bool inject_failure(const char *what) {
    const char *env = getenv("DMC_CUDA_INJECT");
    if (!env || !*env) return false;
    const size_t n = strlen(what);
    for (const char *p = env; *p;) {
        const char *q = strchr(p, ',');
        const size_t len = q ? (size_t)(q - p) : strlen(p);
        if (len == n && !strncmp(p, what, n)) return true;
        if (!q) break;
        p = q + 1;
    }
    return false;
}
cudaError_t dmc_malloc(void **p, size_t bytes) {
    if (inject_failure("malloc")) return cudaErrorMemoryAllocation;
    return cudaMalloc(p, bytes);
}
cudaError_t dmc_malloc_host(void **p, size_t bytes) {
    if (inject_failure("malloc_host")) return cudaErrorMemoryAllocation;
    return cudaMallocHost(p, bytes);
}

// Content fingerprint of a weight buffer: byte length plus a 256-point strided
// sample folded into a 128-bit key -- the reference's residency key
// (compiler/src/gpu.rs:342-358), kept bit-compatible so a weight re-materialised
// at a fresh host address every decode step still hits.
static FpKey fingerprint(const uint8_t *ptr, size_t bytes) {
    uint64_t h1 = 0xcbf29ce484222325ULL ^ (uint64_t)bytes;
    uint64_t h2 = 0x9e3779b97f4a7c15ULL * ((uint64_t)bytes | 1);
    size_t words = bytes / 8;
    if (words > 0) {
        size_t step = words / 256;
        if (step < 1) step = 1;
        // the samples are ~256 cache lines spread over the whole weight: ask for all of them first, so the
        // misses overlap instead of queueing behind the hash chain -- and ask for them to stay cached: the
        // same lines are read again on the next call with this weight (a non-temporal hint made every
        // call miss all the way to DRAM again, ~8 us per call measured)
        if (step >= 8)
            for (size_t i = 0; i < words; i += step) __builtin_prefetch(ptr + 8 * i, 0, 3);
        for (size_t i = 0; i < words; i += step) {
            uint64_t v;
            memcpy(&v, ptr + 8 * i, 8);
            h1 = (h1 ^ v) * 0x00000100000001b3ULL;
            uint64_t t = h2 + v;
            t = (t << 27) | (t >> 37);
            h2 = t * 0xff51afd7ed558ccdULL;
        }
    }
    return FpKey{h1, h2, (uint64_t)bytes};
}

void apply_env_params();

static int init_locked(int device) {
    Context &c = g_ctx;
    if (c.ready) return DMC_CUDA_OK;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        cudaGetLastError();
        return fail(DMC_CUDA_ERR_NO_DEVICE, "no CUDA device is available");
    }
    if (device < 0) {
        const char *env = getenv("DMC_CUDA_DEVICE");
        if (env) device = atoi(env);
        else if (cudaGetDevice(&device) != cudaSuccess) device = 0;
    }
    if (device >= count) return fail(DMC_CUDA_ERR_BAD_ARG, "device %d of %d does not exist", device, count);
    DMC_CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    DMC_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10)
        return fail(DMC_CUDA_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only",
                    device, prop.major, prop.minor);
    c.device = device;
    c.sm_count = prop.multiProcessorCount;
    c.clock_khz = prop.clockRate > 0 ? prop.clockRate : 1900000;
    if (inject_failure("stream")) return fail(DMC_CUDA_ERR_CUDA, "cudaStreamCreateWithFlags failed: injected");
    DMC_CUDA_TRY(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
    DMC_CUDA_TRY(dmc_malloc_host((void **)&c.err_word, sizeof(int)));
    *c.err_word = 0;
    DMC_CUDA_TRY(dmc_malloc_host((void **)&c.done_word, sizeof(unsigned)));
    *c.done_word = 0;
    apply_env_params();
    if (getenv("DMC_CUDA_TIME") && atoi(getenv("DMC_CUDA_TIME")) != 0) g_tuning.timing = 1;
    c.ready = true;
    return DMC_CUDA_OK;
}

// A kernel whose bounded wait ran out leaves a code in the pinned error word.
int check_device_error() {
    Context &c = g_ctx;
    if (c.err_word && *(volatile int *)c.err_word != 0) {
        int code = *(volatile int *)c.err_word;
        *c.err_word = 0;
        return fail(DMC_CUDA_ERR_TIMEOUT, "a device-side wait ran out (code %d): the kernel gave up instead of hanging", code);
    }
    return g_status;
}

int ensure_init() {
    if (g_ctx.ready) {
        int cur = -1;
        if (cudaGetDevice(&cur) == cudaSuccess && cur != g_ctx.device) cudaSetDevice(g_ctx.device);
        return g_status;
    }
    return init_locked(-1);
}

// ---- staging ---------------------------------------------------------------------

static double now_us();

// Wait for the stream.  "spin_sync" polls cudaStreamQuery instead of blocking in
// cudaStreamSynchronize; measured on B200 it is slower (49 vs 35 us per 4096x4096 call: the polling
// competes with the driver's own completion handling), so it is off by default.
//
// When the last thing on the stream is the kernel that delivers a host-pointer call's y, the host
// watches the sequence number that kernel writes last into pinned memory: it sees it about as soon as
// the PCIe write lands, several microseconds before the driver reports the stream idle.  Every ~50 us
// the stream is queried too, so that a failed launch ends the wait.
static cudaError_t stream_wait(cudaStream_t s) {
    Context &c = g_ctx;
    if (c.done_is_last && s == c.stream) {
        const unsigned want = c.done_seq;
        double t_query = now_us();
        for (;;) {
            if ((int)(*(volatile unsigned *)c.done_word - want) >= 0) return cudaSuccess;
#if defined(__x86_64__)
            __builtin_ia32_pause();
#endif
            if (now_us() - t_query > 50.0) {
                cudaError_t e = cudaStreamQuery(s);
                if (e != cudaErrorNotReady) return e;
                t_query = now_us();
            }
        }
    }
    if (!g_tuning.spin_sync) return cudaStreamSynchronize(s);
    for (;;) {
        cudaError_t e = cudaStreamQuery(s);
        if (e != cudaErrorNotReady) return e;
    }
}

static int flush_locked();

static int grow_pair(char **h, char **d, size_t *cap, size_t need) {
    if (need <= *cap) return DMC_CUDA_OK;
    // deferred calls still point into the old buffers: materialise them first
    int rc = flush_locked();
    if (rc) return rc;
    size_t ncap = *cap ? *cap : (size_t)256 << 10;
    while (ncap < need) ncap *= 2;
    if (*h) cudaFreeHost(*h);
    if (*d) cudaFree(*d);
    *h = nullptr;
    *d = nullptr;
    *cap = 0;
    DMC_CUDA_TRY(dmc_malloc_host((void **)h, ncap));
    DMC_CUDA_TRY(dmc_malloc((void **)d, ncap));
    *cap = ncap;
    return DMC_CUDA_OK;
}

static bool overlaps_pending(uintptr_t p, size_t bytes) {
    for (const PendingReadback &r : g_ctx.pending) {
        uintptr_t d0 = (uintptr_t)r.dst;
        if (p < d0 + r.elems * 4 && d0 < p + bytes) return true;
    }
    return false;
}

// Wait for the stream and perform every deferred host readback
// (compiler/src/gpu.rs:306-316 `flush_pending`).
// Outputs that still sit in the device buffer come over in one piece: they are bump-allocated, so one
// span covers them -- a kernel (full-line stores + the completion word) up to 128 KiB, else one copy.
static int deliver_pending_locked() {
    Context &c = g_ctx;
    size_t lo = SIZE_MAX, hi = 0;
    for (PendingReadback &r : c.pending)
        if (r.on_device) {
            lo = std::min(lo, (size_t)((const char *)r.src - c.h_y));
            hi = std::max(hi, (size_t)((const char *)r.src - c.h_y) + r.elems * 4);
            r.on_device = false;
        }
    if (hi <= lo) return DMC_CUDA_OK;
    if (hi - lo <= (128u << 10)) return launch_deliver((const float *)(c.d_y + lo), (float *)(c.h_y + lo), (hi - lo) / 4, c.stream);
    DMC_CUDA_TRY(cudaMemcpyAsync(c.h_y + lo, c.d_y + lo, hi - lo, cudaMemcpyDeviceToHost, c.stream));
    c.done_is_last = false;
    return DMC_CUDA_OK;
}

static int flush_locked() {
    Context &c = g_ctx;
    if (!c.ready) return g_status;
    if (c.pending.empty() && c.x_off == 0 && c.y_off == 0) return g_status;
    int drc = deliver_pending_locked();
    if (drc) return drc;
    DMC_CUDA_TRY(stream_wait(c.stream));
    stream_drained();
    if (check_device_error()) {  // results of a kernel that gave up are not delivered
        c.pending.clear();
        c.x_off = c.y_off = 0;
        return g_status;
    }
    for (const PendingReadback &r : c.pending) memcpy(r.dst, r.src, r.elems * sizeof(float));
    c.pending.clear();
    c.x_off = 0;
    c.y_off = 0;
    return g_status;
}

// ---- resident weights ---------------------------------------------------------------

// Copy a host weight to a fresh device buffer; with `transposed` the [k, n] matrix is stored
// [n, k] (k contiguous) by one device transpose.  Synchronous.
static int upload_weight(uintptr_t r, size_t bytes, int64_t k, int64_t n, size_t wsz, bool transposed, void **out) {
    Context &c = g_ctx;
    void *d = nullptr;
    DMC_CUDA_TRY(dmc_malloc(&d, bytes ? bytes : 16));
    void *staging = d;
    if (transposed) {
        cudaError_t e = dmc_malloc(&staging, bytes);
        if (e != cudaSuccess) {
            cudaFree(d);
            return fail(DMC_CUDA_ERR_OOM, "weight upload: staging allocation failed: %s", cudaGetErrorString(e));
        }
    }
    // On the context's stream, not the legacy default stream: a plain cudaMemcpy from pageable memory
    // may return before its DMA lands, and the non-blocking stream would not wait for it.
    cudaError_t e = cudaMemcpyAsync(staging, (const void *)r, bytes, cudaMemcpyHostToDevice, c.stream);
    if (e == cudaSuccess && !transposed) e = cudaStreamSynchronize(c.stream);
    if (e == cudaSuccess && transposed) {
        int rc = launch_transpose(staging, d, k, n, (int)wsz, c.stream);
        e = rc ? cudaErrorUnknown : cudaStreamSynchronize(c.stream);  // the GEMV may prefetch W before its dependency wait
        cudaFree(staging);
    }
    if (e != cudaSuccess) {
        cudaFree(d);
        return fail(DMC_CUDA_ERR_CUDA, "weight upload failed: %s", cudaGetErrorString(e));
    }
    stream_drained();
    *out = d;
    return DMC_CUDA_OK;
}

// Find or create the device copy of a host weight.  A single [k, n] matrix that the
// row-streaming kernel can take is stored transposed ([n, k], k contiguous) so the one
// bandwidth kernel serves it; *layout says how the returned buffer is laid out.
// The transpose runs once per weight, on the device, at upload.
// `guess`: when not null, a weight last seen at this address with this size is returned without
// reading it, *guess is set to the fingerprint it had then, and the caller must compare that with
// weight_key() before it delivers anything computed from the returned buffer.
static FpKey weight_key(uintptr_t r, size_t bytes, int64_t k, int64_t n, int wdtype, bool may_transpose, bool *transposed) {
    *transposed = may_transpose && g_tuning.store_nk && nk_fast_eligible(k, n, wdtype);
    FpKey key = fingerprint((const uint8_t *)r, bytes);
    key.shape = *transposed ? (((uint64_t)k << 32) | (uint64_t)n) : 0;
    return key;
}

static int resident_weight(uintptr_t r, size_t bytes, int64_t k, int64_t n, int wdtype, bool may_transpose,
                           void **dev, int *layout, FpKey *guess = nullptr, bool *guessed = nullptr) {
    Context &c = g_ctx;
    *layout = DMC_LAYOUT_KN;
    if (guessed) *guessed = false;
    for (const RegisteredRange &rg : c.registered) {
        if (r >= rg.host && r + bytes <= rg.host + rg.bytes) {
            if (rg.k == 0) {  // stored as the host has it
                *dev = (char *)rg.dev + (r - rg.host);
                return DMC_CUDA_OK;
            }
            if (may_transpose && r == rg.host && bytes == rg.bytes && k == rg.k && n == rg.n) {
                *dev = rg.dev;
                *layout = DMC_LAYOUT_NK;
                return DMC_CUDA_OK;
            }
            break;  // a different view of a range stored k-contiguous: served by content below
        }
    }
    const size_t wsz = wdtype == DMC_W_BF16 ? 2 : 4;
    bool transposed = false;
    if (guess) {
        auto g = c.by_address.find(r);
        if (g != c.by_address.end() && g->second.bytes == bytes) {
            transposed = may_transpose && g_tuning.store_nk && nk_fast_eligible(k, n, wdtype);
            const uint64_t shape = transposed ? (((uint64_t)k << 32) | (uint64_t)n) : 0;
            if (g->second.key.shape == shape) {
                *dev = g->second.dev;
                *layout = g->second.layout;
                *guess = g->second.key;
                *guessed = true;
                return DMC_CUDA_OK;
            }
        }
    }
    const FpKey key = weight_key(r, bytes, k, n, wdtype, may_transpose, &transposed);
    auto it = c.by_fingerprint.find(key);
    if (it != c.by_fingerprint.end()) {
        *dev = it->second;
        *layout = transposed ? DMC_LAYOUT_NK : DMC_LAYOUT_KN;
        if (c.by_address.size() > 4096) c.by_address.clear();
        c.by_address[r] = Context::Guess{bytes, key, *dev, *layout};
        return DMC_CUDA_OK;
    }
    if (c.by_fingerprint.size() > 2048) {  // same safety valve as compiler/src/gpu.rs:266
        DMC_CUDA_TRY(cudaStreamSynchronize(c.stream));
        for (auto &kv : c.by_fingerprint) cudaFree(kv.second);
        c.by_fingerprint.clear();
        c.by_address.clear();
        c.resident_bytes = 0;
        for (const RegisteredRange &rg : c.registered) c.resident_bytes += (int64_t)rg.bytes;
    }
    void *d = nullptr;
    int rc = upload_weight(r, bytes, k, n, wsz, transposed, &d);
    if (rc) return rc;
    if (getenv("DMC_CUDA_DEBUG"))
        fprintf(stderr, "[dmc_cuda] upload #%zu %zu MB%s\n", c.by_fingerprint.size() + 1, bytes >> 20,
                transposed ? " (stored k-contiguous)" : "");
    c.by_fingerprint.emplace(key, d);
    c.resident_bytes += (int64_t)bytes;
    *dev = d;
    *layout = transposed ? DMC_LAYOUT_NK : DMC_LAYOUT_KN;
    if (c.by_address.size() > 4096) c.by_address.clear();
    c.by_address[r] = Context::Guess{bytes, key, d, *layout};
    return DMC_CUDA_OK;
}

// ---- the shared host-pointer path (compiler/src/gpu.rs:479-660 `gpu_run`) ------------

struct HostCall {
    const float *l;
    const void *r;
    float *out;
    int64_t m, k, n, batch, ls, rs;
    int layout, wdtype;
    bool defer;
    bool resident;  // keep r on the device across calls
};

static double now_us() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec * 1e6 + ts.tv_nsec * 1e-3;
}

static int run_host_call_locked(const HostCall &h) {
    if (g_status) return g_status;  // sticky: nothing runs after a failure
    if (h.m < 0 || h.k < 0 || h.n < 0 || h.batch < 0 || h.ls < 0 || h.rs < 0)
        return fail(DMC_CUDA_ERR_BAD_ARG, "matmul: negative size (m=%lld k=%lld n=%lld batch=%lld ls=%lld rs=%lld)",
                    (long long)h.m, (long long)h.k, (long long)h.n, (long long)h.batch, (long long)h.ls,
                    (long long)h.rs);
    if (h.m == 0 || h.n == 0 || h.batch == 0) return DMC_CUDA_OK;  // compiler/src/gpu.rs:402, 425
    if (!h.l || !h.r || !h.out) return fail(DMC_CUDA_ERR_BAD_ARG, "matmul: null operand pointer");
    if (h.batch > 1 && h.m != 1) {
        // The JIT only batches m == 1 slices; for anything else the reference runs the slices one
        // after the other (compiler/src/gpu.rs:428-437), and so does this -- on the GPU.
        for (int64_t z = 0; z < h.batch; ++z) {
            HostCall one = h;
            one.l = h.l + z * h.ls;
            one.r = (const char *)h.r + (size_t)z * h.rs * (h.wdtype == DMC_W_BF16 ? 2 : 4);
            one.out = h.out + z * h.m * h.n;
            one.batch = 1;
            one.ls = one.rs = 0;
            int rc = run_host_call_locked(one);
            if (rc) return rc;
        }
        return DMC_CUDA_OK;
    }
    const bool timing = g_tuning.timing != 0;
    const double t0 = timing ? now_us() : 0.0;
    int rc = ensure_init();
    if (rc) return rc;
    Context &c = g_ctx;

    const size_t wsz = h.wdtype == DMC_W_BF16 ? 2 : 4;
    const size_t x_elems = (size_t)(h.batch - 1) * h.ls + (size_t)h.m * h.k;
    const size_t y_elems = (size_t)h.batch * h.m * h.n;
    const size_t w_elems = (size_t)(h.batch - 1) * h.rs + (size_t)h.k * h.n;

    // a call that touches a deferred output materialises it first (compiler/src/gpu.rs:491-499)
    if (!c.pending.empty() &&
        (overlaps_pending((uintptr_t)h.l, x_elems * 4) || overlaps_pending((uintptr_t)h.r, w_elems * wsz) ||
         overlaps_pending((uintptr_t)h.out, y_elems * 4))) {
        rc = flush_locked();
        if (rc) return rc;
    }

    size_t x_base = (c.x_off + 255) & ~(size_t)255;
    size_t y_base = (c.y_off + 255) & ~(size_t)255;
    if (x_base + x_elems * 4 > c.x_cap) {
        rc = grow_pair(&c.h_x, &c.d_x, &c.x_cap, x_base + x_elems * 4);
        if (rc) return rc;
        x_base = (c.x_off + 255) & ~(size_t)255;  // a flush resets the offsets
        y_base = (c.y_off + 255) & ~(size_t)255;
    }
    if (y_base + y_elems * 4 > c.y_cap) {
        rc = grow_pair(&c.h_y, &c.d_y, &c.y_cap, y_base + y_elems * 4);
        if (rc) return rc;
        x_base = (c.x_off + 255) & ~(size_t)255;
        y_base = (c.y_off + 255) & ~(size_t)255;
    }

    // x first: its copy to the device runs while the host looks the weight up (the content
    // fingerprint touches 256 cache lines spread over the whole weight, ~5 us)
    // Up to 64 KiB each way, kernels move x and y instead of the copy engines ("host_io_kernels").
    const bool io_kernels = g_tuning.host_io_kernels != 0;
    memcpy(c.h_x + x_base, h.l, x_elems * 4);
    if (io_kernels && x_elems * 4 <= (64u << 10)) {
        rc = launch_stage_x((const float *)(c.h_x + x_base), (float *)(c.d_x + x_base), x_elems, c.stream);
        if (rc) return rc;
    } else {
        DMC_CUDA_TRY(cudaMemcpyAsync(c.d_x + x_base, c.h_x + x_base, x_elems * 4, cudaMemcpyHostToDevice, c.stream));
        c.done_is_last = false;
    }

    // weights: resident, or (f32 operand that may change between calls) uploaded now
    void *dW = nullptr;
    int layout = h.layout;
    FpKey guess = {};
    bool guessed = false;
    if (h.k > 0) {
        if (h.resident) {
            int stored = DMC_LAYOUT_KN;
            // (with the kernels above the call is short enough for the fingerprint to matter: a weight
            // seen before at this address is used at once and its fingerprint compared while the GPU runs)
            rc = resident_weight((uintptr_t)h.r, w_elems * wsz, h.k, h.n, h.wdtype,
                                 h.layout == DMC_LAYOUT_KN && h.batch == 1, &dW, &stored,
                                 io_kernels ? &guess : nullptr, &guessed);
            if (rc) return rc;
            if (h.layout == DMC_LAYOUT_KN) layout = stored;
        } else {
            bool hit = false;
            for (const RegisteredRange &rg : c.registered)
                if ((uintptr_t)h.r >= rg.host && (uintptr_t)h.r + w_elems * wsz <= rg.host + rg.bytes) {
                    if (rg.k == 0) {
                        dW = (char *)rg.dev + ((uintptr_t)h.r - rg.host);
                        hit = true;
                    } else if ((uintptr_t)h.r == rg.host && w_elems * wsz == rg.bytes && h.k == rg.k && h.n == rg.n &&
                               h.batch == 1 && h.layout == DMC_LAYOUT_KN) {
                        dW = rg.dev;
                        layout = DMC_LAYOUT_NK;
                        hit = true;
                    }
                }
            if (!hit) {
                if (w_elems * wsz > c.tmpw_cap) {
                    DMC_CUDA_TRY(cudaStreamSynchronize(c.stream));
                    stream_drained();
                    if (c.d_tmpw) cudaFree(c.d_tmpw);
                    c.d_tmpw = nullptr;
                    c.tmpw_cap = 0;
                    DMC_CUDA_TRY(dmc_malloc((void **)&c.d_tmpw, w_elems * wsz));
                    c.tmpw_cap = w_elems * wsz;
                }
                // pageable source: the copy returns once the source has been consumed
                DMC_CUDA_TRY(cudaMemcpyAsync(c.d_tmpw, h.r, w_elems * wsz, cudaMemcpyHostToDevice, c.stream));
                c.done_is_last = false;
                dW = c.d_tmpw;
            }
        }
    }
    const double t1 = timing ? now_us() : 0.0;

    // Small outputs (up to 64 KiB) are stored by the kernel straight into the pinned host mirror
    // (device-visible through unified addressing), which saves the device->host copy and its launch
    // latency (measured: 35 vs 39 us per 4096x4096 call); larger ones (an lm-head's 600 KB of logits)
    // would cross PCIe four bytes at a time, so they go through the device buffer and one copy.
    // "zero_copy_y" = 0 always copies.
    const bool deliver = io_kernels && y_elems * 4 <= (64u << 10);
    const bool zc = !deliver && g_tuning.zero_copy_y != 0 && y_elems * 4 <= (64u << 10);
    float *y_target = zc ? (float *)(c.h_y + y_base) : (float *)(c.d_y + y_base);
    const bool timing_events = g_tuning.timing == 1;  // (2 = host clock only: the events themselves serialise the kernels)
    if (timing_events) {
        if (!c.ev0) {
            DMC_CUDA_TRY(cudaEventCreate(&c.ev0));
            DMC_CUDA_TRY(cudaEventCreate(&c.ev1));
        }
        DMC_CUDA_TRY(cudaEventRecord(c.ev0, c.stream));
    }
    rc = launch_gemv(dW, (const float *)(c.d_x + x_base), y_target, h.m, h.k, h.n, h.batch,
                     h.ls, h.rs, layout, h.wdtype, -1, c.stream);
    if (rc) return rc;
    if (timing_events) DMC_CUDA_TRY(cudaEventRecord(c.ev1, c.stream));
    const double t_launched = timing ? now_us() : 0.0;
    if (!deliver && !zc) {
        DMC_CUDA_TRY(cudaMemcpyAsync(c.h_y + y_base, c.d_y + y_base, y_elems * 4, cudaMemcpyDeviceToHost, c.stream));
        c.done_is_last = false;
    }
    if (guessed) {
        // the GPU is running; now read the weight's fingerprint.  If the weight at this address is not
        // the one the launch assumed, nothing of this launch is delivered and the call starts over.
        bool transposed = false;
        const FpKey now = weight_key((uintptr_t)h.r, w_elems * wsz, h.k, h.n, h.wdtype,
                                     h.layout == DMC_LAYOUT_KN && h.batch == 1, &transposed);
        if (!(now == guess)) {
            c.by_address.erase((uintptr_t)h.r);
            cudaError_t we = stream_wait(c.stream);
            if (we != cudaSuccess) return fail(DMC_CUDA_ERR_CUDA, "stream wait failed: %s", cudaGetErrorString(we));
            stream_drained();
            return run_host_call_locked(h);
        }
    }
    const double t2 = timing ? now_us() : 0.0;

    c.pending.push_back(PendingReadback{(const float *)(c.h_y + y_base), h.out, y_elems, deliver});
    c.x_off = x_base + x_elems * 4;  // (also makes the flush below non-trivial when nothing was deferred)
    if (h.defer) {
        c.y_off = y_base + y_elems * 4;
        if (timing)
            fprintf(stderr, "[dmc_cuda time] deferred m=%lld k=%lld n=%lld batch=%lld: weights %.1f us, stage+launch %.1f us\n",
                    (long long)h.m, (long long)h.k, (long long)h.n, (long long)h.batch, t1 - t0, t2 - t1);
        return DMC_CUDA_OK;
    }
    if (!timing) return flush_locked();
    // the flush, taken apart: wait for the stream, then the host copies of every pending output
    const size_t npending = c.pending.size();
    rc = deliver_pending_locked();
    if (rc) return rc;
    cudaError_t we = stream_wait(c.stream);
    const double t3 = now_us();
    if (we != cudaSuccess) return fail(DMC_CUDA_ERR_CUDA, "stream wait failed: %s", cudaGetErrorString(we));
    rc = flush_locked();
    const double t4 = now_us();
    float kms = 0.0f;
    if (timing_events) cudaEventElapsedTime(&kms, c.ev0, c.ev1);
    else fprintf(stderr, "[dmc_cuda time] host clock only: x staged + weight found %.1f us, GEMV launched %.1f us, fingerprint compared %.1f us (the delivery of y is launched by the flush and counted in the wait)\n",
                 t1 - t0, t_launched - t1, t2 - t_launched);
    const double bytes = (double)w_elems * wsz + 4.0 * x_elems + 4.0 * y_elems;
    fprintf(stderr,
            "[dmc_cuda time] m=%lld k=%lld n=%lld batch=%lld %s: weights %.1f us, stage+launch %.1f us, wait %.1f us, "
            "readback %.1f us (%zu outputs), total %.1f us; kernel %.1f us = %.0f GB/s\n",
            (long long)h.m, (long long)h.k, (long long)h.n, (long long)h.batch, layout == DMC_LAYOUT_NK ? "k-contiguous" : "n-contiguous",
            t1 - t0, t2 - t1, t3 - t2, t4 - t3, npending, t4 - t0, kms * 1e3, kms > 0 ? bytes / (kms * 1e-3) / 1e9 : 0.0);
    return rc;
}

static int run_host_call(const HostCall &h) {
    std::lock_guard<std::mutex> lock(g_mutex);
    return run_host_call_locked(h);
}

}  // namespace dmc

using namespace dmc;

// ---- C ABI ------------------------------------------------------------------------------

extern "C" int dmc_cuda_device_count(void) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return count;
}

extern "C" int dmc_cuda_init(int device) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    return init_locked(device);
}

extern "C" void dmc_cuda_shutdown(void) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    Context &c = ctx();
    if (!c.ready) return;
    flush_locked();
    cudaStreamSynchronize(c.stream);
    for (auto &kv : c.by_fingerprint) cudaFree(kv.second);
    c.by_fingerprint.clear();
    c.by_address.clear();
    for (auto &rg : c.registered) cudaFree(rg.dev);
    c.registered.clear();
    if (c.h_x) cudaFreeHost(c.h_x);
    if (c.h_y) cudaFreeHost(c.h_y);
    if (c.d_x) cudaFree(c.d_x);
    if (c.d_y) cudaFree(c.d_y);
    if (c.partial) cudaFree(c.partial);
    if (c.counters) cudaFree(c.counters);
    if (c.d_tmpw) cudaFree(c.d_tmpw);
    if (c.d_tmpx) cudaFree(c.d_tmpx);
    if (c.err_word) cudaFreeHost(c.err_word);
    if (c.done_word) cudaFreeHost(c.done_word);
    if (c.deliver_count) cudaFree(c.deliver_count);
    if (c.ingest_ring) cudaFreeHost(c.ingest_ring);
    if (c.ev0) cudaEventDestroy(c.ev0);
    if (c.ev1) cudaEventDestroy(c.ev1);
    cudaStreamDestroy(c.stream);
    c = Context();
}

extern "C" int dmc_cuda_shard_gemv_host(const void *dW_shard, const float *x_host, float *y_host, int64_t k, int64_t n,
                                        int wdtype) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_status) return g_status;
    if (!dW_shard || !x_host || !y_host || k < 1 || n < 1)
        return fail(DMC_CUDA_ERR_BAD_ARG, "shard_gemv_host: null pointer or empty shape (k=%lld n=%lld)", (long long)k, (long long)n);
    int rc = ensure_init();
    if (rc) return rc;
    Context &c = g_ctx;
    rc = flush_locked();  // deferred calls of the single-GPU path use the same staging buffers
    if (rc) return rc;
    rc = grow_pair(&c.h_x, &c.d_x, &c.x_cap, (size_t)k * 4);
    if (rc) return rc;
    rc = grow_pair(&c.h_y, &c.d_y, &c.y_cap, (size_t)n * 4);
    if (rc) return rc;
    const bool io_kernels = g_tuning.host_io_kernels != 0;
    memcpy(c.h_x, x_host, (size_t)k * 4);
    if (io_kernels && (size_t)k * 4 <= (64u << 10)) {
        rc = launch_stage_x((const float *)c.h_x, (float *)c.d_x, (size_t)k, c.stream);
        if (rc) return rc;
    } else {
        DMC_CUDA_TRY(cudaMemcpyAsync(c.d_x, c.h_x, (size_t)k * 4, cudaMemcpyHostToDevice, c.stream));
        c.done_is_last = false;
    }
    rc = shard_gemv_to_host(dW_shard, (const float *)c.d_x, k, n, wdtype, (float *)c.h_y, c.stream);
    if (rc) return rc;
    if (io_kernels) {  // nothing left to copy: only the completion word, behind everything above
        rc = launch_deliver(nullptr, nullptr, 0, c.stream);
        if (rc) return rc;
    }
    cudaError_t we = stream_wait(c.stream);
    if (we != cudaSuccess) return fail(DMC_CUDA_ERR_CUDA, "stream wait failed: %s", cudaGetErrorString(we));
    stream_drained();
    if (check_device_error()) return g_status;
    memcpy(y_host, c.h_y, (size_t)n * 4);
    return DMC_CUDA_OK;
}

extern "C" int dmc_cuda_status(void) { return dmc::status(); }
extern "C" const char *dmc_cuda_last_error(void) { return g_msg; }
extern "C" void dmc_cuda_clear_error(void) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    g_status = DMC_CUDA_OK;
    g_msg[0] = 0;
    cudaGetLastError();
}

extern "C" void dmc_matmul_bf16_gpu(int64_t l, int64_t r, int64_t out, int64_t m, int64_t k, int64_t n) {
    run_host_call(HostCall{(const float *)l, (const void *)r, (float *)out, m, k, n, 1, 0, 0, DMC_LAYOUT_KN,
                           DMC_W_BF16, false, true});
}

extern "C" void dmc_matmul_bf16_gpu_batched(int64_t l, int64_t r, int64_t out, int64_t m, int64_t k, int64_t n,
                                            int64_t batch, int64_t ls, int64_t rs) {
    run_host_call(HostCall{(const float *)l, (const void *)r, (float *)out, m, k, n, batch, ls, rs, DMC_LAYOUT_KN,
                           DMC_W_BF16, false, true});
}

extern "C" void dmc_matmul_bf16_gpu_batched_deferred(int64_t l, int64_t r, int64_t out, int64_t m, int64_t k,
                                                     int64_t n, int64_t batch, int64_t ls, int64_t rs) {
    run_host_call(HostCall{(const float *)l, (const void *)r, (float *)out, m, k, n, batch, ls, rs, DMC_LAYOUT_KN,
                           DMC_W_BF16, true, true});
}

extern "C" void dmc_matmul_bf16_gpu_flush(void) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    flush_locked();
}

extern "C" void dmc_matmul_f32_gpu(int64_t l, int64_t r, int64_t out, int64_t m, int64_t k, int64_t n) {
    run_host_call(HostCall{(const float *)l, (const void *)r, (float *)out, m, k, n, 1, 0, 0, DMC_LAYOUT_KN,
                           DMC_W_F32, false, false});
}

extern "C" void dmc_matmul_bf16_gpu_nt(int64_t l, int64_t w, int64_t out, int64_t m, int64_t k, int64_t n) {
    run_host_call(HostCall{(const float *)l, (const void *)w, (float *)out, m, k, n, 1, 0, 0, DMC_LAYOUT_NK,
                           DMC_W_BF16, false, true});
}

extern "C" int dmc_cuda_matmul_selected(int flag_on, uint32_t deterministic_depth, int64_t m, int64_t k,
                                        int64_t n, int64_t batch, int rhs_bf16) {
    if (!flag_on || deterministic_depth != 0) return 0;
    if (m <= 0 || k <= 0 || n <= 0 || batch <= 0) return 0;
    const __int128 macs1 = (__int128)m * k * n;
    if (!rhs_bf16) return macs1 >= ((__int128)1 << 17);
    if (batch == 1) return (__int128)k * n >= 4000000;
    // batched projections: m == 1 slices of a width the vector kernels take (compiler/src/jit.rs:19912-19915)
    return m == 1 && n % 4 == 0 && batch <= 65536 && macs1 * batch >= 1000000;
}

extern "C" int dmc_cuda_register_weight(int64_t ptr, int64_t bytes, int64_t k, int64_t n, int layout, int wdtype) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    if (!ptr || bytes <= 0 || (wdtype != DMC_W_BF16 && wdtype != DMC_W_F32))
        return fail(DMC_CUDA_ERR_BAD_ARG, "register_weight: bad range or type");
    const size_t wsz = wdtype == DMC_W_BF16 ? 2 : 4;
    const bool shaped = k > 0 && n > 0;
    if (shaped && ((layout != DMC_LAYOUT_KN && layout != DMC_LAYOUT_NK) || (__int128)k * n * (int64_t)wsz != bytes))
        return fail(DMC_CUDA_ERR_BAD_ARG, "register_weight: %lld bytes is not a [%lld, %lld] matrix of %zu-byte elements",
                    (long long)bytes, (long long)k, (long long)n, wsz);
    int rc = ensure_init();
    if (rc) return rc;
    Context &c = ctx();
    for (const RegisteredRange &rg : c.registered)
        if ((uintptr_t)ptr < rg.host + rg.bytes && rg.host < (uintptr_t)ptr + (size_t)bytes)
            return fail(DMC_CUDA_ERR_BAD_ARG, "register_weight: range overlaps a registered range");
    // A [k, n] matrix (the operand of `x @ w`) is stored k-contiguous, like a weight found by its
    // fingerprint, so that the row-streaming kernel serves it; every other range is kept as it is.
    const bool transposed = shaped && layout == DMC_LAYOUT_KN && tuning().store_nk && nk_fast_eligible(k, n, wdtype);
    void *d = nullptr;
    rc = upload_weight((uintptr_t)ptr, (size_t)bytes, k, n, wsz, transposed, &d);
    if (rc) return rc;
    RegisteredRange rg{(uintptr_t)ptr, (size_t)bytes, d, wdtype};
    if (transposed) rg.k = k, rg.n = n;
    c.registered.push_back(rg);
    c.resident_bytes += bytes;
    return DMC_CUDA_OK;
}

extern "C" int dmc_cuda_unregister_weight(int64_t ptr) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    Context &c = ctx();
    for (size_t i = 0; i < c.registered.size(); ++i)
        if (c.registered[i].host == (uintptr_t)ptr) {
            cudaStreamSynchronize(c.stream);
            cudaFree(c.registered[i].dev);
            c.resident_bytes -= (int64_t)c.registered[i].bytes;
            c.registered.erase(c.registered.begin() + i);
            return DMC_CUDA_OK;
        }
    return DMC_CUDA_ERR_BAD_ARG;  // not an error worth making sticky
}

extern "C" int64_t dmc_cuda_resident_count(void) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    return (int64_t)(ctx().by_fingerprint.size() + ctx().registered.size());
}
extern "C" int64_t dmc_cuda_resident_bytes(void) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    return ctx().resident_bytes;
}
extern "C" void dmc_cuda_drop_resident(void) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    Context &c = ctx();
    if (!c.ready) return;
    cudaStreamSynchronize(c.stream);
    for (auto &kv : c.by_fingerprint) cudaFree(kv.second);
    c.by_fingerprint.clear();
    c.by_address.clear();
    c.resident_bytes = 0;
    for (const RegisteredRange &rg : c.registered) c.resident_bytes += (int64_t)rg.bytes;
}

namespace dmc {
static int apply_param(const char *name, int64_t value) {
    Tuning &t = tuning();
    if (!strcmp(name, "pdl")) t.pdl = (int)value;
    else if (!strcmp(name, "kn_ctas_per_sm")) t.kn_ctas_per_sm = (int)value;
    else if (!strcmp(name, "kn_ksplit")) t.kn_ksplit = (int)value;
    else if (!strcmp(name, "nk_ctas_per_sm")) t.nk_ctas_per_sm = (int)value;
    else if (!strcmp(name, "nk_even_rounds")) t.nk_even_rounds = (int)value;
    else if (!strcmp(name, "tma_ring_kb")) t.tma_ring_kb = (int)value;
    else if (!strcmp(name, "tma_stage_kb")) t.tma_stage_kb = (int)value;
    else if (!strcmp(name, "tma_ctas_per_sm")) t.tma_ctas_per_sm = (int)value;
    else if (!strcmp(name, "store_nk")) t.store_nk = (int)value;
    else if (!strcmp(name, "nk_default")) t.nk_default = (int)value;
    else if (!strcmp(name, "shard_fused")) t.shard_fused = (int)value;
    else if (!strcmp(name, "shard_overlap")) t.shard_overlap = (int)value;
    else if (!strcmp(name, "overlap_independent")) t.overlap_independent = (int)value;
    else if (!strcmp(name, "wait_limit_us")) t.wait_limit_us = (int)value;
    else if (!strcmp(name, "timing")) t.timing = (int)value;
    else if (!strcmp(name, "spin_sync")) t.spin_sync = (int)value;
    else if (!strcmp(name, "host_io_kernels")) t.host_io_kernels = (int)value;
    else if (!strcmp(name, "zero_copy_y")) t.zero_copy_y = (int)value;
    else if (!strcmp(name, "decode_fused")) t.decode_fused = (int)value;
    else if (!strcmp(name, "tc_ksplit")) t.tc_ksplit = (int)value;
    else if (!strcmp(name, "tc_smem_kb")) t.tc_smem_kb = (int)value;
    else if (!strcmp(name, "tc_min_m")) t.tc_min_m = (int)value;
    else return DMC_CUDA_ERR_BAD_ARG;
    return DMC_CUDA_OK;
}

// DMC_CUDA_PARAMS="name=value,name=value": the same knobs as dmc_cuda_set_param, read once at
// context creation (env-var style of the reference's DMC_GPU_PARTS, compiler/src/gpu.rs:552).
void apply_env_params() {
    const char *env = getenv("DMC_CUDA_PARAMS");
    if (!env) return;
    std::string str(env);
    size_t pos = 0;
    while (pos < str.size()) {
        size_t end = str.find(',', pos);
        if (end == std::string::npos) end = str.size();
        std::string kv = str.substr(pos, end - pos);
        size_t eq = kv.find('=');
        if (eq != std::string::npos) apply_param(kv.substr(0, eq).c_str(), atoll(kv.c_str() + eq + 1));
        pos = end + 1;
    }
}
}  // namespace dmc

extern "C" int dmc_cuda_set_param(const char *name, int64_t value) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    return apply_param(name, value);
}

// ---- device-resident path -----------------------------------------------------------------

extern "C" void *dmc_cuda_dev_alloc(int64_t bytes) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status() || ensure_init()) return nullptr;
    void *p = nullptr;
    cudaError_t e = dmc_malloc(&p, bytes > 0 ? (size_t)bytes : 16);
    if (e != cudaSuccess) {
        fail(DMC_CUDA_ERR_OOM, "dev_alloc(%lld) failed: %s", (long long)bytes, cudaGetErrorString(e));
        return nullptr;
    }
    return p;
}
extern "C" void dmc_cuda_dev_free(void *p) {
    if (p) cudaFree(p);
}
extern "C" int dmc_cuda_h2d(void *dst, const void *src, int64_t bytes) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    DMC_CUDA_TRY(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, ctx().stream));
    DMC_CUDA_TRY(cudaStreamSynchronize(ctx().stream));
    stream_drained();
    return DMC_CUDA_OK;
}
extern "C" int dmc_cuda_d2h(void *dst, const void *src, int64_t bytes) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    DMC_CUDA_TRY(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToHost, ctx().stream));
    DMC_CUDA_TRY(cudaStreamSynchronize(ctx().stream));
    stream_drained();
    return DMC_CUDA_OK;
}
extern "C" int dmc_cuda_memset(void *dst, int value, int64_t bytes) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    DMC_CUDA_TRY(cudaMemsetAsync(dst, value, (size_t)bytes, ctx().stream));
    return DMC_CUDA_OK;
}
extern "C" int dmc_cuda_sync(void) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (!ctx().ready) return dmc::status();
    DMC_CUDA_TRY(cudaStreamSynchronize(ctx().stream));
    stream_drained();
    return check_device_error();
}

extern "C" int dmc_cuda_gemv_dev(const void *dW, const float *dx, float *dy, int64_t m, int64_t k, int64_t n,
                                 int layout, int wdtype, int variant) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    int rc = ensure_init();
    if (rc) return rc;
    return launch_gemv(dW, dx, dy, m, k, n, 1, 0, 0, layout, wdtype, variant, ctx().stream);
}

extern "C" int dmc_cuda_gemm_dev(const void *dW, const void *dX, float *dY, int64_t m, int64_t k, int64_t n,
                                 int xdtype) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    int rc = ensure_init();
    if (rc) return rc;
    if (m <= 0 || n <= 0) return DMC_CUDA_OK;
    if (k == 0) {
        DMC_CUDA_TRY(cudaMemsetAsync(dY, 0, (size_t)m * n * sizeof(float), ctx().stream));
        return DMC_CUDA_OK;
    }
    if (!gemm_tc_eligible(m, k, n, dW, dX))
        return fail(DMC_CUDA_ERR_UNSUPPORTED, "gemm: needs k %% 8 == 0 and 16-byte aligned operands (m=%lld k=%lld n=%lld)",
                    (long long)m, (long long)k, (long long)n);
    if (xdtype == DMC_X_BF16) return launch_gemm_tc(dW, dX, dY, m, k, n, 0, ctx().stream);
    if (xdtype == DMC_X_F32) return launch_gemm_tc_f32x(dW, (const float *)dX, dY, m, k, n, ctx().stream);
    return fail(DMC_CUDA_ERR_BAD_ARG, "gemm: unknown activation type %d", xdtype);
}

extern "C" double dmc_cuda_bench_items(const dmc_gemv_item *items, int count, int steps, int warmup,
                                       int use_graph) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status() || ensure_init()) return -1.0;
    if (!items || count <= 0 || steps <= 0 || warmup < 0) {
        fail(DMC_CUDA_ERR_BAD_ARG, "bench_items: need count > 0, steps > 0, warmup >= 0");
        return -1.0;
    }
    Context &c = ctx();
    cudaStream_t s = c.stream;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    double us = -1.0;
    auto one_step = [&]() -> int {
        for (int i = 0; i < count; ++i) {
            const dmc_gemv_item &it = items[i];
            int rc;
            if (it.op == 1) rc = launch_gemm_tc(it.W, it.x, it.y, it.m, it.k, it.n, 0, s);
            else if (it.op == 2) rc = launch_gemm_tc_f32x(it.W, it.x, it.y, it.m, it.k, it.n, s);
            else rc = launch_gemv(it.W, it.x, it.y, it.m, it.k, it.n, it.batch > 1 ? it.batch : 1, it.batch > 1 ? it.ls : 0,
                                  it.batch > 1 ? it.rs : 0, it.layout, it.wdtype, it.variant, s);
            if (rc) return rc;
        }
        return DMC_CUDA_OK;
    };
    auto body = [&]() -> int {
        // one untimed eager step: sizes the split-K scratch (nothing may allocate under capture)
        int rc = one_step();
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
            stream_drained();  // a graph launch is ordered after everything before it in the stream
            if (rc) return rc;
            DMC_CUDA_TRY(ce);
            per_step = c.launches - before;
            DMC_CUDA_TRY(cudaGraphInstantiate(&exec, graph, 0));
        }
        auto run_step = [&]() -> int {
            if (!use_graph) return one_step();
            DMC_CUDA_TRY(cudaGraphLaunch(exec, s));
            c.launches += per_step;  // a replay launches the captured kernels again
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

extern "C" int dmc_cuda_timeline(const void *const *dWs, int count, const float *dx, float *dy, int64_t k, int64_t n,
                                 int dependent, unsigned long long *stamps_out, int64_t stamps_cap_words) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status() || ensure_init()) return -dmc::status();
    return timeline_nk(dWs, count, dx, dy, k, n, dependent, stamps_out, stamps_cap_words, ctx().stream);
}

extern "C" int64_t dmc_cuda_launch_count(void) { return ctx().launches; }
