// no_alloc.cu -- a split-K bf16 GEMV entry point for callers that must not allocate.
//
// Who needs this.  Every other entry point of this library may call cudaMalloc /
// cudaMallocHost behind the caller's back (context set-up, staging, split-K scratch
// that grows on demand).  Some hosts cannot accept that: a runtime that has handed
// the whole device to its own arena under a fixed budget (demoniC gives its Forge a
// hard byte limit and treats any allocation outside it as a bug), or a serving loop
// that shares the GPU with other streams and cannot afford the device-wide
// synchronisation an allocation or free implies in the middle of a decode step.
// For them the split-K partial sums live in a fixed array that is part of the
// library image itself.
//
// The price: the array is file-scope device memory, so every GPU that loads this
// library carries it (about 4 MiB) until the process exits, shapes beyond its
// capacity are refused, and all calls share it -- see the notes on the entry point.
#include <algorithm>
#include <mutex>

#include "gemv.cuh"
#include "runtime.h"

namespace {

constexpr int kMaxN = 16384;      // widest output row the scratch can hold
constexpr int kMaxKsplit = 64;    // most K slices whose partials it can hold
constexpr int kMaxColblocks = kMaxN / 256;
constexpr int kMaxDevices = 64;

struct NoAllocScratch {
    float partial[(size_t)kMaxKsplit * kMaxN];  // [ksplit][n] partial sums, 4 MiB
    unsigned counters[256];                     // one arrival counter per 256-column block
};

// In host code this name is only a handle for the runtime's symbol table, not an
// address a kernel can use: the device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

std::mutex g_setup_mutex;
NoAllocScratch *g_scratch_on_device[kMaxDevices] = {};

// Device address of the scratch array on the current device (looked up on first use).
int scratch_for_current_device(NoAllocScratch **out) {
    int dev = -1;
    DMC_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices)
        return dmc::fail(DMC_CUDA_ERR_UNSUPPORTED, "no-alloc gemv: device ordinal %d is beyond %d", dev, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_on_device[dev]) {
        void *p = nullptr;
        DMC_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        g_scratch_on_device[dev] = static_cast<NoAllocScratch *>(p);
    }
    *out = g_scratch_on_device[dev];
    return DMC_CUDA_OK;
}

}  // namespace

extern "C" int dmc_cuda_gemv_bf16_noalloc(const void *dW, const float *dx, float *dy, int64_t k, int64_t n,
                                          void *stream) {
    using namespace dmc;
    constexpr int TK = 8, U = 8, V = 1, CW = 32 * V * 8;  // 256 columns per CTA
    if (dmc::status()) return dmc::status();
    if (!dW || !dx || !dy || k < 0 || n < 0)
        return fail(DMC_CUDA_ERR_BAD_ARG, "no-alloc gemv: null pointer or negative size (k=%lld n=%lld)",
                    (long long)k, (long long)n);
    if (n == 0) return DMC_CUDA_OK;
    if (n > kMaxN)
        return fail(DMC_CUDA_ERR_UNSUPPORTED,
                    "no-alloc gemv: n=%lld is beyond the built-in scratch (at most %d output columns); "
                    "use dmc_cuda_gemv_dev, which allocates",
                    (long long)n, kMaxN);
    if (k > INT32_MAX)
        return fail(DMC_CUDA_ERR_UNSUPPORTED, "no-alloc gemv: k=%lld is beyond 2^31-1", (long long)k);
    if (n % 8 != 0 || ((uintptr_t)dW % 16) != 0)
        return fail(DMC_CUDA_ERR_UNSUPPORTED,
                    "no-alloc gemv: needs n %% 8 == 0 and a 16-byte aligned weight pointer (n=%lld)", (long long)n);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (k == 0) {  // empty contraction: the row is zero
        DMC_CUDA_TRY(cudaMemsetAsync(dy, 0, (size_t)n * sizeof(float), s));
        return DMC_CUDA_OK;
    }
    NoAllocScratch *scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;

    int sms = 148;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);

    GemvArgs a = {};
    a.W = dW;
    a.x = dx;
    a.y = dy;
    a.K = (int)k;
    a.N = (int)n;
    a.colblocks = (int)((n + CW - 1) / CW);
    int64_t ksplit = ((int64_t)sms * 4 + a.colblocks / 2) / a.colblocks;  // about four CTAs per SM
    const int64_t step = TK * U;
    ksplit = std::max<int64_t>(1, std::min<int64_t>(ksplit, (k + step - 1) / step));
    ksplit = std::min<int64_t>(ksplit, kMaxKsplit);
    int64_t kchunk = (k + ksplit - 1) / ksplit;
    kchunk = (kchunk + TK - 1) / TK * TK;
    ksplit = (k + kchunk - 1) / kchunk;
    a.kchunk = (int)kchunk;
    a.ksplit = (int)ksplit;
    a.partial = scratch->partial;
    a.counters = scratch->counters;
    // The array keeps whatever the previous call left: the arrival counters must start at zero.
    // (The partial sums need no clearing; every slot that is read is written first.)
    DMC_CUDA_TRY(cudaMemsetAsync(scratch->counters, 0, sizeof(scratch->counters), s));
    dmc_wcols_kernel<TK, U, V, 1, uint16_t><<<dim3((unsigned)a.colblocks, (unsigned)ksplit), TK * 32, 0, s>>>(a);
    DMC_CUDA_TRY(cudaGetLastError());
    return DMC_CUDA_OK;
}
