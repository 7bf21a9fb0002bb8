// gemv_launch.cu -- kernel-configuration tables and launch planning for the GEMV kernels.
#include <algorithm>
#include <cstdio>
#include <map>
#include <set>

#include "gemv.cuh"
#include "gemv_tma.cuh"
#include "runtime.h"

namespace dmc {

namespace {

using KernelFn = void (*)(const GemvArgs);

struct KnVariant {
    const char *name;
    int TK, U, V;
    int ctas_per_sm;  // resident-CTA target used to size split-K
    KernelFn bf16[4]; // M = 1, 2, 4, 8
    KernelFn f32[4];
};

#define KN_ROW(TK, U, V, CPS)                                                                    \
    {                                                                                            \
        "kn_tk" #TK "_u" #U "_v" #V, TK, U, V, CPS,                                              \
            {dmc_wcols_kernel<TK, U, V, 1, uint16_t>, nullptr, nullptr, nullptr},                \
            {dmc_wcols_kernel<TK, U, V, 1, float>, nullptr, nullptr, nullptr},                   \
    }

// Index 0 is the multi-row-capable configuration (M up to 8).
static const KnVariant kKn[] = {
    {"kn_tk8_u4_v1", 8, 4, 1, 4,
     {dmc_wcols_kernel<8, 4, 1, 1, uint16_t>, dmc_wcols_kernel<8, 4, 1, 2, uint16_t>,
      dmc_wcols_kernel<8, 4, 1, 4, uint16_t>, dmc_wcols_kernel<8, 4, 1, 8, uint16_t>},
     {dmc_wcols_kernel<8, 4, 1, 1, float>, dmc_wcols_kernel<8, 4, 1, 2, float>,
      dmc_wcols_kernel<8, 4, 1, 4, float>, dmc_wcols_kernel<8, 4, 1, 8, float>}},
    KN_ROW(8, 8, 1, 4),
    KN_ROW(8, 4, 2, 2),
    KN_ROW(8, 8, 2, 2),
    KN_ROW(16, 4, 1, 2),
    KN_ROW(16, 4, 2, 1),
    KN_ROW(16, 8, 1, 2),
    KN_ROW(4, 8, 1, 8),
    KN_ROW(4, 8, 2, 4),
    KN_ROW(4, 16, 1, 6),
    KN_ROW(8, 2, 4, 2),
    KN_ROW(8, 16, 1, 2),
};
constexpr int kKnCount = sizeof(kKn) / sizeof(kKn[0]);

// Narrow matrices (n <= 128: the per-head projections of the batched entry points): 2 or 4 k rows per
// warp-wide load, so that every lane carries a vector.
struct KnNarrow {
    int max_n, NR, TK, U;
    KernelFn bf16, f32;
};
static const KnNarrow kKnNarrow[] = {
    {64, 4, 8, 8, dmc_wcols_kernel<8, 8, 1, 1, uint16_t, 4>, dmc_wcols_kernel<8, 8, 1, 1, float, 2>},   // f32: 4 columns per vector
    {128, 2, 8, 8, dmc_wcols_kernel<8, 8, 1, 1, uint16_t, 2>, dmc_wcols_kernel<8, 8, 1, 1, float, 1>},
};

struct NkVariant {
    const char *name;
    int WARPS, R, U;
    KernelFn bf16, f32;
};
#define NK_ROW(WARPS, R, U)                                                                       \
    {                                                                                             \
        "nk_w" #WARPS "_r" #R "_u" #U, WARPS, R, U, dmc_wrows_kernel<WARPS, R, U, 1, uint16_t>,    \
            dmc_wrows_kernel<WARPS, R, U, 1, float>                                               \
    }
static const NkVariant kNk[] = {
    NK_ROW(8, 2, 8),  NK_ROW(8, 4, 4),  NK_ROW(8, 2, 4),  NK_ROW(8, 1, 8),
    NK_ROW(8, 1, 4),  NK_ROW(16, 2, 4), NK_ROW(16, 1, 8), NK_ROW(4, 2, 8),
    NK_ROW(4, 4, 4),  NK_ROW(8, 4, 2),
};
constexpr int kNkCount = sizeof(kNk) / sizeof(kNk[0]);
constexpr size_t kNkMaxSmem = 200 * 1024;  // staged rows of x per CTA
constexpr int kTcMinRows = 9;                // measured on B200 at 4096x4096 with f32 activations: 8 rows 10.1 us on the CUDA cores
                                             // against 14.2 us on the tensor cores; 16 rows 18.6 against 15.6

// Small batches (2, 4 or 8 activation rows sharing every weight load), one configuration each.
struct NkRows {
    int M, WARPS, R, U;
    KernelFn bf16, f32;
};
static const NkRows kNkRows[] = {
    {2, 8, 2, 8, dmc_wrows_kernel<8, 2, 8, 2, uint16_t>, dmc_wrows_kernel<8, 2, 8, 2, float>},
    {4, 8, 2, 8, dmc_wrows_kernel<8, 2, 8, 4, uint16_t>, dmc_wrows_kernel<8, 2, 8, 4, float>},
    {8, 16, 4, 2, dmc_wrows_kernel<16, 4, 2, 8, uint16_t>, dmc_wrows_kernel<16, 4, 2, 8, float>},
};

// ---- which launches may overlap -----------------------------------------------------------
// Address ranges read and written by the launches since the last point at which the stream was
// known to be drained.  A GEMV that touches none of them in a conflicting way skips the
// programmatic-dependency wait (GemvArgs::nowait) and overlaps whatever is still running; the first
// launch that does conflict after such a kernel is made without the programmatic attribute, i.e.
// it waits for everything before it.
bool overlaps(const std::vector<AddrRange> &list, const void *p, size_t bytes) {
    if (!p || !bytes) return false;
    const uintptr_t lo = (uintptr_t)p, hi = lo + bytes;
    for (const AddrRange &r : list)
        if (lo < r.hi && r.lo < hi) return true;
    return false;
}
void note(std::vector<AddrRange> &list, const void *p, size_t bytes) {
    if (p && bytes) list.push_back(AddrRange{(uintptr_t)p, (uintptr_t)p + bytes});
}

}  // namespace

// ---- host-pointer calls: x in and y out without the copy engines --------------------------
// For the few KiB a GEMV call moves, a copy-engine transfer costs more in start-up than in transfer.
// Two small kernels move the data instead, chained to the GEMV by programmatic dependent launch:
// one reads x from the pinned host mirror, 16 bytes per thread, one PCIe round trip in all; the other
// writes y to the pinned host mirror in full 128-byte lines (the GEMV itself would store it four
// bytes at a time) and then a sequence number, which the waiting host thread polls in its own memory
// instead of asking the driver.
__global__ void __launch_bounds__(1024) dmc_stage_x_kernel(const float *src_host, float *dst, long long elems) {
    griddep_launch_dependents();  // the GEMV behind this kernel loads its first weights meanwhile
    griddep_wait();               // whatever used the staging area before is complete
    const long long nvec = elems / 4;
    for (long long i = (long long)blockIdx.x * 1024 + threadIdx.x; i < nvec; i += (long long)gridDim.x * 1024)
        reinterpret_cast<float4 *>(dst)[i] = __ldcv(reinterpret_cast<const float4 *>(src_host) + i);
    if (blockIdx.x == 0 && threadIdx.x < (int)(elems - nvec * 4)) dst[nvec * 4 + threadIdx.x] = __ldcv(src_host + nvec * 4 + threadIdx.x);
}

__global__ void __launch_bounds__(1024) dmc_deliver_kernel(const float *src, float *dst_host, long long elems,
                                                           unsigned *done_word, unsigned seq, unsigned *arrived) {
    griddep_wait();  // y is complete
    const long long nvec = elems / 4;
    for (long long i = (long long)blockIdx.x * 1024 + threadIdx.x; i < nvec; i += (long long)gridDim.x * 1024)
        reinterpret_cast<float4 *>(dst_host)[i] = __ldcg(reinterpret_cast<const float4 *>(src) + i);
    if (blockIdx.x == 0 && threadIdx.x < (int)(elems - nvec * 4)) dst_host[nvec * 4 + threadIdx.x] = __ldcg(src + nvec * 4 + threadIdx.x);
    // One thread per CTA fences, after the barrier through which it has observed the whole CTA's stores
    // (fences are cumulative): one PCIe round trip, and with a single CTA no arrival counter at all.
    __syncthreads();
    if (threadIdx.x == 0) {
        bool last = true;
        if (gridDim.x > 1) {
            __threadfence_system();
            last = atomicAdd(arrived, 1u) == gridDim.x - 1u;  // the CTA that arrives last writes the sequence number
            if (last) *arrived = 0u;
        }
        if (last) {
            __threadfence_system();
            *(volatile unsigned *)done_word = seq;  // last: the host reads y once it sees this
        }
    }
}

int launch_stage_x(const float *h_src, float *d_dst, size_t elems, cudaStream_t stream) {
    Context &c = ctx();
    long long n = (long long)elems;
    void *params[] = {&h_src, &d_dst, &n};
    const unsigned ctas = (unsigned)std::max<size_t>(1, std::min<size_t>(16, (elems / 4 + 1023) / 1024));
    int rc = launch_ex((const void *)dmc_stage_x_kernel, dim3(ctas), dim3(1024), 0, stream, params, kLaunchTracked);
    if (rc) return rc;
    note(c.inflight_writes, d_dst, elems * 4);
    return DMC_CUDA_OK;
}

int launch_deliver(const float *d_src, float *h_dst, size_t elems, cudaStream_t stream) {
    Context &c = ctx();
    long long n = (long long)elems;
    if (!c.deliver_count) {
        DMC_CUDA_TRY(dmc_malloc((void **)&c.deliver_count, sizeof(unsigned)));
        DMC_CUDA_TRY(cudaMemset(c.deliver_count, 0, sizeof(unsigned)));
    }
    unsigned seq = ++c.done_seq;
    unsigned *word = c.done_word, *arrived = c.deliver_count;
    void *params[] = {&d_src, &h_dst, &n, &word, &seq, &arrived};
    // one CTA per 64 KiB: a single CTA needs no arrival counter (one fence, then the word)
    const unsigned ctas = (unsigned)std::max<size_t>(1, std::min<size_t>(8, (elems * 4 + (64u << 10) - 1) / (64u << 10)));
    int rc = launch_ex((const void *)dmc_deliver_kernel, dim3(ctas), dim3(1024), 0, stream, params, kLaunchTracked);
    if (rc) return rc;
    note(c.inflight_reads, d_src, elems * 4);
    c.done_is_last = true;
    return DMC_CUDA_OK;
}

void stream_drained() {
    Context &c = ctx();
    c.inflight_reads.clear();
    c.inflight_writes.clear();
    c.nowait_inflight = false;
    c.untracked_inflight = false;
}

int launch_ex(const void *fn, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, void **params, int mode) {
    Context &c = ctx();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    int nattr = 0;
    // A kernel that must see everything before it, launched after kernels that skipped their wait,
    // cannot rely on the chain of waits: it is launched fully serialised instead (so is one that
    // arrives when the lists have grown long, which lets them be emptied).
    const bool serialise = mode != kLaunchOverlap &&
                           (c.nowait_inflight || c.inflight_reads.size() + c.inflight_writes.size() > kMaxTrackedRanges);
    if (tuning().pdl && !serialise) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        nattr = 1;
    }
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
    DMC_CUDA_TRY(cudaLaunchKernelExC(&cfg, fn, params));
    c.done_is_last = false;
    if (serialise) stream_drained();  // whatever ran before this kernel is complete when it starts
    if (mode == kLaunchOverlap) c.nowait_inflight = true;
    if (mode == kLaunchUntracked) c.untracked_inflight = true;
    c.launches++;
    return DMC_CUDA_OK;
}

int ensure_scratch(size_t partial_bytes, size_t ncounters) {
    Context &c = ctx();
    if (partial_bytes > c.partial_cap) {
        // in-flight kernels may still use the old buffer
        DMC_CUDA_TRY(cudaStreamSynchronize(c.stream));
        stream_drained();
        if (c.partial) cudaFree(c.partial);
        c.partial = nullptr;
        c.partial_cap = 0;
        size_t cap = std::max(partial_bytes, (size_t)4 << 20);
        DMC_CUDA_TRY(dmc_malloc((void **)&c.partial, cap));
        c.partial_cap = cap;
    }
    if (ncounters > c.counters_cap) {
        DMC_CUDA_TRY(cudaStreamSynchronize(c.stream));
        stream_drained();
        if (c.counters) cudaFree(c.counters);
        c.counters = nullptr;
        c.counters_cap = 0;
        size_t cap = std::max(ncounters, (size_t)4096);
        DMC_CUDA_TRY(dmc_malloc((void **)&c.counters, cap * sizeof(unsigned)));
        DMC_CUDA_TRY(cudaMemset(c.counters, 0, cap * sizeof(unsigned)));
        c.counters_cap = cap;
    }
    return DMC_CUDA_OK;
}

namespace {

// Default configuration per shape (from sweeps on B200 over every configuration in the tables above).
int default_kn_variant(int64_t k, int64_t n) {
    (void)k;
    return n <= 256 ? 1 : 3;  // one vector per lane when a row has no more than 32 of them; else two
}
int default_nk_variant(int64_t k, int64_t n) {
    // B200 sweeps: 8 warps x 2 rows x 8 loads in flight is the best or within 1 % of the best
    // configuration on every shape from 4096x4096 to 65536x8192 (4 rows x 4 loads: 22.0 vs 21.7 us at
    // 8192x8192 in a dependent chain, 81.0 vs 79.6 at 32768x8192).  A matrix with so few rows that two
    // rows per warp would leave SMs without a CTA (a 2048-row output projection: 128 CTAs on 148 SMs)
    // takes one row per warp instead.
    (void)k;
    if ((n + 15) / 16 < ctx().sm_count) return 3;         // nk_w8_r1_u8
    return 0;                                             // nk_w8_r2_u8
}

int launch_kn(const void *dW, const float *dx, float *dy, int64_t m, int64_t k, int64_t n,
              int64_t batch, int64_t ls, int64_t rs, int wdtype, int variant, cudaStream_t stream) {
    Context &c = ctx();
    const int epv = wdtype == DMC_W_BF16 ? 8 : 4;
    const bool vec_ok = n % epv == 0 && rs % epv == 0 && ((uintptr_t)dW % 16) == 0;
    GemvArgs a = {};
    a.W = dW;
    a.K = (int)k;
    a.N = (int)n;
    a.ls = ls;
    a.rs = rs;
    if (!vec_ok) {
        a.x = dx;
        a.y = dy;
        a.ksplit = 1;
        a.kchunk = (int)k;
        a.colblocks = (int)((n + 31) / 32);
        int M = (int)m;
        void *params[] = {&a, &M};
        const void *fn = wdtype == DMC_W_BF16 ? (const void *)dmc_wcols_any_kernel<8, uint16_t>
                                              : (const void *)dmc_wcols_any_kernel<8, float>;
        return launch_ex(fn, dim3((unsigned)(a.colblocks * batch)), dim3(256), 0, stream, params);
    }
    // narrow matrices: the form in which every lane loads (bf16 n <= 128, f32 n <= 64)
    const KnNarrow *narrow = nullptr;
    if (variant < 0 && m == 1)
        for (const KnNarrow &c2 : kKnNarrow)
            if (!narrow && n * (wdtype == DMC_W_BF16 ? 1 : 2) <= c2.max_n) narrow = &c2;
    if (variant < 0 || variant >= kKnCount) variant = default_kn_variant(k, n);
    // rows of x beyond what one kernel instance holds are processed in chunks
    for (int64_t m0 = 0; m0 < m;) {
        const int64_t left = m - m0;
        int mi = left >= 8 ? 3 : left >= 4 ? 2 : left >= 2 ? 1 : 0;
        const int M = 1 << mi;
        KnVariant v = (M == 1) ? kKn[variant] : kKn[0];
        KernelFn fn = wdtype == DMC_W_BF16 ? v.bf16[mi] : v.f32[mi];
        int nr = 1;
        if (narrow) {
            nr = wdtype == DMC_W_BF16 ? narrow->NR : narrow->NR / 2;
            fn = wdtype == DMC_W_BF16 ? narrow->bf16 : narrow->f32;
            v.TK = narrow->TK, v.U = narrow->U, v.V = 1, v.ctas_per_sm = 4;
        }
        const int cw = (32 / nr) * v.V * epv;
        a.colblocks = (int)((n + cw - 1) / cw);
        const int64_t base_ctas = (int64_t)a.colblocks * batch;
        const int cps = tuning().kn_ctas_per_sm > 0 ? tuning().kn_ctas_per_sm : v.ctas_per_sm;
        int64_t ksplit = tuning().kn_ksplit > 0 ? tuning().kn_ksplit
                                                 : ((int64_t)c.sm_count * cps + base_ctas / 2) / base_ctas;
        const int64_t step = (int64_t)v.TK * v.U * nr;
        ksplit = std::max<int64_t>(1, std::min<int64_t>(ksplit, (k + step - 1) / step));
        ksplit = std::min<int64_t>(ksplit, 65535);
        int64_t kchunk = (k + ksplit - 1) / ksplit;
        const int64_t kq = (int64_t)v.TK * nr;
        kchunk = (kchunk + kq - 1) / kq * kq;
        if (kchunk < 1) kchunk = kq;
        ksplit = std::max<int64_t>(1, (k + kchunk - 1) / kchunk);
        a.kchunk = (int)kchunk;
        a.ksplit = (int)ksplit;
        a.x = dx + m0 * k;
        a.y = dy + m0 * n;
        if (ksplit > 1) {
            int rc = ensure_scratch((size_t)batch * ksplit * M * n * sizeof(float), (size_t)base_ctas);
            if (rc) return rc;
            a.partial = c.partial;
            a.counters = c.counters;
        }
        void *params[] = {&a};
        int rc = launch_ex((const void *)fn, dim3((unsigned)base_ctas, (unsigned)ksplit),
                           dim3(v.TK * 32), 0, stream, params);
        if (rc) return rc;
        m0 += M;
    }
    return DMC_CUDA_OK;
}

// ---- NK layout, TMA ring kernel ------------------------------------------------------

using TmaFn = void (*)(const GemvTmaArgs);
#define TMA_ROW(T, CW)                                                                              \
    {dmc_wrows_ring_kernel<1, CW, T>, dmc_wrows_ring_kernel<2, CW, T>, dmc_wrows_ring_kernel<3, CW, T>,     \
     dmc_wrows_ring_kernel<4, CW, T>, dmc_wrows_ring_kernel<5, CW, T>, dmc_wrows_ring_kernel<6, CW, T>,     \
     dmc_wrows_ring_kernel<7, CW, T>, dmc_wrows_ring_kernel<8, CW, T>}
static const TmaFn kTma[2][2][8] = {  // [wdtype][CW == 16][VPL - 1]
    {TMA_ROW(uint16_t, 8), TMA_ROW(uint16_t, 16)},
    {TMA_ROW(float, 8), TMA_ROW(float, 16)},
};
constexpr int kTmaVariantCw8 = kNkCount;       // variant ids after the LDG configurations
constexpr int kTmaVariantCw16 = kNkCount + 1;
constexpr int kNkTotal = kNkCount + 2;

struct TmaPlan {
    bool ok = false;
    int cw = 8, vpl = 1, SR = 1, S = 2, stage_bytes = 0;
    size_t smem = 0;
};

// Ring geometry: stages of whole rows (~tma_stage_kb each), as many as fit the ring
// budget.  The default budget leaves room for the next kernel's CTA on the same SM,
// so its first stages load while this kernel is still running.
TmaPlan plan_tma(int64_t k, int64_t n, int wdtype, int want_cw, const void *dW, const float *dx) {
    TmaPlan p;
    const int wsz = wdtype == DMC_W_BF16 ? 2 : 4;
    const int epv = 16 / wsz;
    if (k % epv || ((uintptr_t)dW % 16) || ((uintptr_t)dx % 16) || n < 1) return p;
    const int64_t nvec = k / epv;
    if (nvec < 256) return p;  // short rows leave most lanes idle: the LDG kernel takes them
    int cw = want_cw;
    if (cw == 0) cw = (nvec + 255) / 256 <= 4 ? 8 : 16;
    int vpl = (int)((nvec + cw * 32 - 1) / (cw * 32));
    if (vpl > 8 && cw == 8) {
        cw = 16;
        vpl = (int)((nvec + cw * 32 - 1) / (cw * 32));
    }
    if (vpl > 8) return p;
    const int64_t rowbytes = k * wsz;
    const int64_t ring = (int64_t)(tuning().tma_ring_kb > 0 ? tuning().tma_ring_kb : 96) * 1024;
    const int64_t stage_target = (int64_t)(tuning().tma_stage_kb > 0 ? tuning().tma_stage_kb : 32) * 1024;
    int64_t SR = std::max<int64_t>(1, stage_target / rowbytes);
    if (SR > 4) SR = SR / 4 * 4;
    SR = std::min<int64_t>(SR, 32);
    int64_t S = ring / (SR * rowbytes);
    while (S < 2 && SR > 1) {
        SR = std::max<int64_t>(1, SR / 2);
        S = ring / (SR * rowbytes);
    }
    if (S < 2) return p;
    S = std::min<int64_t>(S, kTmaMaxStages);
    p.cw = cw;
    p.vpl = vpl;
    p.SR = (int)SR;
    p.S = (int)S;
    p.stage_bytes = (int)(SR * rowbytes);
    p.smem = (size_t)S * p.stage_bytes + (size_t)S * SR * cw * sizeof(float);
    p.ok = p.smem <= 200 * 1024;
    return p;
}

int launch_nk_tma(const TmaPlan &p, const void *dW, const float *dx, float *dy, int64_t m, int64_t k, int64_t n,
                  int wdtype, cudaStream_t stream) {
    Context &c = ctx();
    TmaFn fn = kTma[wdtype][p.cw == 16][p.vpl - 1];
    static bool attr_set[2][2][8] = {};
    if (!attr_set[wdtype][p.cw == 16][p.vpl - 1]) {
        DMC_CUDA_TRY(cudaFuncSetAttribute((const void *)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set[wdtype][p.cw == 16][p.vpl - 1] = true;
    }
    GemvTmaArgs a = {};
    a.W = dW;
    a.err = c.err_word;
    a.N = (int)n;
    a.K = (int)k;
    a.SR = p.SR;
    a.S = p.S;
    a.stage_bytes = p.stage_bytes;
    const int64_t per_sm = tuning().tma_ctas_per_sm > 0 ? tuning().tma_ctas_per_sm : 1;
    const int64_t grid = std::max<int64_t>(1, std::min<int64_t>(n, (int64_t)c.sm_count * per_sm));
    for (int64_t mi = 0; mi < m; ++mi) {
        a.x = dx + mi * k;
        a.y = dy + mi * n;
        void *params[] = {&a};
        int rc = launch_ex((const void *)fn, dim3((unsigned)grid), dim3((p.cw + 2) * 32), p.smem, stream, params);
        if (rc) return rc;
    }
    return DMC_CUDA_OK;
}

// Grid of the NK kernel: one row group per warp when the whole matrix then fits in one wave of
// resident CTAs (no warp idles, no CTA loops); otherwise exactly SMs x resident CTAs, every CTA
// owning the same share of the row groups (the kernel splits them evenly by block index).
int64_t nk_grid(int64_t n, int warps, int r, int sm_count, int cps, int reserve = 0, int even_rounds = 0) {
    const int64_t groups = (n + r - 1) / r;
    const int64_t exact = (groups + warps - 1) / warps;
    const int64_t slots = std::max<int64_t>(1, (int64_t)sm_count * cps - reserve);
    // (when the groups do not even fill one CTA per SM, one group per warp still wins: measured at
    // 4096x4096 with 8 rows of x, 64 full CTAs 10.8 us against 148 CTAs with idle warps 17.0 us)
    if (exact <= slots) return std::max<int64_t>(1, exact);
    // More groups than warps: with `slots` CTAs most warps own rounds - 1 groups and the rest own
    // `rounds`, and those finish the kernel with most of the machine idle.  When they are a minority,
    // fewer CTAs in which every warp owns (all but) exactly `rounds` groups are faster, although fewer
    // CTAs are resident (never below slots * (rounds - 1) / rounds; the stream needs ~8 MB in flight and
    // a CTA holds 64 KB).  Measured on B200, slots -> even, independent / dependent launches, us:
    //   14336x4096 (3 % of the warps own the extra group)  18.05 -> 17.09 / 20.48 -> 18.92
    //    6144x2048 (30 %)                                    5.22 ->  3.88 /  5.76 ->  5.80
    //   11264x2048 (38 %)                                    7.44 ->  6.95 /  9.10 ->  8.61
    //   11008x4096 (32 %)                                   14.04 -> 13.65 / 15.50 -> 15.67
    //    8192x8192 (73 %)                                   20.43 -> 20.65 / 21.73 -> 22.01
    //   32000x2048 (76 %)                                   19.38 -> 19.29 / 21.09 -> 20.84
    const int64_t warps_total = slots * warps;
    const int64_t rounds = (groups + warps_total - 1) / warps_total;
    const int64_t in_last_round = groups - (rounds - 1) * warps_total;  // warps that own `rounds` groups
    const bool even = even_rounds == 2 || (even_rounds == 1 && 2 * in_last_round < warps_total);
    if (!even) return slots;
    return std::min(slots, (groups + rounds * warps - 1) / (rounds * warps));
}

int launch_nk(const void *dW, const float *dx, float *dy, int64_t m, int64_t k, int64_t n,
              int wdtype, int variant, cudaStream_t stream) {
    Context &c = ctx();
    const int epv = wdtype == DMC_W_BF16 ? 8 : 4;
    const size_t xrow = (size_t)((k + 255) / 256 * 256 + 256) * sizeof(float);  // one staged row of x
    const bool vec_ok = k % epv == 0 && ((uintptr_t)dW % 16) == 0 && ((uintptr_t)dx % 16) == 0 &&
                        xrow <= kNkMaxSmem;
    if (c.pro) {
        if (!vec_ok || m != 1)
            return fail(DMC_CUDA_ERR_UNSUPPORTED, "gemv: fused prologue needs m == 1, k %% %d == 0 and aligned buffers", epv);
        if (variant < 0 || variant >= kNkCount) variant = default_nk_variant(k, n);
    }
    if (c.peer) {  // fused exchange lives in the vectorised LDG kernel only
        if (!vec_ok || m != 1)
            return fail(DMC_CUDA_ERR_UNSUPPORTED, "sharded gemv: needs m == 1, k %% %d == 0 and aligned buffers", epv);
        if (variant < 0 || variant >= kNkCount) variant = default_nk_variant(k, n);
    }
    if (variant < 0 && tuning().nk_default >= 0) variant = tuning().nk_default;
    if (variant == kTmaVariantCw8 || variant == kTmaVariantCw16) {
        TmaPlan p = plan_tma(k, n, wdtype, variant == kTmaVariantCw8 ? 8 : 16, dW, dx);
        if (p.ok) return launch_nk_tma(p, dW, dx, dy, m, k, n, wdtype, stream);
        variant = -1;  // shape outside the ring kernel: fall through to the LDG kernel
    }
    GemvArgs a = {};
    a.W = dW;
    a.K = (int)k;
    a.N = (int)n;
    a.ksplit = 1;
    if (!vec_ok) {
        a.x = dx;
        a.y = dy;
        int M = (int)m;
        void *params[] = {&a, &M};
        const void *fn = wdtype == DMC_W_BF16 ? (const void *)dmc_wrows_any_kernel<uint16_t>
                                              : (const void *)dmc_wrows_any_kernel<float>;
        return launch_ex(fn, dim3((unsigned)((n + 7) / 8)), dim3(256), 0, stream, params);
    }
    if (variant < 0 || variant >= kNkCount) variant = default_nk_variant(k, n);
    a.peer = static_cast<const PeerOut *>(c.peer);
    a.yoff = c.peer_yoff;
    a.peer_j = c.peer_j;
    a.pro = c.pro;
    a.pro_add = c.pro_add;
    a.pro_g = c.pro_g;
    a.pro_hout = c.pro_hout;
    a.pro_eps = c.pro_eps;
    a.amax = m == 1 ? c.amax : nullptr;
    // rows of x are taken up to 8 at a time (instances of 8, 4, 2 and 1 rows; 5-7 and 3 rows run in the
    // next larger instance with the missing rows staged as zeros); every instance streams W once
    for (int64_t m0 = 0; m0 < m;) {
        const int64_t left = m - m0;
        int M = left >= 5 ? 8 : left >= 3 ? 4 : left >= 2 ? 2 : 1;
        while (M > 1 && (size_t)M * xrow > kNkMaxSmem) M >>= 1;  // the staged rows must fit in shared memory
        const int mrows = (int)std::min<int64_t>(left, M);
        KernelFn fn;
        int warps, r;
        if (M == 1) {
            const NkVariant &v = kNk[variant];
            fn = wdtype == DMC_W_BF16 ? v.bf16 : v.f32;
            warps = v.WARPS, r = v.R;
        } else {
            const NkRows &v = kNkRows[M == 2 ? 0 : M == 4 ? 1 : 2];
            fn = wdtype == DMC_W_BF16 ? v.bf16 : v.f32;
            warps = v.WARPS, r = v.R;
        }
        const size_t smem = (size_t)M * xrow;
        static std::set<const void *> smem_raised;  // once per kernel instance
        if (!smem_raised.count((const void *)fn)) {
            DMC_CUDA_TRY(cudaFuncSetAttribute((const void *)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kNkMaxSmem));
            smem_raised.insert((const void *)fn);
        }
        // resident CTAs per SM of this instance with this much shared memory (registers decide: 1 or 2)
        static std::map<std::pair<const void *, size_t>, int> occupancy;
        auto key = std::make_pair((const void *)fn, smem);
        auto it = occupancy.find(key);
        if (it == occupancy.end()) {
            int blocks = 1;
            DMC_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, (const void *)fn, warps * 32, smem));
            it = occupancy.emplace(key, std::max(1, blocks)).first;
        }
        int cps = it->second;
        if (tuning().nk_ctas_per_sm > 0) cps = std::min(cps, tuning().nk_ctas_per_sm);
        a.x = dx + m0 * k;
        a.y = dy + m0 * n;
        a.mrows = mrows;
        // May this launch overlap what is still running?  Only if nothing it reads is being written
        // and nothing it writes is being read or written.
        const size_t xbytes = (size_t)mrows * k * 4 * (a.pro == 2 ? 2 : 1), hbytes = (size_t)k * 4;
        const size_t ybytes = a.peer ? 0 : (size_t)mrows * n * 4;  // (a sharded GEMV writes the replicas, which only the gather reads)
        // (a sharded GEMV's replica stores are ordered by the exchange protocol itself; the first of a
        // batch always waits: it follows the kernel that advances the epoch word)
        const bool conflict = (a.peer && (a.peer_j == 0 || !tuning().shard_overlap)) || a.amax || !tuning().overlap_independent || c.untracked_inflight ||
                              c.inflight_reads.size() + c.inflight_writes.size() > kMaxTrackedRanges ||
                              overlaps(c.inflight_writes, a.x, xbytes) || overlaps(c.inflight_writes, a.pro_add, hbytes) ||
                              overlaps(c.inflight_writes, a.y, ybytes) || overlaps(c.inflight_reads, a.y, ybytes) ||
                              overlaps(c.inflight_writes, a.pro_hout, hbytes) || overlaps(c.inflight_reads, a.pro_hout, hbytes);
        a.nowait = conflict ? 0 : 1;
        const int64_t grid = nk_grid(n, warps, r, c.sm_count, cps, a.peer ? kGatherCtas : 0, tuning().nk_even_rounds);
        void *params[] = {&a};
        int rc = launch_ex((const void *)fn, dim3((unsigned)grid), dim3(warps * 32), smem, stream, params,
                           conflict ? kLaunchTracked : kLaunchOverlap);
        if (rc) return rc;
        note(c.inflight_reads, a.x, xbytes);
        note(c.inflight_reads, a.pro_add, hbytes);
        note(c.inflight_writes, a.y, ybytes);
        note(c.inflight_writes, a.pro_hout, hbytes);
        m0 += mrows;
    }
    return DMC_CUDA_OK;
}

}  // namespace

// Time line of a chain of `count` bf16 GEMVs of one shape (W[n][k] copies in dWs), launched back to
// back in one CUDA graph with the default kernel configuration in its stamped instantiation.
// `dependent` != 0: every GEMV waits for its predecessor (as if it consumed its output); 0: none waits.
// stamps_out receives [count][grid][8] words (see GemvArgs::stamps); returns the grid size, < 0 on error.
int timeline_nk(const void *const *dWs, int count, const float *dx, float *dy, int64_t k, int64_t n, int dependent,
                unsigned long long *stamps_out, int64_t stamps_cap_words, cudaStream_t s) {
    Context &c = ctx();
    const size_t xrow = (size_t)((k + 255) / 256 * 256 + 256) * sizeof(float);
    if (k % 8 || xrow > kNkMaxSmem || count < 1)
        return -fail(DMC_CUDA_ERR_UNSUPPORTED, "timeline: needs k %% 8 == 0, a row of x that fits shared memory, count >= 1");
    const void *fn = (const void *)dmc_wrows_kernel<8, 2, 8, 1, uint16_t, true>;
    DMC_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kNkMaxSmem));
    const int64_t grid = nk_grid(n, 8, 2, c.sm_count, 2, 0, tuning().nk_even_rounds);
    if ((int64_t)count * grid * 8 > stamps_cap_words) return -fail(DMC_CUDA_ERR_BAD_ARG, "timeline: stamp buffer too small");
    unsigned long long *d_st = nullptr;
    const size_t bytes = (size_t)count * grid * 8 * sizeof(unsigned long long);
    DMC_CUDA_TRY(dmc_malloc((void **)&d_st, bytes));
    DMC_CUDA_TRY(cudaStreamSynchronize(s));
    stream_drained();
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int rc = DMC_CUDA_OK;
    cudaError_t e = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal);
    for (int i = 0; i < count && e == cudaSuccess && rc == DMC_CUDA_OK; ++i) {
        GemvArgs a = {};
        a.W = dWs[i], a.x = dx, a.y = dy, a.K = (int)k, a.N = (int)n, a.ksplit = 1;
        a.nowait = dependent ? 0 : 1;
        a.stamps = d_st + (size_t)i * grid * 8;
        void *params[] = {&a};
        rc = launch_ex(fn, dim3((unsigned)grid), dim3(256), xrow, s, params, kLaunchTracked);
    }
    if (e == cudaSuccess) e = cudaStreamEndCapture(s, &graph);
    stream_drained();
    if (e == cudaSuccess && rc == DMC_CUDA_OK) e = cudaGraphInstantiate(&exec, graph, 0);
    for (int rep = 0; rep < 4 && e == cudaSuccess && rc == DMC_CUDA_OK; ++rep) e = cudaGraphLaunch(exec, s);  // the last replay's stamps stay
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e == cudaSuccess) e = cudaMemcpy(stamps_out, d_st, bytes, cudaMemcpyDeviceToHost);
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    cudaFree(d_st);
    if (rc) return -rc;
    if (e != cudaSuccess) return -fail(DMC_CUDA_ERR_CUDA, "timeline: %s", cudaGetErrorString(e));
    return (int)grid;
}

bool nk_fast_eligible(int64_t k, int64_t n, int wdtype) {
    const int epv = wdtype == DMC_W_BF16 ? 8 : 4;
    return n >= 1 && k >= 512 && k % epv == 0 && (size_t)((k + 255) / 256 * 256 + 256) * sizeof(float) <= kNkMaxSmem;
}

int launch_transpose(const void *src, void *dst, int64_t rows, int64_t cols, int elem_bytes, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return DMC_CUDA_OK;
    dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64));
    if (grid.y > 65535) return fail(DMC_CUDA_ERR_UNSUPPORTED, "transpose: more than 4M rows");
    if (elem_bytes == 2)
        dmc_transpose_kernel<uint16_t><<<grid, 256, 0, stream>>>((const uint16_t *)src, (uint16_t *)dst, (int)rows, (int)cols);
    else
        dmc_transpose_kernel<uint32_t><<<grid, 256, 0, stream>>>((const uint32_t *)src, (uint32_t *)dst, (int)rows, (int)cols);
    DMC_CUDA_TRY(cudaGetLastError());
    ctx().launches++;
    return DMC_CUDA_OK;
}

int launch_gemv(const void *dW, const float *dx, float *dy, int64_t m, int64_t k, int64_t n,
                int64_t batch, int64_t ls, int64_t rs, int layout, int wdtype, int variant,
                cudaStream_t stream) {
    if (m <= 0 || n <= 0 || batch <= 0) return DMC_CUDA_OK;
    if (k < 0 || k > INT32_MAX || n > INT32_MAX || m > INT32_MAX)
        return fail(DMC_CUDA_ERR_BAD_ARG, "gemv: dimension out of range (m=%lld k=%lld n=%lld)",
                    (long long)m, (long long)k, (long long)n);
    if (wdtype != DMC_W_BF16 && wdtype != DMC_W_F32)
        return fail(DMC_CUDA_ERR_BAD_ARG, "gemv: unknown weight type %d", wdtype);
    if (k == 0) {  // empty contraction: the reference zeroes the row and adds nothing
        DMC_CUDA_TRY(cudaMemsetAsync(dy, 0, (size_t)batch * m * n * sizeof(float), stream));
        return DMC_CUDA_OK;
    }
    if (layout == DMC_LAYOUT_KN) return launch_kn(dW, dx, dy, m, k, n, batch, ls, rs, wdtype, variant, stream);
    if (layout == DMC_LAYOUT_NK) {
        if (batch != 1) return fail(DMC_CUDA_ERR_UNSUPPORTED, "gemv: batched NK layout is not offered");
        // A few activation rows stay on the CUDA cores, with the exact f32 rows of x (the multi-row
        // kernel streams W once for up to 8 rows).  From `tc_min_m` rows on the site is a real
        // contraction and goes to the tensor cores, where x enters as two bf16 terms (16 mantissa bits).
        const int min_m = tuning().tc_min_m > 0 ? tuning().tc_min_m : kTcMinRows;
        if (m >= min_m && wdtype == DMC_W_BF16 && variant < 0 && !ctx().peer && !ctx().pro && gemm_tc_eligible(m, k, n, dW, dx))
            return launch_gemm_tc_f32x(dW, dx, dy, m, k, n, stream);
        return launch_nk(dW, dx, dy, m, k, n, wdtype, variant, stream);
    }
    return fail(DMC_CUDA_ERR_BAD_ARG, "gemv: unknown layout %d", layout);
}

}  // namespace dmc

extern "C" int64_t dmc_cuda_row_kernel_grid(int64_t n, int warps, int rows_per_warp, int sm_count, int ctas_per_sm,
                                            int reserved_ctas, int even_rounds) {
    if (n < 1 || warps < 1 || rows_per_warp < 1 || sm_count < 1 || ctas_per_sm < 1 || reserved_ctas < 0) return 0;
    return dmc::nk_grid(n, warps, rows_per_warp, sm_count, ctas_per_sm, reserved_ctas, even_rounds);
}

extern "C" int dmc_cuda_variant_count(int layout, int wdtype) {
    (void)wdtype;
    return layout == DMC_LAYOUT_KN ? dmc::kKnCount : layout == DMC_LAYOUT_NK ? dmc::kNkTotal : 0;
}

extern "C" const char *dmc_cuda_variant_name(int layout, int wdtype, int variant) {
    (void)wdtype;
    if (layout == DMC_LAYOUT_KN && variant >= 0 && variant < dmc::kKnCount) return dmc::kKn[variant].name;
    if (layout == DMC_LAYOUT_NK && variant >= 0 && variant < dmc::kNkCount) return dmc::kNk[variant].name;
    if (layout == DMC_LAYOUT_NK && variant == dmc::kTmaVariantCw8) return "nk_tma_cw8";
    if (layout == DMC_LAYOUT_NK && variant == dmc::kTmaVariantCw16) return "nk_tma_cw16";
    return "";
}
