// gemv_tma.cuh -- the bandwidth kernel: NK-layout GEMV fed by bulk asynchronous
// copies (TMA, `cp.async.bulk`) into a shared-memory ring.
//
//   y[n] = sum_k W[n][k] * x[k]      W bf16 or f32, K contiguous; x, y f32
//
// One CTA per SM owns a contiguous block of rows, i.e. one contiguous byte range
// of W, so every copy is a plain 1-D bulk copy of whole rows: no tensor map, no
// cluster, no multicast.  A producer warp keeps S stages of SR rows in flight
// (the bytes in flight live in shared memory, not in registers, so the ring can
// hold ~100 KB per SM -- more than the bandwidth-delay product of HBM3e).  The
// weights never depend on an earlier kernel, so the producer starts copying
// before the programmatic-dependency wait: in a chain of GEMVs the next
// kernel's first stages load while the previous kernel drains.
//
// Consumers: CW warps.  A lane keeps its slice of x in registers for the whole
// kernel (x is read once per CTA: lane l of warp w owns the 16-byte vectors
// v = i*CW*32 + w*32 + l of every row), reads W from shared memory with
// conflict-free 128-bit loads, and reduces four rows at a time with a shared
// butterfly.  Per stage the CW warp partials meet in shared memory; a reducer warp
// adds them in a fixed order (results do not vary run to run), stores y and hands
// the stage back to the producer, so the consumers never wait on one another.
// (Measured on B200 it reaches 4.5-6.0 TB/s, behind the LDG kernel of gemv.cuh on the
// decode shapes, which therefore stays the default; this one is selectable as a variant.)
//
// Every wait is bounded: a wait that runs out records a code in *err and the
// CTA leaves; nothing spins forever.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemv.cuh"

namespace dmc {

struct GemvTmaArgs {
    const void *W;
    const float *x;
    float *y;
    int *err;            // device-visible error word (0 = ok)
    int N, K;
    int SR;              // rows per stage
    int S;               // stages
    int stage_bytes;     // SR * K * sizeof(W), multiple of 16
};

constexpr int kTmaMaxStages = 12;
constexpr long long kSpinCycles = 1LL << 31;  // ~1 s at B200 clocks

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *b, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *b, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(b)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint64_t *b, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(b)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false when the limit ran out.  Polls with the non-blocking test_wait: the
// potentially-blocking try_wait parks the thread for a scheduler-defined interval, which a
// pipeline whose stages last well under a microsecond cannot afford.
__device__ __forceinline__ bool mbar_wait(uint64_t *b, uint32_t parity) {
    if (mbar_test_wait(b, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_test_wait(b, parity)) return true;
        if (clock64() - t0 > kSpinCycles) return false;
    }
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Dynamic shared memory: S*stage_bytes (ring) + S*SR*CW floats (warp partials).
// Warps: CW consumers, one reducer (warp CW), one producer (warp CW+1).
template <int VPL, int CW, typename WT>
__global__ void __launch_bounds__((CW + 2) * 32, 1) dmc_wrows_ring_kernel(const GemvTmaArgs a) {
    constexpr int EPV = VecOf<WT>::EPV;
    constexpr int RU = 4;  // rows reduced together
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint64_t full[kTmaMaxStages], empty[kTmaMaxStages], done[kTmaMaxStages];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int N = a.N, K = a.K, S = a.S, SR = a.SR;
    const int nvec = K / EPV;
    const size_t rowbytes = (size_t)K * sizeof(WT);
    float *part = reinterpret_cast<float *>(smem + (size_t)S * a.stage_bytes);

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
            mbar_init(&done[s], CW);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // balanced contiguous row block of this CTA
    const int r0 = (int)(((long long)N * blockIdx.x) / gridDim.x);
    const int r1 = (int)(((long long)N * (blockIdx.x + 1)) / gridDim.x);
    const int nchunks = (r1 - r0 + SR - 1) / SR;

    griddep_launch_dependents();

    if (warp == CW + 1) {  // ---- producer: never waits for the previous kernel, weights are constant ----
        if (lane == 0) {
            const unsigned char *Wb = reinterpret_cast<const unsigned char *>(a.W);
            for (int c = 0; c < nchunks; ++c) {
                const int s = c % S;
                if (c >= S && !mbar_wait(&empty[s], ((c / S) - 1) & 1)) {
                    *(volatile int *)a.err = 1;
                    break;
                }
                const int row0 = r0 + c * SR;
                const int rows = min(SR, r1 - row0);
                const uint32_t bytes = (uint32_t)(rows * rowbytes);
                mbar_expect_tx(&full[s], bytes);
                const unsigned char *src = Wb + (size_t)row0 * rowbytes;
                unsigned char *dst = smem + (size_t)s * a.stage_bytes;
                for (uint32_t off = 0; off < bytes; off += 32768u)
                    bulk_g2s(dst + off, src + off, min(32768u, bytes - off), &full[s]);
            }
        }
        return;
    }

    if (warp == CW) {  // ---- reducer: adds the CW partials of each row in a fixed order, stores y ----
        griddep_wait();  // y may still be read by the previous kernel
        for (int c = 0; c < nchunks; ++c) {
            const int s = c % S;
            if (!mbar_wait(&done[s], (c / S) & 1)) {
                *(volatile int *)a.err = 7;
                return;
            }
            const int row0 = r0 + c * SR;
            const int rows = min(SR, r1 - row0);
            const float *spart = part + (size_t)s * SR * CW;
            for (int r = lane; r < rows; r += 32) {
                float sum = 0.0f;
#pragma unroll
                for (int w = 0; w < CW; ++w) sum += spart[r * CW + w];
                a.y[row0 + r] = sum;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);  // ring slot and its partials are free again
        }
        return;
    }

    // ---- consumers ----
    griddep_wait();  // x may be produced by the previous kernel in the stream
    float xr[VPL][8];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int v = i * (CW * 32) + warp * 32 + lane;
        if (v < nvec) {
            const float4 *xp = reinterpret_cast<const float4 *>(a.x + (size_t)v * EPV);
            float4 lo = __ldcg(xp);
            xr[i][0] = lo.x, xr[i][1] = lo.y, xr[i][2] = lo.z, xr[i][3] = lo.w;
            if constexpr (EPV == 8) {
                float4 hi = __ldcg(xp + 1);
                xr[i][4] = hi.x, xr[i][5] = hi.y, xr[i][6] = hi.z, xr[i][7] = hi.w;
            } else {
                xr[i][4] = xr[i][5] = xr[i][6] = xr[i][7] = 0.0f;
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) xr[i][e] = 0.0f;
        }
    }

    for (int c = 0; c < nchunks; ++c) {
        const int s = c % S;
        if (!mbar_wait(&full[s], (c / S) & 1)) {
            *(volatile int *)a.err = 2;
            return;
        }
        const int rows = min(SR, r1 - (r0 + c * SR));
        const unsigned char *stage = smem + (size_t)s * a.stage_bytes;
        float *spart = part + (size_t)s * SR * CW;

        for (int rb = 0; rb < rows; rb += RU) {
            float acc[RU];
#pragma unroll
            for (int j = 0; j < RU; ++j) acc[j] = 0.0f;
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int v = i * (CW * 32) + warp * 32 + lane;
                // all loads of the batch first (rows past the chunk / vectors past the row read a
                // valid address and are discarded), then the arithmetic
                const int vv = v < nvec ? v : 0;
                uint4 wv[RU];
#pragma unroll
                for (int j = 0; j < RU; ++j) {
                    const int rj = rb + j < rows ? rb + j : rb;
                    wv[j] = *reinterpret_cast<const uint4 *>(stage + (size_t)rj * rowbytes + (size_t)vv * 16);
                }
                const float4 xa = make_float4(xr[i][0], xr[i][1], xr[i][2], xr[i][3]);
                const float4 xb = make_float4(xr[i][4], xr[i][5], xr[i][6], xr[i][7]);
                if (v < nvec) {
#pragma unroll
                    for (int j = 0; j < RU; ++j) acc[j] = dot_vec<WT>(acc[j], wv[j], xa, xb);
                }
            }
            // butterfly over 4 rows: 6 shuffles instead of 20
            const bool h16 = lane & 16;
            float k0 = h16 ? acc[2] : acc[0], s0 = h16 ? acc[0] : acc[2];
            float k1 = h16 ? acc[3] : acc[1], s1 = h16 ? acc[1] : acc[3];
            k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
            k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
            const bool h8 = lane & 8;
            float kk = h8 ? k1 : k0, ss = h8 ? k0 : k1;
            kk += __shfl_xor_sync(0xffffffffu, ss, 8);
            kk += __shfl_xor_sync(0xffffffffu, kk, 4);
            kk += __shfl_xor_sync(0xffffffffu, kk, 2);
            kk += __shfl_xor_sync(0xffffffffu, kk, 1);
            const int rr = rb + ((lane >> 4) << 1) + ((lane >> 3) & 1);
            if ((lane & 7) == 0 && rr < rows) spart[rr * CW + warp] = kk;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&done[s]);  // release: the reducer's wait sees this warp's partials
    }
}

// 64x64-tiled transpose of 16- or 32-bit elements: src[rows][cols] -> dst[cols][rows].
// Runs once per resident weight (the device-side counterpart of the reference's
// `dmc_bf16_transpose_2d`, compiler/src/jit.rs:29801-29834; bit patterns preserved).
template <typename T>
__global__ void __launch_bounds__(256) dmc_transpose_kernel(const T *__restrict__ src, T *__restrict__ dst, int rows,
                                                         int cols) {
    __shared__ T tile[64][64 + 2];
    const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;  // 64 x 4
    for (int i = ty; i < 64; i += 4) {
        const int r = r0 + i, c = c0 + tx;
        if (r < rows && c < cols) tile[i][tx] = src[(size_t)r * cols + c];
    }
    __syncthreads();
    for (int i = ty; i < 64; i += 4) {
        const int c = c0 + i, r = r0 + tx;
        if (r < rows && c < cols) dst[(size_t)c * rows + r] = tile[tx][i];
    }
}

}  // namespace dmc
