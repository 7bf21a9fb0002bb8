// gemm_tc.cuh -- bf16 GEMM on the 5th-generation tensor cores (tcgen05) for
//   Y[m][n] = sum_k X[m][k] * W[n][k]        (`X @ W'`, both operands K-contiguous, f32 out)
// used when an `@` site is a real contraction (several activation rows), where the
// CUDA-core GEMV would run out of FMA throughput before it runs out of HBM bandwidth.
//
// The weight is the MMA's M operand ("swap AB"): a CTA owns 128 rows of W and NB rows of
// X (NB = 16..256, the MMA N), so even a batch of 2 uses full 128-row MMAs and the weight
// stream, which dominates the bytes, is loaded exactly once.
//   warp 0   producer: TMA tiled loads (128-byte swizzle, no multicast) of a 128x64 W tile and
//            an NBx64 X tile per stage into an mbarrier ring
//   warp 1   allocates TMEM; one elected thread issues tcgen05.mma (4 per stage, K = 16 each),
//            accumulating in TMEM; tcgen05.commit hands each stage back to the producer
//   warps 2-5 epilogue: tcgen05.ld the 128 x NB f32 accumulator out of TMEM and store it
// Few W tiles (small n) are spread over more SMs by splitting K across CTAs; partial tiles
// meet in a scratch buffer and the last CTA adds them in a fixed order.
// Every wait is bounded; a wait that runs out sets an error word, and the CTA still frees
// its TMEM before leaving.
#pragma once
#include "gemv.cuh"
#include "tc_ptx.cuh"

namespace dmc {

constexpr int kTcBM = 128;     // W rows per CTA
constexpr int kTcBK = 64;      // K per stage: one 128-byte swizzle atom of bf16
constexpr int kTcMaxStages = 10;
constexpr int kTcWTileBytes = kTcBM * kTcBK * 2;

struct GemmTcArgs {
    float *y;            // [m][n]
    float *partial;      // [ksplit][m][n] when ksplit > 1
    unsigned *counters;  // one per (row tile, batch tile), zero between launches
    int *err;
    int m;               // logical activation rows (output rows)
    int n, k;
    int kblocks_per_split, ksplit;
    int stages;
    int pair;            // 1: X rows come as (hi, lo) pairs, output row j = column 2j + column 2j+1
};

template <int NB>
__global__ void __launch_bounds__(192, 1)
dmc_tc_contract_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const GemmTcArgs a) {
    constexpr int XTILE = NB * kTcBK * 2;
    constexpr int STAGE = kTcWTileBytes + XTILE;
    constexpr uint32_t TMEM_COLS = NB < 32 ? 32 : NB;
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint64_t full[kTcMaxStages], empty[kTcMaxStages], done;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s, s_last;

    unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = a.stages;
    const int tile_n = blockIdx.x, ky = blockIdx.y, tile_m = blockIdx.z;
    const int kblocks_total = (a.k + kTcBK - 1) / kTcBK;
    const int kb0 = ky * a.kblocks_per_split;
    const int nkb = max(0, min(a.kblocks_per_split, kblocks_total - kb0));

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(&done, 1);
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        tc::prefetch_tensormap(&map_w);
        tc::prefetch_tensormap(&map_x);
    }
    if (warp == 1) tc::tmem_alloc(&tmem_base_s, TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = tmem_base_s;

    griddep_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            // The weights never depend on an earlier kernel: their first ring-full of tiles is
            // requested before the programmatic-dependency wait; X (which may) only after it.
            const int pre = min(S, nkb);
            for (int i = 0; i < pre; ++i) {
                mbar_expect_tx(&full[i], STAGE);
                tc::tma_load_2d(smem + (size_t)i * STAGE, &map_w, (kb0 + i) * kTcBK, tile_n * kTcBM, &full[i]);
            }
            griddep_wait();
            for (int i = 0; i < pre; ++i)
                tc::tma_load_2d(smem + (size_t)i * STAGE + kTcWTileBytes, &map_x, (kb0 + i) * kTcBK, tile_m * NB, &full[i]);
            for (int i = pre; i < nkb; ++i) {
                const int s = i % S;
                if (!mbar_wait(&empty[s], ((i / S) - 1) & 1)) {
                    *(volatile int *)a.err = 4;
                    abort_s = 1;
                    break;
                }
                unsigned char *st = smem + (size_t)s * STAGE;
                mbar_expect_tx(&full[s], STAGE);
                tc::tma_load_2d(st, &map_w, (kb0 + i) * kTcBK, tile_n * kTcBM, &full[s]);
                tc::tma_load_2d(st + kTcWTileBytes, &map_x, (kb0 + i) * kTcBK, tile_m * NB, &full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::instr_desc_bf16_f32(kTcBM, NB);
            bool ok = true;
            for (int i = 0; i < nkb && ok; ++i) {
                const int s = i % S;
                if (!mbar_wait(&full[s], (i / S) & 1)) {
                    *(volatile int *)a.err = 5;
                    abort_s = 1;
                    ok = false;
                    break;
                }
                tc::fence_after_sync();
                const uint32_t wa = smem_u32(smem + (size_t)s * STAGE);
                const uint32_t xa = wa + kTcWTileBytes;
#pragma unroll
                for (int kk = 0; kk < kTcBK / 16; ++kk)  // 16 bf16 = 32 bytes along K inside the swizzle atom
                    tc::mma_bf16(tmem_base, tc::smem_desc_k_sw128(wa + kk * 32), tc::smem_desc_k_sw128(xa + kk * 32),
                                 idesc, (i > 0 || kk > 0) ? 1u : 0u);
                tc::mma_commit(&empty[s]);  // stage is free once these MMAs have read it
            }
            if (ok) tc::mma_commit(&done);
        }
    } else {
        // ---- epilogue: TMEM -> registers -> global ----
        const int q = warp & 3;                 // a warp may only touch TMEM lanes 32*(warpid % 4) ..
        const int row = q * 32 + lane;          // accumulator row = W row inside the tile
        const int n = tile_n * kTcBM + row;
        bool ok = nkb > 0;
        griddep_wait();  // y / the split-K scratch may still be in use by the previous kernel
        if (ok && !mbar_wait(&done, 0)) {
            *(volatile int *)a.err = 6;
            abort_s = 1;
            ok = false;
        }
        tc::fence_after_sync();
        const int div = a.pair ? 2 : 1;
        float *dst = a.ksplit == 1 ? a.y : a.partial + (size_t)ky * a.m * a.n;
#pragma unroll 1
        for (int c0 = 0; c0 < NB; c0 += 16) {
            uint32_t r[16];
            if (ok) {
                tc::tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
                tc::tmem_ld_wait();
            } else {
#pragma unroll
                for (int t = 0; t < 16; ++t) r[t] = 0u;  // empty K range: the tile is zero
            }
            if (n < a.n) {
#pragma unroll
                for (int t = 0; t < 16; t += 1) {
                    float v = __uint_as_float(r[t]);
                    if (a.pair) {
                        if (t & 1) continue;
                        v += __uint_as_float(r[t + 1]);
                    }
                    const int mj = (tile_m * NB + c0 + t) / div;
                    if (mj < a.m) dst[(size_t)mj * a.n + n] = v;
                }
            }
        }
    }

    // ---- split-K: the CTA that arrives last adds the partial tiles in a fixed order ----
    if (a.ksplit > 1) {
        __threadfence();
        __syncthreads();
        const int group = tile_m * gridDim.x + tile_n;
        if (tid == 0) s_last = (atomicAdd(&a.counters[group], 1u) == (unsigned)a.ksplit - 1u);
        __syncthreads();
        if (s_last) {
            __threadfence();
            const int div = a.pair ? 2 : 1;
            const int m0 = tile_m * NB / div, m1 = min(a.m, (tile_m + 1) * NB / div);
            const int n0 = tile_n * kTcBM, nn = min(kTcBM, a.n - n0);
            const size_t slab = (size_t)a.m * a.n;  // one split's partial matrix
            if ((a.n & 3) == 0 && (nn & 3) == 0) {
                // 128-bit loads, eight splits in flight per thread, summed in split order
                const int nv = nn >> 2;
                for (int idx = tid; idx < (m1 - m0) * nv; idx += blockDim.x) {
                    const size_t off = (size_t)(m0 + idx / nv) * a.n + n0 + (size_t)(idx % nv) * 4;
                    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int j0 = 0; j0 < a.ksplit; j0 += 8) {
                        float4 v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            v[j] = (j0 + j < a.ksplit)
                                       ? __ldcg(reinterpret_cast<const float4 *>(a.partial + (size_t)(j0 + j) * slab + off))
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            s.x += v[j].x;
                            s.y += v[j].y;
                            s.z += v[j].z;
                            s.w += v[j].w;
                        }
                    }
                    *reinterpret_cast<float4 *>(a.y + off) = s;
                }
            } else {
                for (int idx = tid; idx < (m1 - m0) * nn; idx += blockDim.x) {
                    const int mj = m0 + idx / nn, n = n0 + idx % nn;
                    float s = 0.0f;
                    for (int j = 0; j < a.ksplit; ++j) s += __ldcg(&a.partial[(size_t)j * slab + (size_t)mj * a.n + n]);
                    a.y[(size_t)mj * a.n + n] = s;
                }
            }
            if (tid == 0) a.counters[group] = 0u;
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem_base, TMEM_COLS);
}

// f32 activations -> (hi, lo) bf16 row pairs, so the tensor cores see x to 16 mantissa bits:
// row 2j = bf16(x_j) and row 2j+1 = bf16(x_j - hi), both round-to-nearest-even.
__global__ void __launch_bounds__(256) dmc_split_x_kernel(const float *__restrict__ x, uint16_t *__restrict__ xs, int m,
                                                      int k) {
    const long long total = (long long)m * k;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int j = (int)(i / k), c = (int)(i % k);
        const float v = x[i];
        auto rne = [](float f) -> uint32_t {
            uint32_t u = __float_as_uint(f);
            return (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
        };
        const uint32_t hi = rne(v);
        const float rem = v - __uint_as_float(hi << 16);
        xs[(size_t)(2 * j) * k + c] = (uint16_t)hi;
        xs[(size_t)(2 * j + 1) * k + c] = (uint16_t)rne(rem);
    }
}

}  // namespace dmc
