// gemv.cuh -- memory-bound weight-streaming GEMV kernels for sm_100a.
//
// Two weight layouts:
//   KN  W[k][n], n contiguous  (`x @ W`; what the reference's builtins receive:
//       compiler/src/gpu.rs:397-399, kernel analogue compiler/src/gpu.rs:115-153)
//   NK  W[n][k], k contiguous  (`x @ W'` consumed without the transpose pass of
//       compiler/src/jit.rs:29801-29834)
// Weights are bf16 bit patterns (widen = bits << 16, compiler/src/jit.rs:29224-29227)
// or f32; activations and outputs are f32; accumulation is f32 FMA.  The
// summation order differs from the reference's ascending-k chain (split across
// lanes / warps / CTAs), which the reference allows for its own GPU path
// ("within f32 reduction-order tolerance", compiler/src/gpu.rs:35-37).
//
// Every weight byte is read exactly once with 128-bit streaming loads that
// bypass L1; algorithmic traffic per GEMV is n*k*sizeof(W) + 4k + 4n bytes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "peer.cuh"

namespace dmc {

struct GemvArgs {
    const void *W;       // weights, layout per kernel
    const float *x;      // activations [M][K] (+ z*ls per batch slice)
    float *y;            // outputs [M][N] (+ z*M*N per batch slice)
    float *partial;      // split-K scratch [batch][ksplit][M][N]
    unsigned *counters;  // split-K arrival counters [batch][colblocks], zero between launches
    int K, N;
    int kchunk, ksplit;  // KN: rows of k per CTA along grid.y
    int colblocks;       // KN: CTAs along n per batch slice
    long long ls, rs;    // batch strides in elements (x: f32, W: weight elements)
    // NK kernel: 1 = nothing this launch reads or writes is touched by a kernel that may still be
    // running, so the programmatic-dependency wait is skipped and the launch overlaps its
    // predecessors freely (set by the launch planner, never by a caller)
    int nowait;
    int mrows;           // NK kernel with M > 1: rows of x actually present (1..M); the others are staged as zeros
    const PeerOut *peer; // NK kernel, sharded path: store y into every rank's replica (else null)
    long long yoff;      // first row of this rank's slice within the replicated y
    int peer_j;          // position of this exchange in the current batch of launches
    // NK kernel: an elementwise op applied to x while it is staged into shared memory (0 = none)
    //   1  x = rms_norm(x + add) * g; CTA 0 also stores the sum x + add to hout (the residual stream)
    //   2  x[i] = silu(x[i]) * x[K + i]  (SwiGLU over a [gate | up] vector of 2K floats)
    int pro;
    const float *pro_add, *pro_g;
    float *pro_hout;
    float pro_eps;
    // NK kernel, M == 1: if non-null, the arg-max of y is folded into the kernel.  The word receives,
    // by atomic maximum, (order-preserving bits of the value) << 32 | (0xFFFFFFFF - row): the greatest
    // value wins and, among equal values, the lowest row -- the reference's first strict maximum
    // (compiler/src/interp.rs:13529-13538).  The caller zeroes it beforehand.
    unsigned long long *amax;
    // Time-line instantiation only (STAMP = true): per CTA {kernel entry, wait returned, x staged,
    // first row group done, last row group done} in globaltimer nanoseconds, plus the SM id.
    unsigned long long *stamps;
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Order-preserving map f32 -> u32 (greater float <=> greater unsigned) and the packed arg-max key.
__device__ __forceinline__ unsigned long long amax_key(float v, int row) {
    const unsigned u = __float_as_uint(v);
    const unsigned ord = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)ord << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)row);
}

// ---- small device helpers ---------------------------------------------------

__device__ __forceinline__ uint4 ldg_stream16(const void *p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p));
    return v;
}

// Programmatic dependent launch: everything before the wait (address setup and
// the first weight loads, which no earlier kernel writes) overlaps the tail of
// the previous kernel in the stream; x is only read after it.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ float bf16lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

template <typename WT> struct VecOf;
template <> struct VecOf<uint16_t> { static constexpr int EPV = 8; };
template <> struct VecOf<float> { static constexpr int EPV = 4; };

// acc[e] += x * w[e] over the EPV elements of one 16-byte vector (KN layout).
template <typename WT>
__device__ __forceinline__ void axpy_vec(float *acc, const uint4 &w, float xv) {
    if constexpr (sizeof(WT) == 2) {
        acc[0] = fmaf(xv, bf16lo(w.x), acc[0]);
        acc[1] = fmaf(xv, bf16hi(w.x), acc[1]);
        acc[2] = fmaf(xv, bf16lo(w.y), acc[2]);
        acc[3] = fmaf(xv, bf16hi(w.y), acc[3]);
        acc[4] = fmaf(xv, bf16lo(w.z), acc[4]);
        acc[5] = fmaf(xv, bf16hi(w.z), acc[5]);
        acc[6] = fmaf(xv, bf16lo(w.w), acc[6]);
        acc[7] = fmaf(xv, bf16hi(w.w), acc[7]);
    } else {
        acc[0] = fmaf(xv, __uint_as_float(w.x), acc[0]);
        acc[1] = fmaf(xv, __uint_as_float(w.y), acc[1]);
        acc[2] = fmaf(xv, __uint_as_float(w.z), acc[2]);
        acc[3] = fmaf(xv, __uint_as_float(w.w), acc[3]);
    }
}

// The EPV elements of one 16-byte weight vector, widened to f32.
template <typename WT>
__device__ __forceinline__ void widen_vec(const uint4 &w, float (&f)[8]) {
    if constexpr (sizeof(WT) == 2) {
        f[0] = bf16lo(w.x), f[1] = bf16hi(w.x), f[2] = bf16lo(w.y), f[3] = bf16hi(w.y);
        f[4] = bf16lo(w.z), f[5] = bf16hi(w.z), f[6] = bf16lo(w.w), f[7] = bf16hi(w.w);
    } else {
        f[0] = __uint_as_float(w.x), f[1] = __uint_as_float(w.y), f[2] = __uint_as_float(w.z), f[3] = __uint_as_float(w.w);
        f[4] = f[5] = f[6] = f[7] = 0.0f;
    }
}

// acc += dot(w[0..EPV), x[0..EPV)) (NK layout); xa holds x[0..4), xb x[4..8).
template <typename WT>
__device__ __forceinline__ float dot_vec(float acc, const uint4 &w, const float4 &xa, const float4 &xb) {
    if constexpr (sizeof(WT) == 2) {
        acc = fmaf(xa.x, bf16lo(w.x), acc);
        acc = fmaf(xa.y, bf16hi(w.x), acc);
        acc = fmaf(xa.z, bf16lo(w.y), acc);
        acc = fmaf(xa.w, bf16hi(w.y), acc);
        acc = fmaf(xb.x, bf16lo(w.z), acc);
        acc = fmaf(xb.y, bf16hi(w.z), acc);
        acc = fmaf(xb.z, bf16lo(w.w), acc);
        acc = fmaf(xb.w, bf16hi(w.w), acc);
    } else {
        acc = fmaf(xa.x, __uint_as_float(w.x), acc);
        acc = fmaf(xa.y, __uint_as_float(w.y), acc);
        acc = fmaf(xa.z, __uint_as_float(w.z), acc);
        acc = fmaf(xa.w, __uint_as_float(w.w), acc);
    }
    return acc;
}

// Split-K epilogue: the CTA that arrives last at the group's counter adds the
// partials in a fixed order (so results do not vary from run to run), writes y
// and re-arms the counter for the next launch.
//   partial index: ((z*ksplit + j)*M + m)*N + col
template <int THREADS>
__device__ __forceinline__ void splitk_finish(const GemvArgs &a, int z, int group, int M, int col0,
                                              int ncols, int *s_last) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned t = atomicAdd(&a.counters[group], 1u);
        *s_last = (t == (unsigned)a.ksplit - 1u);
    }
    __syncthreads();
    if (!*s_last) return;
    __threadfence();
    for (int m = 0; m < M; ++m) {
        for (int c = threadIdx.x; c < ncols; c += THREADS) {
            int col = col0 + c;
            if (col >= a.N) continue;
            float s = 0.0f;
            for (int j = 0; j < a.ksplit; ++j)
                s += __ldcg(&a.partial[(((size_t)z * a.ksplit + j) * M + m) * a.N + col]);
            a.y[((size_t)z * M + m) * a.N + col] = s;
        }
    }
    if (threadIdx.x == 0) a.counters[group] = 0u;
}

// ---- KN layout ----------------------------------------------------------------
//
// CTA = TK warps over the same CW = 32*V*EPV columns; the warps interleave over
// the k rows of the CTA's k range (grid.y splits K), U rows in flight per warp.
// Per row a warp reads V contiguous 512-byte segments.  Warp partials meet in
// shared memory; CTA partials of a split K meet in `partial` (splitk_finish).
// grid.x = colblocks * batch, grid.y = ksplit.  Needs N % EPV == 0, rs % EPV == 0
// and a 16-byte aligned W.
// NR > 1 is the form for narrow matrices (per-head projections with n = 128 or 64): a warp-wide load
// covers NR consecutive k rows of 32/NR vectors each instead of one row of 32, so no lane idles; the NR
// partial rows meet by shuffle at the end.
template <int TK, int U, int V, int M, typename WT, int NR = 1>
__global__ void __launch_bounds__(TK * 32) dmc_wcols_kernel(const GemvArgs a) {
    constexpr int EPV = VecOf<WT>::EPV;
    constexpr int LPR = 32 / NR;           // lanes per k row
    constexpr int CW = LPR * V * EPV;
    constexpr int THREADS = TK * 32;
    static_assert(NR == 1 || NR == 2 || NR == 4, "rows per warp-wide load");
    __shared__ __align__(16) float red[TK][CW];
    __shared__ int s_last;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lcol = lane % LPR, sub = lane / LPR;  // position within a k row, and which of the NR rows
    const int cb = blockIdx.x % a.colblocks, z = blockIdx.x / a.colblocks;
    const int K = a.K, N = a.N;
    const WT *Wz = (const WT *)a.W + (size_t)z * a.rs;
    const float *xz = a.x + (size_t)z * a.ls;
    const int kbeg = blockIdx.y * a.kchunk;
    const int kend = (int)min((long long)K, (long long)kbeg + a.kchunk);  // 64-bit: kbeg + kchunk may pass 2^31

    int col[V];
    bool cok[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
        col[v] = cb * CW + (v * LPR + lcol) * EPV;
        cok[v] = col[v] < N;
    }

    float acc[M][V][EPV];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int v = 0; v < V; ++v)
#pragma unroll
            for (int e = 0; e < EPV; ++e) acc[m][v][e] = 0.0f;

    uint4 w[U][V];
    auto load_w = [&](int k) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int kk = k + u * TK * NR;
#pragma unroll
            for (int v = 0; v < V; ++v)
                w[u][v] = (kk < kend && cok[v]) ? ldg_stream16(Wz + (size_t)kk * N + col[v])
                                                : make_uint4(0, 0, 0, 0);
        }
    };
    auto consume = [&](int k) {
        float xv[M][U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int kk = k + u * TK * NR;
#pragma unroll
            for (int m = 0; m < M; ++m) xv[m][u] = kk < kend ? __ldcg(xz + (size_t)m * K + kk) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int m = 0; m < M; ++m)
#pragma unroll
                for (int v = 0; v < V; ++v) axpy_vec<WT>(acc[m][v], w[u][v], xv[m][u]);
    };

    int k = kbeg + warp * NR + sub;
    if (k < kend) load_w(k);
    griddep_launch_dependents();
    griddep_wait();
    if (k < kend) {
        consume(k);
        k += TK * U * NR;
    }
    for (; k < kend; k += TK * U * NR) {
        load_w(k);
        consume(k);
    }
    if constexpr (NR > 1) {  // the NR partial rows of a warp meet in its first LPR lanes
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
            for (int v = 0; v < V; ++v)
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    float s = acc[m][v][e];
                    s += __shfl_xor_sync(0xffffffffu, s, 16);
                    if constexpr (NR == 4) s += __shfl_xor_sync(0xffffffffu, s, 8);
                    acc[m][v][e] = s;
                }
    }

    // warps -> CTA, one x row at a time (keeps shared memory at TK*CW floats)
#pragma unroll
    for (int m = 0; m < M; ++m) {
        if (m) __syncthreads();
#pragma unroll
        for (int v = 0; v < V; ++v) {
            if (sub == 0) {
                float4 *dst = reinterpret_cast<float4 *>(&red[warp][(v * LPR + lcol) * EPV]);
                dst[0] = make_float4(acc[m][v][0], acc[m][v][1], acc[m][v][2], acc[m][v][3]);
                if constexpr (EPV == 8)
                    dst[1] = make_float4(acc[m][v][4], acc[m][v][5], acc[m][v][6], acc[m][v][7]);
            }
        }
        __syncthreads();
        for (int c = threadIdx.x; c < CW; c += THREADS) {
            const int cc = cb * CW + c;
            if (cc >= N) continue;
            float s = 0.0f;
#pragma unroll
            for (int t = 0; t < TK; ++t) s += red[t][c];
            if (a.ksplit == 1)
                a.y[((size_t)z * M + m) * N + cc] = s;
            else
                a.partial[(((size_t)z * a.ksplit + blockIdx.y) * M + m) * N + cc] = s;
        }
    }
    if (a.ksplit > 1) splitk_finish<THREADS>(a, z, z * a.colblocks + cb, M, cb * CW, CW, &s_last);
}

// Any-shape fallback (odd n, unaligned strides): one column per thread, the
// TK warps of a CTA split k, partials meet in shared memory.  Not a bandwidth
// kernel; it exists so no shape ever leaves the GPU.  Reference analogue:
// `gemv_bf16_tiled2d`, compiler/src/gpu.rs:158-183.
template <int TK, typename WT>
__global__ void __launch_bounds__(TK * 32) dmc_wcols_any_kernel(const GemvArgs a, int M) {
    __shared__ float red[TK][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cb = blockIdx.x % a.colblocks, z = blockIdx.x / a.colblocks;
    const int n = cb * 32 + lane;
    const WT *Wz = (const WT *)a.W + (size_t)z * a.rs;
    const float *xz = a.x + (size_t)z * a.ls;
    griddep_wait();
    for (int m = 0; m < M; ++m) {
        float acc = 0.0f;
        if (n < a.N) {
            for (int k = warp; k < a.K; k += TK) {
                float wv;
                if constexpr (sizeof(WT) == 2)
                    wv = __uint_as_float((uint32_t)Wz[(size_t)k * a.N + n] << 16);
                else
                    wv = Wz[(size_t)k * a.N + n];
                acc = fmaf(__ldcg(xz + (size_t)m * a.K + k), wv, acc);
            }
        }
        if (m) __syncthreads();
        red[warp][lane] = acc;
        __syncthreads();
        if (warp == 0 && n < a.N) {
            float s = 0.0f;
#pragma unroll
            for (int t = 0; t < TK; ++t) s += red[t][lane];
            a.y[((size_t)z * M + m) * a.N + n] = s;
        }
    }
}

// ---- NK layout ----------------------------------------------------------------
//
// The M rows of x (M = 1 for a GEMV; 2, 4 or 8 for a small batch, which shares
// every weight load among its rows) are staged once per CTA in shared memory,
// each row permuted so that a lane's two float4 reads are conflict-free.  A CTA
// owns a contiguous block of row groups (R adjacent weight rows each) and deals
// them to its warps; a warp streams a group with U 16-byte loads in flight per
// row, keeps R*M accumulators and reduces across lanes with shuffles.  The grid
// is either one group per warp (when that fits in one wave) or exactly
// SMs x resident CTAs, every CTA with the same share of the rows.
// Needs K % EPV == 0 and a 16-byte aligned W.  Dynamic shared memory: M rows of
// K floats, each rounded up to a multiple of 256 floats plus 256 zeros.
// STAMP = true is the same kernel with five time stamps per CTA (GemvArgs::stamps), used only by the
// time-line measurement; the product instantiations carry none of it.
template <int WARPS, int R, int U, int M, typename WT, bool STAMP = false>
__global__ void __launch_bounds__(WARPS * 32) dmc_wrows_kernel(const GemvArgs a) {
    constexpr int EPV = VecOf<WT>::EPV;
    constexpr int THREADS = WARPS * 32;
    constexpr int NACC = M == 1 ? 2 : 1;  // a single row keeps two accumulator chains per weight row
    extern __shared__ __align__(16) float xs[];
    float4 *xs4 = reinterpret_cast<float4 *>(xs);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = a.K, N = a.N;
    const int nvec = K / EPV;
    const int xpad4 = (K + 255) / 256 * 64;  // float4 slots of one staged row of x ...
    const int xrow4 = xpad4 + 64;            // ... followed by a block of zeros
    const uint4 *W4 = reinterpret_cast<const uint4 *>(a.W);

    // this CTA's block of row groups
    const int groups = (N + R - 1) / R;
    const int g0 = (int)(((long long)groups * blockIdx.x) / gridDim.x);
    const int g1 = (int)(((long long)groups * (blockIdx.x + 1)) / gridDim.x);

    uint4 w[R][U];
    auto load_w = [&](int row0, int c) {
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const int row = row0 + j;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int cc = c + 32 * u;
                w[j][u] = (row < N && cc < nvec) ? ldg_stream16(W4 + (size_t)row * nvec + cc)
                                                 : make_uint4(0, 0, 0, 0);
            }
        }
    };
    float acc[R][M][NACC];
    auto consume = [&](int c) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            // vectors past the end of a row (loaded as zeros) read a block of zeros kept behind the staged row,
            // instead of predicating every shared-memory read
            const int cc = c + 32 * u;
            // per 32 vectors: low halves first, then high halves
            const int xi = cc < nvec ? (EPV == 8 ? (cc >> 5) * 64 + (cc & 31) : cc) : xpad4;
            if constexpr (M == 1) {
                const float4 xa = xs4[xi];
                const float4 xb = EPV == 8 ? xs4[xi + 32] : make_float4(0, 0, 0, 0);
#pragma unroll
                for (int j = 0; j < R; ++j) acc[j][0][u & 1] = dot_vec<WT>(acc[j][0][u & 1], w[j][u], xa, xb);
            } else {
                // several rows of x: widen each weight vector once, reuse it for every row
                float wf[R][8];
#pragma unroll
                for (int j = 0; j < R; ++j) widen_vec<WT>(w[j][u], wf[j]);
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const float4 xa = xs4[m * xrow4 + xi];
                    const float4 xb = EPV == 8 ? xs4[m * xrow4 + xi + 32] : make_float4(0, 0, 0, 0);
#pragma unroll
                    for (int j = 0; j < R; ++j) {
                        float s = acc[j][m][0];
                        s = fmaf(xa.x, wf[j][0], s);
                        s = fmaf(xa.y, wf[j][1], s);
                        s = fmaf(xa.z, wf[j][2], s);
                        s = fmaf(xa.w, wf[j][3], s);
                        if constexpr (EPV == 8) {
                            s = fmaf(xb.x, wf[j][4], s);
                            s = fmaf(xb.y, wf[j][5], s);
                            s = fmaf(xb.z, wf[j][6], s);
                            s = fmaf(xb.w, wf[j][7], s);
                        }
                        acc[j][m][0] = s;
                    }
                }
            }
        }
    };

    unsigned long long t_entry = 0, t_wait = 0, t_x = 0, t_first = 0;
    if (STAMP && threadIdx.x == 0) t_entry = globaltimer_ns();
    // (the first exchange of a batch lets its dependents go only after its own wait: they read the
    // epoch word that the end of the previous batch advances)
    const bool hold_dependents = a.peer != nullptr && a.peer_j == 0;
    if (!hold_dependents) griddep_launch_dependents();
    int g = g0 + warp;
    if (g < g1) load_w(g * R, lane);  // weights depend on no earlier kernel: first loads go out before the wait
    // The exchange descriptor is copied into shared memory once per CTA: read through the global
    // pointer, every field would have to be reloaded after each output store (the compiler cannot
    // rule out that a store hits the descriptor).
    __shared__ PeerOut s_peer;
    static_assert(sizeof(PeerOut) % 4 == 0, "PeerOut is copied word by word");
    if (a.peer) {
        for (int i = threadIdx.x; i < (int)(sizeof(PeerOut) / 4); i += THREADS)
            reinterpret_cast<unsigned *>(&s_peer)[i] = __ldg(reinterpret_cast<const unsigned *>(a.peer) + i);
    }
    if (!a.nowait) griddep_wait();
    if (hold_dependents) griddep_launch_dependents();
    if (STAMP && threadIdx.x == 0) t_wait = globaltimer_ns();
    // after the wait: an earlier kernel (the end of the previous batch) is what advances the epoch word
    const PeerOut *peer = a.peer ? &s_peer : nullptr;
    if (a.peer) __syncthreads();  // the descriptor copy is complete
    const unsigned epoch = peer ? peer_epoch(peer, a.peer_j) : 0u;
    // the replica buffer of this exchange must be free again: the words that say so are requested here
    // and looked at once x is staged; the barrier there orders every warp's stores after the check
    __shared__ __align__(16) unsigned guard_words[kMaxPeers];
    const bool guard = peer != nullptr && threadIdx.x == 0 && epoch >= 3u;
    if (guard) peer_guard_load(peer, guard_words);

    // stage x (after the dependency wait: an earlier kernel may produce it)
    {
        const int n4 = K / 4;
        auto slot = [&](int m, int i) -> float4 & {
            if constexpr (EPV == 8) {
                const int blk = i >> 6, idx = i & 63;
                return xs4[m * xrow4 + blk * 64 + (idx & 1) * 32 + (idx >> 1)];
            } else {
                return xs4[m * xrow4 + i];
            }
        };
        const float4 *x4 = reinterpret_cast<const float4 *>(a.x);
        for (int i = threadIdx.x; i < 64 * M; i += THREADS) xs4[(i >> 6) * xrow4 + xpad4 + (i & 63)] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (M == 1 && a.pro == 1) {
            // RMSNorm of the residual stream fused into the staging (f32 form of the JIT,
            // compiler/src/jit.rs:23776-23847): every CTA normalises its own copy of x
            // Loads are issued in batches (x, the residual and the gain of up to PG elements per thread
            // before anything is used): the staging sits on the critical path of a dependent chain, and
            // every separate round trip to L2 costs ~0.3 us there.
            __shared__ float red[WARPS];
            constexpr int PG = 4;
            const float4 *add4 = reinterpret_cast<const float4 *>(a.pro_add);
            const float4 *g4 = reinterpret_cast<const float4 *>(a.pro_g);
            float4 *h4 = reinterpret_cast<float4 *>(a.pro_hout);
            float4 v[PG], gg[PG];
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < PG; ++j) {
                const int i = threadIdx.x + j * THREADS;
                v[j] = i < n4 ? __ldcg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            if (add4) {
#pragma unroll
                for (int j = 0; j < PG; ++j) {
                    const int i = threadIdx.x + j * THREADS;
                    if (i < n4) {
                        const float4 d = __ldcg(add4 + i);
                        v[j].x += d.x, v[j].y += d.y, v[j].z += d.z, v[j].w += d.w;
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < PG; ++j) {
                const int i = threadIdx.x + j * THREADS;
                gg[j] = i < n4 ? __ldg(g4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < PG; ++j) {
                const int i = threadIdx.x + j * THREADS;
                if (i < n4) {
                    if (h4 && blockIdx.x == 0) h4[i] = v[j];
                    ss = fmaf(v[j].x, v[j].x, fmaf(v[j].y, v[j].y, fmaf(v[j].z, v[j].z, fmaf(v[j].w, v[j].w, ss))));
                }
            }
            for (int i = threadIdx.x + PG * THREADS; i < n4; i += THREADS) {  // rows longer than PG * THREADS vectors
                float4 t = __ldcg(x4 + i);
                if (add4) {
                    const float4 d = __ldcg(add4 + i);
                    t.x += d.x, t.y += d.y, t.z += d.z, t.w += d.w;
                }
                if (h4 && blockIdx.x == 0) h4[i] = t;
                ss = fmaf(t.x, t.x, fmaf(t.y, t.y, fmaf(t.z, t.z, fmaf(t.w, t.w, ss))));
                slot(0, i) = t;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) red[warp] = ss;
            __syncthreads();
            float tot = 0.0f;
#pragma unroll
            for (int w2 = 0; w2 < WARPS; ++w2) tot += red[w2];
            const float inv = 1.0f / sqrtf(tot / (float)K + a.pro_eps);
#pragma unroll
            for (int j = 0; j < PG; ++j) {  // the first PG elements per thread never left the registers
                const int i = threadIdx.x + j * THREADS;
                if (i < n4) {
                    float4 t = v[j];
                    t.x = t.x * gg[j].x * inv, t.y = t.y * gg[j].y * inv, t.z = t.z * gg[j].z * inv, t.w = t.w * gg[j].w * inv;
                    slot(0, i) = t;
                }
            }
            for (int i = threadIdx.x + PG * THREADS; i < n4; i += THREADS) {  // each thread rescales what it stored itself
                float4 t = slot(0, i);
                const float4 g1 = __ldg(g4 + i);
                t.x = t.x * g1.x * inv, t.y = t.y * g1.y * inv, t.z = t.z * g1.z * inv, t.w = t.w * g1.w * inv;
                slot(0, i) = t;
            }
        } else if (M == 1 && a.pro == 2) {
            // SwiGLU (silu = x / (1 + e^-x), compiler/src/interp.rs:13418) of a [gate | up] vector
            constexpr int PG = 4;
            for (int i0 = threadIdx.x; i0 < n4; i0 += PG * THREADS) {
                float4 gt[PG], up[PG];
#pragma unroll
                for (int j = 0; j < PG; ++j) {
                    const int i = i0 + j * THREADS;
                    if (i < n4) gt[j] = __ldcg(x4 + i), up[j] = __ldcg(x4 + n4 + i);
                }
#pragma unroll
                for (int j = 0; j < PG; ++j) {
                    const int i = i0 + j * THREADS;
                    if (i < n4) {
                        float4 v;
                        v.x = gt[j].x / (1.0f + __expf(-gt[j].x)) * up[j].x;
                        v.y = gt[j].y / (1.0f + __expf(-gt[j].y)) * up[j].y;
                        v.z = gt[j].z / (1.0f + __expf(-gt[j].z)) * up[j].z;
                        v.w = gt[j].w / (1.0f + __expf(-gt[j].w)) * up[j].w;
                        slot(0, i) = v;
                    }
                }
            }
        } else {
#pragma unroll
            for (int m = 0; m < M; ++m)
                for (int i = threadIdx.x; i < n4; i += THREADS)
                    slot(m, i) = (M == 1 || m < a.mrows) ? __ldcg(x4 + (size_t)m * n4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (guard && !peer_guard_ok(peer, epoch, guard_words)) peer_wait_buffer_free(peer, epoch);
        __syncthreads();
    }
    if (STAMP && threadIdx.x == 0) t_x = globaltimer_ns();

    unsigned long long best = 0ull;  // arg-max epilogue: this warp's best (value, row) so far
    bool first = true;  // the warp's first row group: chunk 0 is already in registers
    for (; g < g1; g += WARPS) {
        const int row0 = g * R;
#pragma unroll
        for (int j = 0; j < R; ++j)
#pragma unroll
            for (int m = 0; m < M; ++m)
#pragma unroll
                for (int t = 0; t < NACC; ++t) acc[j][m][t] = 0.0f;
        for (int c = lane; c < nvec; c += 32 * U) {
            if (!(first && c == lane)) load_w(row0, c);
            consume(c);
        }
        first = false;
        float mine = 0.0f;  // sharded path: lane j keeps the sum of row j
#pragma unroll
        for (int j = 0; j < R; ++j) {
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float s = acc[j][m][0];
                if constexpr (NACC == 2) s += acc[j][m][1];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);  // every lane ends with the sum
                const int row = row0 + j;
                if (M == 1 && peer) {
                    if (lane == j) mine = s;
                } else if (lane == 0 && row < N && (M == 1 || m < a.mrows)) {
                    a.y[(size_t)m * N + row] = s;
                }
                if (M == 1 && a.amax && row < N && s == s) {  // (a NaN is never a maximum)
                    const unsigned long long key = amax_key(s, row);
                    best = key > best ? key : best;
                }
            }
        }
        // The R rows of a warp are adjacent, so lanes 0..R-1 store them together: one R*8-byte write per
        // replica instead of R separate ones (fewer, larger NVLink packets).
        if (M == 1 && peer && lane < R && row0 + lane < N) peer_store(peer, epoch, a.yoff + row0 + lane, mine);
        if (STAMP && threadIdx.x == 0 && t_first == 0) t_first = globaltimer_ns();
    }
    if (STAMP) {
        __syncthreads();  // every warp of the CTA has finished its rows
        if (threadIdx.x == 0) {
            unsigned smid;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            unsigned long long *st = a.stamps + (size_t)blockIdx.x * 8;
            st[0] = t_entry, st[1] = t_wait, st[2] = t_x, st[3] = t_first, st[4] = globaltimer_ns(), st[5] = smid;
        }
    }
    if (M == 1 && a.amax) {  // one atomic per CTA
        __shared__ unsigned long long s_best[WARPS];
        if (lane == 0) s_best[warp] = best;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long b = s_best[0];
#pragma unroll
            for (int w2 = 1; w2 < WARPS; ++w2) b = s_best[w2] > b ? s_best[w2] : b;
            if (b) atomicMax(a.amax, b);
        }
    }
}

// Any-shape NK fallback: one warp per row, scalar loads.
template <typename WT>
__global__ void __launch_bounds__(256) dmc_wrows_any_kernel(const GemvArgs a, int M) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    griddep_wait();
    if (row >= a.N) return;
    const WT *Wr = (const WT *)a.W + (size_t)row * a.K;
    for (int m = 0; m < M; ++m) {
        float acc = 0.0f;
        for (int k = lane; k < a.K; k += 32) {
            float wv;
            if constexpr (sizeof(WT) == 2)
                wv = __uint_as_float((uint32_t)Wr[k] << 16);
            else
                wv = Wr[k];
            acc = fmaf(__ldcg(a.x + (size_t)m * a.K + k), wv, acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) a.y[(size_t)m * a.N + row] = acc;
    }
}

}  // namespace dmc
