// decode_ops.cuh -- the small kernels around the GEMVs of one decode step of a decoder-only
// transformer built from the reference's own ops.  Each restates the f32 form the JIT emits:
//   rms_norm   compiler/src/jit.rs:23776-23847 (x * g / sqrt(mean(x^2) + eps))
//   rope       docs/STDLIB.md:185-202, compiler/src/interp.rs:13636-13678 (pairs (2i, 2i+1))
//   attention  compiler/src/jit.rs:20303-20506 (q.K^T, scale 1/sqrt(d), softmax, p.V) over a KV cache
//   silu       compiler/src/interp.rs:13418 (x / (1 + e^-x)); SwiGLU = silu(gate) * up
//   embed      compiler/src/interp.rs:13494-13516 (ids clamp to [0, V-1])
//   argmax     compiler/src/interp.rs:13529-13538 (first strict maximum)
// They are tolerance-matched companions (sums run in parallel, not sequentially), not
// roofline-graded; all activations stay on the device between them.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemv.cuh"

namespace dmc {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over a CTA of up to 1024 threads; every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float *red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < nw; ++i) t += red[i];
    return t;
}

// h[d] = widen(vocab[clamp(id)][d])
__global__ void embed_kernel(const uint16_t *__restrict__ vocab, int V, int D, const int *__restrict__ id_ptr,
                             float *__restrict__ h, unsigned long long *__restrict__ amax_key) {
    griddep_wait();
    if (amax_key && blockIdx.x == 0 && threadIdx.x == 0) *amax_key = 0ull;  // re-armed for this step's lm-head
    int id = *id_ptr;
    id = id < 0 ? 0 : (id > V - 1 ? V - 1 : id);
    for (int d = blockIdx.x * blockDim.x + threadIdx.x; d < D; d += gridDim.x * blockDim.x)
        h[d] = __uint_as_float((uint32_t)vocab[(size_t)id * D + d] << 16);
}

// y = x * g * rsqrt-free form of the JIT: inv = 1 / sqrt(sum(x^2)/d + eps).  One CTA.
// If `add` is non-null the input is first updated in place: x += add (the residual connection).
__global__ void __launch_bounds__(1024) rmsnorm_kernel(float *__restrict__ x, const float *__restrict__ add,
                                                        const float *__restrict__ g, float *__restrict__ y, int D,
                                                        float eps) {
    __shared__ float red[32];
    griddep_launch_dependents();
    griddep_wait();
    float ss = 0.0f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = x[i];
        if (add) {
            v += add[i];
            x[i] = v;
        }
        ss = fmaf(v, v, ss);
    }
    const float tot = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(tot / (float)D + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) y[i] = x[i] * g[i] * inv;
}

// RoPE on q and k (pairs (2i, 2i+1) of each head, angle row `pos` of the cos/sin tables) and the
// KV-cache append: K[h][pos] = rope(k_h), V[h][pos] = v_h.  qkv = [q | k | v], each H*hd floats.
// Cache layout [H][cap][hd] f32 (the reference's KV[B,H,~,D] with B = 1).
__global__ void rope_append_kernel(float *__restrict__ qkv, const float *__restrict__ cs, const float *__restrict__ sn,
                                   float *__restrict__ kc, float *__restrict__ vc, int H, int hd, int cap,
                                   const int *__restrict__ pos_ptr) {
    griddep_launch_dependents();
    griddep_wait();
    const int pos = *pos_ptr;
    const int half = hd / 2, total = H * half;
    float *q = qkv, *k = qkv + H * hd, *v = qkv + 2 * H * hd;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int h = i / half, p = i % half;
        const float c = cs[(size_t)pos * half + p], s = sn[(size_t)pos * half + p];
        const int e = h * hd + 2 * p;
        const float qa = q[e], qb = q[e + 1];
        q[e] = qa * c - qb * s;
        q[e + 1] = qa * s + qb * c;
        const float ka = k[e], kb = k[e + 1];
        const size_t ce = ((size_t)h * cap + pos) * hd + 2 * p;
        kc[ce] = ka * c - kb * s;
        kc[ce + 1] = ka * s + kb * c;
        vc[ce] = v[e];
        vc[ce + 1] = v[e + 1];
    }
}

// Decode attention, split over the keys: CTA (h, z) handles keys [z*chunk, (z+1)*chunk) of head h with an
// online softmax, and leaves (max, sum, unnormalised output[hd]) for the combine kernel.  hd == 128:
// a lane owns 4 dims, a warp one key at a time.  part layout [H][splits][hd + 2].
__global__ void __launch_bounds__(128) attn_partial_kernel(const float *__restrict__ qkv, const float *__restrict__ kc,
                                                            const float *__restrict__ vc, float *__restrict__ part,
                                                            int H, int cap, const int *__restrict__ pos_ptr, int chunk) {
    constexpr int HD = 128;
    __shared__ float sm_m[4], sm_l[4], sm_o[4][HD];
    griddep_launch_dependents();
    griddep_wait();
    const int len = *pos_ptr + 1;  // keys 0..pos (the new token was just appended)
    const int h = blockIdx.x, z = blockIdx.y, splits = gridDim.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t0 = z * chunk, t1 = min(len, t0 + chunk);
    const float scale = 1.0f / sqrtf((float)HD);
    const float4 q4 = reinterpret_cast<const float4 *>(qkv + (size_t)h * HD)[lane];
    float m = -INFINITY, l = 0.0f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int t = t0 + warp; t < t1; t += 4) {
        const float4 k4 = __ldcs(reinterpret_cast<const float4 *>(kc + ((size_t)h * cap + t) * HD) + lane);
        const float4 v4 = __ldcs(reinterpret_cast<const float4 *>(vc + ((size_t)h * cap + t) * HD) + lane);
        float s = q4.x * k4.x + q4.y * k4.y + q4.z * k4.z + q4.w * k4.w;
        s = warp_sum(s) * scale;
        const float mn = fmaxf(m, s);
        const float corr = __expf(m - mn), p = __expf(s - mn);
        l = l * corr + p;
        o.x = o.x * corr + p * v4.x;
        o.y = o.y * corr + p * v4.y;
        o.z = o.z * corr + p * v4.z;
        o.w = o.w * corr + p * v4.w;
        m = mn;
    }
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
    reinterpret_cast<float4 *>(sm_o[warp])[lane] = o;
    __syncthreads();
    // merge the four warps
    float M = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
    const int d = threadIdx.x;  // 128 threads, one dim each
    float L = 0.0f, O = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const float c = (sm_m[w] == -INFINITY) ? 0.0f : __expf(sm_m[w] - M);
        L += sm_l[w] * c;
        O += sm_o[w][d] * c;
    }
    float *dst = part + ((size_t)h * splits + z) * (HD + 2);
    dst[d] = O;
    if (d == 0) {
        dst[HD] = M;
        dst[HD + 1] = L;
    }
}

// out[h][d] = sum_z O_z e^(m_z - M) / sum_z l_z e^(m_z - M)
__global__ void __launch_bounds__(128) attn_combine_kernel(const float *__restrict__ part, float *__restrict__ out,
                                                            int splits) {
    constexpr int HD = 128;
    griddep_launch_dependents();
    griddep_wait();
    const int h = blockIdx.x, d = threadIdx.x;
    const float *p = part + (size_t)h * splits * (HD + 2);
    float M = -INFINITY;
    for (int z = 0; z < splits; ++z) M = fmaxf(M, p[(size_t)z * (HD + 2) + HD]);
    float L = 0.0f, O = 0.0f;
    for (int z = 0; z < splits; ++z) {
        const float mz = p[(size_t)z * (HD + 2) + HD];
        const float c = (mz == -INFINITY) ? 0.0f : __expf(mz - M);
        L += p[(size_t)z * (HD + 2) + HD + 1] * c;
        O += p[(size_t)z * (HD + 2) + d] * c;
    }
    out[(size_t)h * HD + d] = L > 0.0f ? O / L : 0.0f;
}

// The three kernels above in one launch: CTA (h, z) rotates q_h itself, the CTA whose key range
// holds `pos` rotates and appends the new k/v (and uses them from shared memory), every CTA runs the
// online softmax over its keys, and the CTA that arrives last at the head's counter merges the
// splits into out[h].  cnt: one counter per head, zero between launches.
__global__ void __launch_bounds__(128) attn_fused_kernel(const float *__restrict__ qkv, const float *__restrict__ cs,
                                                          const float *__restrict__ sn, float *__restrict__ kc,
                                                          float *__restrict__ vc, float *__restrict__ part,
                                                          float *__restrict__ out, unsigned *__restrict__ cnt, int H, int cap,
                                                          const int *__restrict__ pos_ptr, int chunk) {
    constexpr int HD = 128;
    __shared__ __align__(16) float qs[HD], ks[HD], vs[HD];
    __shared__ float sm_m[4], sm_l[4];
    __shared__ __align__(16) float sm_o[4][HD];
    __shared__ int s_last;
    griddep_launch_dependents();
    const int h = blockIdx.x, z = blockIdx.y, splits = gridDim.y;
    const int d = threadIdx.x, lane = d & 31, warp = d >> 5;
    const int t0 = z * chunk;
    constexpr int KU = 8;  // keys in flight per warp: the loop is bound by memory latency, not by arithmetic
    // `pos` is written by a copy that completed before the first kernel of the step started, and the
    // cached rows below `pos` by earlier steps: neither depends on the kernel before this one, so both
    // are read BEFORE the dependency wait and the whole cache of the layer is in flight while the qkv
    // projection is still finishing.  (The row at `pos` is the one this launch appends: it is taken
    // from shared memory below, never from the cache.)
    const int pos = *pos_ptr, len = pos + 1;
    const int t1 = min(len, t0 + chunk);
    const bool owns_new = pos >= t0 && pos < t0 + chunk;
    // key ranges beyond the current length take no part at all: they leave before the dependency wait,
    // and the head's arrival counter and merge count only the ranges that hold keys
    const int active = min(splits, (len + chunk - 1) / chunk);
    if (z >= active) return;
    float4 k4[KU], v4[KU];
    auto load_batch = [&](int tb) {
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            const int t = tb + 4 * u;
            if (t >= t1 || t == pos) {
                k4[u] = v4[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            } else {
                k4[u] = __ldcg(reinterpret_cast<const float4 *>(kc + ((size_t)h * cap + t) * HD) + lane);
                v4[u] = __ldcg(reinterpret_cast<const float4 *>(vc + ((size_t)h * cap + t) * HD) + lane);
            }
        }
    };
    load_batch(t0 + warp);
    const float c = cs[(size_t)pos * (HD / 2) + (d >> 1)], s = sn[(size_t)pos * (HD / 2) + (d >> 1)];  // constant tables
    griddep_wait();  // q, k, v of this token come from the projection before this kernel
    {   // RoPE, pairs (2i, 2i+1): thread d holds element d and reads its partner
        const float *q = qkv + (size_t)h * HD, *k = qkv + (size_t)(H + h) * HD, *v = qkv + (size_t)(2 * H + h) * HD;
        const float qa = q[d & ~1], qb = q[d | 1];
        qs[d] = (d & 1) ? qa * s + qb * c : qa * c - qb * s;
        if (owns_new) {
            const float ka = k[d & ~1], kb = k[d | 1];
            const float kr = (d & 1) ? ka * s + kb * c : ka * c - kb * s;
            ks[d] = kr;
            vs[d] = v[d];
            kc[((size_t)h * cap + pos) * HD + d] = kr;
            vc[((size_t)h * cap + pos) * HD + d] = v[d];
        }
    }
    __syncthreads();
    const float scale = 1.0f / sqrtf((float)HD);
    const float4 q4 = reinterpret_cast<const float4 *>(qs)[lane];
    float m = -INFINITY, l = 0.0f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int tb = t0 + warp; tb < t1; tb += 4 * KU) {
        if (tb != t0 + warp) load_batch(tb);
        // the scores of the batch first: KU independent shuffle reductions overlap, where one key at a
        // time each would wait for the one before it
        float sc[KU];
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            if (tb + 4 * u == pos) {
                k4[u] = reinterpret_cast<const float4 *>(ks)[lane];
                v4[u] = reinterpret_cast<const float4 *>(vs)[lane];
            }
            sc[u] = q4.x * k4[u].x + q4.y * k4[u].y + q4.z * k4[u].z + q4.w * k4[u].w;
        }
#pragma unroll
        for (int u = 0; u < KU; ++u) sc[u] = warp_sum(sc[u]) * scale;
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            const int t = tb + 4 * u;
            if (t >= t1) break;
            const float s = sc[u];
            const float mn = fmaxf(m, s);
            const float corr = __expf(m - mn), p = __expf(s - mn);
            l = l * corr + p;
            o.x = o.x * corr + p * v4[u].x;
            o.y = o.y * corr + p * v4[u].y;
            o.z = o.z * corr + p * v4[u].z;
            o.w = o.w * corr + p * v4[u].w;
            m = mn;
        }
    }
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
    reinterpret_cast<float4 *>(sm_o[warp])[lane] = o;
    __syncthreads();
    const float M = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
    float L = 0.0f, O = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const float c = (sm_m[w] == -INFINITY) ? 0.0f : __expf(sm_m[w] - M);
        L += sm_l[w] * c;
        O += sm_o[w][d] * c;
    }
    float *dst = part + ((size_t)h * splits + z) * (HD + 2);
    dst[d] = O;
    if (d == 0) {
        dst[HD] = M;
        dst[HD + 1] = L;
    }
    // last CTA of the head merges the splits (in split order: fixed)
    __threadfence();
    __syncthreads();
    if (d == 0) s_last = (atomicAdd(&cnt[h], 1u) == (unsigned)active - 1u);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // splits <= 32.  Every load of the merge goes out at once -- a thread's value of each split and, in
    // warp 0, one (max, sum) pair per lane -- so the merge costs one round trip to L2, not one per group
    // of splits; the weights e^(m_z - M) then go through shared memory.
    const float *p = part + (size_t)h * splits * (HD + 2);
    __shared__ float cz[32], Lsum;
    float pv[32];
#pragma unroll
    for (int u = 0; u < 32; ++u) pv[u] = u < active ? __ldcg(&p[(size_t)u * (HD + 2) + d]) : 0.0f;
    if (warp == 0) {
        const float mz = lane < active ? __ldcg(&p[(size_t)lane * (HD + 2) + HD]) : -INFINITY;
        const float lz = lane < active ? __ldcg(&p[(size_t)lane * (HD + 2) + HD + 1]) : 0.0f;
        float Mx = mz;
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) Mx = fmaxf(Mx, __shfl_xor_sync(0xffffffffu, Mx, o2));
        const float c = (mz == -INFINITY) ? 0.0f : __expf(mz - Mx);
        cz[lane] = c;
        const float Ls = warp_sum(lz * c);
        if (lane == 0) Lsum = Ls;
    }
    __syncthreads();
    float Os = 0.0f;
#pragma unroll
    for (int u = 0; u < 32; ++u) Os += pv[u] * cz[u];  // (split order: fixed; absent splits have weight 0)
    out[(size_t)h * HD + d] = Lsum > 0.0f ? Os / Lsum : 0.0f;
    if (d == 0) cnt[h] = 0u;
}

// act[i] = silu(gate[i]) * up[i], gu = [gate | up]
__global__ void swiglu_kernel(const float *__restrict__ gu, float *__restrict__ act, int F) {
    griddep_launch_dependents();
    griddep_wait();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < F; i += gridDim.x * blockDim.x) {
        const float g = gu[i];
        act[i] = (g / (1.0f + __expf(-g))) * gu[F + i];
    }
}

// First strict maximum of x[0..n) (ties: lowest index).  gridDim.x CTAs scan slices; the CTA that
// arrives last at `cnt` merges the per-CTA candidates.  scratch: gridDim.x (value, index) pairs.
__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ x, int n, int *__restrict__ out,
                                                      float *__restrict__ sval, int *__restrict__ sidx,
                                                      unsigned *__restrict__ cnt) {
    __shared__ float bv[8];
    __shared__ int bi[8];
    __shared__ int s_last;
    griddep_wait();
    auto better = [](float v, int i, float bv_, int bi_) { return v > bv_ || (v == bv_ && i < bi_); };
    auto block_best = [&](float &best, int &idx) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float v2 = __shfl_xor_sync(0xffffffffu, best, o);
            const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
            if (better(v2, i2, best, idx)) {
                best = v2;
                idx = i2;
            }
        }
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        __syncthreads();
        if (lane == 0) {
            bv[warp] = best;
            bi[warp] = idx;
        }
        __syncthreads();
        best = bv[0];
        idx = bi[0];
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (better(bv[w], bi[w], best, idx)) {
                best = bv[w];
                idx = bi[w];
            }
    };
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = __ldcg(x + i);
        if (better(v, i, best, idx)) {
            best = v;
            idx = i;
        }
    }
    block_best(best, idx);
    if (threadIdx.x == 0) {
        sval[blockIdx.x] = best;
        sidx[blockIdx.x] = idx;
        __threadfence();
        s_last = (atomicAdd(cnt, 1u) == gridDim.x - 1u);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    best = -INFINITY;
    idx = 0x7fffffff;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) {
        const float v = __ldcg(sval + i);
        const int j = __ldcg(sidx + i);
        if (better(v, j, best, idx)) {
            best = v;
            idx = j;
        }
    }
    block_best(best, idx);
    if (threadIdx.x == 0) {
        *out = idx == 0x7fffffff ? 0 : idx;
        *cnt = 0u;
    }
}

}  // namespace dmc
