// decode.cu -- one decode step of a decoder-only transformer, fully on the device: every
// projection goes through the GEMV path, the companions of decode_ops.cuh sit between them, and
// the whole step (43 launches in the fused arrangement) is captured once into a CUDA graph and replayed per token, so the
// per-call host<->device traffic the reference ABI forces (compiler/src/gpu.rs:528-531, 649-651)
// disappears: a token id goes in, a token id comes out.
#include <cstring>
#include <utility>
#include <vector>

#include "decode_ops.cuh"
#include "runtime.h"

namespace dmc {
namespace {

struct Layer {
    uint16_t *wqkv = nullptr, *wo = nullptr, *wgu = nullptr, *wd = nullptr;  // [3D,D] [D,D] [2F,D] [D,F] bf16, k contiguous
    float *g1 = nullptr, *g2 = nullptr;                                      // RMSNorm gains [D]
    float *kc = nullptr, *vc = nullptr;                                      // KV cache [H][cap][hd] f32
};

struct Decoder {
    dmc_decoder_config cfg;
    std::vector<Layer> layers;
    uint16_t *embed = nullptr, *lm_head = nullptr;  // [V,D] bf16
    float *gf = nullptr, *rope_cos = nullptr, *rope_sin = nullptr;
    float *h2 = nullptr;        // second residual-stream buffer (the fused RMSNorm ping-pongs between h and h2)
    unsigned *attn_cnt = nullptr;
    unsigned long long *am_key = nullptr;  // arg-max key the lm-head GEMV leaves (fused arrangement)
    float *am_val = nullptr;    // argmax per-CTA candidates (unfused arrangement)
    int *am_idx = nullptr;
    unsigned *am_cnt = nullptr;
    int fused = 1;              // 1: RMSNorm / SwiGLU fused into the GEMVs' staging, RoPE + append + combine into attention
    float *h = nullptr, *xn = nullptr, *qkv = nullptr, *ao = nullptr, *d1 = nullptr, *gu = nullptr, *act = nullptr,
          *d2 = nullptr, *logits = nullptr, *part = nullptr;
    int *d_token = nullptr, *d_pos = nullptr, *d_next = nullptr;
    int splits = 32;            // key ranges per head in the attention kernels
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int64_t launches_per_step = 0;
};

template <typename T>
int dalloc(T **p, size_t count) {
    DMC_CUDA_TRY(dmc_malloc((void **)p, count * sizeof(T)));
    DMC_CUDA_TRY(cudaMemset(*p, 0, count * sizeof(T)));
    return DMC_CUDA_OK;
}

template <typename... Args>
int launch_small(void (*fn)(Args...), dim3 grid, dim3 block, cudaStream_t s, Args... args) {
    void *params[] = {(void *)&args...};
    return launch_ex((const void *)fn, grid, block, 0, s, params);
}

// y = W . prologue(x) with the prologue fused into the GEMV's x staging (see GemvArgs::pro).
int gemv_pro(const void *W, const float *x, float *y, int64_t k, int64_t n, int pro, const float *add, const float *g,
             float *hout, float eps, cudaStream_t s) {
    Context &c = ctx();
    c.pro = pro;
    c.pro_add = add;
    c.pro_g = g;
    c.pro_hout = hout;
    c.pro_eps = eps;
    int rc = launch_gemv(W, x, y, 1, k, n, 1, 0, 0, DMC_LAYOUT_NK, DMC_W_BF16, -1, s);
    c.pro = 0;
    c.pro_add = c.pro_g = nullptr;
    c.pro_hout = nullptr;
    return rc;
}

// All launches of one step, in order, on `s`: 5 per layer (43 in all for 8 layers).
int enqueue_step_fused(Decoder &d, cudaStream_t s) {
    const dmc_decoder_config &c = d.cfg;
    const int D = c.d_model, H = c.heads, F = c.ffn, V = c.vocab, cap = c.max_len;
    int rc;
    float *hin = d.h, *hout = d.h2;
    if ((rc = launch_small(embed_kernel, dim3(8), dim3(256), s, (const uint16_t *)d.embed, V, D, (const int *)d.d_token, hin,
                           d.am_key)))
        return rc;
    const float *carry = nullptr;
    const int chunk = (cap + d.splits - 1) / d.splits;
    for (int l = 0; l < c.layers; ++l) {
        Layer &L = d.layers[l];
        // qkv = Wqkv . rms_norm(h + carry);  h' = h + carry
        if ((rc = gemv_pro(L.wqkv, hin, d.qkv, D, 3 * D, 1, carry, L.g1, hout, c.eps, s))) return rc;
        std::swap(hin, hout);
        if ((rc = launch_small(attn_fused_kernel, dim3(H, d.splits), dim3(128), s, (const float *)d.qkv,
                               (const float *)d.rope_cos, (const float *)d.rope_sin, L.kc, L.vc, d.part, d.ao, d.attn_cnt, H,
                               cap, (const int *)d.d_pos, chunk)))
            return rc;
        if ((rc = launch_gemv(L.wo, d.ao, d.d1, 1, D, D, 1, 0, 0, DMC_LAYOUT_NK, DMC_W_BF16, -1, s))) return rc;
        // gu = Wgu . rms_norm(h + d1);  h' = h + d1
        if ((rc = gemv_pro(L.wgu, hin, d.gu, D, 2 * F, 1, d.d1, L.g2, hout, c.eps, s))) return rc;
        std::swap(hin, hout);
        // d2 = Wd . (silu(gate) * up)
        if ((rc = gemv_pro(L.wd, d.gu, d.d2, F, D, 2, nullptr, nullptr, nullptr, 0.0f, s))) return rc;
        carry = d.d2;
    }
    // logits = lm_head . rms_norm(h + carry), and their arg-max in the same kernel
    ctx().amax = d.am_key;
    rc = gemv_pro(d.lm_head, hin, d.logits, D, V, 1, carry, d.gf, nullptr, c.eps, s);
    ctx().amax = nullptr;
    return rc;
}

// The unfused sequence (9 launches per layer), kept as the reference arrangement of the same math.
int enqueue_step_plain(Decoder &d, cudaStream_t s) {
    const dmc_decoder_config &c = d.cfg;
    const int D = c.d_model, H = c.heads, hd = c.head_dim, F = c.ffn, V = c.vocab, cap = c.max_len;
    int rc;
    if ((rc = launch_small(embed_kernel, dim3(8), dim3(256), s, (const uint16_t *)d.embed, V, D, (const int *)d.d_token, d.h,
                           (unsigned long long *)nullptr)))
        return rc;
    const float *carry = nullptr;  // residual branch output waiting to be added to h
    const int chunk = (cap + d.splits - 1) / d.splits;
    for (int l = 0; l < c.layers; ++l) {
        Layer &L = d.layers[l];
        if ((rc = launch_small(rmsnorm_kernel, dim3(1), dim3(1024), s, d.h, carry, (const float *)L.g1, d.xn, D, c.eps))) return rc;
        if ((rc = launch_gemv(L.wqkv, d.xn, d.qkv, 1, D, 3 * D, 1, 0, 0, DMC_LAYOUT_NK, DMC_W_BF16, -1, s))) return rc;
        if ((rc = launch_small(rope_append_kernel, dim3(4), dim3(256), s, d.qkv, (const float *)d.rope_cos,
                               (const float *)d.rope_sin, L.kc, L.vc, H, hd, cap, (const int *)d.d_pos)))
            return rc;
        if ((rc = launch_small(attn_partial_kernel, dim3(H, d.splits), dim3(128), s, (const float *)d.qkv,
                               (const float *)L.kc, (const float *)L.vc, d.part, H, cap, (const int *)d.d_pos, chunk)))
            return rc;
        if ((rc = launch_small(attn_combine_kernel, dim3(H), dim3(128), s, (const float *)d.part, d.ao, d.splits))) return rc;
        if ((rc = launch_gemv(L.wo, d.ao, d.d1, 1, D, D, 1, 0, 0, DMC_LAYOUT_NK, DMC_W_BF16, -1, s))) return rc;
        if ((rc = launch_small(rmsnorm_kernel, dim3(1), dim3(1024), s, d.h, (const float *)d.d1, (const float *)L.g2, d.xn, D, c.eps)))
            return rc;
        if ((rc = launch_gemv(L.wgu, d.xn, d.gu, 1, D, 2 * F, 1, 0, 0, DMC_LAYOUT_NK, DMC_W_BF16, -1, s))) return rc;
        if ((rc = launch_small(swiglu_kernel, dim3(8), dim3(256), s, (const float *)d.gu, d.act, F))) return rc;
        if ((rc = launch_gemv(L.wd, d.act, d.d2, 1, F, D, 1, 0, 0, DMC_LAYOUT_NK, DMC_W_BF16, -1, s))) return rc;
        carry = d.d2;
    }
    if ((rc = launch_small(rmsnorm_kernel, dim3(1), dim3(1024), s, d.h, carry, (const float *)d.gf, d.xn, D, c.eps))) return rc;
    if ((rc = launch_gemv(d.lm_head, d.xn, d.logits, 1, D, V, 1, 0, 0, DMC_LAYOUT_NK, DMC_W_BF16, -1, s))) return rc;
    return launch_small(argmax_kernel, dim3(64), dim3(256), s, (const float *)d.logits, V, d.d_next, d.am_val, d.am_idx, d.am_cnt);
}

int enqueue_step(Decoder &d, cudaStream_t s) { return d.fused ? enqueue_step_fused(d, s) : enqueue_step_plain(d, s); }

int ensure_graph(Decoder &d) {
    if (d.exec) return DMC_CUDA_OK;
    Context &c = ctx();
    int rc = enqueue_step(d, c.stream);  // eager once: kernel attributes and scratch are set up outside capture
    if (rc) return rc;
    DMC_CUDA_TRY(cudaStreamSynchronize(c.stream));
    const int64_t before = c.launches;
    DMC_CUDA_TRY(cudaStreamBeginCapture(c.stream, cudaStreamCaptureModeThreadLocal));
    rc = enqueue_step(d, c.stream);
    cudaError_t ce = cudaStreamEndCapture(c.stream, &d.graph);
    if (rc) return rc;
    DMC_CUDA_TRY(ce);
    d.launches_per_step = c.launches - before;
    DMC_CUDA_TRY(cudaGraphInstantiate(&d.exec, d.graph, 0));
    return DMC_CUDA_OK;
}

void *weight_slot(Decoder &d, int which, int layer, size_t *bytes) {
    const dmc_decoder_config &c = d.cfg;
    const size_t D = c.d_model, F = c.ffn, V = c.vocab;
    if (which == DMC_DEC_EMBED) { *bytes = V * D * 2; return d.embed; }
    if (which == DMC_DEC_LM_HEAD) { *bytes = V * D * 2; return d.lm_head; }
    if (which == DMC_DEC_GAIN_FINAL) { *bytes = D * 4; return d.gf; }
    if (layer < 0 || layer >= c.layers) return nullptr;
    Layer &L = d.layers[layer];
    switch (which) {
        case DMC_DEC_WQKV: *bytes = 3 * D * D * 2; return L.wqkv;
        case DMC_DEC_WO: *bytes = D * D * 2; return L.wo;
        case DMC_DEC_WGU: *bytes = 2 * F * D * 2; return L.wgu;
        case DMC_DEC_WD: *bytes = D * F * 2; return L.wd;
        case DMC_DEC_GAIN1: *bytes = D * 4; return L.g1;
        case DMC_DEC_GAIN2: *bytes = D * 4; return L.g2;
        default: return nullptr;
    }
}

}  // namespace
}  // namespace dmc

using namespace dmc;

extern "C" int dmc_decoder_create(const dmc_decoder_config *cfg, void **out) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    if (!cfg || !out || cfg->layers < 1 || cfg->d_model < 8 || cfg->heads < 1 || cfg->head_dim != 128 ||
        cfg->heads * cfg->head_dim != cfg->d_model || cfg->ffn < 8 || cfg->vocab < 1 || cfg->max_len < 1 ||
        cfg->d_model % 8 || cfg->ffn % 8)
        return fail(DMC_CUDA_ERR_BAD_ARG, "decoder_create: unsupported configuration (head_dim must be 128, "
                                          "heads*head_dim == d_model, d_model and ffn multiples of 8)");
    int rc = ensure_init();
    if (rc) return rc;
    Decoder *d = new Decoder();
    d->cfg = *cfg;
    const size_t D = cfg->d_model, F = cfg->ffn, V = cfg->vocab, H = cfg->heads, hd = cfg->head_dim, cap = cfg->max_len;
    d->layers.resize(cfg->layers);
    rc = dalloc(&d->embed, V * D) || dalloc(&d->lm_head, V * D) || dalloc(&d->gf, D) || dalloc(&d->rope_cos, cap * hd / 2) ||
         dalloc(&d->rope_sin, cap * hd / 2) || dalloc(&d->h, D) || dalloc(&d->xn, D) || dalloc(&d->qkv, 3 * D) ||
         dalloc(&d->ao, D) || dalloc(&d->d1, D) || dalloc(&d->gu, 2 * F) || dalloc(&d->act, F) || dalloc(&d->d2, D) ||
         dalloc(&d->logits, V) || dalloc(&d->part, H * (size_t)d->splits * (hd + 2)) || dalloc(&d->d_token, 1) ||
         dalloc(&d->d_pos, 1) || dalloc(&d->d_next, 1) || dalloc(&d->h2, D) || dalloc(&d->attn_cnt, H) ||
         dalloc(&d->am_val, 64) || dalloc(&d->am_idx, 64) || dalloc(&d->am_cnt, 1) || dalloc(&d->am_key, 1);
    d->fused = tuning().decode_fused;
    for (Layer &L : d->layers)
        rc = rc || dalloc(&L.wqkv, 3 * D * D) || dalloc(&L.wo, D * D) || dalloc(&L.wgu, 2 * F * D) || dalloc(&L.wd, D * F) ||
             dalloc(&L.g1, D) || dalloc(&L.g2, D) || dalloc(&L.kc, H * cap * hd) || dalloc(&L.vc, H * cap * hd);
    if (rc) return dmc::status();
    *out = d;
    return DMC_CUDA_OK;
}

extern "C" int dmc_decoder_load(void *dec, int which, int layer, const void *host, int64_t bytes) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    Decoder *d = static_cast<Decoder *>(dec);
    size_t want = 0;
    void *dst = nullptr;
    if (which == DMC_DEC_ROPE_COS || which == DMC_DEC_ROPE_SIN) {
        want = (size_t)d->cfg.max_len * d->cfg.head_dim / 2 * 4;
        dst = which == DMC_DEC_ROPE_COS ? d->rope_cos : d->rope_sin;
    } else if (which == DMC_DEC_KCACHE || which == DMC_DEC_VCACHE) {
        if (layer < 0 || layer >= d->cfg.layers) return fail(DMC_CUDA_ERR_BAD_ARG, "decoder_load: bad layer %d", layer);
        want = (size_t)d->cfg.heads * d->cfg.max_len * d->cfg.head_dim * 4;
        dst = which == DMC_DEC_KCACHE ? d->layers[layer].kc : d->layers[layer].vc;
    } else {
        dst = weight_slot(*d, which, layer, &want);
    }
    if (!dst || !host || (size_t)bytes != want)
        return fail(DMC_CUDA_ERR_BAD_ARG, "decoder_load: tensor %d layer %d wants %zu bytes, got %lld", which, layer, want,
                    (long long)bytes);
    DMC_CUDA_TRY(cudaMemcpyAsync(dst, host, want, cudaMemcpyHostToDevice, ctx().stream));
    DMC_CUDA_TRY(cudaStreamSynchronize(ctx().stream));
    return DMC_CUDA_OK;
}

extern "C" int dmc_decoder_step(void *dec, int token, int pos, int *next_token, float *logits_out) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return dmc::status();
    Decoder *d = static_cast<Decoder *>(dec);
    if (pos < 0 || pos >= d->cfg.max_len) return fail(DMC_CUDA_ERR_BAD_ARG, "decoder_step: pos %d outside the cache", pos);
    cudaStream_t s = ctx().stream;
    const int tp[2] = {token, pos};
    DMC_CUDA_TRY(cudaMemcpyAsync(d->d_token, &tp[0], 4, cudaMemcpyHostToDevice, s));
    DMC_CUDA_TRY(cudaMemcpyAsync(d->d_pos, &tp[1], 4, cudaMemcpyHostToDevice, s));
    DMC_CUDA_TRY(cudaStreamSynchronize(s));  // tp lives on this stack frame
    // (the first call also runs the step once eagerly before capturing it: token and pos are already
    // in place, so that run writes the same cache slot with the same values)
    int rc = ensure_graph(*d);
    if (rc) return rc;
    DMC_CUDA_TRY(cudaGraphLaunch(d->exec, s));
    ctx().launches += d->launches_per_step;
    int next = 0;
    unsigned long long key = 0ull;
    if (d->fused) DMC_CUDA_TRY(cudaMemcpyAsync(&key, d->am_key, 8, cudaMemcpyDeviceToHost, s));
    else DMC_CUDA_TRY(cudaMemcpyAsync(&next, d->d_next, 4, cudaMemcpyDeviceToHost, s));
    if (logits_out) DMC_CUDA_TRY(cudaMemcpyAsync(logits_out, d->logits, (size_t)d->cfg.vocab * 4, cudaMemcpyDeviceToHost, s));
    DMC_CUDA_TRY(cudaStreamSynchronize(s));
    stream_drained();
    if (d->fused) next = key ? (int)(0xFFFFFFFFu - (unsigned)(key & 0xFFFFFFFFull)) : 0;  // low half: 0xFFFFFFFF - row
    if (next_token) *next_token = next;
    return dmc::status();
}

extern "C" double dmc_decoder_bench(void *dec, int token, int pos, int steps, int warmup) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dmc::status()) return -1.0;
    Decoder *d = static_cast<Decoder *>(dec);
    cudaStream_t s = ctx().stream;
    if (steps < 1 || warmup < 0 || pos < 0 || pos >= d->cfg.max_len) {
        fail(DMC_CUDA_ERR_BAD_ARG, "decoder_bench: bad steps/warmup/pos");
        return -1.0;
    }
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    double us = -1.0;
    auto body = [&]() -> int {
        const int tp[2] = {token, pos};
        DMC_CUDA_TRY(cudaMemcpyAsync(d->d_token, &tp[0], 4, cudaMemcpyHostToDevice, s));
        DMC_CUDA_TRY(cudaMemcpyAsync(d->d_pos, &tp[1], 4, cudaMemcpyHostToDevice, s));
        DMC_CUDA_TRY(cudaStreamSynchronize(s));
        int rc = ensure_graph(*d);
        if (rc) return rc;
        DMC_CUDA_TRY(cudaEventCreate(&e0));
        DMC_CUDA_TRY(cudaEventCreate(&e1));
        for (int i = 0; i < warmup; ++i) DMC_CUDA_TRY(cudaGraphLaunch(d->exec, s));
        DMC_CUDA_TRY(cudaStreamSynchronize(s));
        DMC_CUDA_TRY(cudaEventRecord(e0, s));
        for (int i = 0; i < steps; ++i) DMC_CUDA_TRY(cudaGraphLaunch(d->exec, s));
        DMC_CUDA_TRY(cudaEventRecord(e1, s));
        DMC_CUDA_TRY(cudaStreamSynchronize(s));
        ctx().launches += d->launches_per_step * (warmup + steps);
        float ms = 0.0f;
        DMC_CUDA_TRY(cudaEventElapsedTime(&ms, e0, e1));
        us = (double)ms * 1000.0 / steps;
        return DMC_CUDA_OK;
    };
    body();
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    return dmc::status() ? -1.0 : us;
}

extern "C" int64_t dmc_decoder_launches_per_step(void *dec) { return static_cast<Decoder *>(dec)->launches_per_step; }

extern "C" void dmc_decoder_destroy(void *dec) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    Decoder *d = static_cast<Decoder *>(dec);
    if (!d) return;
    if (ctx().ready) cudaStreamSynchronize(ctx().stream);
    if (d->exec) cudaGraphExecDestroy(d->exec);
    if (d->graph) cudaGraphDestroy(d->graph);
    void *singles[] = {d->embed, d->lm_head, d->gf, d->rope_cos, d->rope_sin, d->h, d->xn, d->qkv, d->ao, d->d1, d->gu,
                       d->act, d->d2, d->logits, d->part, d->d_token, d->d_pos, d->d_next, d->h2, d->attn_cnt, d->am_val, d->am_idx, d->am_cnt,
                       d->am_key};
    for (void *p : singles)
        if (p) cudaFree(p);
    for (Layer &L : d->layers) {
        void *ps[] = {L.wqkv, L.wo, L.wgu, L.wd, L.g1, L.g2, L.kc, L.vc};
        for (void *p : ps)
            if (p) cudaFree(p);
    }
    delete d;
}
