"""CPU restatement of one decode step from the oracle's pieces (test infrastructure): RMSNorm
(compiler/src/jit.rs:23776-23847), RoPE (compiler/src/interp.rs:13636-13678), KV attention
(compiler/src/jit.rs:20303-20506), SwiGLU with silu of compiler/src/interp.rs:13418, every projection
the interpreter's `@` (compiler/src/interp.rs:9270-9287) on the widened bf16 weights."""
import numpy as np

import oracle


def step(cfg, model, token: int, pos: int):
    d, h, hd, f = cfg.d_model, cfg.heads, cfg.head_dim, cfg.ffn
    x = oracle.embed_bf16(model["embed"], token)
    cs, sn = model["rope_cos"][pos], model["rope_sin"][pos]
    for L in model["layers"]:
        xn = oracle.rms_norm_f32(x, L["gain1"], cfg.eps)
        qkv = oracle.gemm_bf16_nt(xn.reshape(1, d), L["wqkv"])[0]
        q, k, v = qkv[:d].copy(), qkv[d:2 * d].copy(), qkv[2 * d:].copy()
        ao = np.empty(d, np.float32)
        for i in range(h):
            sl = slice(i * hd, (i + 1) * hd)
            q[sl] = oracle.rope_row(q[sl], cs, sn)
            L["kc"][i, pos] = oracle.rope_row(k[sl], cs, sn)
            L["vc"][i, pos] = v[sl]
            ao[sl] = oracle.kv_attention_head(q[sl], L["kc"][i, :pos + 1], L["vc"][i, :pos + 1])
        x = x + oracle.gemm_bf16_nt(ao.reshape(1, d), L["wo"])[0]
        xn = oracle.rms_norm_f32(x, L["gain2"], cfg.eps)
        gu = oracle.gemm_bf16_nt(xn.reshape(1, d), L["wgu"])[0]
        act = (oracle.silu(gu[:f]) * gu[f:]).astype(np.float32)
        x = x + oracle.gemm_bf16_nt(act.reshape(1, f), L["wd"])[0]
    xn = oracle.rms_norm_f32(x, model["gain_final"], cfg.eps)
    logits = oracle.gemm_bf16_nt(xn.reshape(1, d), model["lm_head"])[0]
    return oracle.argmax(logits), logits
