"""Host side of the device-resident decode step (``dmc_decoder_*``): a random-init model with the
benchmark configuration's shapes and the thin wrapper that loads it and steps it."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib, synth

EMBED, WQKV, WO, WGU, WD, GAIN1, GAIN2, GAIN_FINAL, LM_HEAD, ROPE_COS, ROPE_SIN, KCACHE, VCACHE = range(13)


@dataclass
class Config:
    layers: int = 8
    d_model: int = 2048
    heads: int = 16
    head_dim: int = 128
    ffn: int = 5632
    vocab: int = 32000
    max_len: int = 513          # 512 cached positions + the token being decoded
    eps: float = 1e-6
    rope_theta: float = 10000.0

    def weight_bytes(self) -> int:
        d, f, v = self.d_model, self.ffn, self.vocab
        return 2 * (self.layers * (4 * d * d + 3 * d * f) + v * d)     # 57 GEMVs; the embedding row read is not counted

    def kv_bytes(self, length: int) -> int:
        return self.layers * 2 * self.heads * length * self.head_dim * 4


def rope_tables(cfg: Config):
    """cos/sin [max_len, head_dim/2] in f32; angle(s, i) = s * theta^(-2i/head_dim)."""
    half = cfg.head_dim // 2
    inv = cfg.rope_theta ** (-np.arange(half, dtype=np.float64) * 2.0 / cfg.head_dim)
    ang = np.arange(cfg.max_len, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def random_model(cfg: Config, seed: int = synth.DEFAULT_SEED, cache_len: int = 512) -> dict:
    """bf16 weights N(0, 0.02), unit gains perturbed a little, KV cache filled N(0, 1) for `cache_len` positions."""
    rng = np.random.default_rng(seed)
    d, f, v, h, hd = cfg.d_model, cfg.ffn, cfg.vocab, cfg.heads, cfg.head_dim
    m = {"embed": synth.bf16_weights(rng, (v, d)), "lm_head": synth.bf16_weights(rng, (v, d)),
         "gain_final": (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32), "layers": []}
    m["rope_cos"], m["rope_sin"] = rope_tables(cfg)
    for _ in range(cfg.layers):
        kc = np.zeros((h, cfg.max_len, hd), np.float32)
        vc = np.zeros((h, cfg.max_len, hd), np.float32)
        kc[:, :cache_len] = rng.standard_normal((h, cache_len, hd), dtype=np.float32)
        vc[:, :cache_len] = rng.standard_normal((h, cache_len, hd), dtype=np.float32)
        m["layers"].append({
            "wqkv": synth.bf16_weights(rng, (3 * d, d)), "wo": synth.bf16_weights(rng, (d, d)),
            "wgu": synth.bf16_weights(rng, (2 * f, d)), "wd": synth.bf16_weights(rng, (d, f)),
            "gain1": (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32),
            "gain2": (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32), "kc": kc, "vc": vc})
    return m


class Decoder:
    def __init__(self, cfg: Config, model: dict):
        self.cfg = cfg
        lib = _lib.load()
        c = _lib.DecoderConfig(cfg.layers, cfg.d_model, cfg.heads, cfg.head_dim, cfg.ffn, cfg.vocab, cfg.max_len, cfg.eps)
        self.handle = C.c_void_p()
        lib.dmc_decoder_create(C.byref(c), C.byref(self.handle))
        _lib.check()
        self._load(EMBED, 0, model["embed"])
        self._load(LM_HEAD, 0, model["lm_head"])
        self._load(GAIN_FINAL, 0, model["gain_final"])
        self._load(ROPE_COS, 0, model["rope_cos"])
        self._load(ROPE_SIN, 0, model["rope_sin"])
        for i, L in enumerate(model["layers"]):
            for which, key in ((WQKV, "wqkv"), (WO, "wo"), (WGU, "wgu"), (WD, "wd"), (GAIN1, "gain1"), (GAIN2, "gain2"),
                               (KCACHE, "kc"), (VCACHE, "vc")):
                self._load(which, i, L[key])

    def _load(self, which: int, layer: int, a: np.ndarray) -> None:
        a = np.ascontiguousarray(a)
        _lib.load().dmc_decoder_load(self.handle, which, layer, a.ctypes.data_as(C.c_void_p), a.nbytes)
        _lib.check()

    def step(self, token: int, pos: int, want_logits: bool = False):
        nxt = C.c_int()
        logits = np.empty(self.cfg.vocab, np.float32) if want_logits else None
        _lib.load().dmc_decoder_step(self.handle, token, pos, C.byref(nxt),
                                     logits.ctypes.data_as(C.c_void_p) if want_logits else None)
        _lib.check()
        return (nxt.value, logits) if want_logits else nxt.value

    def bench(self, token: int, pos: int, steps: int, warmup: int = 3) -> float:
        us = _lib.load().dmc_decoder_bench(self.handle, token, pos, steps, warmup)
        _lib.check()
        return float(us)

    @property
    def launches_per_step(self) -> int:
        return int(_lib.load().dmc_decoder_launches_per_step(self.handle))

    def close(self) -> None:
        if self.handle:
            _lib.load().dmc_decoder_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
