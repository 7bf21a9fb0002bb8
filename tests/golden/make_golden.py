"""Generates tests/golden/matmul_golden.npz: seeded inputs (by seed) and the
CPU oracle's outputs for a handful of matmul cases.

The reference cannot be run where this repository is developed (Rust crate, no
toolchain), so the expected values come from the oracle, which is itself pinned
to the reference's known-answer tests by tests/test_oracle_pins.py.  Inputs are
regenerated from the stored seed; a SHA-256 of the regenerated inputs is stored
to catch generator drift.

    python tests/golden/make_golden.py
"""
import hashlib
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402
from demonic_b200 import synth  # noqa: E402

# name, kind, m, k, n, batch, ls_kind, rs_kind, seed
CASES = [
    ("bf16_gemv_256x512", "bf16", 1, 256, 512, 1, 0, 0, 11),
    ("bf16_gemv_1000x264", "bf16", 1, 1000, 264, 1, 0, 0, 12),
    ("bf16_gemv_odd_37x13", "bf16", 1, 37, 13, 1, 0, 0, 13),
    ("bf16_gemm_m3_64x40", "bf16", 3, 64, 40, 1, 0, 0, 14),
    ("bf16_gemm_m5_640x136", "bf16", 5, 640, 136, 1, 0, 0, 15),
    ("bf16_batched_qproj_b8", "bf16", 1, 320, 128, 8, "zero", "full", 16),   # [1,1,K] @ [H,K,N]
    ("bf16_batched_wo_b4", "bf16", 1, 128, 320, 4, "full", "full", 17),      # [H,1,K] @ [H,K,N]
    ("bf16_batched_bcast_w_b3", "bf16", 1, 96, 64, 3, "full", "zero", 18),   # shared weight
    ("f32_gemv_300x260", "f32", 1, 300, 260, 1, 0, 0, 19),
    ("f32_gemm_96", "f32", 96, 96, 96, 1, 0, 0, 20),
    ("bf16_nt_gemv_520x264", "nt", 1, 264, 520, 1, 0, 0, 21),
]


def make_inputs(kind, m, k, n, batch, ls_kind, rs_kind, seed):
    rng = np.random.default_rng(seed)
    ls = m * k if ls_kind == "full" else 0
    rs = k * n if rs_kind == "full" else 0
    l = synth.activations(rng, ((batch - 1) * ls + m * k,))
    if kind == "f32":
        r = synth.f32_weights(rng, ((batch - 1) * rs + k * n,))
    else:
        r = synth.bf16_weights(rng, ((batch - 1) * rs + k * n,))
    return l, r, ls, rs


def expected(kind, l, r, m, k, n, batch, ls, rs):
    if kind == "f32":
        return oracle.gemm_f32_fma(l.reshape(m, k), r.reshape(k, n))
    if kind == "nt":        # r is stored [n, k]; the reference transposes then multiplies
        w_kn = oracle.bf16_transpose_2d(r, n, k)
        return oracle.gemm_bf16_fma(l.reshape(m, k), w_kn)
    if batch == 1:
        return oracle.gemm_bf16_fma(l.reshape(m, k), r.reshape(k, n))
    return oracle.bf16_gemv_batched(l, r, k, n, batch, ls, rs)


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def main():
    out = {}
    for name, kind, m, k, n, batch, lsk, rsk, seed in CASES:
        l, r, ls, rs = make_inputs(kind, m, k, n, batch, lsk, rsk, seed)
        y = expected(kind, l, r, m, k, n, batch, ls, rs)
        out[name + "/y"] = np.ascontiguousarray(y, np.float32).reshape(-1)
        out[name + "/sha"] = np.frombuffer(digest(l, r).encode(), np.uint8)
    np.savez_compressed(Path(__file__).with_name("matmul_golden.npz"), **out)
    print("wrote", len(CASES), "cases")


if __name__ == "__main__":
    main()
