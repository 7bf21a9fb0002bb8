"""Parity metrics shared by the GPU tests.

The GPU path sums in a different order than the reference's ascending-k chain
(K is split across warps and CTAs), so agreement is tolerance-equal, as the
reference accepts for its own GPU backend (compiler/src/gpu.rs:35-37) and for
`--blas` (docs/NUMERICS.md §2.2).  Bars: <= 1e-2 for bf16 weights and <= 1e-5
for f32, on max|y_gpu - y_ref| / max|y_ref| per output vector (elementwise
relative error is meaningless where N(0,0.02) x U(-1,1) sums land near zero),
plus the reference oracle's elementwise allclose(rtol=1e-3, atol=1e-4)
(tools/numpy_oracle.py:41-42)."""
import numpy as np

TOL_BF16 = 1e-2
TOL_F32 = 1e-5
RTOL, ATOL = 1e-3, 1e-4


def scaled_err(got: np.ndarray, ref: np.ndarray) -> float:
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    scale = max(float(np.max(np.abs(ref))) if ref.size else 0.0, 1e-30)
    return float(np.max(np.abs(got - ref))) / scale if ref.size else 0.0


def assert_parity(got, ref, tol, what=""):
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    err = scaled_err(got, ref)
    assert err <= tol, f"{what}: scaled error {err:.3e} > {tol:g}"
    assert np.allclose(np.asarray(got).reshape(-1), np.asarray(ref).reshape(-1), rtol=RTOL, atol=ATOL), \
        f"{what}: outside rtol={RTOL} atol={ATOL}"
    return err
