#!/usr/bin/env python3
"""numpy_oracle_cuda.py -- the NumPy oracle of tools/numpy_oracle.py, pointed at the CUDA matmul path.

The reference's harness runs tensor programs through `dmc run` and compares what they print with
an independent NumPy computation (tools/numpy_oracle.py:1-22).  This is the same gate for the one
operator the B200 backend takes over: `@`.  Inputs are drawn in NumPy from the harness's own seed
(0xDEC0DE; the first case draws the very numbers of its `matmul` case), handed to `libdmc_cuda`
through the builtins the JIT binds (raw host addresses, all-i64 ABI), and the result is compared
with a float64 NumPy reference written from the operator's definition -- deliberately not from the
library's code -- under the harness's tolerances (rtol 1e-3, atol 1e-4, tools/numpy_oracle.py:41-42)
plus the backend's own bar: max|y - ref| / max|ref| <= 1e-2 for bf16 weights, <= 1e-5 for f32.

    python3 numpy_oracle_cuda.py [--lib PATH/libdmc_cuda.so] [--verbose] [--meta-test]

`--meta-test` confirms the harness has teeth: a correct result checked against a deliberately
wrong reference must be flagged.  Diagnostics are machine-greppable: `oracle: name: kind: message`.
Exit status: 0 all cases match, 1 a mismatch, 2 no library or no CUDA device.
"""
from __future__ import annotations

import argparse
import ctypes as C
import sys
from pathlib import Path

import numpy as np

RTOL = 1e-3
ATOL = 1e-4
TOL_BF16 = 1e-2
TOL_F32 = 1e-5
I64 = C.c_int64
DEFAULT_LIB = Path(__file__).resolve().parents[2] / "demonic_b200" / "libdmc_cuda.so"


def load(path: Path) -> C.CDLL:
    lib = C.CDLL(str(path))
    for name, n in (("dmc_matmul_bf16_gpu", 6), ("dmc_matmul_f32_gpu", 6), ("dmc_matmul_bf16_gpu_nt", 6),
                    ("dmc_matmul_bf16_gpu_batched", 9), ("dmc_matmul_bf16_gpu_batched_deferred", 9)):
        getattr(lib, name).argtypes = [I64] * n
        getattr(lib, name).restype = None
    lib.dmc_matmul_bf16_gpu_flush.restype = None
    lib.dmc_cuda_last_error.restype = C.c_char_p
    return lib


def to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bf16 bit patterns (how the benchmark's weights are made)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)


def widen(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


class Case:
    def __init__(self, name, run, expected, tol):
        self.name, self.run, self.expected, self.tol = name, run, np.asarray(expected, np.float64), tol


def build_cases(lib, rng: np.random.Generator) -> list[Case]:
    cases: list[Case] = []
    f32 = np.float32

    # the reference harness's own `matmul` case: same draws, same shapes (tools/numpy_oracle.py:118-121)
    A = rng.uniform(-2, 2, (3, 4))
    B = rng.uniform(-2, 2, (4, 2))
    a32, b32 = np.ascontiguousarray(A, f32), np.ascontiguousarray(B, f32)

    def run_small():
        out = np.zeros((3, 2), f32)
        lib.dmc_matmul_f32_gpu(a32.ctypes.data, b32.ctypes.data, out.ctypes.data, 3, 4, 2)
        return out
    cases.append(Case("matmul", run_small, a32.astype(np.float64) @ b32.astype(np.float64), TOL_F32))

    # the decode GEMV `x @ m.w`, bf16 weight [K, N], at a shape the flag selects (k*n >= 4e6)
    k, n = 2560, 2048
    w = to_bf16(rng.standard_normal((k, n)) * 0.02)
    x = rng.uniform(-1, 1, (1, k)).astype(f32)

    def run_gemv():
        out = np.zeros((1, n), f32)
        lib.dmc_matmul_bf16_gpu(x.ctypes.data, w.ctypes.data, out.ctypes.data, 1, k, n)
        return out
    cases.append(Case("matmul_bf16_gemv", run_gemv, x.astype(np.float64) @ widen(w).astype(np.float64), TOL_BF16))

    # `x @ m.w'` with the weight stored [N, K]
    wt = np.ascontiguousarray(w.T)

    def run_nt():
        out = np.zeros((1, n), f32)
        lib.dmc_matmul_bf16_gpu_nt(x.ctypes.data, wt.ctypes.data, out.ctypes.data, 1, k, n)
        return out
    cases.append(Case("matmul_bf16_transposed", run_nt, x.astype(np.float64) @ widen(w).astype(np.float64), TOL_BF16))

    # prefill rows (m > 1): a few rows, and enough rows to reach the tensor cores
    for m in (4, 32):
        xm = rng.uniform(-1, 1, (m, k)).astype(f32)

        def run_rows(xm=xm, m=m):
            out = np.zeros((m, n), f32)
            lib.dmc_matmul_bf16_gpu_nt(xm.ctypes.data, wt.ctypes.data, out.ctypes.data, m, k, n)
            return out
        cases.append(Case(f"matmul_bf16_rows_{m}", run_rows, xm.astype(np.float64) @ widen(w).astype(np.float64), TOL_BF16))

    # a batched per-head projection [1, K] @ [H, K, N] (x broadcast), synchronous and deferred + flush
    H, kk, nn = 8, 2560, 128
    wh = to_bf16(rng.standard_normal((H, kk, nn)) * 0.02)
    xh = rng.uniform(-1, 1, (1, kk)).astype(f32)
    ref_h = np.stack([xh[0].astype(np.float64) @ widen(wh[h]).astype(np.float64) for h in range(H)])

    def run_batched():
        out = np.zeros((H, nn), f32)
        lib.dmc_matmul_bf16_gpu_batched(xh.ctypes.data, wh.ctypes.data, out.ctypes.data, 1, kk, nn, H, 0, kk * nn)
        return out

    def run_deferred():
        out = np.zeros((H, nn), f32)
        lib.dmc_matmul_bf16_gpu_batched_deferred(xh.ctypes.data, wh.ctypes.data, out.ctypes.data, 1, kk, nn, H, 0, kk * nn)
        lib.dmc_matmul_bf16_gpu_flush()
        return out
    cases.append(Case("matmul_bf16_batched", run_batched, ref_h, TOL_BF16))
    cases.append(Case("matmul_bf16_batched_deferred", run_deferred, ref_h, TOL_BF16))

    # f32 weights through the f32 builtin (the `--blas`-sized site)
    wf = (rng.standard_normal((512, 384)) * 0.02).astype(f32)
    xf = rng.uniform(-1, 1, (2, 512)).astype(f32)

    def run_f32():
        out = np.zeros((2, 384), f32)
        lib.dmc_matmul_f32_gpu(xf.ctypes.data, wf.ctypes.data, out.ctypes.data, 2, 512, 384)
        return out
    cases.append(Case("matmul_f32", run_f32, xf.astype(np.float64) @ wf.astype(np.float64), TOL_F32))
    return cases


def mismatch(got: np.ndarray, expected: np.ndarray, tol: float) -> str | None:
    if got.shape != expected.shape:
        return f"shape {got.shape} != numpy {expected.shape}"
    if not np.all(np.isfinite(got)):
        return "non-finite output"
    scale = max(float(np.max(np.abs(expected))), 1e-30)
    err = float(np.max(np.abs(got - expected)))
    if err / scale > tol:
        return f"max|d|/max|ref|={err / scale:.2e} exceeds {tol:g}"
    if not np.allclose(got, expected, rtol=RTOL, atol=ATOL):
        return f"max|d|={err:.2e} exceeds rtol={RTOL} atol={ATOL}"
    return None


def main() -> int:
    ap = argparse.ArgumentParser(description="numpy reference oracle for the CUDA matmul path")
    ap.add_argument("--lib", type=Path, default=DEFAULT_LIB)
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--meta-test", action="store_true", help="assert the harness catches a deliberately-wrong reference")
    args = ap.parse_args()
    if not args.lib.exists():
        print(f"oracle: error: library not found at {args.lib} (build it with `python -m demonic_b200.build`)", file=sys.stderr)
        return 2
    lib = load(args.lib)
    if lib.dmc_cuda_device_count() < 1:
        print("oracle: error: no CUDA device (the backend has no CPU fallback to check instead)", file=sys.stderr)
        return 2
    rng = np.random.default_rng(0xDEC0DE)
    cases = build_cases(lib, rng)
    failures = []
    for c in cases:
        got = np.asarray(c.run(), np.float64)
        if lib.dmc_cuda_status() != 0:
            print(f"oracle: {c.name}: error: library status {lib.dmc_cuda_status()}: {lib.dmc_cuda_last_error().decode()}", file=sys.stderr)
            return 1
        why = mismatch(got, c.expected, c.tol)
        if why:
            print(f"oracle: {c.name}: error: {why}", file=sys.stderr)
            failures.append(c.name)
        elif args.verbose:
            print(f"oracle: {c.name}: ok")
    if args.meta_test:
        c = next(x for x in cases if x.name == "matmul_bf16_gemv")
        got = np.asarray(c.run(), np.float64)
        wrong = c.expected * 1.02 + 0.01        # a reference that is off by 2 %
        if mismatch(got, wrong, c.tol) is None:
            print("oracle: meta-test: error: harness did NOT catch a wrong reference", file=sys.stderr)
            return 1
        print("oracle: meta-test: ok -- wrong reference correctly flagged")
    print(f"oracle: {len(cases) - len(failures)}/{len(cases)} matmul cases match numpy (rtol={RTOL}, atol={ATOL}; "
          f"scaled {TOL_BF16:g} bf16 / {TOL_F32:g} f32)")
    return 1 if failures else 0


if __name__ == "__main__":
    sys.exit(main())
