#!/usr/bin/env python3
"""diff_backends_cuda.py -- the `--cuda` column of the reference's backend differential.

tools/diff_backends.py asserts that `dmc run` and `dmc jit` print the same thing for every
example the JIT can run.  `dmc jit --cuda` cannot be held to byte equality -- the GPU sums in its
own order, like `--blas` (docs/NUMERICS.md §2.2) -- so its column compares numbers, not bytes:

  with a dmc binary (`--dmc PATH`, built with `--features cuda`):
      every example under `--examples` is run with `dmc jit` and with `dmc jit --cuda`; the two
      outputs must have the same text once numbers are masked out, and every pair of numbers
      must agree within rtol 1e-3 / atol 1e-4 (tools/numpy_oracle.py:41-42).  Files `dmc jit`
      refuses land in `jit-unsupported`, as in the reference's gate; a timeout fails the run.
      (Written against the reference's CLI; not run where this was written -- no cargo, no dmc.)

  without one (default):
      the matmul sites themselves are replayed: for each (m, k, n, batch) site shape of the
      reference's examples and benchmarks the CUDA builtin the JIT would bind is called with
      seeded inputs and compared with the CPU kernel the JIT would otherwise call
      (`dmc_matmul_bf16` / `dmc_matmul_par`, restated in this repository's oracle/), under the
      same tolerances plus the backend's bar (1e-2 scaled for bf16 weights, 1e-5 for f32).
      Sites the selection rule does not send to the GPU are listed as `not-selected` and must
      be left alone by the flag (the predicate says so; nothing is called).

Output is machine-greppable (`site-or-file: kind: message`); exit status 0 only if every compared
pair agrees.
"""
from __future__ import annotations

import argparse
import ctypes as C
import re
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
RTOL, ATOL = 1e-3, 1e-4
NUM = re.compile(r"[-+]?(?:\d+\.\d*|\.\d+|\d+)(?:[eE][-+]?\d+)?")

# (label, m, k, n, batch, bf16 weight?) -- matmul sites of the reference's examples and benches
SITES = [
    ("transformer ffn 2560x9728 (jit.rs:29961)", 1, 2560, 9728, 1, True),
    ("q-proj [32,2560,128] (gpu.rs:784)", 1, 2560, 128, 32, True),
    ("kv-proj [8,2560,128] (gpu.rs:786)", 1, 2560, 128, 8, True),
    ("wo [32,128,2560] (gpu.rs:788)", 1, 128, 2560, 32, True),
    ("decode 4096x4096", 1, 4096, 4096, 1, True),
    ("prefill 16x4096x4096", 16, 4096, 4096, 1, True),
    ("tiny field matmul [1,2]@[2,3] (jit.rs:42643)", 1, 2, 3, 1, True),
    ("attention scores, per head, small", 1, 128, 64, 16, True),
    ("blas probe 96^3 (jit.rs:39022)", 96, 96, 96, 1, False),
    ("f32 linear 2x512x384", 2, 512, 384, 1, False),
]


def compare_numbers(a: str, b: str) -> str | None:
    """None when two program outputs agree: same text around the numbers, numbers within tolerance."""
    if NUM.sub("#", a) != NUM.sub("#", b):
        return "outputs differ in text, not only in numbers"
    xs, ys = [float(t) for t in NUM.findall(a)], [float(t) for t in NUM.findall(b)]
    if xs and not np.allclose(xs, ys, rtol=RTOL, atol=ATOL):
        worst = max(abs(p - q) for p, q in zip(xs, ys))
        return f"numbers differ beyond rtol={RTOL} atol={ATOL} (max |d| = {worst:.3e})"
    return None


def run_programs(dmc: Path, examples: Path, timeout: int) -> int:
    counts = {"matched": 0, "jit-unsupported": 0, "diverged": 0, "timed-out": 0}
    for path in sorted(examples.rglob("*.dmc")):
        outs = []
        for flags in ([], ["--cuda"]):
            try:
                p = subprocess.run([str(dmc), "jit", *flags, str(path)], capture_output=True, text=True,
                                   timeout=timeout, stdin=subprocess.DEVNULL)
                outs.append((p.returncode, p.stdout))
            except subprocess.TimeoutExpired:
                outs.append((None, ""))
        if any(rc is None for rc, _ in outs):
            print(f"{path}: timed-out: exceeded {timeout}s")
            counts["timed-out"] += 1
        elif outs[0][0] != 0:
            counts["jit-unsupported"] += 1
        elif outs[1][0] != 0:
            print(f"{path}: diverged: `dmc jit --cuda` exited {outs[1][0]} where `dmc jit` succeeded")
            counts["diverged"] += 1
        else:
            why = compare_numbers(outs[0][1], outs[1][1])
            if why:
                print(f"{path}: diverged: {why}")
                counts["diverged"] += 1
            else:
                counts["matched"] += 1
    print("diff_backends_cuda: " + ", ".join(f"{v} {k}" for k, v in counts.items()))
    return 1 if counts["diverged"] or counts["timed-out"] else 0


def run_sites(lib_path: Path, verbose: bool) -> int:
    sys.path.insert(0, str(ROOT))
    import oracle                                   # the CPU kernels the JIT calls without the flag, restated
    from demonic_b200 import synth
    lib = C.CDLL(str(lib_path))
    I64 = C.c_int64
    lib.dmc_matmul_bf16_gpu.argtypes = lib.dmc_matmul_f32_gpu.argtypes = [I64] * 6
    lib.dmc_matmul_bf16_gpu_batched.argtypes = [I64] * 9
    lib.dmc_cuda_matmul_selected.argtypes = [C.c_int, C.c_uint32, I64, I64, I64, I64, C.c_int]
    lib.dmc_cuda_last_error.restype = C.c_char_p
    if lib.dmc_cuda_device_count() < 1:
        print("diff_backends_cuda: error: no CUDA device", file=sys.stderr)
        return 2
    rng = np.random.default_rng(0xDEC0DE)
    counts = {"matched": 0, "not-selected": 0, "diverged": 0}
    for label, m, k, n, batch, bf16 in SITES:
        if not lib.dmc_cuda_matmul_selected(1, 0, m, k, n, batch, int(bf16)):
            counts["not-selected"] += 1
            if verbose:
                print(f"{label}: not-selected: stays on the CPU kernel with the flag on")
            continue
        if lib.dmc_cuda_matmul_selected(1, 1, m, k, n, batch, int(bf16)) or lib.dmc_cuda_matmul_selected(0, 0, m, k, n, batch, int(bf16)):
            print(f"{label}: diverged: selected inside @deterministic or with the flag off")
            counts["diverged"] += 1
            continue
        x = synth.activations(rng, (m, k))
        if bf16:
            w = synth.bf16_weights(rng, (batch, k, n))
            cpu = np.stack([oracle.dmc_matmul_bf16(x, w[z]) for z in range(batch)])
            got = np.zeros((batch, m, n), np.float32)
            if batch == 1:
                lib.dmc_matmul_bf16_gpu(x.ctypes.data, w.ctypes.data, got.ctypes.data, m, k, n)
            else:
                lib.dmc_matmul_bf16_gpu_batched(x.ctypes.data, w.ctypes.data, got.ctypes.data, m, k, n, batch, 0, k * n)
            tol = 1e-2
        else:
            w = synth.f32_weights(rng, (k, n), std=1.0)
            cpu = oracle.dmc_matmul_par(x, w)[None]
            got = np.zeros((1, m, n), np.float32)
            lib.dmc_matmul_f32_gpu(x.ctypes.data, w.ctypes.data, got.ctypes.data, m, k, n)
            tol = 1e-5
        if lib.dmc_cuda_status() != 0:
            print(f"{label}: diverged: library status {lib.dmc_cuda_status()}: {lib.dmc_cuda_last_error().decode()}")
            return 1
        scale = max(float(np.max(np.abs(cpu))), 1e-30)
        err = float(np.max(np.abs(got.astype(np.float64) - cpu.astype(np.float64)))) / scale
        if err > tol or not np.allclose(got, cpu, rtol=RTOL, atol=ATOL):
            print(f"{label}: diverged: scaled error {err:.3e} (bar {tol:g}, rtol={RTOL} atol={ATOL})")
            counts["diverged"] += 1
        else:
            counts["matched"] += 1
            if verbose:
                print(f"{label}: matched: scaled error {err:.2e}")
    print("diff_backends_cuda: " + ", ".join(f"{v} {k}" for k, v in counts.items()))
    return 1 if counts["diverged"] else 0


def main() -> int:
    ap = argparse.ArgumentParser(description="`dmc jit` vs `dmc jit --cuda` differential")
    ap.add_argument("--dmc", type=Path, default=None, help="a dmc binary built with --features cuda: compare whole programs")
    ap.add_argument("--examples", type=Path, default=Path("examples"))
    ap.add_argument("--timeout", type=int, default=320)
    ap.add_argument("--lib", type=Path, default=ROOT / "demonic_b200" / "libdmc_cuda.so")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    if args.dmc is not None:
        return run_programs(args.dmc, args.examples, args.timeout)
    return run_sites(args.lib, args.verbose)


if __name__ == "__main__":
    sys.exit(main())
