#!/usr/bin/env python
"""Benchmark of the bf16-weight GEMV path (metric: achieved HBM GB/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1 (default): one step is the batch-1 decode-shape GEMV sweep
(rows x cols in {4096x4096, 11008x4096, 4096x11008, 14336x4096, 4096x14336},
y = W.x with bf16 W ~ N(0, 0.02), f32 x ~ U(-1, 1), f32 accumulate), each shape
rotating over enough distinct weight buffers that its working set exceeds L2.
N > 1 (under torchrun): the 65536x8192 weight row-sharded over the ranks, output
slices all-gathered.  Rank 0 prints ONE JSON line.  `--impl reference` times the
reference's CPU kernel (restated in oracle/, the reference being a Rust crate
that cannot be built here) on the same workload and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SWEEP = [(4096, 4096), (11008, 4096), (4096, 11008), (14336, 4096), (4096, 14336)]   # (rows = n_out, cols = k)
SHARDED = (65536, 8192)
L2_BYTES = 126 << 20
ROTATE_BYTES = 512 << 20          # per-shape working set (>= 4 x L2)
METRIC = "bf16_gemv_hbm_bandwidth"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_PEAK_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            t0 = time.time()
            while not self.lines and time.time() - t0 < 5.0:      # nvidia-smi is up and sampling
                time.sleep(0.02)
        except OSError:
            self.proc = None
        self.before = len(self.lines)
        return self

    def samples_under_load(self) -> int:
        """Samples taken since the timed region began."""
        return len(self.lines) - self.before

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines[getattr(self, "before", 0):] or self.lines:
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = max(mx, float(f[1]))
            except ValueError:
                continue
            for name, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# workload

def make_shape_inputs(rows: int, cols: int, seed: int):
    """W [rows, cols] bf16 bits (k contiguous, "y = W.x") and x [cols] f32."""
    from demonic_b200 import synth
    rng = np.random.default_rng(seed)
    return synth.bf16_weights(rng, (rows, cols)), synth.activations(rng, (cols,))


def cpu_pass(cases) -> None:
    """One pass of the reference's CPU kernel over the workload: `dmc_matmul_bf16` with its
    own thread policy (compiler/src/jit.rs:29488-29566) on the [k, n] weights it would see."""
    import oracle
    for w_kn, x, out in cases:
        oracle.dmc_matmul_bf16(x, w_kn, out)


def cpu_cases(shapes, seed):
    import oracle
    cases = []
    for i, (rows, cols) in enumerate(shapes):
        w_nk, x = make_shape_inputs(rows, cols, seed + i)
        w_kn = oracle.bf16_transpose_2d(w_nk, rows, cols)       # what `x @ w'` materialises (jit.rs:29801)
        cases.append((w_kn, x.reshape(1, cols), np.empty((1, rows), np.float32)))
    return cases


def cpu_threads(shapes) -> int:
    import oracle
    return max(oracle.bf16_colsplit_ways(c, r) for r, c in shapes)


def run_reference(args, shapes, workload: str, rank: int, world: int) -> None:
    """Reference arm: the reference's own CPU implementation of the path on the host cores."""
    if rank != 0:
        return
    from demonic_b200 import synth
    cases = cpu_cases(shapes, synth.DEFAULT_SEED)
    alg = sum(synth.gemv_bytes(r, c) for r, c in shapes)
    for _ in range(max(args.warmup, 1)):
        cpu_pass(cases)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pass(cases)
    dt = (time.perf_counter() - t0) / args.steps
    gbs = alg / dt / 1e9
    cores = cpu_threads(shapes)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "f32", "weights": "bf16 (widened exactly, f32 FMA accumulate)", "data": "synthetic",
        "config": {"workload": workload, "timed": "one pass of the CPU kernel over the workload per step"},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port", "host_cores": os.cpu_count(),
                         "sample": f"{args.steps} passes over the workload; dmc_matmul_bf16 order and thread policy "
                                   f"(column split over {cores} threads), gcc -O3 -march=x86-64-v3"},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def cpu_blas_baseline(host, alg_bytes: int) -> dict:
    """cblas_sgemm(RowMajor, NoTrans, NoTrans, 1, n, k) on the widened [k, n] weights, ~5 s."""
    from demonic_b200 import synth
    cases = []
    for w_nk, x in host:
        w_kn = np.ascontiguousarray(synth.bf16_to_f32(w_nk).T)          # [k, n] f32, as `x @ w` sees it
        cases.append((x.reshape(1, -1), w_kn, np.empty((1, w_kn.shape[1]), np.float32)))
    threads, lib_name = None, "unknown"
    try:
        from threadpoolctl import threadpool_info
        for info in threadpool_info():
            if info.get("user_api") == "blas":
                threads, lib_name = info.get("num_threads"), f"{info.get('internal_api')} {info.get('version')}"
    except Exception:
        pass
    for x, w, out in cases:
        np.matmul(x, w, out=out)
    t0 = time.perf_counter()
    passes = 0
    while time.perf_counter() - t0 < 5.0:
        for x, w, out in cases:
            np.matmul(x, w, out=out)
        passes += 1
    dt = (time.perf_counter() - t0) / passes
    return {"value": alg_bytes / dt / 1e9, "unit": UNIT, "cores": threads, "kind": "port", "blas": lib_name,
            "note": "GB/s counted on the bf16 algorithmic bytes; the BLAS itself streams the 2x larger f32 copy",
            "sample": f"{passes} passes over the five sweep shapes (~5 s), np.matmul -> sgemm on f32-widened [k, n] weights"}


# --------------------------------------------------------------------------------------------
# our arm, one GPU

def run_single(args) -> None:
    import demonic_b200 as dmc
    from demonic_b200 import backend, synth

    lib = dmc.load()
    if lib.dmc_cuda_device_count() < 1:
        raise SystemExit("bench: no CUDA device (this backend has no CPU fallback)")
    peak, peak_kind = measured_peak()
    seed = synth.DEFAULT_SEED

    # resident weights: per shape, enough distinct copies that a pass over them exceeds L2 four times
    dev, host = [], []
    for i, (rows, cols) in enumerate(SWEEP):
        w, x = make_shape_inputs(rows, cols, seed + i)
        copies = max(2, -(-ROTATE_BYTES // w.nbytes))
        bufs = [backend.DeviceBuffer.from_host(w) for _ in range(copies)]
        dev.append((rows, cols, bufs, backend.DeviceBuffer.from_host(x), backend.DeviceBuffer(rows * 4)))
        host.append((w, x))

    def items_for(entries, layout=backend.LAYOUT_NK):
        out = []
        for rows, cols, bufs, dx, dy in entries:
            out += [(b, dx, dy, 1, cols, rows, layout, backend.W_BF16, -1) for b in bufs]
        return out

    step_items = items_for(dev)
    step_bytes = sum(synth.gemv_bytes(r, c) * len(b) for r, c, b, _, _ in dev)
    step_flops = sum(synth.gemv_flops(r, c) * len(b) for r, c, b, _, _ in dev)

    # ---- timed region: K steps, device-timed with CUDA events on the launching stream ----
    backend.sync()
    launches0 = lib.dmc_cuda_launch_count()
    with ClockSampler() as clocks:
        us_step = backend.bench_items(step_items, args.steps, args.warmup, use_graph=True)
        backend.sync()
        # a short timed region can fall between two samples: keep the same load running, untimed,
        # until the sampler has seen it a few times
        t_tail = time.time()
        while clocks.samples_under_load() < 3 and time.time() - t_tail < 2.0:
            backend.bench_items(step_items, args.steps, 0, use_graph=True)
    launches_total = lib.dmc_cuda_launch_count() - launches0
    # bench_items runs 1 eager sizing step + 1 captured step + warmup + K timed replays
    per_step = len(step_items)
    gpu_launches = per_step * args.steps
    value = step_bytes / us_step / 1e3

    # ---- per-shape numbers (same protocol, one shape at a time) ----
    shapes_out = []
    for entry in dev:
        rows, cols, bufs, dx, dy = entry
        us = backend.bench_items(items_for([entry]), max(args.steps, 5), args.warmup) / len(bufs)
        b = synth.gemv_bytes(rows, cols)
        shapes_out.append({"shape": f"{rows}x{cols}", "us_per_gemv": round(us, 3), "gbs": round(b / us / 1e3, 1),
                           "tflops": round(synth.gemv_flops(rows, cols) / us / 1e6, 3),
                           "frac_of_measured_peak": round(b / us / 1e3 / peak, 4),
                           "frac_of_nominal_8tbs": round(b / us / 1e3 / NOMINAL_HBM_GBS, 4), "copies": len(bufs)})

    # ---- end to end through the C ABI with host buffers (H2D of x, D2H of y every call) ----
    outs = [np.empty((1, r), np.float32) for r, _ in SWEEP]
    for w, _ in host:      # the vault-load hook: weights resident by registered range, as loaded ([n, k])
        rc = lib.dmc_cuda_register_weight(w.ctypes.data, w.nbytes, backend.W_BF16)
        assert rc == 0, lib.dmc_cuda_last_error()

    def e2e_step():
        for (w, x), out, (rows, cols) in zip(host, outs, SWEEP):
            lib.dmc_matmul_bf16_gpu_nt(x.ctypes.data, w.ctypes.data, out.ctypes.data, 1, cols, rows)

    for _ in range(args.warmup):
        e2e_step()
    dmc.check()
    backend.sync()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    backend.sync()
    e2e_dt = (time.perf_counter() - t0) / args.steps
    dmc.check()
    e2e_bytes = sum(synth.gemv_bytes(r, c) for r, c in SWEEP)
    e2e = {"value": e2e_bytes / e2e_dt / 1e9, "unit": UNIT, "h2d_bytes_per_step": sum(4 * c for _, c in SWEEP),
           "d2h_bytes_per_step": sum(4 * r for r, _ in SWEEP), "ms_per_step": e2e_dt * 1e3,
           "note": "5 synchronous dmc_matmul_bf16_gpu_nt calls per step with host x/out; weights resident"}

    # ---- CPU baseline: the reference's CPU kernel on the host cores, bounded sample ----
    cases = cpu_cases(SWEEP, seed)
    cpu_pass(cases)
    t0 = time.perf_counter()
    passes = 0
    while time.perf_counter() - t0 < 10.0:
        cpu_pass(cases)
        passes += 1
    cpu_dt = (time.perf_counter() - t0) / passes
    cpu = {"value": e2e_bytes / cpu_dt / 1e9, "unit": UNIT, "cores": cpu_threads(SWEEP), "kind": "port",
           "host_cores": os.cpu_count(),
           "sample": f"{passes} passes over the five sweep shapes (~10 s), dmc_matmul_bf16 order and thread policy"}

    # ---- the `--blas` form of the CPU path: sgemm on f32-widened weights (--blas applies to f32 x f32
    # only, compiler/src/jit.rs:20811, 29375-29400), through the BLAS bundled with NumPy ----
    cpu_blas = cpu_blas_baseline(host, e2e_bytes)

    extras = run_extras(args, lib, backend, synth, dev[0][2], peak)

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": us_step / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "weights": "bf16 (widened exactly, f32 FMA accumulate)", "data": "synthetic",
        "config": {"workload": "batch-1 decode-shape bf16 GEMV sweep (BASELINE config 2), y = W.x, W [rows, cols] k-contiguous",
                   "shapes": [f"{r}x{c}" for r, c in SWEEP], "gemvs_per_step": per_step,
                   "l2": f"inputs larger than L2: each shape rotates over >= {ROTATE_BYTES >> 20} MiB of distinct weight copies",
                   "launch": "one CUDA graph replay per step, programmatic dependent launch between GEMVs"},
        "tflops": step_flops / us_step / 1e6,
        "frac_of_nominal_8tbs": value / NOMINAL_HBM_GBS,
        "roofline": {"bound": "hbm", "achieved": value, "peak": peak, "unit": UNIT, "frac": value / peak,
                     "peak_kind": f"of {peak_kind}", "traffic": step_bytes / per_step * TRAFFIC_RATIO,
                     "algorithmic_bytes_per_launch": step_bytes / per_step,
                     "kernel": "gemv_nk_kernel (all launches of the timed region)"},
        "shapes": shapes_out,
        "e2e": e2e,
        "cpu_baseline": cpu,
        "cpu_blas": cpu_blas,
        "clocks": clocks.summary(),
        "gpu_launches": gpu_launches,
        "gpu_launches_including_warmup": launches_total,
    }
    line.update(extras)
    print(json.dumps(line), flush=True)


def run_extras(args, lib, backend, synth, w4096_bufs, hbm_peak) -> dict:
    """The other single-GPU configurations, reported beside the headline (not part of `value`):
    small-batch X @ W' with the GEMV -> tcgen05 crossover (config 3), the tcgen05 GEMM on a dense
    contraction against the measured bf16 tensor peak, and one decode step (config 4)."""
    out = {}
    k = n = 4096
    rng = np.random.default_rng(synth.DEFAULT_SEED + 77)
    rows = []
    for m in (1, 2, 4, 8, 16):
        xb = synth.bf16_weights(rng, (m, k))                      # bf16 activations N(0, 0.02)
        dXb = backend.DeviceBuffer.from_host(xb)
        dXf = backend.DeviceBuffer.from_host(synth.bf16_to_f32(xb))
        dY = backend.DeviceBuffer(m * n * 4)
        alg = n * k * 2 + m * k * 2 + m * n * 4
        us_gemv = backend.bench_items([(b, dXf, dY, m, k, n, backend.LAYOUT_NK, backend.W_BF16, 3) for b in w4096_bufs],
                                      max(args.steps, 5), args.warmup) / len(w4096_bufs)
        us_tc = backend.bench_items([(b, dXb, dY, m, k, n, backend.LAYOUT_NK, backend.W_BF16, -1, 1) for b in w4096_bufs],
                                    max(args.steps, 5), args.warmup) / len(w4096_bufs)
        best = min(us_gemv, us_tc)
        rows.append({"n": m, "us_gemv_kernel_per_row": round(us_gemv, 2), "us_tcgen05_gemm": round(us_tc, 2),
                     "winner": "gemv" if us_gemv <= us_tc else "tcgen05", "gbs": round(alg / best / 1e3, 1),
                     "frac_of_measured_peak": round(alg / best / 1e3 / hbm_peak, 4)})
    cross = next((r["n"] for r in rows if r["winner"] == "tcgen05"), None)
    out["small_batch"] = {"workload": "X bf16 [N,4096] @ W' with W bf16 [4096,4096] (BASELINE config 3), f32 out",
                          "rows": rows, "crossover_to_tcgen05_at_n": cross}
    # dense contraction on the tensor cores
    try:
        tpeak = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        t_burst, t_kind = float(tpeak["bf16_tflops"]), "measured"
    except Exception:
        t_burst, t_kind = 1590.0, "fallback"
    M = 8192
    dW = backend.DeviceBuffer.from_host(synth.bf16_weights(rng, (M, M)))
    dX = backend.DeviceBuffer.from_host(synth.bf16_weights(rng, (M, M)))
    dY = backend.DeviceBuffer(M * M * 4)
    us = backend.bench_items([(dW, dX, dY, M, M, M, backend.LAYOUT_NK, backend.W_BF16, -1, 1)], 5, 2)
    tf = 2.0 * M * M * M / us / 1e6
    out["dense_gemm"] = {"workload": "bf16 8192^3 X @ W' on tcgen05/TMEM, f32 out", "us": round(us, 1),
                         "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": t_burst, "unit": "TFLOP/s",
                                      "frac": round(tf / t_burst, 4), "peak_kind": f"of {t_kind} (cuBLAS burst)"}}
    for b in (dW, dX, dY):
        b.free()
    # one decode step (config 4)
    from demonic_b200 import decoder
    cfg = decoder.Config()
    dec = decoder.Decoder(cfg, decoder.random_model(cfg, cache_len=512))
    us = dec.bench(1234, 512, max(args.steps, 20), args.warmup)
    byt = cfg.weight_bytes() + cfg.kv_bytes(513)
    out["decode"] = {"workload": "one decode step, 8 layers, d_model 2048, 16x128 heads, FFN 5632, vocab 32000, bf16 weights, "
                                 "KV length 512 (+ the new token), batch 1 (BASELINE config 4), device resident, one CUDA graph",
                     "us_per_step": round(us, 1), "tokens_per_s": round(1e6 / us, 1), "launches_per_step": dec.launches_per_step,
                     "bytes_per_step": byt, "gbs": round(byt / us / 1e3, 1), "frac_of_measured_peak": round(byt / us / 1e3 / hbm_peak, 4),
                     "tokens_per_s_bound_at_measured_peak": round(hbm_peak * 1e9 / byt, 1)}
    dec.close()
    # weight ingest: a stored .npz (what numpy.savez writes) from the page cache into HBM
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        rows_i, cols_i = 32768, 8192                                   # 512 MiB of bf16
        path = os.path.join(tmp, "w.npz")
        np.savez(path, w=synth.bf16_weights(rng, (rows_i, cols_i)))
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            buf, _ = backend.load_npz(path, "w", rows_i, cols_i)
            dt = time.perf_counter() - t0
            buf.free()
            best = dt if best is None else min(best, dt)
        out["ingest"] = {"workload": "dmc_cuda_load_npz of a stored 32768x8192 bf16 entry (512 MiB), file in the page cache",
                         "ms": round(best * 1e3, 1), "gbs": round(rows_i * cols_i * 2 / best / 1e9, 2)}
    return out


# dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu capture of the 4096x4096 case
# summarised in profiles/gemv_nk_ldg_4096x4096_full.md (33,617,152 B against 33,587,200 algorithmic:
# ratio 1.0009), scaled to the sweep's mean launch by the algorithmic bytes (traffic is the weight
# stream, which grows in proportion).
TRAFFIC_RATIO = 33617152 / 33587200


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    if args.impl == "reference":
        if world > 1:
            run_reference(args, [SHARDED], "row-sharded 65536x8192 bf16 GEMV (BASELINE config 5), whole matrix on the host", rank, world)
        else:
            run_reference(args, SWEEP, "batch-1 decode-shape bf16 GEMV sweep (BASELINE config 2)", rank, world)
        return
    if world > 1:
        from demonic_b200 import sharded_bench
        sharded_bench.run(args, rank, world)
        return
    run_single(args)


if __name__ == "__main__":
    main()
