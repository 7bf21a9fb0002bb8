#!/usr/bin/env python
"""Benchmark of the bf16-weight GEMV path (metric: achieved HBM GB/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1 (default): one step is the batch-1 decode-shape GEMV sweep
(rows x cols in {4096x4096, 11008x4096, 4096x11008, 14336x4096, 4096x14336},
y = W.x with bf16 W ~ N(0, 0.02), f32 x ~ U(-1, 1), f32 accumulate), each shape
rotating over enough distinct weight buffers that its working set exceeds L2.
N > 1 (under torchrun): the 65536x8192 weight row-sharded over the ranks, output
slices exchanged into a replicated y (bench_sharded.py).  Rank 0 prints ONE JSON
line.  `--impl reference` times the reference's CPU kernel (restated in oracle/,
the reference being a Rust crate that cannot be built here) on the same workload
and prints the same line shape.

    python bench.py --case 4096x4096 [--layout nk|kn] [--launches L] [--m M] [--op O] [--decode S] [--e2e C]

runs one small fixed case and prints its device time: the command profilers are
pointed at (a few launches of one shape over rotating weight copies, a few hundred
MiB on the device).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

from bench_common import (METRIC, NOMINAL_HBM_GBS, ROOT, ROTATE_BYTES, SHARDED, SWEEP, UNIT, ClockSampler,
                          make_shape_inputs, measured_peak, measured_tensor_peak, shard_weights, sharded_x, workload_text)

sys.path.insert(0, str(ROOT))

# the reference's own GPU bench shapes (compiler/src/gpu.rs:784-796): (name, batch, k, n)
REFERENCE_GPU_SHAPES = [("q-proj", 32, 2560, 128), ("kv-proj", 8, 2560, 128), ("wo", 32, 128, 2560),
                        ("ffn", 1, 2560, 9728), ("lm-head", 1, 2560, 151936)]

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture of the 4096x4096 case
# (33,615,104 B against 33,587,200 algorithmic: ratio 1.0008), scaled to the sweep's mean launch by the
# algorithmic bytes (traffic is the weight stream, which grows in proportion).
TRAFFIC_RATIO = 33615104 / 33587200


# --------------------------------------------------------------------------------------------
# the reference arm: the reference's CPU kernel on the host cores

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
        if (rows, cols) == SHARDED:
            w_nk, x = shard_weights(0, rows, seed), sharded_x(seed)
        else:
            w_nk, x = make_shape_inputs(rows, cols, seed + i)
        w_kn = oracle.bf16_transpose_2d(w_nk, rows, cols)       # what `x @ w'` materialises (jit.rs:29801)
        cases.append((w_kn, x.reshape(1, cols), np.empty((1, rows), np.float32)))
    return cases


def cpu_threads(shapes) -> int:
    import oracle
    return max(oracle.bf16_colsplit_ways(c, r) for r, c in shapes)


def run_reference(args, shapes, rank: int, world: int) -> None:
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
        "config": {"workload": workload_text(world)},
        "timed": "one pass of the CPU kernel over the workload per step, whole matrix on the host",
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
# this repo's arm, one GPU

def run_single(args) -> None:
    import demonic_b200 as dmc
    import oracle                      # the checker of the results the timed region produced, never timed itself
    from demonic_b200 import backend, synth
    from tests.parity import scaled_err

    lib = dmc.load()
    if lib.dmc_cuda_device_count() < 1:
        raise SystemExit("bench: no CUDA device (this backend has no CPU fallback)")
    peak, peak_kind = measured_peak()
    seed = synth.DEFAULT_SEED

    # resident weights: per shape, enough distinct copies that a pass over them exceeds L2 four times;
    # every GEMV of a step has its own output slot, so the results can be checked afterwards
    dev, host = [], []
    for i, (rows, cols) in enumerate(SWEEP):
        w, x = make_shape_inputs(rows, cols, seed + i)
        copies = max(2, -(-ROTATE_BYTES // w.nbytes))
        bufs = [backend.DeviceBuffer.from_host(w) for _ in range(copies)]
        dev.append((rows, cols, bufs, backend.DeviceBuffer.from_host(x), backend.DeviceBuffer(copies * rows * 4)))
        host.append((w, x))

    def items_for(entries, layout=backend.LAYOUT_NK):
        out = []
        for rows, cols, bufs, dx, dy in entries:
            out += [(b, dx, (dy, j * rows * 4), 1, cols, rows, layout, backend.W_BF16, -1) for j, b in enumerate(bufs)]
        return out

    step_items = items_for(dev)
    step_bytes = sum(synth.gemv_bytes(r, c) * len(b) for r, c, b, _, _ in dev)
    step_flops = sum(synth.gemv_flops(r, c) * len(b) for r, c, b, _, _ in dev)
    per_step = len(step_items)

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
    gpu_launches = per_step * args.steps
    value = step_bytes / us_step / 1e3

    # ---- what the timed region computed, against the oracle: every GEMV of the step ----
    parity = {"checked_gemvs": 0, "scaled_err_max": 0.0}
    for (rows, cols, bufs, dx, dy), (w, x) in zip(dev, host):
        ys = dy.download(np.float32, len(bufs) * rows).reshape(len(bufs), rows)
        ref = oracle.gemm_bf16_nt(x.reshape(1, cols), w).reshape(-1)
        for j in range(len(bufs)):
            parity["scaled_err_max"] = max(parity["scaled_err_max"], scaled_err(ys[j], ref))
            parity["checked_gemvs"] += 1
    if not parity["scaled_err_max"] <= 1e-2:
        raise SystemExit(f"bench: the timed region's results are off by {parity['scaled_err_max']:.3e} (> 1e-2)")

    # ---- the same step with every GEMV waiting for the one before it (a chain in which each x could be the
    # previous y): what a dependent sequence of these shapes costs ----
    lib.dmc_cuda_set_param(b"overlap_independent", 0)
    us_chain = backend.bench_items(step_items, args.steps, args.warmup, use_graph=True)
    lib.dmc_cuda_set_param(b"overlap_independent", 1)

    # ---- per-shape numbers (same protocol, one shape at a time), both ways ----
    shapes_out = []
    for entry in dev:
        rows, cols, bufs, dx, dy = entry
        b = synth.gemv_bytes(rows, cols)
        us = backend.bench_items(items_for([entry]), max(args.steps, 5), args.warmup) / len(bufs)
        lib.dmc_cuda_set_param(b"overlap_independent", 0)
        us_dep = backend.bench_items(items_for([entry]), max(args.steps, 5), args.warmup) / len(bufs)
        lib.dmc_cuda_set_param(b"overlap_independent", 1)
        shapes_out.append({"shape": f"{rows}x{cols}", "us_per_gemv": round(us, 3), "gbs": round(b / us / 1e3, 1),
                           "tflops": round(synth.gemv_flops(rows, cols) / us / 1e6, 3),
                           "frac_of_measured_peak": round(b / us / 1e3 / peak, 4),
                           "frac_of_nominal_8tbs": round(b / us / 1e3 / NOMINAL_HBM_GBS, 4),
                           "dependent_chain": {"us_per_gemv": round(us_dep, 3), "gbs": round(b / us_dep / 1e3, 1),
                                               "frac_of_nominal_8tbs": round(b / us_dep / 1e3 / NOMINAL_HBM_GBS, 4)},
                           "copies": len(bufs)})

    e2e = run_e2e(args, lib, dmc, backend, synth, host)

    # ---- CPU baseline: the reference's CPU kernel on the host cores, bounded sample ----
    e2e_bytes = sum(synth.gemv_bytes(r, c) for r, c in SWEEP)
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
    del cases

    # ---- the `--blas` form of the CPU path: sgemm on f32-widened weights (--blas applies to f32 x f32
    # only, compiler/src/jit.rs:20811, 29375-29400), through the BLAS bundled with NumPy ----
    cpu_blas = cpu_blas_baseline(host, e2e_bytes)

    extras = run_extras(args, lib, backend, synth, dev[0][2], peak)
    for _, _, bufs, dx, dy in dev:
        for b in bufs:
            b.free()
    extras["sharded_1gpu"] = run_sharded_one_gpu(args, lib, backend, synth, peak)

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": us_step / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "weights": "bf16 (widened exactly, f32 FMA accumulate)", "data": "synthetic",
        "config": {"workload": workload_text(1)},
        "protocol": {"shapes": [f"{r}x{c}" for r, c in SWEEP], "gemvs_per_step": per_step,
                     "l2": f"inputs larger than L2: each shape rotates over >= {ROTATE_BYTES >> 20} MiB of distinct weight copies",
                     "launch": "one CUDA graph replay per step, programmatic dependent launch between GEMVs",
                     "independence": "the GEMVs of a step share x and write distinct outputs; the library sees that none "
                                     "of them touches what another writes and lets them overlap (no dependency wait). "
                                     "`dependent_chain` is the same step with every GEMV waiting for its predecessor"},
        "tflops": step_flops / us_step / 1e6,
        "frac_of_nominal_8tbs": value / NOMINAL_HBM_GBS,
        "roofline": {"bound": "hbm", "achieved": value, "peak": peak, "unit": UNIT, "frac": value / peak,
                     "peak_kind": f"of {peak_kind}", "traffic": step_bytes / per_step * TRAFFIC_RATIO,
                     "algorithmic_bytes_per_launch": step_bytes / per_step,
                     "kernel": "dmc_wrows_kernel (all launches of the timed region)"},
        "dependent_chain": {"value": step_bytes / us_chain / 1e3, "unit": UNIT, "ms_per_step": us_chain / 1e3,
                            "frac_of_measured_peak": step_bytes / us_chain / 1e3 / peak,
                            "frac_of_nominal_8tbs": step_bytes / us_chain / 1e3 / NOMINAL_HBM_GBS},
        "parity": parity,
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


def run_e2e(args, lib, dmc, backend, synth, host) -> dict:
    """The sweep end to end through the C ABI with HOST buffers: every call copies its x to the device
    and its y back.  Headline form: the symbol the JIT binds (`dmc_matmul_bf16_gpu`, [k, n] weights found
    resident by fingerprint), one synchronous call per GEMV.  Beside it: the `x @ w'` form on registered
    [n, k] weights, and five deferred calls + one flush (compiler/src/jit.rs:8726-8744, 19908-19957)."""
    outs = [np.empty((1, r), np.float32) for r, _ in SWEEP]
    xs = [x.reshape(1, -1) for _, x in host]
    w_kn = [np.ascontiguousarray(w.T) for w, _ in host]                # [k, n]: what `x @ m.w` hands over
    e2e_bytes = sum(synth.gemv_bytes(r, c) for r, c in SWEEP)

    def timed(step):
        for _ in range(max(args.warmup, 1)):
            step()
        dmc.check()
        backend.sync()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step()
        backend.sync()
        dt = (time.perf_counter() - t0) / args.steps
        dmc.check()
        return dt

    # JIT-emitted code passes raw host addresses (i64): they are taken once, outside the timed loops
    calls_kn = [(x.ctypes.data, w.ctypes.data, out.ctypes.data, cols, rows)
                for w, x, out, (rows, cols) in zip(w_kn, xs, outs, SWEEP)]
    calls_nt = [(x.ctypes.data, w.ctypes.data, out.ctypes.data, cols, rows)
                for (w, _), x, out, (rows, cols) in zip(host, xs, outs, SWEEP)]

    def step_jit():
        for ax, aw, ao, cols, rows in calls_kn:
            lib.dmc_matmul_bf16_gpu(ax, aw, ao, 1, cols, rows)

    def step_deferred():
        for ax, aw, ao, cols, rows in calls_kn:
            lib.dmc_matmul_bf16_gpu_batched_deferred(ax, aw, ao, 1, cols, rows, 1, 0, 0)
        lib.dmc_matmul_bf16_gpu_flush()

    def step_nt():
        for ax, aw, ao, cols, rows in calls_nt:
            lib.dmc_matmul_bf16_gpu_nt(ax, aw, ao, 1, cols, rows)

    dt_jit = timed(step_jit)
    dt_def = timed(step_deferred)
    for w, _ in host:      # the vault-load hook: weights resident by registered range, as loaded ([n, k])
        rc = lib.dmc_cuda_register_weight(w.ctypes.data, w.nbytes, 0, 0, 0, backend.W_BF16)
        assert rc == 0, lib.dmc_cuda_last_error()
    dt_nt = timed(step_nt)
    for w, _ in host:
        lib.dmc_cuda_unregister_weight(w.ctypes.data)
    lib.dmc_cuda_drop_resident()
    h2d, d2h = sum(4 * c for _, c in SWEEP), sum(4 * r for r, _ in SWEEP)
    return {"value": e2e_bytes / dt_jit / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "ms_per_step": dt_jit * 1e3, "us_per_call": dt_jit * 1e6 / len(SWEEP),
            "note": "5 synchronous dmc_matmul_bf16_gpu calls per step on [k, n] host weights (resident by fingerprint), host x/out",
            "deferred": {"value": e2e_bytes / dt_def / 1e9, "unit": UNIT, "ms_per_step": dt_def * 1e3,
                         "note": "5 dmc_matmul_bf16_gpu_batched_deferred calls + one dmc_matmul_bf16_gpu_flush per step"},
            "nt_registered": {"value": e2e_bytes / dt_nt / 1e9, "unit": UNIT, "ms_per_step": dt_nt * 1e3,
                              "note": "5 synchronous dmc_matmul_bf16_gpu_nt calls per step on registered [n, k] weights"}}


def run_sharded_one_gpu(args, lib, backend, synth, peak) -> dict:
    """BASELINE config 5 on one GPU (the 1 of the 1/2/4/8 curve): the whole 65536x8192 weight (1 GiB, larger
    than L2 by itself) through the sharded entry point in a world of one."""
    from demonic_b200 import sharded
    rows, cols = SHARDED
    w = shard_weights(0, rows, synth.DEFAULT_SEED)
    dW = backend.DeviceBuffer.from_host(w)
    dx = backend.DeviceBuffer.from_host(sharded_x(synth.DEFAULT_SEED))
    del w
    sharded.init(0, 1, None, rows)
    try:
        us = sharded.bench([dW], dx, cols, rows, max(args.steps, 10), args.warmup, use_graph=True)
    finally:
        sharded.shutdown()
    dW.free()
    b = synth.gemv_bytes(rows, cols)
    return {"workload": workload_text(2), "us": round(us, 2), "gbs": round(b / us / 1e3, 1), "frac": round(b / us / 1e3 / peak, 4),
            "frac_of_nominal_8tbs": round(b / us / 1e3 / NOMINAL_HBM_GBS, 4)}


def run_extras(args, lib, backend, synth, w4096_bufs, hbm_peak) -> dict:
    """The other single-GPU configurations, reported beside the headline (not part of `value`):
    small-batch X @ W' with the GEMV -> tcgen05 crossover (config 3), the reference's own GPU bench shapes
    through the batched path, the tcgen05 GEMM on a dense contraction against the measured bf16 tensor
    peak, one decode step (config 4) and the weight ingest."""
    out = {}
    k = n = 4096
    rng = np.random.default_rng(synth.DEFAULT_SEED + 77)
    reps = max(args.steps, 5)
    rows = []
    for m in (1, 2, 4, 8, 16):
        xb = synth.bf16_weights(rng, (m, k))                      # bf16 activations N(0, 0.02)
        dXb = backend.DeviceBuffer.from_host(xb)
        dXf = backend.DeviceBuffer.from_host(synth.bf16_to_f32(xb))
        dY = backend.DeviceBuffer(len(w4096_bufs) * m * n * 4)
        ys = [(dY, j * m * n * 4) for j in range(len(w4096_bufs))]
        alg = n * k * 2 + m * k * 2 + m * n * 4
        lib.dmc_cuda_set_param(b"tc_min_m", 1 << 20)              # keep every row count on the CUDA cores for this column
        us_rows = backend.bench_items([(b, dXf, y, m, k, n, backend.LAYOUT_NK, backend.W_BF16, -1) for b, y in zip(w4096_bufs, ys)],
                                      reps, args.warmup) / len(w4096_bufs)
        lib.dmc_cuda_set_param(b"tc_min_m", 0)
        us_tc = backend.bench_items([(b, dXb, y, m, k, n, backend.LAYOUT_NK, backend.W_BF16, -1, 1) for b, y in zip(w4096_bufs, ys)],
                                    reps, args.warmup) / len(w4096_bufs)
        us_tcf = backend.bench_items([(b, dXf, y, m, k, n, backend.LAYOUT_NK, backend.W_BF16, -1, 2) for b, y in zip(w4096_bufs, ys)],
                                     reps, args.warmup) / len(w4096_bufs)
        us_lib = backend.bench_items([(b, dXf, y, m, k, n, backend.LAYOUT_NK, backend.W_BF16, -1) for b, y in zip(w4096_bufs, ys)],
                                     reps, args.warmup) / len(w4096_bufs)
        best = min(us_rows, us_tc)
        rows.append({"n": m, "us_cuda_core_rows_f32x": round(us_rows, 2), "us_tcgen05_bf16x": round(us_tc, 2),
                     "us_tcgen05_f32x_two_terms": round(us_tcf, 2), "us_library_choice_f32x": round(us_lib, 2),
                     "winner_bf16x": "cuda-core rows" if us_rows <= us_tc else "tcgen05", "gbs": round(alg / best / 1e3, 1),
                     "frac_of_measured_peak": round(alg / best / 1e3 / hbm_peak, 4)})
        for b in (dXb, dXf, dY):
            b.free()
    cross = next((r["n"] for r in rows if r["winner_bf16x"] == "tcgen05"), None)
    out["small_batch"] = {"workload": "X [N,4096] @ W' with W bf16 [4096,4096] (BASELINE config 3), f32 out; columns: the multi-row "
                                      "CUDA-core kernel with exact f32 X, the tcgen05 GEMM with bf16 X and with f32 X split in two bf16 terms",
                          "rows": rows, "crossover_to_tcgen05_at_n": cross}

    # the reference's own GPU bench shapes (compiler/src/gpu.rs:784-796, harness 698-808)
    shapes = []
    for name, batch, kk, nn in REFERENCE_GPU_SHAPES:
        wbytes = batch * kk * nn * 2
        copies = max(1, -(-ROTATE_BYTES // wbytes)) if wbytes < ROTATE_BYTES else 1
        w = synth.bf16_weights(rng, (batch, kk, nn))
        x = synth.activations(rng, (1, kk))
        alg = wbytes + 4 * kk + 4 * batch * nn
        dx = backend.DeviceBuffer.from_host(x)
        dy = backend.DeviceBuffer(copies * batch * nn * 4)
        if batch > 1:   # batched projection: x broadcast over the heads, the n-contiguous split-K kernel
            bufs = [backend.DeviceBuffer.from_host(w) for _ in range(copies)]
            items = [(b, dx, (dy, j * batch * nn * 4), 1, kk, nn, backend.LAYOUT_KN, backend.W_BF16, -1, 0, (batch, 0, kk * nn))
                     for j, b in enumerate(bufs)]
            kernel = "dmc_wcols_kernel (batched, split-K)"
        else:           # a single matrix is kept k-contiguous on the device and served by the row-streaming kernel
            wt = np.ascontiguousarray(w[0].T)
            bufs = [backend.DeviceBuffer.from_host(wt) for _ in range(copies)]
            items = [(b, dx, (dy, j * nn * 4), 1, kk, nn, backend.LAYOUT_NK, backend.W_BF16, -1) for j, b in enumerate(bufs)]
            kernel = "dmc_wrows_kernel"
        us = backend.bench_items(items, reps, args.warmup) / copies
        for b in bufs:
            b.free()
        # end to end through the reference's entry point with host buffers
        outb = np.empty((batch, nn), np.float32)
        ax, aw, ao = x.ctypes.data, w.ctypes.data, outb.ctypes.data
        call = (lambda: lib.dmc_matmul_bf16_gpu_batched(ax, aw, ao, 1, kk, nn, batch, 0, kk * nn)) \
            if batch > 1 else (lambda: lib.dmc_matmul_bf16_gpu(ax, aw, ao, 1, kk, nn))
        for _ in range(3):
            call()
        t0 = time.perf_counter()
        for _ in range(reps):
            call()
        dt = (time.perf_counter() - t0) / reps
        lib.dmc_cuda_drop_resident()
        shapes.append({"shape": f"{name} [{batch},{kk},{nn}]", "kernel": kernel, "us": round(us, 2),
                       "roofline": {"bound": "hbm", "achieved": round(alg / us / 1e3, 1), "peak": hbm_peak, "unit": UNIT,
                                    "frac": round(alg / us / 1e3 / hbm_peak, 4)},
                       "e2e_us_per_call": round(dt * 1e6, 1), "e2e_gbs": round(alg / dt / 1e9, 1), "copies": copies})
        dx.free(), dy.free()
    out["reference_gpu_bench_shapes"] = {"workload": "the shapes of the reference's own Metal benchmark, x [1,k] broadcast over `batch` "
                                                     "[k,n] bf16 weights; device-timed kernel and the reference entry point with host buffers",
                                         "shapes": shapes}

    # dense contraction on the tensor cores
    t_burst, t_kind = measured_tensor_peak()
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


# --------------------------------------------------------------------------------------------
# one small fixed case (what a profiler is pointed at)

def run_case(args) -> None:
    import demonic_b200 as dmc
    from demonic_b200 import backend, synth
    lib = dmc.load()
    for kv in args.param:
        name, val = kv.split("=")
        assert lib.dmc_cuda_set_param(name.encode(), int(val)) == 0, name
    if args.decode:
        from demonic_b200 import decoder
        cfg = decoder.Config()
        dec = decoder.Decoder(cfg, decoder.random_model(cfg, cache_len=512))
        for _ in range(args.decode):
            tok = dec.step(1234, 512)
        print(f"decode: {args.decode} steps, {dec.launches_per_step} launches per step, next token {tok}")
        return
    rows, cols = (int(t) for t in args.case.split("x"))
    rng = np.random.default_rng(synth.DEFAULT_SEED)
    if args.timeline:
        run_timeline(args, lib, backend, synth, rows, cols, rng)
        return
    if args.e2e:
        # host-pointer calls through the symbol the JIT binds: [k, n] host weight, host x and out
        w_kn = synth.bf16_weights(rng, (cols, rows))
        x = synth.activations(rng, (1, cols))
        out = np.empty((1, rows), np.float32)
        ax, aw, ao = x.ctypes.data, w_kn.ctypes.data, out.ctypes.data
        for _ in range(3):
            lib.dmc_matmul_bf16_gpu(ax, aw, ao, 1, cols, rows)
        launches0 = lib.dmc_cuda_launch_count()
        t0 = time.perf_counter()
        for _ in range(args.e2e):
            lib.dmc_matmul_bf16_gpu(ax, aw, ao, 1, cols, rows)
        dt = (time.perf_counter() - t0) / args.e2e
        assert lib.dmc_cuda_status() == 0, lib.dmc_cuda_last_error().decode()
        print(f"{args.case} e2e: {dt * 1e6:.1f} us per dmc_matmul_bf16_gpu call, "
              f"{(lib.dmc_cuda_launch_count() - launches0) // args.e2e} kernel launches per call")
        return
    w = synth.bf16_weights(rng, (rows, cols))
    x = synth.bf16_weights(rng, (args.m, cols)) if args.op == 1 else synth.activations(rng, (args.m, cols))
    copies = max(2, -(-(args.mib << 20) // w.nbytes))
    layout = backend.LAYOUT_NK if args.layout == "nk" else backend.LAYOUT_KN
    bufs = [backend.DeviceBuffer.from_host(w) for _ in range(copies)]
    dx, dy = backend.DeviceBuffer.from_host(x), backend.DeviceBuffer(args.launches * args.m * rows * 4)
    items = [(bufs[i % copies], dx, (dy, i * args.m * rows * 4), args.m, cols, rows, layout, backend.W_BF16, args.variant, args.op)
             for i in range(args.launches)]
    us = backend.bench_items(items, steps=1, warmup=1, use_graph=False) / len(items)
    b = synth.gemv_bytes(rows, cols, m=args.m)
    print(f"{args.case} {args.layout} m={args.m} op={args.op} variant={args.variant}: {us:.2f} us/launch, {b / us / 1e3:.0f} GB/s "
          f"(algorithmic bytes {b})")


def run_timeline(args, lib, backend, synth, rows, cols, rng) -> None:
    """Where the time between two GEMVs of a chain goes: per-CTA time stamps of `--launches` back-to-back
    GEMVs of one shape (dmc_cuda_timeline), once with every GEMV waiting for its predecessor and once with
    none waiting, reported relative to the moment the previous GEMV's last CTA finished."""
    import ctypes as C
    w = synth.bf16_weights(rng, (rows, cols))
    count = max(args.launches, 6)
    bufs = [backend.DeviceBuffer.from_host(w) for _ in range(count)]
    dx = backend.DeviceBuffer.from_host(synth.activations(rng, (cols,)))
    dy = backend.DeviceBuffer(rows * 4)
    ptrs = (C.c_void_p * count)(*[b.ptr for b in bufs])
    cap = count * 1024 * 8
    stamps = np.zeros(cap, np.uint64)
    b = synth.gemv_bytes(rows, cols)
    names = ["entry", "wait returned", "x staged", "first group done", "last group done"]
    for dependent in (1, 0):
        grid = lib.dmc_cuda_timeline(C.cast(ptrs, C.c_void_p), count, dx.ptr, dy.ptr, cols, rows, dependent,
                                     stamps.ctypes.data_as(C.c_void_p), cap)
        assert grid > 0, lib.dmc_cuda_last_error().decode()
        st = stamps[:count * grid * 8].reshape(count, grid, 8).astype(np.int64)
        ends = st[:, :, 4].max(axis=1)
        periods = np.diff(ends)[2:]
        print(f"{args.case} {'every GEMV waits for its predecessor' if dependent else 'no GEMV waits'}: grid {grid} CTAs, "
              f"period {np.median(periods) / 1e3:.2f} us per GEMV = {b / np.median(periods):.0f} GB/s "
              f"(min {periods.min() / 1e3:.2f}, max {periods.max() / 1e3:.2f} over {len(periods)} links)")
        print("  ns after the previous GEMV's last CTA finished: min / median / max over the CTAs, median over the links")
        rel = st[3:, :, :5] - ends[2:-1, None, None]
        for j, name in enumerate(names):
            col = rel[:, :, j]
            print(f"    {name:18s} {int(np.median(col.min(axis=1))):7d} / {int(np.median(np.median(col, axis=1))):7d} / {int(np.median(col.max(axis=1))):7d}")
        sms = st[3, :, 5]
        per_sm = np.bincount(sms.astype(int))
        print(f"  CTAs per SM in one launch: {dict(zip(*np.unique(per_sm[per_sm > 0], return_counts=True)))}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--case", default=None, help="rows x cols of W: run this one small case instead of the benchmark")
    ap.add_argument("--layout", default="nk", choices=["nk", "kn"])
    ap.add_argument("--launches", type=int, default=8)
    ap.add_argument("--variant", type=int, default=-1)
    ap.add_argument("--mib", type=int, default=256, help="--case: distinct weight bytes to rotate over")
    ap.add_argument("--m", type=int, default=1, help="--case: activation rows")
    ap.add_argument("--op", type=int, default=0, help="--case: 0 GEMV kernels, 1 tcgen05 GEMM (bf16 x), 2 tcgen05 GEMM (f32 x)")
    ap.add_argument("--e2e", type=int, default=0, help="--case: run this many host-pointer calls (dmc_matmul_bf16_gpu) on the shape instead")
    ap.add_argument("--decode", type=int, default=0, help="--case: run this many decode steps of the benchmark model instead")
    ap.add_argument("--param", action="append", default=[], help="--case: tuning knob name=value")
    ap.add_argument("--timeline", action="store_true", help="--case: per-CTA time stamps of a chain of GEMVs of this shape")
    args = ap.parse_args()
    if args.case or args.decode:
        run_case(args)
        return
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    if args.impl == "reference":
        run_reference(args, [SHARDED] if world > 1 else SWEEP, rank, world)
        return
    if world > 1:
        import bench_sharded
        bench_sharded.run(args, rank, world)
        return
    run_single(args)


if __name__ == "__main__":
    main()
