"""bench.py's multi-GPU arm: the 65536x8192 bf16 weight row-sharded over the ranks
(BASELINE config 5), output slices all-gathered inside the library, device-timed,
maximum over ranks.  Launched by torchrun, one rank per GPU; torch.distributed (gloo)
carries only host plumbing: the NCCL id, barriers and the max over ranks.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np

ROWS, COLS = 65536, 8192
BLOCK = 4096                      # rows generated per seed, so any rank can rebuild any row block
ROTATE_BYTES = 512 << 20


FUSED_FROM_WORLD = 2              # the library's own rule (shard_fused = -1): fused exchange from this many ranks up
EXCHANGE_TEXT = {
    "fused_peer_stores": "by the GEMV kernel itself (epoch-tagged peer stores over NVLink, validated by a gather kernel)",
    "nccl_allgather": "ncclAllGather after the kernel",
}


def block_weights(block: int, seed: int) -> np.ndarray:
    from . import synth
    return synth.bf16_weights(np.random.default_rng(seed + 1000 + block), (BLOCK, COLS))


def shard_weights(r0: int, r1: int, seed: int) -> np.ndarray:
    out = np.empty((r1 - r0, COLS), np.uint16)
    for b in range(r0 // BLOCK, -(-r1 // BLOCK)):
        w = block_weights(b, seed)
        lo, hi = max(r0, b * BLOCK), min(r1, (b + 1) * BLOCK)
        out[lo - r0:hi - r0] = w[lo - b * BLOCK:hi - b * BLOCK]
    return out


def run(args, rank: int, world: int) -> None:
    import torch.distributed as dist

    import demonic_b200 as dmc
    from . import backend, sharded, synth

    local = int(os.environ.get("LOCAL_RANK", rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lib = dmc.load()
    assert lib.dmc_cuda_init(local) == 0, lib.dmc_cuda_last_error().decode()
    ids = [sharded.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    sharded.init(rank, world, ids[0], ROWS)

    seed = synth.DEFAULT_SEED
    r0, r1 = sharded.shard_range(ROWS, rank, world)
    w = shard_weights(r0, r1, seed)
    x = synth.activations(np.random.default_rng(seed), (COLS,))
    copies = max(1, -(-ROTATE_BYTES // w.nbytes)) if w.nbytes < ROTATE_BYTES else 1
    bufs = [backend.DeviceBuffer.from_host(w) for _ in range(copies)]
    dx = backend.DeviceBuffer.from_host(x)

    # sanity check of 64 rows of this rank's slice against a float64 NumPy dot product
    sharded.gemv(bufs[0], dx, COLS, ROWS)
    y = sharded.output(ROWS)
    rows = np.linspace(0, r1 - r0 - 1, 64).astype(int)
    ref = synth.bf16_to_f32(w[rows]).astype(np.float64) @ x.astype(np.float64)
    err = float(np.max(np.abs(y[r0 + rows] - ref)) / max(np.max(np.abs(ref)), 1e-30))
    assert err <= 1e-2, f"rank {rank}: sharded GEMV off by {err:.3e}"
    # every rank must hold the same replicated y
    digest = [float(np.sum(y.astype(np.float64)))]
    alld = [None] * world
    dist.all_gather_object(alld, digest)
    assert all(abs(d[0] - alld[0][0]) == 0.0 for d in alld), f"replicas differ: {alld}"

    peak_file = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        peak, peak_kind = float(json.load(open(peak_file))["hbm_gbs"]), "measured"
    except Exception:
        peak, peak_kind = 6650.0, "fallback"

    import bench as bench_mod
    dist.barrier()
    backend.sync()
    launches0 = lib.dmc_cuda_launch_count()
    with bench_mod.ClockSampler(local) as clocks:
        us = sharded.bench(bufs, dx, COLS, ROWS, args.steps, args.warmup, use_graph=True)
        backend.sync()
        launches_timed_run = lib.dmc_cuda_launch_count() - launches0
        allt = [None] * world
        dist.all_gather_object(allt, [us])
        us_max = max(v[0] for v in allt)
        # The timed region lasts a few milliseconds: the same load, untimed, keeps running for ~0.3 s so
        # that the clock samples are taken under it.  The exchange is collective: every rank must run the
        # same number of steps, hence the count comes from the maximum over ranks, not from its own time.
        sharded.bench(bufs, dx, COLS, ROWS, max(1, int(3e5 / max(us_max, 1.0))), 0, use_graph=True)
        backend.sync()
    # dmc_cuda_bench_shard runs 1 eager step + 1 captured step + warmup + K timed replays
    launches_per_step = launches_timed_run // (2 + args.warmup + args.steps)
    dist.barrier()
    # the same step with each exchange forced: fused into the kernel (peer stores + flags) and ncclAllGather
    forced = {}
    for name, mode in (("fused_peer_stores", 1), ("nccl_allgather", 0)):
        lib.dmc_cuda_set_param(b"shard_fused", mode)
        dist.barrier()
        u = sharded.bench(bufs, dx, COLS, ROWS, args.steps, args.warmup, use_graph=True)
        backend.sync()
        allu = [None] * world
        dist.all_gather_object(allu, [u])
        forced[name] = max(v[0] for v in allu) / copies
    lib.dmc_cuda_set_param(b"shard_fused", -1)
    chosen = "fused_peer_stores" if world >= FUSED_FROM_WORLD else "nccl_allgather"
    alg = synth.gemv_bytes(ROWS, COLS)            # whole job: every weight byte once + x + y
    value = alg * copies / us_max / 1e3

    # end to end: host x in, replicated y out, every step
    for _ in range(args.warmup):
        dx.upload(x)
        sharded.gemv(bufs[0], dx, COLS, ROWS)
        sharded.output(ROWS)
    dist.barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        dx.upload(x)
        sharded.gemv(bufs[i % copies], dx, COLS, ROWS)
        sharded.output(ROWS)
    dt = (time.perf_counter() - t0) / args.steps
    alle = [None] * world
    dist.all_gather_object(alle, [dt])
    dt_max = max(v[0] for v in alle)
    dist.barrier()

    if rank == 0:
        line = {
            "metric": bench_mod.METRIC, "value": value, "unit": bench_mod.UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": us_max / 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "weights": "bf16 (widened exactly, f32 FMA accumulate)", "data": "synthetic",
            "config": {"workload": f"row-sharded bf16 GEMV {ROWS}x{COLS} (BASELINE config 5), rows split evenly over "
                                   f"{world} GPUs, output slices exchanged into a replicated y: "
                                   + EXCHANGE_TEXT[chosen],
                       "gemvs_per_step": copies, "rows_per_rank": r1 - r0,
                       "l2": f"inputs larger than L2: each rank rotates over {copies} distinct copies of its "
                             f"{w.nbytes >> 20} MiB shard",
                       "launch": "one CUDA graph replay per step",
                       "timing": "CUDA events per rank on the launching stream, max over ranks"},
            "tflops": synth.gemv_flops(ROWS, COLS) * copies / us_max / 1e6,
            "us_per_sharded_gemv": us_max / copies,
            "us_per_sharded_gemv_by_exchange": forced,
            "frac_of_nominal_8tbs": value / (bench_mod.NOMINAL_HBM_GBS * world),
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": bench_mod.UNIT,
                         "frac": value / world / peak, "peak_kind": f"of {peak_kind}", "traffic": None,
                         "note": "per GPU: whole-job algorithmic bytes / world / step time (includes the exchange)"},
            "e2e": {"value": alg / dt_max / 1e9, "unit": bench_mod.UNIT, "h2d_bytes_per_step": 4 * COLS,
                    "d2h_bytes_per_step": 4 * ROWS, "ms_per_step": dt_max * 1e3,
                    "note": "per step and rank: H2D of x, sharded GEMV with fused exchange, D2H of the whole y; max over ranks"},
            "cpu_baseline": None,
            "clocks": clocks.summary(),
            "gpu_launches": launches_per_step * args.steps,
            "gpu_launches_including_warmup": launches_timed_run,
            "parity": {"scaled_err_vs_f64_dot_rank0": err},
        }
        print(json.dumps(line), flush=True)
    sharded.shutdown()
    dist.destroy_process_group()
