"""bench.py's multi-GPU arm: the 65536x8192 bf16 weight row-sharded over the ranks
(BASELINE config 5), output slices exchanged inside the library into a replicated y,
device-timed, maximum over ranks.  Launched by torchrun, one rank per GPU;
torch.distributed (gloo) carries only host plumbing: the NCCL id, barriers, the max over
ranks and the oracle slices of the parity check.

Before the sharded region rank 0 also times the whole matrix on its own GPU, so that the
line carries the one-GPU time of the same run and the speed-up can be read from it.
After the timed region, and after each run with a forced exchange, every rank compares
its whole replicated y (both buffers of the pair) with the CPU oracle.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np

from bench_common import (METRIC, NOMINAL_HBM_GBS, ROTATE_BYTES, SHARDED, UNIT, ClockSampler,
                          measured_peak, shard_weights, sharded_x, workload_text)

ROWS, COLS = SHARDED
EXCHANGE_TEXT = {
    "fused_peer_stores": "by the GEMV kernel itself (epoch-tagged peer stores over NVLink, validated by a gather kernel)",
    "nccl_allgather": "ncclAllGather after the kernel",
}


def oracle_full_y(rank: int, world: int, w_shard: np.ndarray, x: np.ndarray, r0: int, r1: int, dist) -> np.ndarray:
    """The whole y from the CPU oracle: every rank computes the rows of its own shard, the slices are
    gathered over gloo.  (The checker of the results; nothing here is timed.)"""
    import oracle
    mine = oracle.gemm_bf16_nt(x.reshape(1, COLS), w_shard).reshape(-1)
    parts = [None] * world
    dist.all_gather_object(parts, (r0, mine))
    y = np.empty(ROWS, np.float32)
    for a, piece in parts:
        y[a:a + piece.size] = piece
    return y


def run(args, rank: int, world: int) -> None:
    import torch.distributed as dist

    import demonic_b200 as dmc
    from demonic_b200 import backend, sharded, synth
    from tests.parity import scaled_err

    local = int(os.environ.get("LOCAL_RANK", rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lib = dmc.load()
    assert lib.dmc_cuda_init(local) == 0, lib.dmc_cuda_last_error().decode()
    peak, peak_kind = measured_peak()
    seed = synth.DEFAULT_SEED
    x = sharded_x(seed)
    dx = backend.DeviceBuffer.from_host(x)

    # ---- one GPU, same run: rank 0 streams the whole matrix (1 GiB, larger than L2 by itself) ----
    one_gpu_us = None
    if rank == 0:
        w_full = shard_weights(0, ROWS, seed)
        dfull = backend.DeviceBuffer.from_host(w_full)
        del w_full
        dy1 = backend.DeviceBuffer(ROWS * 4)
        one_gpu_us = backend.bench_items([(dfull, dx, dy1, 1, COLS, ROWS, backend.LAYOUT_NK, backend.W_BF16, -1)],
                                         max(args.steps, 10), args.warmup, use_graph=True)
        dfull.free()
        dy1.free()
    dist.barrier()

    ids = [sharded.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    sharded.init(rank, world, ids[0], ROWS)
    r0, r1 = sharded.shard_range(ROWS, rank, world)
    w = shard_weights(r0, r1, seed)
    # at least four GEMVs per step (a batch of independent exchanges: adjacent ones overlap), over distinct
    # copies of the shard that together exceed L2 several times
    copies = max(4, -(-ROTATE_BYTES // w.nbytes))
    bufs = [backend.DeviceBuffer.from_host(w) for _ in range(copies)]
    y_ref = oracle_full_y(rank, world, w, x, r0, r1, dist)

    def check(label: str) -> float:
        """This rank's whole replicated y, both buffers of the pair, against the oracle."""
        err = max(scaled_err(sharded.output(ROWS), y_ref), scaled_err(sharded.output_previous(ROWS), y_ref))
        errs = [None] * world
        dist.all_gather_object(errs, err)
        worst = max(errs)
        if not worst <= 1e-2:
            raise SystemExit(f"bench: {label}: replicated y off by {worst:.3e} on some rank (> 1e-2)")
        return worst

    parity = {"rows_checked_per_rank": ROWS, "buffers_checked": 2}
    sharded.gemv(bufs[0], dx, COLS, ROWS)
    sharded.gemv(bufs[-1], dx, COLS, ROWS)
    parity["before_timing"] = check("before the timed region")

    dist.barrier()
    backend.sync()
    launches0 = lib.dmc_cuda_launch_count()
    with ClockSampler(local) as clocks:
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
    parity["after_timed_region"] = check("after the timed region")
    chosen = "fused_peer_stores" if lib.dmc_cuda_shard_uses_fused(COLS, ROWS) else "nccl_allgather"
    dist.barrier()
    # the same step with each exchange forced: fused into the kernel (peer stores) and ncclAllGather
    forced, per_exchange = {}, {}
    for name, mode, overlap in (("fused_peer_stores", 1, 1), ("fused_peer_stores_one_exchange_at_a_time", 1, 0),
                                ("nccl_allgather", 0, 1)):
        lib.dmc_cuda_set_param(b"shard_fused", mode)
        lib.dmc_cuda_set_param(b"shard_overlap", overlap)
        dist.barrier()
        u = sharded.bench(bufs, dx, COLS, ROWS, args.steps, args.warmup, use_graph=True)
        backend.sync()
        allu = [None] * world
        dist.all_gather_object(allu, [u])
        forced[name] = max(v[0] for v in allu) / copies
        per_exchange[name] = check(f"after the run with {name}")
    lib.dmc_cuda_set_param(b"shard_fused", -1)
    lib.dmc_cuda_set_param(b"shard_overlap", 1)
    parity["per_exchange"] = per_exchange
    parity["scaled_err_max_over_ranks"] = max([parity["before_timing"], parity["after_timed_region"], *per_exchange.values()])
    alg = synth.gemv_bytes(ROWS, COLS)            # whole job: every weight byte once + x + y
    value = alg * copies / us_max / 1e3

    # end to end: host x in, the whole replicated y out in host memory on every rank, every step
    y_host = np.empty(ROWS, np.float32)
    ax, ay = x.ctypes.data, y_host.ctypes.data       # raw host addresses, taken once (what JIT-emitted code passes)
    for _ in range(args.warmup):
        sharded.gemv_host(bufs[0], x, y_host, COLS, ROWS)
    dist.barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        lib.dmc_cuda_shard_gemv_host(bufs[i % copies].ptr, ax, ay, COLS, ROWS, backend.W_BF16)
    dt = (time.perf_counter() - t0) / args.steps
    assert lib.dmc_cuda_status() == 0, lib.dmc_cuda_last_error().decode()
    e2e_err = scaled_err(y_host, y_ref)
    alle = [None] * world
    dist.all_gather_object(alle, [dt, e2e_err])
    dt_max = max(v[0] for v in alle)
    parity["e2e_host_pointers"] = max(v[1] for v in alle)
    if not parity["e2e_host_pointers"] <= 1e-2:
        raise SystemExit(f"bench: e2e: y off by {parity['e2e_host_pointers']:.3e} on some rank (> 1e-2)")
    dist.barrier()

    if rank == 0:
        us_gemv = us_max / copies
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": us_max / 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "weights": "bf16 (widened exactly, f32 FMA accumulate)", "data": "synthetic",
            "config": {"workload": workload_text(world)},
            "protocol": {"exchange": EXCHANGE_TEXT[chosen], "gemvs_per_step": copies, "rows_per_rank": r1 - r0,
                         "l2": f"inputs larger than L2: each rank rotates over {copies} distinct copies of its "
                               f"{w.nbytes >> 20} MiB shard",
                         "launch": "one CUDA graph replay per step",
                         "timing": "CUDA events per rank on the launching stream, max over ranks"},
            "tflops": synth.gemv_flops(ROWS, COLS) * copies / us_max / 1e6,
            "us_per_sharded_gemv": us_gemv,
            "one_gpu_us": one_gpu_us,
            "one_gpu_gbs": alg / one_gpu_us / 1e3,
            "speedup_vs_one_gpu": one_gpu_us / us_gemv,
            "efficiency": one_gpu_us / us_gemv / world,
            "us_per_sharded_gemv_by_exchange": forced,
            "frac_of_nominal_8tbs": value / (NOMINAL_HBM_GBS * world),
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": UNIT,
                         "frac": value / world / peak, "peak_kind": f"of {peak_kind}", "traffic": None,
                         "note": "per GPU: whole-job algorithmic bytes / world / step time (includes the exchange)"},
            "e2e": {"value": alg / dt_max / 1e9, "unit": UNIT, "h2d_bytes_per_step": 4 * COLS,
                    "d2h_bytes_per_step": 4 * ROWS, "ms_per_step": dt_max * 1e3,
                    "note": "per step and rank: one synchronous dmc_cuda_shard_gemv_host call (host x in, sharded GEMV with its exchange, the whole y in host memory); max over ranks"},
            "cpu_baseline": None,
            "clocks": clocks.summary(),
            "gpu_launches": launches_per_step * args.steps,
            "gpu_launches_including_warmup": launches_timed_run,
            "parity": parity,
        }
        print(json.dumps(line), flush=True)
    sharded.shutdown()
    dist.destroy_process_group()
