"""Pieces shared by the benchmark's arms (bench.py, bench_sharded.py): workload descriptions,
the measured roofline denominator, the clock sampler and the seeded weight blocks."""
from __future__ import annotations

import json
import subprocess
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent

SWEEP = [(4096, 4096), (11008, 4096), (4096, 11008), (14336, 4096), (4096, 14336)]   # (rows = n_out, cols = k)
SHARDED = (65536, 8192)
BLOCK = 4096                      # rows of the sharded weight generated per seed, so any rank can rebuild any block
ROTATE_BYTES = 512 << 20          # per-shape working set (>= 4 x L2)
METRIC = "bf16_gemv_hbm_bandwidth"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0

# `config.workload` of a line: the same text for this repo's arm and for the reference arm at a given N
WORKLOAD_SWEEP = ("batch-1 decode-shape bf16 GEMV sweep (BASELINE config 2): y = W.x for W [rows, cols] in "
                  "{4096x4096, 11008x4096, 4096x11008, 14336x4096, 4096x14336}, bf16 W ~ N(0, 0.02), f32 x ~ U(-1, 1), f32 accumulate")
WORKLOAD_SHARDED = ("row-sharded bf16 GEMV 65536x8192 (BASELINE config 5): bf16 W ~ N(0, 0.02), f32 x ~ U(-1, 1), rows split "
                    "evenly over the GPUs, output slices exchanged into a replicated y")


def workload_text(world: int) -> str:
    return WORKLOAD_SHARDED if world > 1 else WORKLOAD_SWEEP


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_PEAK_GBS, "fallback"


def measured_tensor_peak():
    try:
        return float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


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


def make_shape_inputs(rows: int, cols: int, seed: int):
    """W [rows, cols] bf16 bits (k contiguous, "y = W.x") and x [cols] f32."""
    from demonic_b200 import synth
    rng = np.random.default_rng(seed)
    return synth.bf16_weights(rng, (rows, cols)), synth.activations(rng, (cols,))


def block_weights(block: int, seed: int) -> np.ndarray:
    """Rows [block * BLOCK, (block + 1) * BLOCK) of the sharded 65536x8192 weight."""
    from demonic_b200 import synth
    return synth.bf16_weights(np.random.default_rng(seed + 1000 + block), (BLOCK, SHARDED[1]))


def shard_weights(r0: int, r1: int, seed: int) -> np.ndarray:
    out = np.empty((r1 - r0, SHARDED[1]), np.uint16)
    for b in range(r0 // BLOCK, -(-r1 // BLOCK)):
        w = block_weights(b, seed)
        lo, hi = max(r0, b * BLOCK), min(r1, (b + 1) * BLOCK)
        out[lo - r0:hi - r0] = w[lo - b * BLOCK:hi - b * BLOCK]
    return out


def sharded_x(seed: int) -> np.ndarray:
    from demonic_b200 import synth
    return synth.activations(np.random.default_rng(seed), (SHARDED[1],))
