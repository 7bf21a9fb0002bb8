"""Small fixed case for profilers: a few bf16 GEMV launches of one shape over rotating
weight copies (inputs larger than L2, a few hundred MiB on the device).

    python -m demonic_b200.profile_case --shape 4096x4096 --layout nk --launches 8 [--variant V]

Prints the device-timed microseconds per launch.  Used for the ncu captures summarised
under profiles/ (capture with: ncu --set full --clock-control none -k regex:gemv -c 3 ...).
"""
from __future__ import annotations

import argparse

import numpy as np

from . import _lib, backend, synth


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="4096x4096", help="rows x cols of W (y = W.x)")
    ap.add_argument("--layout", default="nk", choices=["nk", "kn"])
    ap.add_argument("--launches", type=int, default=8)
    ap.add_argument("--variant", type=int, default=-1)
    ap.add_argument("--mib", type=int, default=256, help="distinct weight bytes to rotate over")
    ap.add_argument("--m", type=int, default=1, help="activation rows")
    ap.add_argument("--op", type=int, default=0, help="0 GEMV kernels, 1 tcgen05 GEMM (bf16 x), 2 tcgen05 GEMM (f32 x)")
    ap.add_argument("--decode", type=int, default=0, help="run this many decode steps of the benchmark model instead")
    ap.add_argument("--param", action="append", default=[], help="tuning knob name=value")
    args = ap.parse_args()
    rows, cols = (int(t) for t in args.shape.split("x"))
    lib = _lib.load()
    for kv in args.param:
        name, val = kv.split("=")
        assert lib.dmc_cuda_set_param(name.encode(), int(val)) == 0, name
    if args.decode:
        from . import decoder
        cfg = decoder.Config()
        dec = decoder.Decoder(cfg, decoder.random_model(cfg, cache_len=512))
        for _ in range(args.decode):
            tok = dec.step(1234, 512)
        print(f"decode: {args.decode} steps, {dec.launches_per_step} launches per step, next token {tok}")
        return
    rng = np.random.default_rng(synth.DEFAULT_SEED)
    w = synth.bf16_weights(rng, (rows, cols))
    x = synth.bf16_weights(rng, (args.m, cols)) if args.op == 1 else synth.activations(rng, (args.m, cols))
    copies = max(2, -(-(args.mib << 20) // w.nbytes))
    layout = backend.LAYOUT_NK if args.layout == "nk" else backend.LAYOUT_KN
    bufs = [backend.DeviceBuffer.from_host(w) for _ in range(copies)]
    dx, dy = backend.DeviceBuffer.from_host(x), backend.DeviceBuffer(args.m * rows * 4)
    items = [(bufs[i % copies], dx, dy, args.m, cols, rows, layout, backend.W_BF16, args.variant, args.op)
             for i in range(args.launches)]
    us = backend.bench_items(items, steps=1, warmup=1, use_graph=False) / len(items)
    b = synth.gemv_bytes(rows, cols, m=args.m)
    print(f"{args.shape} {args.layout} m={args.m} op={args.op} variant={args.variant}: {us:.2f} us/launch, {b / us / 1e3:.0f} GB/s "
          f"(algorithmic bytes {b})")


if __name__ == "__main__":
    main()
