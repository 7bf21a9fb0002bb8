"""Row-sharded GEMV on the GPU: world 1 in-process; world 2 as child processes when two GPUs exist."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import demonic_b200 as dmc
import oracle
from demonic_b200 import _lib, backend, sharded, synth
from tests.parity import TOL_BF16, assert_parity

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("exchange", [3, 2, 1], ids=["tagged", "counted", "flags"])
def test_world_of_one_is_the_plain_gemv(exchange):
    lib = _lib.load()
    lib.dmc_cuda_clear_error()
    n, k = 3001, 4096                       # odd row count
    rng = np.random.default_rng(41)
    w = synth.bf16_weights(rng, (n, k))
    x = synth.activations(rng, (k,))
    lib.dmc_cuda_set_param(b"shard_exchange", exchange)      # read when the shard context is created
    sharded.init(0, 1, None, n)
    try:
        dW, dx = backend.DeviceBuffer.from_host(w), backend.DeviceBuffer.from_host(x)
        ref = oracle.gemm_bf16_fma(x.reshape(1, k), np.ascontiguousarray(w.T))
        for fused in (1, 0, 1, 1):          # the fused epilogue (a world of one stores only to itself) and the plain path
            lib.dmc_cuda_set_param(b"shard_fused", fused)
            sharded.gemv(dW, dx, k, n)
            assert_parity(sharded.output(n), ref, TOL_BF16, f"fused={fused}")
        lib.dmc_cuda_set_param(b"shard_fused", 1)
        us = sharded.bench([dW, dW, dW], dx, k, n, steps=3, warmup=1)      # graph replays advance the epoch on the device
        assert us > 0
        sharded.gemv(dW, dx, k, n)
        assert_parity(sharded.output(n), ref, TOL_BF16, "after graph replays")
    finally:
        lib.dmc_cuda_set_param(b"shard_fused", -1)
        lib.dmc_cuda_set_param(b"shard_exchange", 3)
        sharded.shutdown()
    assert lib.dmc_cuda_status() == 0


CHILD = r"""
import os, sys
import numpy as np
sys.path.insert(0, {root!r})
import torch.distributed as dist
import demonic_b200 as dmc
from demonic_b200 import backend, sharded, synth
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
lib = dmc.load()
assert lib.dmc_cuda_init(rank) == 0
for exchange in (3, 2, 1):                  # tagged elements, counted arrivals, flags by the last CTA
  lib.dmc_cuda_set_param(b"shard_exchange", exchange)
  ids = [sharded.unique_id() if rank == 0 else None]
  dist.broadcast_object_list(ids, src=0)
  for n in (8192, 1001):                    # even split (all-gather) and ragged split (broadcast group)
    k = 2048
    rng = np.random.default_rng(5)
    w = synth.bf16_weights(rng, (n, k)); x = synth.activations(rng, (k,))
    if n == 8192: sharded.init(rank, world, ids[0], 8192)
    r0, r1 = sharded.shard_range(n, rank, world)
    dW, dx = backend.DeviceBuffer.from_host(w[r0:r1]), backend.DeviceBuffer.from_host(x)
    ref = synth.bf16_to_f32(w).astype(np.float64) @ x.astype(np.float64)
    for fused in (1, 1, 0, 1):               # peer-store epilogue (twice: both y buffers), NCCL exchange, fused again
        lib.dmc_cuda_set_param(b"shard_fused", fused)
        sharded.gemv(dW, dx, k, n)
        y = sharded.output(n)
        err = float(np.max(np.abs(y - ref)) / np.max(np.abs(ref)))
        assert err < 1e-5, (rank, n, exchange, fused, err)
    lib.dmc_cuda_set_param(b"shard_fused", 1)
    us = sharded.bench([dW, dW, dW], dx, k, n, steps=5, warmup=2)
    sharded.gemv(dW, dx, k, n)
    y = sharded.output(n)
    assert float(np.max(np.abs(y - ref)) / np.max(np.abs(ref))) < 1e-5, "after graph replays"
    np.save(os.path.join({out!r}, f"y{{rank}}_{{n}}_{{exchange}}.npy"), y)
  assert lib.dmc_cuda_status() == 0, lib.dmc_cuda_last_error()
  dist.barrier()
  sharded.shutdown()
dist.destroy_process_group()
"""


def test_two_ranks_on_two_gpus(tmp_path):
    if _lib.load().dmc_cuda_device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "child.py"
    script.write_text(CHILD.format(root=str(ROOT), out=str(tmp_path)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                           "--master-addr", "127.0.0.1", "--master-port", "29517", str(script)],
                          env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    for exchange in (3, 2, 1):
        for n in (8192, 1001):
            y0, y1 = np.load(tmp_path / f"y0_{n}_{exchange}.npy"), np.load(tmp_path / f"y1_{n}_{exchange}.npy")
            assert np.array_equal(y0, y1), "the two replicas of y differ"
