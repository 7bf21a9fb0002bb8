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


def test_world_of_one_is_the_plain_gemv():
    lib = _lib.load()
    lib.dmc_cuda_clear_error()
    n, k = 3001, 4096                       # odd row count
    rng = np.random.default_rng(41)
    w = synth.bf16_weights(rng, (n, k))
    x = synth.activations(rng, (k,))
    sharded.init(0, 1, None, n)
    try:
        dW, dx = backend.DeviceBuffer.from_host(w), backend.DeviceBuffer.from_host(x)
        ref = oracle.gemm_bf16_fma(x.reshape(1, k), np.ascontiguousarray(w.T))
        for fused in (1, 0, 1, 1):          # the fused epilogue (a world of one stores only to itself) and the plain path
            lib.dmc_cuda_set_param(b"shard_fused", fused)
            assert lib.dmc_cuda_shard_uses_fused(k, n) == fused
            sharded.gemv(dW, dx, k, n)
            assert_parity(sharded.output(n), ref, TOL_BF16, f"fused={fused}")
            for io in (1, 0):               # host pointers in and out: kernels + completion word, or the copy engines
                lib.dmc_cuda_set_param(b"host_io_kernels", io)
                out = np.full(n, np.nan, np.float32)
                sharded.gemv_host(dW, x, out, k, n)
                assert_parity(out, ref, TOL_BF16, f"host pointers, fused={fused}, host_io_kernels={io}")
            lib.dmc_cuda_set_param(b"host_io_kernels", 1)
        lib.dmc_cuda_set_param(b"shard_fused", 1)
        us = sharded.bench([dW, dW, dW], dx, k, n, steps=3, warmup=1)      # graph replays advance the epoch on the device
        assert us > 0
        sharded.gemv(dW, dx, k, n)
        assert_parity(sharded.output(n), ref, TOL_BF16, "after graph replays")
        assert_parity(sharded.output_previous(n), ref, TOL_BF16, "the other buffer of the pair")
    finally:
        lib.dmc_cuda_set_param(b"shard_fused", -1)
        lib.dmc_cuda_set_param(b"host_io_kernels", 1)
        sharded.shutdown()
    assert lib.dmc_cuda_status() == 0


def test_batch_of_independent_sharded_gemvs_overlaps_and_keeps_every_result():
    """Six sharded GEMVs of one x in a batch (they may overlap: exchange i + 1 starts while exchange i is
    still landing; the replica buffer of exchange i is reused by exchange i + 2 under the guard), each
    with its own destination; then a GEMV that consumes one of the results, which must wait for it."""
    lib = _lib.load()
    lib.dmc_cuda_clear_error()
    n, k = 2048, 2048
    rng = np.random.default_rng(45)
    ws = [synth.bf16_weights(rng, (n, k)) for _ in range(6)]
    x = synth.activations(rng, (k,))
    lib.dmc_cuda_set_param(b"shard_fused", 1)
    sharded.init(0, 1, None, n)
    try:
        dWs = [backend.DeviceBuffer.from_host(w) for w in ws]
        dx = backend.DeviceBuffer.from_host(x)
        dys = [backend.DeviceBuffer(n * 4) for _ in ws]
        refs = [oracle.gemm_bf16_fma(x.reshape(1, k), np.ascontiguousarray(w.T)).reshape(-1) for w in ws]
        for rep in range(3):
            sharded.gemv_batch(dWs, dx, dys, k, n)
            sharded.gemv(dWs[0], dys[5], k, n)            # x = the last result of the batch: a true dependency
            backend.sync()
            for i, (dy, ref) in enumerate(zip(dys, refs)):
                assert_parity(dy.download(np.float32, n), ref, TOL_BF16, f"rep {rep} batch member {i}")
            chained = oracle.gemm_bf16_fma(refs[5].reshape(1, k), np.ascontiguousarray(ws[0].T))
            assert_parity(sharded.output(n), chained, TOL_BF16, f"rep {rep} consumer of a batch result")
        us = sharded.bench(dWs, dx, k, n, steps=5, warmup=2)
        assert us > 0
        sharded.gemv_batch(dWs, dx, None, k, n)
        assert_parity(sharded.output(n), refs[5], TOL_BF16, "last of a batch without destinations")
        assert_parity(sharded.output_previous(n), refs[4], TOL_BF16, "the one before it")
    finally:
        lib.dmc_cuda_set_param(b"shard_fused", -1)
        sharded.shutdown()
    assert lib.dmc_cuda_status() == 0, lib.dmc_cuda_last_error().decode()


def test_a_wait_that_runs_out_reports_timeout_and_leaves_the_gpu_usable():
    """The bounded device-side wait, made to run out in the permitted way: the arrival check runs for
    an exchange nobody writes, with a 2 ms limit.  Expected: status 6, nothing delivered, and the next
    sharded GEMV on the same context is right."""
    lib = _lib.load()
    lib.dmc_cuda_clear_error()
    n, k = 2048, 1024
    rng = np.random.default_rng(43)
    w = synth.bf16_weights(rng, (n, k))
    x = synth.activations(rng, (k,))
    lib.dmc_cuda_set_param(b"wait_limit_us", 2000)           # read by shard_init
    lib.dmc_cuda_set_param(b"shard_fused", 1)
    sharded.init(0, 1, None, n)
    try:
        rc = lib.dmc_cuda_shard_probe_timeout(n)
        assert rc == 6 and lib.dmc_cuda_status() == 6, lib.dmc_cuda_last_error().decode()
        assert b"wait ran out" in lib.dmc_cuda_last_error()
        # sticky: nothing runs until the host clears the error
        dW, dx = None, None
        assert lib.dmc_cuda_shard_gemv(None, None, k, n, backend.W_BF16) == 6
        lib.dmc_cuda_clear_error()
        dW, dx = backend.DeviceBuffer.from_host(w), backend.DeviceBuffer.from_host(x)
        ref = oracle.gemm_bf16_fma(x.reshape(1, k), np.ascontiguousarray(w.T))
        for _ in range(2):
            sharded.gemv(dW, dx, k, n)
            assert_parity(sharded.output(n), ref, TOL_BF16, "after the timeout")
    finally:
        lib.dmc_cuda_clear_error()
        lib.dmc_cuda_set_param(b"wait_limit_us", 0)
        lib.dmc_cuda_set_param(b"shard_fused", -1)
        sharded.shutdown()
    assert lib.dmc_cuda_status() == 0


def test_injected_host_failures_are_sticky_and_leave_nothing_behind(monkeypatch):
    """cudaMalloc, ncclCommInitRank and cudaIpcOpenMemHandle made to fail on the host (DMC_CUDA_INJECT):
    the call reports its status, `out` stays untouched, and after clearing the error the same call works."""
    lib = _lib.load()
    lib.dmc_cuda_clear_error()
    lib.dmc_cuda_drop_resident()
    k, n = 1024, 512
    rng = np.random.default_rng(44)
    w = synth.bf16_weights(rng, (k, n))
    x = synth.activations(rng, (1, k))
    out = np.full((1, n), 7.0, np.float32)
    monkeypatch.setenv("DMC_CUDA_INJECT", "malloc")
    lib.dmc_matmul_bf16_gpu(x.ctypes.data, w.ctypes.data, out.ctypes.data, 1, k, n)      # first sight: needs an upload
    assert lib.dmc_cuda_status() == 4 and np.all(out == 7.0)
    lib.dmc_matmul_bf16_gpu(x.ctypes.data, w.ctypes.data, out.ctypes.data, 1, k, n)      # sticky
    assert lib.dmc_cuda_status() == 4 and np.all(out == 7.0)
    assert lib.dmc_cuda_resident_count() == 0
    monkeypatch.setenv("DMC_CUDA_INJECT", "nccl_init")
    lib.dmc_cuda_clear_error()
    assert lib.dmc_cuda_shard_init(0, 1, None, n) == 5
    lib.dmc_cuda_clear_error()
    monkeypatch.setenv("DMC_CUDA_INJECT", "ipc_open")        # not an error: the NCCL exchange is kept instead
    lib.dmc_cuda_set_param(b"shard_fused", 1)
    try:
        assert lib.dmc_cuda_shard_init(0, 1, None, n) == 0
        assert lib.dmc_cuda_shard_uses_fused(k, n) == 0
        wt = np.ascontiguousarray(w.T)
        dW, dx = backend.DeviceBuffer.from_host(wt), backend.DeviceBuffer.from_host(x)
        sharded.gemv(dW, dx, k, n)
        assert_parity(sharded.output(n), oracle.gemm_bf16_fma(x, w), TOL_BF16, "plain path after a failed mapping")
    finally:
        lib.dmc_cuda_set_param(b"shard_fused", -1)
        sharded.shutdown()
    monkeypatch.delenv("DMC_CUDA_INJECT")
    lib.dmc_cuda_clear_error()
    dmc.matmul_bf16_gpu(x, w, out, 1, k, n)
    assert_parity(out, oracle.gemm_bf16_fma(x, w), TOL_BF16, "after the injected failures")
    lib.dmc_cuda_drop_resident()


CHILD = r"""
import os, sys
import numpy as np
sys.path.insert(0, {root!r})
import torch.distributed as dist
import demonic_b200 as dmc
import oracle
from demonic_b200 import backend, sharded, synth
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
lib = dmc.load()
assert lib.dmc_cuda_init(rank) == 0
ids = [sharded.unique_id() if rank == 0 else None]
dist.broadcast_object_list(ids, src=0)
sharded.init(rank, world, ids[0], 8192)
for n in (8192, 1001, 1):                   # even split, ragged split, fewer rows than ranks (an empty slice)
    k = 2048
    rng = np.random.default_rng(5)
    w = synth.bf16_weights(rng, (n, k)); x = synth.activations(rng, (k,))
    r0, r1 = sharded.shard_range(n, rank, world)
    dW = backend.DeviceBuffer.from_host(w[r0:r1]) if r1 > r0 else backend.DeviceBuffer(16)
    dx = backend.DeviceBuffer.from_host(x)
    ref = oracle.gemm_bf16_fma(x.reshape(1, k), np.ascontiguousarray(w.T)).reshape(-1)     # the whole y, every rank
    for fused in (1, 1, 0, 1):               # peer-store epilogue (twice: both y buffers), NCCL exchange, fused again
        lib.dmc_cuda_set_param(b"shard_fused", fused)
        assert lib.dmc_cuda_shard_uses_fused(k, n) == fused
        sharded.gemv(dW, dx, k, n)
        y = sharded.output(n)
        err = float(np.max(np.abs(y - ref)) / np.max(np.abs(ref)))
        assert err < 1e-5, (rank, n, fused, err)
        for rep in range(2):                 # host pointers in and out (both buffers of the exchange's pair)
            out = np.full(n, np.nan, np.float32)
            sharded.gemv_host(dW, x, out, k, n)
            err = float(np.max(np.abs(out - ref)) / np.max(np.abs(ref)))
            assert err < 1e-5, ("host pointers", rank, n, fused, rep, err)
    lib.dmc_cuda_set_param(b"shard_fused", 1)
    dys = [backend.DeviceBuffer(n * 4) for _ in range(5)]
    for rep in range(3):                     # a batch of independent exchanges: adjacent ones overlap
        sharded.gemv_batch([dW] * 5, dx, dys, k, n)
        backend.sync()
        for i, dy in enumerate(dys):
            y = dy.download(np.float32, n)
            assert float(np.max(np.abs(y - ref)) / np.max(np.abs(ref))) < 1e-5, ("batch", rank, n, rep, i)
    us = sharded.bench([dW, dW, dW], dx, k, n, steps=5, warmup=2)
    sharded.gemv(dW, dx, k, n)
    for name, y in (("last", sharded.output(n)), ("previous", sharded.output_previous(n))):
        assert float(np.max(np.abs(y - ref)) / np.max(np.abs(ref))) < 1e-5, ("after graph replays", name)
    np.save(os.path.join({out!r}, f"y{{rank}}_{{n}}.npy"), sharded.output(n))
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
    for n in (8192, 1001, 1):
        y0, y1 = np.load(tmp_path / f"y0_{n}.npy"), np.load(tmp_path / f"y1_{n}.npy")
        assert np.array_equal(y0, y1), "the two replicas of y differ"
