"""Host side of the row-sharded GEMV: the shard plan and the per-rank driver.

One process per GPU.  Rank r owns rows n*r/world .. n*(r+1)/world of W[n][k]; the ranks only
share the 128-byte NCCL id (any host channel will do; the benchmark uses torch.distributed) and
then exchange output slices inside the library.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib, backend


def shard_range(n: int, rank: int, world: int) -> tuple[int, int]:
    """Rows [r0, r1) owned by `rank` (``dmc_cuda_shard_range``)."""
    r0, r1 = C.c_int64(), C.c_int64()
    _lib.load().dmc_cuda_shard_range(n, rank, world, C.byref(r0), C.byref(r1))
    return r0.value, r1.value


def unique_id() -> bytes:
    buf = (C.c_uint8 * 128)()
    _lib.load().dmc_cuda_shard_unique_id(C.cast(buf, C.c_void_p))
    _lib.check()
    return bytes(buf)


def init(rank: int, world: int, uid: bytes | None, max_n: int) -> None:
    buf = (C.c_uint8 * 128)(*uid) if uid is not None else None
    _lib.load().dmc_cuda_shard_init(rank, world, C.cast(buf, C.c_void_p) if buf is not None else None, max_n)
    _lib.check()


def shutdown() -> None:
    _lib.load().dmc_cuda_shard_shutdown()


def gemv(dW_shard: backend.DeviceBuffer, dx: backend.DeviceBuffer, k: int, n: int,
         wdtype: int = backend.W_BF16) -> None:
    _lib.load().dmc_cuda_shard_gemv(dW_shard.ptr, dx.ptr, k, n, wdtype)
    _lib.check()


def gemv_host(dW_shard: backend.DeviceBuffer, x: np.ndarray, out: np.ndarray, k: int, n: int,
              wdtype: int = backend.W_BF16) -> None:
    """``dmc_cuda_shard_gemv_host``: x and the whole y in host memory, synchronous, collective."""
    assert x.dtype == np.float32 and out.dtype == np.float32 and x.size >= k and out.size >= n
    assert x.flags.c_contiguous and out.flags.c_contiguous
    _lib.load().dmc_cuda_shard_gemv_host(dW_shard.ptr, x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p),
                                         k, n, wdtype)
    _lib.check()


def gemv_batch(dW_shards: list[backend.DeviceBuffer], dx: backend.DeviceBuffer, dys: list[backend.DeviceBuffer] | None,
               k: int, n: int, wdtype: int = backend.W_BF16) -> None:
    """``dmc_cuda_shard_gemv_batch``: independent sharded GEMVs of one x; ``dys[i]`` receives the whole y of GEMV i."""
    arr = (C.c_void_p * len(dW_shards))(*[b.ptr for b in dW_shards])
    outs = (C.c_void_p * len(dys))(*[b.ptr for b in dys]) if dys is not None else None
    _lib.load().dmc_cuda_shard_gemv_batch(C.cast(arr, C.c_void_p), len(dW_shards), dx.ptr,
                                          C.cast(outs, C.c_void_p) if outs is not None else None, k, n, wdtype)
    _lib.check()


def output(n: int) -> np.ndarray:
    """The replicated y (first n floats), copied to the host after a sync."""
    lib = _lib.load()
    lib.dmc_cuda_sync()
    out = np.empty(n, np.float32)
    lib.dmc_cuda_d2h(out.ctypes.data_as(C.c_void_p), lib.dmc_cuda_shard_output(), out.nbytes)
    _lib.check()
    return out


def output_previous(n: int) -> np.ndarray:
    """The replicated y of the sharded GEMV before the last one (the other buffer of the pair)."""
    lib = _lib.load()
    out = np.empty(n, np.float32)
    lib.dmc_cuda_d2h(out.ctypes.data_as(C.c_void_p), lib.dmc_cuda_shard_output_previous(), out.nbytes)
    _lib.check()
    return out


def bench(dW_shards: list[backend.DeviceBuffer], dx: backend.DeviceBuffer, k: int, n: int, steps: int,
          warmup: int, use_graph: bool = True, wdtype: int = backend.W_BF16) -> float:
    arr = (C.c_void_p * len(dW_shards))(*[b.ptr for b in dW_shards])
    us = _lib.load().dmc_cuda_bench_shard(C.cast(arr, C.c_void_p), len(dW_shards), dx.ptr, k, n, wdtype, steps,
                                          warmup, int(use_graph))
    _lib.check()
    return float(us)
