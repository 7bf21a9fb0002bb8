"""Host-side mirror of the reference's GPU builtins over NumPy buffers.

Each function hands the library the raw addresses of caller-owned host arrays,
exactly as JIT-emitted code passes Forge pointers as i64 (reference:
compiler/src/jit.rs:19951, 20945), then converts the library's sticky status
into an exception.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

LAYOUT_KN, LAYOUT_NK = 0, 1
W_BF16, W_F32 = 0, 1


def _addr(a: np.ndarray) -> int:
    return a.ctypes.data


def _need(a: np.ndarray, dtype, name: str) -> np.ndarray:
    if a.dtype != dtype or not a.flags.c_contiguous:
        raise TypeError(f"{name} must be a C-contiguous {np.dtype(dtype).name} array")
    return a


def matmul_selected(flag_on: bool, deterministic_depth: int, m: int, k: int, n: int,
                    batch: int = 1, rhs_bf16: bool = True) -> bool:
    """Selection predicate of the opt-in flag (see ``dmc_cuda_matmul_selected``)."""
    return bool(_lib.load().dmc_cuda_matmul_selected(int(flag_on), deterministic_depth, m, k, n, batch,
                                                     int(rhs_bf16)))


def matmul_bf16_gpu(l: np.ndarray, r_bits: np.ndarray, out: np.ndarray, m: int, k: int, n: int) -> None:
    """``dmc_matmul_bf16_gpu(l, r, out, m, k, n)`` -- compiler/src/gpu.rs:400."""
    _need(l, np.float32, "l"), _need(r_bits, np.uint16, "r"), _need(out, np.float32, "out")
    _lib.load().dmc_matmul_bf16_gpu(_addr(l), _addr(r_bits), _addr(out), m, k, n)
    _lib.check()


def matmul_bf16_gpu_batched(l, r_bits, out, m, k, n, batch, ls, rs) -> None:
    """``dmc_matmul_bf16_gpu_batched`` -- compiler/src/gpu.rs:421."""
    _need(l, np.float32, "l"), _need(r_bits, np.uint16, "r"), _need(out, np.float32, "out")
    _lib.load().dmc_matmul_bf16_gpu_batched(_addr(l), _addr(r_bits), _addr(out), m, k, n, batch, ls, rs)
    _lib.check()


def matmul_bf16_gpu_batched_deferred(l, r_bits, out, m, k, n, batch, ls, rs) -> None:
    """``dmc_matmul_bf16_gpu_batched_deferred`` -- compiler/src/gpu.rs:449.
    ``out`` must stay alive and untouched until the next synchronous call or flush."""
    _need(l, np.float32, "l"), _need(r_bits, np.uint16, "r"), _need(out, np.float32, "out")
    _lib.load().dmc_matmul_bf16_gpu_batched_deferred(_addr(l), _addr(r_bits), _addr(out), m, k, n, batch, ls, rs)
    _lib.check()


def matmul_bf16_gpu_flush() -> None:
    """``dmc_matmul_bf16_gpu_flush`` -- compiler/src/gpu.rs:468."""
    _lib.load().dmc_matmul_bf16_gpu_flush()
    _lib.check()


def matmul_f32_gpu(l, r, out, m, k, n) -> None:
    """f32 `@` on the GPU; ABI of ``dmc_matmul_par`` (compiler/src/jit.rs:29415)."""
    _need(l, np.float32, "l"), _need(r, np.float32, "r"), _need(out, np.float32, "out")
    _lib.load().dmc_matmul_f32_gpu(_addr(l), _addr(r), _addr(out), m, k, n)
    _lib.check()


def matmul_bf16_gpu_nt(l, w_bits, out, m, k, n) -> None:
    """`x @ w'` with w stored [n, k]: no transpose pass (compiler/src/jit.rs:29801)."""
    _need(l, np.float32, "l"), _need(w_bits, np.uint16, "w"), _need(out, np.float32, "out")
    _lib.load().dmc_matmul_bf16_gpu_nt(_addr(l), _addr(w_bits), _addr(out), m, k, n)
    _lib.check()


class DeviceBuffer:
    """A device allocation owned by the library (device-resident path)."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        self.ptr = _lib.load().dmc_cuda_dev_alloc(self.nbytes)
        _lib.check()
        if not self.ptr:
            raise MemoryError(f"dmc_cuda_dev_alloc({nbytes}) returned NULL")

    @classmethod
    def from_host(cls, a: np.ndarray) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        buf = cls(a.nbytes)
        buf.upload(a)
        return buf

    def upload(self, a: np.ndarray) -> None:
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        _lib.load().dmc_cuda_h2d(self.ptr, a.ctypes.data_as(C.c_void_p), a.nbytes)
        _lib.check()

    def download(self, dtype, count: int) -> np.ndarray:
        out = np.empty(count, dtype)
        assert out.nbytes <= self.nbytes
        _lib.load().dmc_cuda_d2h(out.ctypes.data_as(C.c_void_p), self.ptr, out.nbytes)
        _lib.check()
        return out

    def free(self) -> None:
        if self.ptr:
            _lib.load().dmc_cuda_dev_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def npz_locate(path: str, key: str) -> dict:
    """Describe entry ``key`` of a ``.npz`` archive (``dmc_npz_locate``; host only, no device)."""
    e = _lib.NpzEntry()
    rc = _lib.load().dmc_npz_locate(str(path).encode(), key.encode(), C.byref(e))
    if rc != 0:
        raise OSError(f"vault.load_npz: cannot locate `{key}` in `{path}` (status {rc})")
    return {"data_offset": e.data_offset, "data_bytes": e.data_bytes, "shape": tuple(e.shape[:e.ndim]),
            "itemsize": e.itemsize, "fortran_order": bool(e.fortran_order), "method": e.method,
            "descr": e.descr.decode()}


def load_npz(path: str, key: str, rows: int, cols: int, wdtype: int = W_BF16, rank: int = 0, world: int = 1,
             host_dst: np.ndarray | None = None) -> tuple[DeviceBuffer, int]:
    """``vault.load_npz`` straight into HBM (``dmc_cuda_load_npz``): returns the device buffer holding
    this rank's rows of the ``[rows, cols]`` array and the number of rows loaded.  With ``host_dst``
    the bytes are also written there and the host range is registered as resident (the library then
    owns the device buffer: the returned object will not free it)."""
    dev = C.c_void_p()
    got = C.c_int64()
    _lib.load().dmc_cuda_load_npz(str(path).encode(), key.encode(), rows, cols, wdtype, rank, world,
                                  0 if host_dst is None else host_dst.ctypes.data, C.byref(dev), C.byref(got))
    _lib.check()
    buf = DeviceBuffer.__new__(DeviceBuffer)
    buf.nbytes = got.value * cols * (2 if wdtype == W_BF16 else 4)
    buf.ptr = dev.value
    if host_dst is not None:
        buf.free = lambda: None          # owned by the registration
    return buf, got.value


def gemv_dev(dW: DeviceBuffer, dx: DeviceBuffer, dy: DeviceBuffer, m: int, k: int, n: int,
             layout: int = LAYOUT_KN, wdtype: int = W_BF16, variant: int = -1) -> None:
    """Asynchronous device-resident GEMV (``dmc_cuda_gemv_dev``)."""
    _lib.load().dmc_cuda_gemv_dev(dW.ptr, dx.ptr, dy.ptr, m, k, n, layout, wdtype, variant)
    _lib.check()


def bench_items(items: list[tuple], steps: int, warmup: int = 3, use_graph: bool = True) -> float:
    """Device-timed microseconds per step (``dmc_cuda_bench_items``).  Each item is
    ``(dW, dx, dy, m, k, n, layout, wdtype, variant[, op[, (batch, ls, rs)]])``; ``dW`` / ``dx`` / ``dy``
    are DeviceBuffers or ``(DeviceBuffer, byte offset)`` pairs; ``op`` 0 (default) is the GEMV path,
    1 / 2 the tensor-core GEMM with bf16 / f32 activations."""
    def addr(b):
        return b[0].ptr + b[1] if isinstance(b, tuple) else b.ptr
    arr = (_lib.GemvItem * len(items))()
    for slot, item in zip(arr, items):
        dW, dx, dy, m, k, n, layout, wdtype, variant = item[:9]
        slot.W, slot.x, slot.y = addr(dW), addr(dx), addr(dy)
        slot.m, slot.k, slot.n = m, k, n
        slot.layout, slot.wdtype, slot.variant = layout, wdtype, variant
        slot.op = item[9] if len(item) > 9 else 0
        slot.batch, slot.ls, slot.rs = item[10] if len(item) > 10 else (1, 0, 0)
    us = _lib.load().dmc_cuda_bench_items(C.cast(arr, C.c_void_p), len(items), steps, warmup, int(use_graph))
    _lib.check()
    return float(us)


def bench_gemv(dWs: list[DeviceBuffer], dx: DeviceBuffer, dy: DeviceBuffer, m: int, k: int, n: int,
               layout: int, wdtype: int, variant: int, reps: int = 4, warmup: int = 1,
               use_graph: bool = True) -> float:
    """Microseconds per launch of one shape, rotating over the weight copies in ``dWs``."""
    items = [(w, dx, dy, m, k, n, layout, wdtype, variant) for w in dWs]
    return bench_items(items, reps, warmup, use_graph) / len(dWs)


def sync() -> None:
    _lib.load().dmc_cuda_sync()
    _lib.check()
