"""ctypes binding of libdmc_cuda.so (the C ABI in include/dmc_cuda.h).

There is no CPU fallback: if the library is missing, or a call fails on the
device, this module raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libdmc_cuda.so"

I64 = C.c_int64
VP = C.c_void_p

# name -> (restype, argtypes); every symbol include/dmc_cuda.h declares
SIGNATURES = {
    "dmc_cuda_device_count": (C.c_int, []),
    "dmc_cuda_init": (C.c_int, [C.c_int]),
    "dmc_cuda_shutdown": (None, []),
    "dmc_cuda_status": (C.c_int, []),
    "dmc_cuda_last_error": (C.c_char_p, []),
    "dmc_cuda_clear_error": (None, []),
    "dmc_matmul_bf16_gpu": (None, [I64] * 6),
    "dmc_matmul_bf16_gpu_batched": (None, [I64] * 9),
    "dmc_matmul_bf16_gpu_batched_deferred": (None, [I64] * 9),
    "dmc_matmul_bf16_gpu_flush": (None, []),
    "dmc_matmul_f32_gpu": (None, [I64] * 6),
    "dmc_matmul_bf16_gpu_nt": (None, [I64] * 6),
    "dmc_cuda_matmul_selected": (C.c_int, [C.c_int, C.c_uint32, I64, I64, I64, I64, C.c_int]),
    "dmc_cuda_register_weight": (C.c_int, [I64, I64, I64, I64, C.c_int, C.c_int]),
    "dmc_cuda_unregister_weight": (C.c_int, [I64]),
    "dmc_cuda_resident_count": (I64, []),
    "dmc_cuda_resident_bytes": (I64, []),
    "dmc_cuda_drop_resident": (None, []),
    "dmc_cuda_dev_alloc": (VP, [I64]),
    "dmc_cuda_dev_free": (None, [VP]),
    "dmc_cuda_h2d": (C.c_int, [VP, VP, I64]),
    "dmc_cuda_d2h": (C.c_int, [VP, VP, I64]),
    "dmc_cuda_memset": (C.c_int, [VP, C.c_int, I64]),
    "dmc_cuda_sync": (C.c_int, []),
    "dmc_cuda_gemv_dev": (C.c_int, [VP, VP, VP, I64, I64, I64, C.c_int, C.c_int, C.c_int]),
    "dmc_cuda_gemv_bf16_noalloc": (C.c_int, [VP, VP, VP, I64, I64, VP]),
    "dmc_cuda_shard_gemv_host": (C.c_int, [VP, VP, VP, I64, I64, C.c_int]),
    "dmc_cuda_shard_range": (None, [I64, C.c_int, C.c_int, C.POINTER(I64), C.POINTER(I64)]),
    "dmc_cuda_shard_unique_id": (C.c_int, [VP]),
    "dmc_cuda_shard_init": (C.c_int, [C.c_int, C.c_int, VP, I64]),
    "dmc_cuda_shard_shutdown": (None, []),
    "dmc_cuda_shard_gemv": (C.c_int, [VP, VP, I64, I64, C.c_int]),
    "dmc_cuda_shard_gemv_batch": (C.c_int, [VP, C.c_int, VP, VP, I64, I64, C.c_int]),
    "dmc_cuda_shard_output": (VP, []),
    "dmc_cuda_shard_output_previous": (VP, []),
    "dmc_cuda_shard_uses_fused": (C.c_int, [I64, I64]),
    "dmc_cuda_shard_probe_timeout": (C.c_int, [I64]),
    "dmc_cuda_row_kernel_grid": (I64, [I64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "dmc_cuda_shard_path": (C.c_int, [C.c_int, C.c_int, C.c_int, I64, I64]),
    "dmc_cuda_bench_shard": (C.c_double, [VP, C.c_int, VP, I64, I64, C.c_int, C.c_int, C.c_int, C.c_int]),
    "dmc_cuda_gemm_dev": (C.c_int, [VP, VP, VP, I64, I64, I64, C.c_int]),
    "dmc_decoder_create": (C.c_int, [VP, C.POINTER(VP)]),
    "dmc_decoder_load": (C.c_int, [VP, C.c_int, C.c_int, VP, I64]),
    "dmc_decoder_step": (C.c_int, [VP, C.c_int, C.c_int, C.POINTER(C.c_int), VP]),
    "dmc_decoder_bench": (C.c_double, [VP, C.c_int, C.c_int, C.c_int, C.c_int]),
    "dmc_decoder_launches_per_step": (I64, [VP]),
    "dmc_decoder_destroy": (None, [VP]),
    "dmc_npz_locate": (C.c_int, [C.c_char_p, C.c_char_p, VP]),
    "dmc_cuda_load_npz": (C.c_int, [C.c_char_p, C.c_char_p, I64, I64, C.c_int, C.c_int, C.c_int, I64, C.POINTER(VP),
                                    C.POINTER(I64)]),
    "dmc_cuda_timeline": (C.c_int, [VP, C.c_int, VP, VP, I64, I64, C.c_int, VP, I64]),
    "dmc_cuda_bench_items": (C.c_double, [VP, C.c_int, C.c_int, C.c_int, C.c_int]),
    "dmc_cuda_variant_count": (C.c_int, [C.c_int, C.c_int]),
    "dmc_cuda_variant_name": (C.c_char_p, [C.c_int, C.c_int, C.c_int]),
    "dmc_cuda_set_param": (C.c_int, [C.c_char_p, I64]),
    "dmc_cuda_launch_count": (I64, []),
}



class NpzEntry(C.Structure):
    """``dmc_npz_entry`` of include/dmc_cuda.h."""
    _fields_ = [("data_offset", I64), ("data_bytes", I64), ("shape", I64 * 4), ("ndim", C.c_int),
                ("itemsize", C.c_int), ("fortran_order", C.c_int), ("method", C.c_int), ("descr", C.c_char * 16)]


class GemvItem(C.Structure):
    """``dmc_gemv_item`` of include/dmc_cuda.h."""
    _fields_ = [("W", VP), ("x", VP), ("y", VP), ("m", I64), ("k", I64), ("n", I64),
                ("layout", C.c_int), ("wdtype", C.c_int), ("variant", C.c_int), ("op", C.c_int),
                ("batch", I64), ("ls", I64), ("rs", I64)]




class DecoderConfig(C.Structure):
    """``dmc_decoder_config`` of include/dmc_cuda.h."""
    _fields_ = [("layers", C.c_int), ("d_model", C.c_int), ("heads", C.c_int), ("head_dim", C.c_int),
                ("ffn", C.c_int), ("vocab", C.c_int), ("max_len", C.c_int), ("eps", C.c_float)]


_lib = None


class DmcCudaError(RuntimeError):
    """A libdmc_cuda call failed; carries the library's status code."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"runtime error: dmc_cuda status {code}: {msg}")
        self.code = code


def load() -> C.CDLL:
    """Load the in-tree library; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m demonic_b200.build` "
                "(there is no CPU fallback)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)     # AttributeError if the .so lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check() -> None:
    """Turn the library's sticky status into an exception (what the host's
    `runtime error:` + exit(1) convention would do)."""
    lib = load()
    code = lib.dmc_cuda_status()
    if code != 0:
        raise DmcCudaError(code, lib.dmc_cuda_last_error().decode())
