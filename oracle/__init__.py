"""ctypes front of the CPU oracle (``dmc_oracle.c``).

TEST INFRASTRUCTURE ONLY: the checker the CUDA backend is compared against and
the timed CPU baseline of the benchmark.  The product package never imports
this module.  Each wrapper names the reference function the C code restates
(paths relative to the reference project root).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libdmc_oracle.so"
CFLAGS = ["-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fPIC", "-shared", "-pthread",
          "-fvisibility=hidden"]


def build(force: bool = False) -> Path:
    """Compile ``dmc_oracle.c`` (same flags as the Makefile beside it)."""
    src = HERE / "dmc_oracle.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run([os.environ.get("CC", "gcc"), *CFLAGS, "-o", str(LIB_PATH), str(src), "-lm"],
                       check=True)
    return LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        _lib = C.CDLL(str(LIB_PATH))
        _lib.orc_bf16_bits_to_f32.restype = C.c_float
        _lib.orc_bf16_bits_to_f32.argtypes = [C.c_uint16]
        _lib.orc_dot_two_rounding.restype = C.c_float
        _lib.orc_silu.restype = C.c_float
        _lib.orc_silu.argtypes = [C.c_float]
        _lib.orc_matmul_threads.restype = C.c_int64
        _lib.orc_bf16_colsplit_ways.restype = C.c_int64
        _lib.orc_argmax.restype = C.c_int64
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u16(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint16)


_i64 = C.c_int64


# ---- bf16 helpers ----------------------------------------------------------

def bf16_bits_to_f32(bits) -> np.ndarray:
    """compiler/src/jit.rs:29224-29227 — widen = bits << 16."""
    b = _u16(bits)
    out = np.empty(b.shape, np.float32)
    lib().orc_bf16_upconvert(_p(b), _p(out), _i64(b.size))
    return out


def f32_to_bf16_trunc(x) -> np.ndarray:
    """compiler/src/jit.rs:29783-29792 — truncating f32→bf16 store."""
    x = _f32(x)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16_trunc(_p(x), _p(out), _i64(x.size))
    return out


def f32_to_bf16_rne(x) -> np.ndarray:
    """Round-to-nearest-even f32→bf16 (input generation only: the benchmark
    configs draw N(0, 0.02) weights "rounded to bf16").  Not a reference
    function: the reference only ever truncates."""
    u = _f32(x).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_transpose_2d(w, m: int, n: int) -> np.ndarray:
    """compiler/src/jit.rs:29801-29834."""
    w = _u16(w).reshape(m, n)
    out = np.empty((n, m), np.uint16)
    lib().orc_bf16_transpose_2d(_p(w), _p(out), _i64(m), _i64(n))
    return out


def fingerprint(buf: np.ndarray) -> tuple[int, int]:
    """compiler/src/gpu.rs:342-358."""
    b = np.ascontiguousarray(buf).view(np.uint8).reshape(-1)
    out = (C.c_uint64 * 2)()
    lib().orc_fingerprint(_p(b), C.c_uint64(b.size), out)
    return int(out[0]), int(out[1])


# ---- `@` semantics ---------------------------------------------------------

def gemm_f32_fma(a, b) -> np.ndarray:
    """compiler/src/interp.rs:9270-9287 — the reference semantics of `@`."""
    a = _f32(a)
    b = _f32(b)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = np.empty((m, n), np.float32)
    lib().orc_gemm_f32_fma(_p(a), _p(b), _p(c), _i64(m), _i64(k), _i64(n))
    return c


def gemm_bf16_fma(a, w_bits) -> np.ndarray:
    """The interpreter's `@` on widened bf16 weights (``w_bits`` is [k, n])."""
    a = _f32(a)
    w = _u16(w_bits)
    m, k = a.shape
    k2, n = w.shape
    assert k == k2
    c = np.empty((m, n), np.float32)
    lib().orc_gemm_bf16_fma(_p(a), _p(w), _p(c), _i64(m), _i64(k), _i64(n))
    return c


def gemm_bf16_nt(a, w_nk_bits) -> np.ndarray:
    """`x @ w'` for w stored [n, k]: transpose (compiler/src/jit.rs:29801-29834) then the interpreter's
    `@` (compiler/src/interp.rs:9270-9287), computed without materialising the transpose."""
    a = _f32(a)
    w = _u16(w_nk_bits)
    m, k = a.shape
    n, k2 = w.shape
    assert k == k2
    c = np.empty((m, n), np.float32)
    lib().orc_gemm_bf16_nt(_p(a), _p(w), _p(c), _i64(m), _i64(k), _i64(n))
    return c


def dot_two_rounding(a, b_col) -> float:
    """compiler/src/jit.rs:37403-37412 — the non-contracted hand loop."""
    a = _f32(a)
    b = _f32(b_col)
    return float(lib().orc_dot_two_rounding(_p(a), _p(b), _i64(a.size), _i64(1)))


def dmc_matmul_par(a, b) -> np.ndarray:
    """compiler/src/jit.rs:29415-29441 (threaded f32 runtime kernel)."""
    a = _f32(a)
    b = _f32(b)
    m, k = a.shape
    _, n = b.shape
    c = np.empty((m, n), np.float32)
    lib().orc_dmc_matmul_par(_p(a), _p(b), _p(c), _i64(m), _i64(k), _i64(n))
    return c


def simd_matmul_f32(a, b) -> np.ndarray:
    """compiler/src/jit.rs:20525-20712 (inline default f32 kernel order)."""
    a = _f32(a)
    b = _f32(b)
    m, k = a.shape
    _, n = b.shape
    assert n % 4 == 0
    c = np.empty((m, n), np.float32)
    lib().orc_simd_matmul_f32(_p(a), _p(b), _p(c), _i64(m), _i64(k), _i64(n))
    return c


def dmc_matmul_bf16(a, w_bits, out: np.ndarray | None = None) -> np.ndarray:
    """compiler/src/jit.rs:29488-29566 (CPU bf16 decode GEMV/GEMM with its
    thread policy).  ``w_bits`` is [k, n] bf16 bit patterns."""
    a = _f32(a)
    w = _u16(w_bits)
    m, k = a.shape
    _, n = w.shape
    c = out if out is not None else np.empty((m, n), np.float32)
    lib().orc_dmc_matmul_bf16(_p(a), _p(w), _p(c), _i64(m), _i64(k), _i64(n))
    return c


def bf16_gemv_batched(l, r, k: int, n: int, batch: int, ls: int, rs: int) -> np.ndarray:
    """compiler/src/gpu.rs:384-391 — batch of m==1 slices at affine offsets."""
    l = _f32(l).reshape(-1)
    r = _u16(r).reshape(-1)
    assert l.size >= (batch - 1) * ls + k and r.size >= (batch - 1) * rs + k * n
    c = np.empty((batch, n), np.float32)
    lib().orc_bf16_gemv_batched(_p(l), _p(r), _p(c), _i64(k), _i64(n), _i64(batch), _i64(ls), _i64(rs))
    return c


def matmul_broadcast_f32(a, b) -> np.ndarray:
    """compiler/src/interp.rs:9330-9374 — batched `@` with broadcast batch dims."""
    a = _f32(a)
    b = _f32(b)
    m, k = a.shape[-2:]
    k2, n = b.shape[-2:]
    assert k == k2
    br = max(a.ndim, b.ndim) - 2
    ab = (1,) * (br - (a.ndim - 2)) + a.shape[:-2]
    bb = (1,) * (br - (b.ndim - 2)) + b.shape[:-2]
    ob = tuple(max(x, y) for x, y in zip(ab, bb))
    for x, y in zip(ab, bb):
        if x != y and x != 1 and y != 1:
            raise ValueError(f"batched matmul: batch dims cannot broadcast: {ab} vs {bb}")
    out = np.empty(ob + (m, n), np.float32)
    A = (C.c_int64 * max(br, 1))(*ab)
    B = (C.c_int64 * max(br, 1))(*bb)
    lib().orc_matmul_broadcast_f32(_p(a), A, _p(b), B, _i64(br), _i64(m), _i64(k), _i64(n), _p(out))
    return out


def matmul_threads(m: int, k: int, n: int) -> int:
    """compiler/src/jit.rs:29471-29479."""
    return int(lib().orc_matmul_threads(_i64(m), _i64(k), _i64(n)))


def bf16_colsplit_ways(k: int, n: int) -> int:
    """compiler/src/jit.rs:29527-29529."""
    return int(lib().orc_bf16_colsplit_ways(_i64(k), _i64(n)))


def set_thread_cap(cap: int) -> None:
    lib().orc_set_thread_cap(C.c_int(cap))


# ---- decode companions -----------------------------------------------------

def rms_norm_f32(x, g, eps: float = 1e-6) -> np.ndarray:
    """compiler/src/jit.rs:23776-23847 (f32 lowering)."""
    x = _f32(x)
    g = _f32(g)
    y = np.empty_like(x)
    lib().orc_rms_norm_f32(_p(x), _p(g), _p(y), _i64(x.size), C.c_float(eps))
    return y


def rms_norm_f64(x, g, eps: float = 1e-6) -> np.ndarray:
    """compiler/src/interp.rs:13559-13590 (interpreter, f64)."""
    x = _f32(x)
    g = _f32(g)
    y = np.empty_like(x)
    lib().orc_rms_norm_f64(_p(x), _p(g), _p(y), _i64(x.size), C.c_double(eps))
    return y


def rope_row(x, cos, sin) -> np.ndarray:
    """compiler/src/interp.rs:13636-13678 for one [d] row."""
    x = _f32(x)
    cos = _f32(cos)
    sin = _f32(sin)
    y = np.empty_like(x)
    lib().orc_rope_row(_p(x), _p(cos), _p(sin), _p(y), _i64(x.size))
    return y


def softmax_row(x) -> np.ndarray:
    """compiler/src/interp.rs:13451-13489 for one row."""
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_softmax_row(_p(x), _p(y), _i64(x.size))
    return y


def silu(x) -> np.ndarray:
    """compiler/src/interp.rs:13418."""
    x = _f32(x)
    return np.array([lib().orc_silu(C.c_float(float(v))) for v in x.reshape(-1)],
                    np.float32).reshape(x.shape)


def kv_attention_head(q, kc, vc) -> np.ndarray:
    """compiler/src/jit.rs:20303-20506 — one head over a [len, d] KV cache."""
    q = _f32(q)
    kc = _f32(kc)
    vc = _f32(vc)
    ln, d = kc.shape
    out = np.empty(d, np.float32)
    scratch = np.empty(ln, np.float32)
    lib().orc_kv_attention_head(_p(q), _p(kc), _p(vc), _p(out), _p(scratch), _i64(ln), _i64(d))
    return out


def embed_bf16(vocab_bits, idx: int) -> np.ndarray:
    """compiler/src/interp.rs:13494-13516 (ids clamp)."""
    v = _u16(vocab_bits)
    out = np.empty(v.shape[1], np.float32)
    lib().orc_embed_bf16(_p(v), _i64(v.shape[0]), _i64(v.shape[1]), _i64(idx), _p(out))
    return out


def argmax(x) -> int:
    """compiler/src/interp.rs:13529-13538."""
    x = _f32(x)
    return int(lib().orc_argmax(_p(x), _i64(x.size)))
