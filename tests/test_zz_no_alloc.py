"""The allocation-free GEMV entry point (`dmc_cuda_gemv_bf16_noalloc`).

Some hosts cannot let this library allocate for them: a runtime that keeps the whole device inside
its own budgeted arena, or a decode loop that cannot take the device-wide stall of an allocation
while other streams run.  For them one entry point keeps its split-K scratch in a fixed array
inside the library.  This test drives it through the C ABI on device buffers the *caller*
allocated, twice in a row (the second call finds the first call's leftovers in the shared array),
and compares each result with the ordinary entry point's on the same inputs and with the CPU
oracle, and checks that the free device memory is the same after the calls as before them.
It passes alone in a fresh process and after the other tests.
"""
import ctypes

import numpy as np
import pytest

import demonic_b200 as dmc
import oracle
from demonic_b200 import _lib, backend, synth
from tests.parity import TOL_BF16, assert_parity

pytestmark = pytest.mark.gpu
F = np.float32


def cudart():
    """The CUDA runtime, for a caller-owned stream and for waiting on it (the entry point itself
    never synchronises)."""
    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaStreamCreate.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
    rt.cudaStreamSynchronize.argtypes = [ctypes.c_void_p]
    rt.cudaStreamDestroy.argtypes = [ctypes.c_void_p]
    rt.cudaMemGetInfo.argtypes = [ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)]
    return rt


def free_device_bytes(rt) -> int:
    free, total = ctypes.c_size_t(), ctypes.c_size_t()
    assert rt.cudaMemGetInfo(ctypes.byref(free), ctypes.byref(total)) == 0
    return free.value


def test_noalloc_entry_matches_the_allocating_one_twice_in_a_row():
    lib = _lib.load()
    assert lib.dmc_cuda_device_count() > 0, "no CUDA device"
    lib.dmc_cuda_clear_error()
    k, n = 4096, 4096
    rng = np.random.default_rng(2024)
    w = synth.bf16_weights(rng, (k, n))
    xs = [synth.activations(rng, (k,)), synth.activations(rng, (k,)) * F(3.0)]
    dW = backend.DeviceBuffer.from_host(w)              # the caller's allocations
    dx = backend.DeviceBuffer(k * 4)
    dy_ref, dy_new = backend.DeviceBuffer(n * 4), backend.DeviceBuffer(n * 4)
    rt = cudart()
    stream = ctypes.c_void_p()
    assert rt.cudaStreamCreate(ctypes.byref(stream)) == 0
    for call, x in enumerate(xs):
        dx.upload(x)
        backend.gemv_dev(dW, dx, dy_ref, 1, k, n, backend.LAYOUT_KN, backend.W_BF16)
        backend.sync()
        want = dy_ref.download(F, n)
        lib.dmc_cuda_memset(dy_new.ptr, 0xFF, n * 4)
        backend.sync()
        free_before = free_device_bytes(rt)
        rc = lib.dmc_cuda_gemv_bf16_noalloc(dW.ptr, dx.ptr, dy_new.ptr, k, n, stream)
        assert rc == 0, lib.dmc_cuda_last_error().decode()
        assert rt.cudaStreamSynchronize(stream) == 0
        if call == 0:
            # the first call on a device makes the CUDA runtime load this kernel's part of the library image,
            # which includes the fixed scratch array: a one-time cost of the image, a few MiB, not an allocation
            assert free_before - free_device_bytes(rt) <= 32 << 20
        else:
            assert free_device_bytes(rt) == free_before, "the entry point allocated (or freed) device memory"
        got = dy_new.download(F, n)
        assert_parity(got, want, TOL_BF16, f"call {call + 1} vs the allocating entry point")
        assert_parity(got, oracle.gemm_bf16_fma(x.reshape(1, k), w), TOL_BF16, f"call {call + 1} vs the CPU oracle")
    # a second shape through the same array (fewer K slices, ragged last column block)
    k2, n2 = 1000, 264
    w2 = synth.bf16_weights(rng, (k2, n2))
    x2 = synth.activations(rng, (k2,))
    dW2, dx2 = backend.DeviceBuffer.from_host(w2), backend.DeviceBuffer.from_host(x2)
    backend.gemv_dev(dW2, dx2, dy_ref, 1, k2, n2, backend.LAYOUT_KN, backend.W_BF16)
    backend.sync()
    want2 = dy_ref.download(F, n2)
    assert lib.dmc_cuda_gemv_bf16_noalloc(dW2.ptr, dx2.ptr, dy_new.ptr, k2, n2, stream) == 0
    assert rt.cudaStreamSynchronize(stream) == 0
    assert_parity(dy_new.download(F, n2), want2, TOL_BF16, "second shape")
    assert_parity(dy_new.download(F, n2), oracle.gemm_bf16_fma(x2.reshape(1, k2), w2), TOL_BF16, "second shape vs the CPU oracle")
    assert rt.cudaStreamDestroy(stream) == 0


def test_noalloc_entry_refuses_what_its_scratch_cannot_hold():
    lib = _lib.load()
    lib.dmc_cuda_clear_error()
    d = backend.DeviceBuffer(1 << 16)
    rc = lib.dmc_cuda_gemv_bf16_noalloc(d.ptr, d.ptr, d.ptr, 64, 16384 + 8, None)
    assert rc == 7 and "beyond the built-in scratch" in lib.dmc_cuda_last_error().decode()
    lib.dmc_cuda_clear_error()
    rc = lib.dmc_cuda_gemv_bf16_noalloc(d.ptr, d.ptr, d.ptr, 64, 100, None)        # n % 8 != 0
    assert rc == 7
    lib.dmc_cuda_clear_error()
    assert lib.dmc_cuda_status() == 0
