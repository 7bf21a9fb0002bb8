"""tcgen05 / TMEM GEMM (`X @ W'`, bf16 operands, f32 accumulate) against the CPU oracle: the
interpreter's `@` order applied to the widened operands (compiler/src/interp.rs:9270-9287)."""
import numpy as np
import pytest

import demonic_b200 as dmc
import oracle
from demonic_b200 import _lib, backend, synth
from tests.parity import TOL_BF16, assert_parity

pytestmark = pytest.mark.gpu
F = np.float32


def run_gemm(w, x, m, k, n, xdtype):
    lib = _lib.load()
    dW, dX = backend.DeviceBuffer.from_host(w), backend.DeviceBuffer.from_host(x)
    dY = backend.DeviceBuffer(m * n * 4)
    lib.dmc_cuda_memset(dY.ptr, 0xFF, m * n * 4)
    rc = lib.dmc_cuda_gemm_dev(dW.ptr, dX.ptr, dY.ptr, m, k, n, xdtype)
    assert rc == 0, lib.dmc_cuda_last_error().decode()
    backend.sync()
    return dY.download(F, m * n).reshape(m, n)


@pytest.fixture(autouse=True)
def clean():
    lib = _lib.load()
    lib.dmc_cuda_clear_error()
    yield
    for knob in (b"tc_ksplit", b"tc_smem_kb"):
        lib.dmc_cuda_set_param(knob, 0)
    assert lib.dmc_cuda_status() == 0, lib.dmc_cuda_last_error().decode()


@pytest.mark.parametrize("m", [1, 2, 4, 8, 16])
def test_small_batch_config(m):
    # BASELINE config 3: X bf16 [N, 4096] @ W' with W bf16 [4096, 4096], both N(0, 0.02)
    k = n = 4096
    rng = np.random.default_rng(300 + m)
    w = synth.bf16_weights(rng, (n, k))
    x = synth.bf16_weights(rng, (m, k))
    ref = oracle.gemm_bf16_fma(synth.bf16_to_f32(x), np.ascontiguousarray(w.T))
    for ksplit in (0, 1, 3):
        _lib.load().dmc_cuda_set_param(b"tc_ksplit", ksplit)
        got = run_gemm(w, x, m, k, n, 0)
        for j in range(m):
            assert_parity(got[j], ref[j], TOL_BF16, f"m={m} row {j} ksplit={ksplit}")


@pytest.mark.parametrize("m,k,n", [(17, 512, 300), (33, 1032, 136), (64, 64, 128), (100, 2048, 257), (130, 328, 520),
                                   (300, 1024, 384), (3, 8, 5), (256, 4096, 128)])
def test_ragged_shapes_and_dense_tiles(m, k, n):
    rng = np.random.default_rng(m * 7 + k + n)
    w = synth.bf16_weights(rng, (n, k), std=1.0)
    x = synth.bf16_weights(rng, (m, k), std=1.0)
    ref = oracle.gemm_bf16_fma(synth.bf16_to_f32(x), np.ascontiguousarray(w.T))
    got = run_gemm(w, x, m, k, n, 0)
    assert_parity(got, ref, 1e-5, f"{m}x{k}x{n}")       # bf16 x bf16 products are exact in f32: only the order differs
    _lib.load().dmc_cuda_set_param(b"tc_smem_kb", 48)    # shallow ring: stages wrap many times
    assert_parity(run_gemm(w, x, m, k, n, 0), ref, 1e-5, f"{m}x{k}x{n} shallow ring")


@pytest.mark.parametrize("m,k,n", [(1, 4096, 4096), (5, 2048, 1000), (16, 4096, 512), (40, 1024, 256)])
def test_f32_activations_split_in_two_bf16_terms(m, k, n):
    rng = np.random.default_rng(m + k)
    w = synth.bf16_weights(rng, (n, k))
    x = synth.activations(rng, (m, k))
    ref = oracle.gemm_bf16_fma(x, np.ascontiguousarray(w.T))
    got = run_gemm(w, x, m, k, n, 1)
    for j in range(m):
        assert_parity(got[j], ref[j], TOL_BF16, f"row {j}")
    err = float(np.max(np.abs(got - ref)) / np.max(np.abs(ref)))
    assert err < 1e-4, f"two-term split should carry ~16 mantissa bits of x, got {err:.2e}"


def test_unsupported_k_is_refused():
    lib = _lib.load()
    d = backend.DeviceBuffer(1 << 16)
    assert lib.dmc_cuda_gemm_dev(d.ptr, d.ptr, d.ptr, 2, 12, 8, 0) == 7
    lib.dmc_cuda_clear_error()
