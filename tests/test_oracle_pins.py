"""Pins the CPU oracle to the known-answer tests the reference carries for the
matmul path.  Every case cites the reference test it restates (paths relative to
the reference project root).  CPU only."""
import numpy as np
import pytest

import oracle
from oracle import exact

F = np.float32


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_bf16_widen_kats():
    # compiler/src/jit.rs:30171-30178 `bf16_widen_to_f32`
    got = oracle.bf16_bits_to_f32(np.array([0x0000, 0x3F80, 0xBF80, 0x4000, 0x4049], np.uint16))
    assert got[0] == 0.0 and got[1] == 1.0 and got[2] == -1.0 and got[3] == 2.0
    assert bits(got)[4] == 0x40490000


def test_f32_to_bf16_is_truncation():
    # compiler/src/jit.rs:29783-29792: bits >> 16, so 1.0 + 2^-8 + 2^-9 keeps only the top 16 bits
    x = np.array([1.0, -2.5, 3.14159274, 1.99999988], F)
    t = oracle.f32_to_bf16_trunc(x)
    assert list(t) == [int(b) >> 16 for b in bits(x)]
    assert t[3] == 0x3FFF  # RNE would have produced 0x4000


def test_bf16_matmul_bit_identical_to_widened():
    # compiler/src/jit.rs:30204-30243, m,k,n = 3,5,4
    m, k, n = 3, 5, 4
    a = (np.arange(m * k, dtype=F) * F(0.5) - F(3.0)).reshape(m, k)
    w = oracle.f32_to_bf16_trunc(np.arange(k * n, dtype=F) * F(0.25) - F(2.0)).reshape(k, n)
    got = oracle.dmc_matmul_bf16(a, w)
    wf = oracle.bf16_bits_to_f32(w)
    # reference expectation: widen then the same kk-ascending mul_add chain
    want = np.array(exact.gemm_f32_fma(a.tolist(), wf.tolist()), F)
    assert np.array_equal(bits(got), bits(want))
    assert np.array_equal(bits(oracle.gemm_f32_fma(a, wf)), bits(want))
    assert np.array_equal(bits(oracle.gemm_bf16_fma(a, w)), bits(want))
    assert np.array_equal(bits(oracle.dmc_matmul_par(a, wf)), bits(want))


def test_integer_goldens():
    # compiler/src/jit.rs:32602-32617 -> 415
    a = np.array([[1, 2, 3], [4, 5, 6]], F)
    b = np.array([[7, 8], [9, 10], [11, 12]], F)
    assert int(oracle.gemm_f32_fma(a, b).sum()) == 415
    # compiler/src/jit.rs:32692-32709 -> 136 (A @ I = A)
    A = np.arange(1, 17, dtype=F).reshape(4, 4)
    assert int(oracle.simd_matmul_f32(A, np.eye(4, dtype=F)).sum()) == 136
    # compiler/src/jit.rs:32711-32730 -> 40
    assert int(oracle.simd_matmul_f32(np.diag(np.array([1, 2, 3, 4], F)), np.ones((4, 4), F)).sum()) == 40
    # compiler/src/jit.rs:34513-34537 -> 30300
    A = np.zeros((4, 4), F)
    A[0] = [1, 2, 3, 4]
    B = np.zeros((4, 4), F)
    B[:, 0] = [10, 20, 30, 40]
    B[:, 1] = [100, 200, 300, 400]
    Cm = oracle.gemm_f32_fma(A, B)
    assert int(Cm[0, 0] + Cm[0, 1] * F(10.0)) == 30300
    # compiler/src/jit.rs:42643-42655 `jit_bf16_field_matmul` -> 6
    x = np.ones((1, 2), F)
    w = oracle.f32_to_bf16_trunc(np.ones((2, 3), F)).reshape(2, 3)
    assert int(oracle.dmc_matmul_bf16(x, w).sum()) == 6


def _fill_a():
    i, j = np.meshgrid(np.arange(8), np.arange(16), indexing="ij")
    return ((i * 16 + j).astype(F) * F(0.7) + F(0.1)) / F(3.0)


def _fill_b(n, stride):
    i, j = np.meshgrid(np.arange(16), np.arange(n), indexing="ij")
    return ((i * stride + j).astype(F) * F(0.3) + F(0.2)) / F(7.0)


def test_result_does_not_depend_on_unrelated_columns():
    # compiler/src/jit.rs:37353-37386: C[0,0] is the same number for n = 3, 4, 15, 16
    a = _fill_a()
    got = {n: int(bits(oracle.gemm_f32_fma(a, _fill_b(n, 97)))[0, 0]) for n in (3, 4, 15, 16)}
    assert len(set(got.values())) == 1
    assert int(bits(oracle.simd_matmul_f32(a, _fill_b(16, 97)))[0, 0]) == got[16]
    assert int(bits(oracle.dmc_matmul_par(a, _fill_b(15, 97)))[0, 0]) == got[15]
    want = exact.gemm_f32_fma(a[:1].tolist(), _fill_b(3, 97).tolist())[0][0]
    assert exact.f32_bits(want) == got[3]


def test_matmul_contracts_and_says_so():
    # compiler/src/jit.rs:37388-37422: the FMA answer differs from the two-rounding answer
    a, b = _fill_a(), _fill_b(16, 16)
    contracted = oracle.gemm_f32_fma(a, b)[0, 0]
    two = oracle.dot_two_rounding(a[0], b[:, 0])
    assert exact.f32_bits(float(contracted)) != exact.f32_bits(two)
    want = exact.gemm_f32_fma(a[:1].tolist(), b[:, :1].tolist())[0][0]
    assert exact.f32_bits(want) == exact.f32_bits(float(contracted))
    # the hand loop really rounds twice
    s = F(0.0)
    for i in range(16):
        s = F(s + F(a[0, i] * b[i, 0]))
    assert exact.f32_bits(float(s)) == exact.f32_bits(two)


def test_batched_matmul_contracts_too():
    # compiler/src/jit.rs:37424-37438: [2,4,8] @ [2,8,4], element [1,2,3]
    nn, i, j = np.meshgrid(np.arange(2), np.arange(4), np.arange(8), indexing="ij")
    a = ((nn * 32 + i * 8 + j).astype(F) * F(0.7) + F(0.1)) / F(3.0)
    nn, i, j = np.meshgrid(np.arange(2), np.arange(8), np.arange(4), indexing="ij")
    b = ((nn * 32 + i * 4 + j).astype(F) * F(0.3) + F(0.2)) / F(7.0)
    out = oracle.matmul_broadcast_f32(a, b)
    want = exact.gemm_f32_fma(a[1, 2:3].tolist(), b[1][:, 3:4].tolist())[0][0]
    assert exact.f32_bits(float(out[1, 2, 3])) == exact.f32_bits(want)


def test_broadcast_batch_dims():
    # compiler/src/interp.rs:9330-9374 and compiler/src/interp_tests.rs:533-590
    rng = np.random.default_rng(5)
    a = rng.uniform(-1, 1, (2, 1, 3, 4)).astype(F)
    b = rng.uniform(-1, 1, (5, 4, 2)).astype(F)
    out = oracle.matmul_broadcast_f32(a, b)
    assert out.shape == (2, 5, 3, 2)
    for p in range(2):
        for q in range(5):
            assert np.array_equal(bits(out[p, q]), bits(oracle.gemm_f32_fma(a[p, 0], b[q])))
    with pytest.raises(ValueError):
        oracle.matmul_broadcast_f32(np.zeros((2, 3, 4), F), np.zeros((3, 4, 2), F))


def test_cpu_bf16_gemv_bench_pin():
    # compiler/src/jit.rs:29961-29965, 30016-30030: k=2560, n=9728, kernel == scalar chain, bit for bit
    k, n = 2560, 9728
    a = ((np.arange(k) % 13).astype(F) * F(0.1)).reshape(1, k)
    w = (0x3F00 | (np.arange(k * n, dtype=np.uint64) & 0x7F)).astype(np.uint16).reshape(k, n)
    assert oracle.bf16_colsplit_ways(k, n) == 4          # 47.5 MiB of weights -> 4-way split
    got = oracle.dmc_matmul_bf16(a, w)
    want = oracle.gemm_bf16_fma(a, w)
    assert np.array_equal(bits(got), bits(want))
    # a few columns against the exact-rational chain
    wf = oracle.bf16_bits_to_f32(w[:, [0, 4097, n - 1]])
    ex = exact.gemm_f32_fma(a.tolist(), wf.tolist())[0]
    assert [exact.f32_bits(v) for v in ex] == [int(v) for v in bits(got)[0, [0, 4097, n - 1]]]


def test_bf16_transpose_2d_preserves_bits():
    # compiler/src/jit.rs:30249-30263
    m, n = 2, 3
    src = (0x3F00 + np.arange(m * n) * 0x80).astype(np.uint16).reshape(m, n)
    dst = oracle.bf16_transpose_2d(src, m, n)
    assert np.array_equal(dst, src.T)
    big = np.random.default_rng(1).integers(0, 65536, (130, 67)).astype(np.uint16)
    assert np.array_equal(oracle.bf16_transpose_2d(big, 130, 67), big.T)


def test_thread_policy():
    # compiler/src/jit.rs:29527-29529 and 29471-29479
    assert oracle.bf16_colsplit_ways(512, 1024) == 1            # 1 MiB
    assert oracle.bf16_colsplit_ways(2048, 2048) == 2           # 8 MiB
    assert oracle.bf16_colsplit_ways(4096, 4096) == 4           # 32 MiB
    assert oracle.matmul_threads(1, 4096, 4096) == 1            # m == 1 never threads rows
    assert oracle.matmul_threads(2, 16, 16) == 1                # below 2^20 MACs
    assert 1 <= oracle.matmul_threads(64, 512, 512) <= 16


def _py_fingerprint(buf: bytes):
    M = (1 << 64) - 1
    n = len(buf)
    h1 = 0xCBF29CE484222325 ^ n
    h2 = (0x9E3779B97F4A7C15 * (n | 1)) & M
    words = n // 8
    if words:
        step = max(words // 256, 1)
        for i in range(0, words, step):
            v = int.from_bytes(buf[8 * i:8 * i + 8], "little")
            h1 = ((h1 ^ v) * 0x00000100000001B3) & M
            t = (h2 + v) & M
            t = ((t << 27) | (t >> 37)) & M
            h2 = (t * 0xFF51AFD7ED558CCD) & M
    return h1, h2


def test_fingerprint_matches_definition():
    # compiler/src/gpu.rs:342-358
    rng = np.random.default_rng(9)
    for nbytes in (0, 7, 8, 4096, 8 * 257, 100_003):
        b = rng.integers(0, 256, nbytes).astype(np.uint8)
        assert oracle.fingerprint(b) == _py_fingerprint(b.tobytes())


def test_numpy_oracle_matmul_case():
    # tools/numpy_oracle.py:118-121,192: (3x4)@(4x2), U(-2,2), seed 0xDEC0DE, literals printed %.5f,
    # rtol 1e-3 / atol 1e-4 (tools/numpy_oracle.py:41-42); --meta-test: a wrong reference is caught.
    rng = np.random.default_rng(0xDEC0DE)
    A = rng.uniform(-2, 2, (3, 4))
    B = rng.uniform(-2, 2, (4, 2))
    a = np.array([[float(f"{v:.5f}") for v in row] for row in A], F)
    b = np.array([[float(f"{v:.5f}") for v in row] for row in B], F)
    got = oracle.gemm_f32_fma(a, b).astype(np.float64)
    assert np.allclose(got, A @ B, rtol=1e-3, atol=1e-4)
    assert not np.allclose(got, (A @ B) * 1.5 + 1.0, rtol=1e-3, atol=1e-4)


def test_decode_companions_known_answers():
    # examples/rope.dmc:72-150: 90 degree rotation of [3,4,1,2] -> [-4,3,-2,1]; identity at angle 0
    x = np.array([3, 4, 1, 2], F)
    assert np.allclose(oracle.rope_row(x, np.zeros(2, F), np.ones(2, F)), [-4, 3, -2, 1])
    assert np.array_equal(oracle.rope_row(x, np.ones(2, F), np.zeros(2, F)), x)
    # examples/transformer.dmc:61-79: rms_norm gives unit RMS with unit gain; gain is linear
    v = np.random.default_rng(3).normal(0, 3, 64).astype(F)
    y = oracle.rms_norm_f32(v, np.ones(64, F))
    assert abs(float(np.sqrt(np.mean(y.astype(np.float64) ** 2))) - 1.0) < 1e-4
    assert np.allclose(oracle.rms_norm_f32(v, np.full(64, 2, F)), 2 * y, rtol=1e-6)
    assert np.allclose(oracle.rms_norm_f64(v, np.ones(64, F)), y, rtol=1e-5, atol=1e-6)
    # examples/kvcache.dmc:64-137: two-step uniform cache -> attention weights 0.5/0.5
    q = np.ones(4, F)
    kc = np.ones((2, 4), F)
    vc = np.array([[1, 0, 0, 0], [0, 1, 0, 0]], F)
    assert np.allclose(oracle.kv_attention_head(q, kc, vc), [0.5, 0.5, 0, 0])
    # tools/numpy_oracle.py:154-174 softmax / silu definitions
    z = np.array([0.5, -1.0, 2.0], F)
    e = np.exp(z - z.max())
    assert np.allclose(oracle.softmax_row(z), e / e.sum(), rtol=1e-6)
    assert np.allclose(oracle.silu(z), z / (1 + np.exp(-z)), rtol=1e-6)
    assert np.array_equal(oracle.softmax_row(np.full(3, -np.inf, F)), np.zeros(3, F))
    vocab = oracle.f32_to_bf16_trunc(np.arange(12, dtype=F)).reshape(4, 3)
    assert np.array_equal(oracle.embed_bf16(vocab, 99), [9, 10, 11])      # ids clamp
    assert np.array_equal(oracle.embed_bf16(vocab, -5), [0, 1, 2])
    assert oracle.argmax(np.array([1, 7, 7, 3], F)) == 1                 # first strict maximum
