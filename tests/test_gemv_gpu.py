"""GPU parity tests: the CUDA path, called through the C ABI with host buffers
the way JIT-emitted code calls it, against the CPU oracle on the same seeded
inputs and against the committed golden fixture."""
import numpy as np
import pytest

import demonic_b200 as dmc
import oracle
from demonic_b200 import _lib, backend, lowering, synth
from tests.golden import make_golden as mg
from tests.parity import TOL_BF16, TOL_F32, assert_parity, scaled_err

pytestmark = pytest.mark.gpu
F = np.float32
GOLD = np.load(mg.Path(mg.__file__).with_name("matmul_golden.npz"))


@pytest.fixture(autouse=True)
def clean_status():
    lib = _lib.load()
    assert lib.dmc_cuda_device_count() > 0, "no CUDA device: the GPU tests cannot run on a CPU fallback"
    lib.dmc_cuda_clear_error()
    yield
    lib.dmc_matmul_bf16_gpu_flush()
    assert lib.dmc_cuda_status() == 0, lib.dmc_cuda_last_error().decode()


def gpu_bf16(l, w, m, k, n):
    out = np.full((m, n), np.nan, F)
    dmc.matmul_bf16_gpu(l, w, out, m, k, n)
    return out


# ---- golden fixture ----------------------------------------------------------------

@pytest.mark.parametrize("case", mg.CASES, ids=[c[0] for c in mg.CASES])
def test_golden_fixture(case):
    name, kind, m, k, n, batch, lsk, rsk, seed = case
    l, r, ls, rs = mg.make_inputs(kind, m, k, n, batch, lsk, rsk, seed)
    out = np.full(batch * m * n, np.nan, F)
    if kind == "f32":
        dmc.matmul_f32_gpu(l, r, out, m, k, n)
        tol = TOL_F32
    elif kind == "nt":
        dmc.matmul_bf16_gpu_nt(l, r, out, m, k, n)
        tol = TOL_BF16
    elif batch == 1:
        dmc.matmul_bf16_gpu(l, r, out, m, k, n)
        tol = TOL_BF16
    else:
        dmc.matmul_bf16_gpu_batched(l, r, out, m, k, n, batch, ls, rs)
        tol = TOL_BF16
    ref = GOLD[name + "/y"]
    if batch == 1:
        assert_parity(out, ref, tol, name)
    else:
        for z in range(batch):
            assert_parity(out[z * n:(z + 1) * n], ref[z * n:(z + 1) * n], tol, f"{name}[{z}]")


# ---- the reference's own known answers, through the GPU -------------------------------

def test_reference_known_answers_on_gpu():
    # compiler/src/jit.rs:30204-30243 (3x5x4): exact here because every product and sum is exact in f32
    m, k, n = 3, 5, 4
    a = (np.arange(m * k, dtype=F) * F(0.5) - F(3.0)).reshape(m, k)
    w = oracle.f32_to_bf16_trunc(np.arange(k * n, dtype=F) * F(0.25) - F(2.0)).reshape(k, n)
    assert np.array_equal(gpu_bf16(a, w, m, k, n), oracle.gemm_bf16_fma(a, w))
    # compiler/src/jit.rs:42643-42655: ones [1,2] @ [2,3] -> sum 6
    assert int(gpu_bf16(np.ones((1, 2), F), np.full((2, 3), 0x3F80, np.uint16), 1, 2, 3).sum()) == 6
    # compiler/src/jit.rs:32602-32617 -> 415 and 34513-34537 -> 30300, via the f32 entry point
    a = np.array([[1, 2, 3], [4, 5, 6]], F)
    b = np.array([[7, 8], [9, 10], [11, 12]], F)
    out = np.zeros((2, 2), F)
    dmc.matmul_f32_gpu(a, b, out, 2, 3, 2)
    assert int(out.sum()) == 415
    A = np.zeros((4, 4), F)
    A[0] = [1, 2, 3, 4]
    B = np.zeros((4, 4), F)
    B[:, 0] = [10, 20, 30, 40]
    B[:, 1] = [100, 200, 300, 400]
    out = np.zeros((4, 4), F)
    dmc.matmul_f32_gpu(A, B, out, 4, 4, 4)
    assert int(out[0, 0] + out[0, 1] * F(10.0)) == 30300
    # compiler/src/jit.rs:29961-29965: the 2560x9728 FFN shape with the bench's formula inputs
    k, n = 2560, 9728
    x = ((np.arange(k) % 13).astype(F) * F(0.1)).reshape(1, k)
    w = (0x3F00 | (np.arange(k * n, dtype=np.uint64) & 0x7F)).astype(np.uint16).reshape(k, n)
    assert_parity(gpu_bf16(x, w, 1, k, n), oracle.gemm_bf16_fma(x, w), 1e-5, "ffn pin")


def test_blas_probe_shape_f32():
    # compiler/src/jit.rs:39022-39054: 96^3 GEMM, relative < 1e-5 on sum(c)*100
    i, j = np.meshgrid(np.arange(96), np.arange(96), indexing="ij")
    a = (((i + j) % 7).astype(F) * F(0.125))
    b = (((i * 3 + j) % 5).astype(F) * F(0.25))
    out = np.zeros((96, 96), F)
    dmc.matmul_f32_gpu(np.ascontiguousarray(a), np.ascontiguousarray(b), out, 96, 96, 96)
    ref = oracle.gemm_f32_fma(a, b)
    s_gpu, s_ref = float(out.sum(dtype=np.float64)) * 100, float(ref.sum(dtype=np.float64)) * 100
    assert abs(s_gpu - s_ref) / max(abs(s_ref), 1.0) < 1e-5


# ---- benchmark configurations at full size --------------------------------------------

CONFIG_SHAPES = [(2048, 2048), (4096, 4096), (11008, 4096), (4096, 11008), (14336, 4096), (4096, 14336)]


@pytest.mark.parametrize("rows,cols", CONFIG_SHAPES)
def test_config_shapes_both_layouts(rows, cols):
    """y = W.x with W [rows, cols] row-major: directly (NK entry) and in the
    reference's native order (transpose to [cols, rows], then `x @ W`)."""
    rng = np.random.default_rng(synth.DEFAULT_SEED + rows + cols)
    w_nk = synth.bf16_weights(rng, (rows, cols))
    x = synth.activations(rng, (1, cols))
    w_kn = oracle.bf16_transpose_2d(w_nk, rows, cols)
    ref = oracle.dmc_matmul_bf16(x, w_kn)
    out = np.full((1, rows), np.nan, F)
    dmc.matmul_bf16_gpu_nt(x, w_nk, out, 1, cols, rows)
    assert_parity(out, ref, TOL_BF16, "NK")
    assert_parity(gpu_bf16(x, w_kn, 1, cols, rows), ref, TOL_BF16, "KN")
    # meta-test (tools/numpy_oracle.py:216-226): a deliberately wrong reference is caught
    assert scaled_err(out, ref * 1.5) > TOL_BF16
    dmc.load().dmc_cuda_drop_resident()


def test_linearity_at_full_size():
    # size-independent property: W.(a*x1 + x2) == a*W.x1 + W.x2 within the parity bar
    k, n = 4096, 14336
    rng = np.random.default_rng(3)
    w = synth.bf16_weights(rng, (k, n))
    x1, x2 = synth.activations(rng, (1, k)), synth.activations(rng, (1, k))
    y1, y2 = gpu_bf16(x1, w, 1, k, n), gpu_bf16(x2, w, 1, k, n)
    y3 = gpu_bf16(F(0.5) * x1 + x2, w, 1, k, n)
    assert scaled_err(y3, F(0.5) * y1 + y2) < 1e-5
    assert dmc.load().dmc_cuda_resident_count() == 1       # one weight, three calls
    dmc.load().dmc_cuda_drop_resident()


# ---- edge cases --------------------------------------------------------------------------

@pytest.mark.parametrize("m,k,n", [(1, 1, 8), (1, 7, 8), (1, 8, 24), (1, 31, 1), (1, 33, 7), (2, 9, 10), (1, 513, 520),
                                   (1, 4096, 8), (1, 16, 4104), (7, 128, 264), (16, 256, 512), (19, 100, 72)])
def test_ragged_and_small_shapes(m, k, n):
    rng = np.random.default_rng(m * 1000003 + k * 1009 + n)
    x = synth.activations(rng, (m, k))
    w = synth.bf16_weights(rng, (k, n), std=1.0)
    assert_parity(gpu_bf16(x, w, m, k, n), oracle.gemm_bf16_fma(x, w), 1e-5, f"{m}x{k}x{n}")
    wn = np.ascontiguousarray(w.T)
    out = np.full((m, n), np.nan, F)
    dmc.matmul_bf16_gpu_nt(x, wn, out, m, k, n)
    assert_parity(out, oracle.gemm_bf16_fma(x, w), 1e-5, f"nt {m}x{k}x{n}")
    wf = synth.bf16_to_f32(w)
    out = np.full((m, n), np.nan, F)
    dmc.matmul_f32_gpu(x, wf, out, m, k, n)
    assert_parity(out, oracle.gemm_f32_fma(x, wf), TOL_F32, f"f32 {m}x{k}x{n}")


def test_empty_shapes():
    x = np.ones((1, 8), F)
    w = np.full((8, 8), 0x3F80, np.uint16)
    out = np.full((1, 8), 5.0, F)
    dmc.matmul_bf16_gpu(x, w, out, 0, 8, 8)       # m == 0 / n == 0 return (compiler/src/gpu.rs:402)
    dmc.matmul_bf16_gpu(x, w, out, 1, 8, 0)
    assert np.all(out == 5.0)
    dmc.matmul_bf16_gpu(x, w, out, 1, 0, 8)       # k == 0: the row is zeroed and nothing is added
    assert np.all(out == 0.0)
    dmc.matmul_bf16_gpu_batched(x, w, out, 1, 8, 8, 0, 0, 0)


@pytest.mark.parametrize("batch,ls_full,rs_full", [(1, True, True), (2, True, True), (3, False, True),
                                                   (3, True, False), (32, False, True), (8, True, True)])
def test_batched_strides(batch, ls_full, rs_full):
    # compiler/src/gpu.rs:784-790 decode projection shapes, scaled down
    k, n = 320, 128
    rng = np.random.default_rng(batch * 7 + ls_full * 2 + rs_full)
    ls, rs = (k if ls_full else 0), (k * n if rs_full else 0)
    l = synth.activations(rng, ((batch - 1) * ls + k,))
    r = synth.bf16_weights(rng, ((batch - 1) * rs + k * n,), std=1.0)
    out = np.full((batch, n), np.nan, F)
    dmc.matmul_bf16_gpu_batched(l, r, out, 1, k, n, batch, ls, rs)
    ref = oracle.bf16_gemv_batched(l, r, k, n, batch, ls, rs)
    for z in range(batch):
        assert_parity(out[z], ref[z], 1e-5, f"slice {z}")


@pytest.mark.parametrize("n", [8, 32, 64, 72, 128, 136])
@pytest.mark.parametrize("k", [128, 1000, 2560])
def test_narrow_per_head_projections(n, k):
    """Narrow matrices (the per-head projections: n = 128 or 64) run in the form where a warp-wide load
    covers 2 or 4 k rows; widths around the switch points, k not a multiple of the row tiling, several
    split-K factors, bf16 and f32."""
    lib = dmc.load()
    batch = 5
    rng = np.random.default_rng(1000 * n + k)
    x = synth.activations(rng, (1, k))
    w = synth.bf16_weights(rng, (batch, k, n))
    ref = np.stack([oracle.gemm_bf16_fma(x, w[z])[0] for z in range(batch)])
    for ksplit in (0, 1, 3):
        lib.dmc_cuda_set_param(b"kn_ksplit", ksplit)
        out = np.full((batch, n), np.nan, F)
        dmc.matmul_bf16_gpu_batched(x, w, out, 1, k, n, batch, 0, k * n)
        for z in range(batch):
            assert_parity(out[z], ref[z], TOL_BF16, f"bf16 n={n} k={k} ksplit={ksplit} slice {z}")
    lib.dmc_cuda_set_param(b"kn_ksplit", 0)
    wf = synth.f32_weights(rng, (k, n), std=1.0)
    out = np.full((1, n), np.nan, F)
    dmc.matmul_f32_gpu(x, wf, out, 1, k, n)
    assert_parity(out, oracle.gemm_f32_fma(x, wf), TOL_F32, f"f32 n={n} k={k}")


def test_batched_unaligned_stride_uses_generic_kernel():
    k, n, batch = 33, 12, 3          # rs = 396, not a multiple of 8
    rng = np.random.default_rng(77)
    l = synth.activations(rng, (batch * k,))
    r = synth.bf16_weights(rng, (batch * k * n,), std=1.0)
    out = np.full((batch, n), np.nan, F)
    dmc.matmul_bf16_gpu_batched(l, r, out, 1, k, n, batch, k, k * n)
    assert_parity(out, oracle.bf16_gemv_batched(l, r, k, n, batch, k, k * n), 1e-5)


def test_deferred_calls_materialise_on_flush():
    # compiler/src/gpu.rs:441-474: deferred output is written by the next sync call or the flush
    k, n = 512, 1024
    rng = np.random.default_rng(5)
    w1, w2 = synth.bf16_weights(rng, (k, n)), synth.bf16_weights(rng, (k, n))
    x = synth.activations(rng, (1, k))
    o1 = np.full((1, n), -7.0, F)
    o2 = np.full((1, n), -7.0, F)
    o3 = np.full((1, n), -7.0, F)
    dmc.matmul_bf16_gpu_batched_deferred(x, w1, o1, 1, k, n, 1, 0, 0)
    dmc.matmul_bf16_gpu_batched_deferred(x, w2, o2, 1, k, n, 1, 0, 0)
    assert np.all(o1 == -7.0) and np.all(o2 == -7.0), "a deferred call must not write `out`"
    dmc.matmul_bf16_gpu_batched(x, w1, o3, 1, k, n, 1, 0, 0)      # sync call materialises its neighbours
    assert_parity(o1, oracle.gemm_bf16_fma(x, w1), TOL_BF16)
    assert_parity(o2, oracle.gemm_bf16_fma(x, w2), TOL_BF16)
    assert np.array_equal(o1, o3)
    o4 = np.full((1, n), -7.0, F)
    dmc.matmul_bf16_gpu_batched_deferred(x, w2, o4, 1, k, n, 1, 0, 0)
    dmc.matmul_bf16_gpu_flush()
    assert np.array_equal(o4, o2)
    dmc.matmul_bf16_gpu_flush()                                   # idempotent


def test_deferred_output_read_by_next_call_is_flushed_first():
    # compiler/src/gpu.rs:491-499: a call that reads a deferred output as its activation flushes first
    k = n = 256
    rng = np.random.default_rng(6)
    w = synth.bf16_weights(rng, (k, n), std=0.1)
    x = synth.activations(rng, (1, k))
    h = np.zeros((1, n), F)
    y = np.zeros((1, n), F)
    dmc.matmul_bf16_gpu_batched_deferred(x, w, h, 1, k, n, 1, 0, 0)
    dmc.matmul_bf16_gpu_batched(h, w, y, 1, k, n, 1, 0, 0)
    href = oracle.gemm_bf16_fma(x, w)
    assert_parity(h, href, TOL_BF16)
    assert_parity(y, oracle.gemm_bf16_fma(h, w), TOL_BF16)


def test_many_deferred_calls_grow_staging():
    k, n, calls = 256, 4096, 40          # 40 x 16 KiB of outputs > the initial 256 KiB staging
    rng = np.random.default_rng(8)
    w = synth.bf16_weights(rng, (k, n))
    xs = [synth.activations(rng, (1, k)) for _ in range(calls)]
    outs = [np.zeros((1, n), F) for _ in range(calls)]
    for x, o in zip(xs, outs):
        dmc.matmul_bf16_gpu_batched_deferred(x, w, o, 1, k, n, 1, 0, 0)
    dmc.matmul_bf16_gpu_flush()
    for x, o in zip(xs, outs):
        assert_parity(o, oracle.gemm_bf16_fma(x, w), TOL_BF16)


def test_weights_stay_resident_across_fresh_addresses():
    # compiler/src/gpu.rs:195-200: same bytes at a new address every decode step must hit the memo
    lib = dmc.load()
    lib.dmc_cuda_drop_resident()
    k, n = 1024, 2048
    rng = np.random.default_rng(9)
    w = synth.bf16_weights(rng, (k, n))
    x = synth.activations(rng, (1, k))
    ref = oracle.gemm_bf16_fma(x, w)
    for _ in range(4):
        w_again = w.copy()                     # fresh host address, identical content
        assert_parity(gpu_bf16(x, w_again, 1, k, n), ref, TOL_BF16)
    assert lib.dmc_cuda_resident_count() == 1
    assert lib.dmc_cuda_resident_bytes() == k * n * 2
    w2 = w.copy()
    w2[::7] ^= 0x0040                          # different content -> a second resident buffer
    assert_parity(gpu_bf16(x, w2, 1, k, n), oracle.gemm_bf16_fma(x, w2), TOL_BF16)
    assert lib.dmc_cuda_resident_count() == 2
    lib.dmc_cuda_drop_resident()
    assert lib.dmc_cuda_resident_count() == 0


def test_registered_weight_range():
    lib = dmc.load()
    k, n = 512, 768
    rng = np.random.default_rng(10)
    blob = synth.bf16_weights(rng, (3 * k * n,))       # three layers in one vault buffer
    assert lib.dmc_cuda_register_weight(blob.ctypes.data, blob.nbytes, 0, 0, 0, backend.W_BF16) == 0      # opaque range
    before = lib.dmc_cuda_resident_count()
    x = synth.activations(rng, (1, k))
    for layer in range(3):
        w = blob[layer * k * n:(layer + 1) * k * n]
        out = np.zeros((1, n), F)
        lib.dmc_matmul_bf16_gpu(x.ctypes.data, w.ctypes.data, out.ctypes.data, 1, k, n)
        _lib.check()
        assert_parity(out, oracle.gemm_bf16_fma(x, w.reshape(k, n)), TOL_BF16)
    assert lib.dmc_cuda_resident_count() == before      # served from the registered range, no new uploads
    assert lib.dmc_cuda_unregister_weight(blob.ctypes.data) == 0


def test_registered_matrix_is_stored_k_contiguous():
    """A registered [k, n] matrix (the vault-load hook with its shape) gets the same k-contiguous
    residency as a weight found by fingerprint: one transpose at registration, then the row kernel."""
    lib = dmc.load()
    k, n = 4096, 1024
    rng = np.random.default_rng(11)
    w = synth.bf16_weights(rng, (k, n))
    x = synth.activations(rng, (1, k))
    before = lib.dmc_cuda_launch_count()
    assert lib.dmc_cuda_register_weight(w.ctypes.data, w.nbytes, k, n, backend.LAYOUT_KN, backend.W_BF16) == 0
    assert lib.dmc_cuda_launch_count() - before == 1, "one transpose kernel at registration"
    resident = lib.dmc_cuda_resident_count()
    assert_parity(gpu_bf16(x, w, 1, k, n), oracle.gemm_bf16_fma(x, w), TOL_BF16)
    # x in, the GEMV, y out
    assert lib.dmc_cuda_launch_count() - before == 1 + 3 and lib.dmc_cuda_resident_count() == resident
    # another view of the same bytes is served by content, not from the transposed copy
    assert_parity(gpu_bf16(x[:, :2048], w.reshape(2048, 2048), 1, 2048, 2048),
                  oracle.gemm_bf16_fma(x[:, :2048], w.reshape(2048, 2048)), TOL_BF16)
    assert lib.dmc_cuda_unregister_weight(w.ctypes.data) == 0
    assert lib.dmc_cuda_register_weight(w.ctypes.data, w.nbytes - 2, k, n, backend.LAYOUT_KN, backend.W_BF16) == 2   # not k*n elements
    lib.dmc_cuda_clear_error()
    lib.dmc_cuda_drop_resident()


@pytest.mark.parametrize("m", [2, 3, 4, 5, 7, 8, 9, 16])
def test_small_batch_keeps_f32_rows_on_the_cuda_cores(m):
    """x @ w' with a few f32 rows of x on a k-contiguous weight: up to 8 rows share every weight load
    in the multi-row kernel with exact f32 activations (parity at the f32-order level, far inside 1e-2);
    more rows go to the tensor cores.  With `tc_min_m` raised, 9 and 16 rows stay on the CUDA cores too."""
    k, n = 4096, 4096
    rng = np.random.default_rng(700 + m)
    w = synth.bf16_weights(rng, (n, k))
    x = synth.activations(rng, (m, k))
    out = np.full((m, n), np.nan, F)
    lib = dmc.load()
    lib.dmc_cuda_set_param(b"host_io_kernels", 0)               # count the GEMV launches only: x and y by the copy engines
    try:
        before = lib.dmc_cuda_launch_count()
        dmc.matmul_bf16_gpu_nt(x, w, out, m, k, n)
        dmc.matmul_bf16_gpu_nt(x, w, out, m, k, n)              # the weight is resident now: count this call's launches
        launches = (lib.dmc_cuda_launch_count() - before) // 2
        ref = oracle.gemm_bf16_fma(x, np.ascontiguousarray(w.T))
        err = assert_parity(out, ref, TOL_BF16, f"m={m}")
        if m <= 8:
            assert err < 1e-5, f"m={m}: the CUDA-core rows use exact f32 activations (got {err:.2e})"
            assert launches == 1, "up to 8 rows in one instance: W streamed once"
        lib.dmc_cuda_set_param(b"tc_min_m", 1 << 20)            # every row count on the CUDA cores
        out2 = np.full((m, n), np.nan, F)
        before = lib.dmc_cuda_launch_count()
        dmc.matmul_bf16_gpu_nt(x, w, out2, m, k, n)
        assert lib.dmc_cuda_launch_count() - before == -(-m // 8)
        assert assert_parity(out2, ref, TOL_BF16, f"m={m} cuda cores") < 1e-5
    finally:
        lib.dmc_cuda_set_param(b"tc_min_m", 0)
        lib.dmc_cuda_set_param(b"host_io_kernels", 1)


def test_batched_slices_with_several_rows_run_on_the_gpu():
    # compiler/src/gpu.rs:428-437: batch > 1 with m != 1 runs slice by slice; here on the GPU, not refused
    lib = dmc.load()
    m, k, n, batch = 3, 512, 256, 4
    rng = np.random.default_rng(15)
    l = synth.activations(rng, (batch, m, k))
    r = synth.bf16_weights(rng, (batch, k, n))
    out = np.full((batch, m, n), np.nan, F)
    dmc.matmul_bf16_gpu_batched(l, r, out, m, k, n, batch, m * k, k * n)
    for z in range(batch):
        assert_parity(out[z], oracle.gemm_bf16_fma(l[z], r[z]), TOL_BF16, f"slice {z}")
    assert not backend.matmul_selected(True, 0, m, k, n, batch)        # ... though the JIT gate never selects it
    # whatever the predicate selects, the entry points accept
    for (mm, kk, nn, bb) in [(1, 2560, 128, 8), (1, 128, 2560, 32), (1, 4096, 4096, 1), (1, 1000, 1000, 4)]:
        if backend.matmul_selected(True, 0, mm, kk, nn, bb):
            l2 = synth.activations(rng, (bb, mm, kk))
            r2 = synth.bf16_weights(rng, (bb, kk, nn))
            o2 = np.zeros((bb, mm, nn), F)
            dmc.matmul_bf16_gpu_batched(l2, r2, o2, mm, kk, nn, bb, mm * kk, kk * nn)
            assert lib.dmc_cuda_status() == 0
            assert_parity(o2[bb - 1], oracle.gemm_bf16_fma(l2[bb - 1], r2[bb - 1]), TOL_BF16)


def test_independent_gemvs_overlap_and_dependent_ones_do_not():
    """A GEMV whose operands no running kernel touches skips its dependency wait; one that consumes
    an earlier result must still see it.  Same numbers with the overlap on and off."""
    lib = dmc.load()
    k = n = 2048
    rng = np.random.default_rng(16)
    ws = [synth.bf16_weights(rng, (n, k)) for _ in range(4)]
    x = synth.activations(rng, (k,)) 
    dWs = [backend.DeviceBuffer.from_host(w) for w in ws]
    dx = backend.DeviceBuffer.from_host(x)
    dys = [backend.DeviceBuffer(n * 4) for _ in range(4)]
    dchain = [backend.DeviceBuffer(n * 4) for _ in range(3)]
    results = {}
    for overlap in (1, 0):
        lib.dmc_cuda_set_param(b"overlap_independent", overlap)
        for rep in range(3):
            for dW, dy in zip(dWs, dys):                           # four independent GEMVs of the same x
                backend.gemv_dev(dW, dx, dy, 1, k, n, backend.LAYOUT_NK)
            backend.gemv_dev(dWs[0], dx, dchain[0], 1, k, n, backend.LAYOUT_NK)          # a chain: each consumes the previous y
            backend.gemv_dev(dWs[1], dchain[0], dchain[1], 1, k, n, backend.LAYOUT_NK)
            backend.gemv_dev(dWs[2], dchain[1], dchain[2], 1, k, n, backend.LAYOUT_NK)
            backend.gemv_dev(dWs[3], dx, dchain[0], 1, k, n, backend.LAYOUT_NK)          # overwrites what the chain's 2nd link read
        backend.sync()
        results[overlap] = [d.download(F, n) for d in dys + dchain]
    lib.dmc_cuda_set_param(b"overlap_independent", 1)
    for a, b in zip(results[1], results[0]):
        assert np.array_equal(a, b), "overlapping launches changed a result"
    xs = x.reshape(1, k)
    for w, y in zip(ws, results[1][:4]):
        assert_parity(y, oracle.gemm_bf16_fma(xs, np.ascontiguousarray(w.T)), TOL_BF16)
    y0 = oracle.gemm_bf16_fma(xs, np.ascontiguousarray(ws[0].T))
    y1 = oracle.gemm_bf16_fma(y0, np.ascontiguousarray(ws[1].T))
    y2 = oracle.gemm_bf16_fma(y1, np.ascontiguousarray(ws[2].T))
    assert_parity(results[1][5], y1, TOL_BF16, "second link")
    assert_parity(results[1][6], y2, TOL_BF16, "third link")
    assert_parity(results[1][4], oracle.gemm_bf16_fma(xs, np.ascontiguousarray(ws[3].T)), TOL_BF16, "the overwrite comes last")


def test_f32_operand_is_not_cached_by_fingerprint():
    # an arbitrary f32 right operand may change between calls at unsampled positions
    k, n = 2048, 1024
    rng = np.random.default_rng(12)
    b = synth.f32_weights(rng, (k, n), std=1.0)
    x = synth.activations(rng, (1, k))
    out = np.zeros((1, n), F)
    dmc.matmul_f32_gpu(x, b, out, 1, k, n)
    assert_parity(out, oracle.gemm_f32_fma(x, b), TOL_F32)
    b[5, 3] += 100.0                       # index 5*1024+3 is not a fingerprint sample
    dmc.matmul_f32_gpu(x, b, out, 1, k, n)
    assert_parity(out, oracle.gemm_f32_fma(x, b), TOL_F32)


def test_bad_arguments_set_sticky_status():
    lib = dmc.load()
    x = np.ones((1, 8), F)
    w = np.full((8, 8), 0x3F80, np.uint16)
    out = np.full((1, 8), 9.0, F)
    with pytest.raises(dmc.DmcCudaError) as ei:
        dmc.matmul_bf16_gpu(x, w, out, 1, -8, 8)
    assert ei.value.code == 2
    # sticky: later calls do nothing until the host clears (it would have exited)
    lib.dmc_matmul_bf16_gpu(x.ctypes.data, w.ctypes.data, out.ctypes.data, 1, 8, 8)
    assert np.all(out == 9.0) and lib.dmc_cuda_status() == 2
    lib.dmc_cuda_clear_error()
    dmc.matmul_bf16_gpu(x, w, out, 1, 8, 8)
    assert np.all(out == 8.0)


# ---- every kernel configuration, device-resident path ------------------------------------

@pytest.mark.parametrize("layout", [backend.LAYOUT_KN, backend.LAYOUT_NK])
@pytest.mark.parametrize("wdtype", [backend.W_BF16, backend.W_F32])
def test_every_kernel_variant(layout, wdtype):
    lib = dmc.load()
    k, n = 1544, 2072            # not multiples of any tile: exercises every edge predicate
    rng = np.random.default_rng(13 + layout * 2 + wdtype)
    x = synth.activations(rng, (1, k))
    if wdtype == backend.W_BF16:
        w = synth.bf16_weights(rng, (k, n))
        ref = oracle.gemm_bf16_fma(x, w)
    else:
        w = synth.f32_weights(rng, (k, n))
        ref = oracle.gemm_f32_fma(x, w)
    w_dev = w if layout == backend.LAYOUT_KN else np.ascontiguousarray(w.T)
    dW, dx = backend.DeviceBuffer.from_host(w_dev), backend.DeviceBuffer.from_host(x)
    dy = backend.DeviceBuffer(n * 4)
    tol = TOL_BF16 if wdtype == backend.W_BF16 else TOL_F32
    count = lib.dmc_cuda_variant_count(layout, wdtype)
    assert count > 0
    for v in range(count):
        for ksplit in ((0, 1, 5) if layout == backend.LAYOUT_KN else (0,)):
            lib.dmc_cuda_set_param(b"kn_ksplit", ksplit)
            lib.dmc_cuda_memset(dy.ptr, 0xFF, n * 4)
            backend.gemv_dev(dW, dx, dy, 1, k, n, layout, wdtype, v)
            backend.sync()
            got = dy.download(F, n)
            assert_parity(got, ref, tol, lib.dmc_cuda_variant_name(layout, wdtype, v).decode() + f" ksplit={ksplit}")
    lib.dmc_cuda_set_param(b"kn_ksplit", 0)


@pytest.mark.parametrize("wdtype", [backend.W_BF16, backend.W_F32])
@pytest.mark.parametrize("k,n", [(2048, 300), (2560, 1000), (4096, 4096), (6144, 777), (8192, 148), (11008, 512),
                                 (14336, 301), (16384, 64), (28672, 100), (4096, 1), (4096, 147), (2048 + 8, 149)])
def test_tma_ring_kernel(k, n, wdtype):
    """The bulk-copy ring kernel across its register-slice widths, both consumer-warp
    counts, ragged row counts (fewer rows than CTAs, partial last stage) and ring shapes."""
    lib = dmc.load()
    if wdtype == backend.W_F32 and k > 16384:
        pytest.skip("f32 rows this long go to the LDG kernel")
    rng = np.random.default_rng(k * 31 + n + wdtype)
    x = synth.activations(rng, (1, k))
    if wdtype == backend.W_BF16:
        w = synth.bf16_weights(rng, (n, k))
        ref = oracle.gemm_bf16_fma(x, np.ascontiguousarray(w.T))
        tol = TOL_BF16
    else:
        w = synth.f32_weights(rng, (n, k))
        ref = oracle.gemm_f32_fma(x, np.ascontiguousarray(w.T))
        tol = TOL_F32
    dW, dx, dy = backend.DeviceBuffer.from_host(w), backend.DeviceBuffer.from_host(x), backend.DeviceBuffer(n * 4)
    total = lib.dmc_cuda_variant_count(backend.LAYOUT_NK, wdtype)
    try:
        for variant in (total - 2, total - 1):                   # nk_tma_cw8, nk_tma_cw16
            for ring, stage in ((0, 0), (64, 8), (192, 64), (128, 16)):
                lib.dmc_cuda_set_param(b"tma_ring_kb", ring)
                lib.dmc_cuda_set_param(b"tma_stage_kb", stage)
                lib.dmc_cuda_memset(dy.ptr, 0xFF, n * 4)
                backend.gemv_dev(dW, dx, dy, 1, k, n, backend.LAYOUT_NK, wdtype, variant)
                backend.sync()
                name = lib.dmc_cuda_variant_name(backend.LAYOUT_NK, wdtype, variant).decode()
                assert_parity(dy.download(F, n), ref, tol, f"{name} ring={ring} stage={stage}")
    finally:
        lib.dmc_cuda_set_param(b"tma_ring_kb", 0)
        lib.dmc_cuda_set_param(b"tma_stage_kb", 0)


def test_host_call_moves_x_and_y_with_kernels_and_still_checks_the_weight():
    """Up to 64 KiB each way, a host-pointer call is three kernels (x in, GEMV, y out + completion word)
    and launches before it has read the weight's fingerprint.  The fingerprint is still compared on every
    call: a weight changed in place at the same address gives the new product, never the old one; the
    copy-engine path ("host_io_kernels" = 0) gives bit-identical results; deferred calls deliver at the flush."""
    lib = dmc.load()
    lib.dmc_cuda_drop_resident()
    k, n = 2048, 1536
    rng = np.random.default_rng(77)
    w = synth.bf16_weights(rng, (k, n))
    x = synth.activations(rng, (1, k))
    first = gpu_bf16(x, w, 1, k, n)
    before = lib.dmc_cuda_launch_count()
    again = gpu_bf16(x, w, 1, k, n)
    assert lib.dmc_cuda_launch_count() - before == 3
    assert np.array_equal(first, again)
    assert_parity(again, oracle.gemm_bf16_fma(x, w), TOL_BF16)
    # same address, new content (every 4th row, so that the sampled words certainly change)
    w[::4, :] = synth.bf16_weights(rng, (k // 4, n))
    changed = gpu_bf16(x, w, 1, k, n)
    assert_parity(changed, oracle.gemm_bf16_fma(x, w), TOL_BF16)
    assert not np.array_equal(changed, first)
    assert np.array_equal(gpu_bf16(x, w, 1, k, n), changed)
    # many different x at one weight: each call's y belongs to its own x
    for i in range(8):
        xi = synth.activations(rng, (1, k))
        assert_parity(gpu_bf16(xi, w, 1, k, n), oracle.gemm_bf16_fma(xi, w), TOL_BF16, f"call {i}")
    # the copy-engine path computes the same bits
    lib.dmc_cuda_set_param(b"host_io_kernels", 0)
    try:
        assert np.array_equal(gpu_bf16(x, w, 1, k, n), changed)
    finally:
        lib.dmc_cuda_set_param(b"host_io_kernels", 1)
    # deferred calls: nothing is delivered before the flush, everything after it
    outs = [np.full((1, n), np.nan, F) for _ in range(3)]
    xs = [synth.activations(rng, (1, k)) for _ in range(3)]
    for xi, oi in zip(xs, outs):
        lib.dmc_matmul_bf16_gpu_batched_deferred(xi.ctypes.data, w.ctypes.data, oi.ctypes.data, 1, k, n, 1, 0, 0)
    assert all(np.isnan(oi).all() for oi in outs)
    lib.dmc_matmul_bf16_gpu_flush()
    _lib.check()
    for xi, oi in zip(xs, outs):
        assert_parity(oi, oracle.gemm_bf16_fma(xi, w), TOL_BF16)
    lib.dmc_cuda_drop_resident()


def test_resident_kn_weight_is_stored_k_contiguous_once():
    # a [k, n] weight the row-streaming kernel can take is transposed on the device at upload; later calls reuse it
    lib = dmc.load()
    lib.dmc_cuda_drop_resident()
    k, n = 4096, 1024
    rng = np.random.default_rng(31)
    w = synth.bf16_weights(rng, (k, n))
    x = synth.activations(rng, (1, k))
    ref = oracle.gemm_bf16_fma(x, w)
    first = lib.dmc_cuda_launch_count()
    assert_parity(gpu_bf16(x, w, 1, k, n), ref, TOL_BF16)
    after_first = lib.dmc_cuda_launch_count()
    assert_parity(gpu_bf16(x, w.copy(), 1, k, n), ref, TOL_BF16)
    assert after_first - first == 2 + 2, "upload = one transpose kernel + one GEMV (+ x in, y out)"
    assert lib.dmc_cuda_launch_count() - after_first == 1 + 2, "second call = one GEMV, no re-upload"
    assert lib.dmc_cuda_resident_count() == 1
    # the same bytes viewed with another shape are a different resident entry
    assert_parity(gpu_bf16(x[:, :2048], w.reshape(2048, 2048), 1, 2048, 2048),
                  oracle.gemm_bf16_fma(x[:, :2048], w.reshape(2048, 2048)), TOL_BF16)
    assert lib.dmc_cuda_resident_count() == 2
    lib.dmc_cuda_drop_resident()


def test_lowering_plan_runs_through_the_abi():
    # the whole compile-time decision + runtime call, as the JIT would make it, vs the interpreter's batched `@`
    low = lowering.Lowering(cuda=True)
    rng = np.random.default_rng(21)
    l = synth.activations(rng, (1, 1, 1, 2560))
    r = synth.bf16_weights(rng, (8, 2560, 128))
    plan = low.lower(l.shape, r.shape)
    out = np.zeros(plan.out_shape, F)
    left = lowering.run(plan, l, r, out)
    assert left == [] and plan.calls[0].symbol == lowering.SYM_BATCHED
    ref = oracle.matmul_broadcast_f32(l, synth.bf16_to_f32(r))
    for h in range(8):
        assert_parity(out[0, h], ref[0, h], TOL_BF16)
    with low.deterministic():
        plan = low.lower(l.shape, r.shape)
        assert all(not c.on_gpu for c in plan.calls)
