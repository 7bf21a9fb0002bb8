"""`dmc_cuda_load_npz` on a GPU: the weight that arrives in HBM from the archive is the one
`vault.load_npz` would have produced on the host (compiler/src/jit.rs:29836-29927), checked by
reading it back and by running the GEMV path on it against the CPU oracle."""
import numpy as np
import pytest

import demonic_b200 as dmc
import oracle
from demonic_b200 import _lib, backend, sharded, synth
from tests.parity import TOL_BF16, assert_parity

pytestmark = pytest.mark.gpu
F = np.float32


@pytest.fixture(autouse=True)
def clean_status():
    lib = _lib.load()
    assert lib.dmc_cuda_device_count() > 0, "no CUDA device: the GPU tests cannot run on a CPU fallback"
    lib.dmc_cuda_clear_error()
    yield
    lib.dmc_cuda_clear_error()


@pytest.fixture(scope="module")
def archive(tmp_path_factory):
    rng = np.random.default_rng(11)
    n, k = 1536, 2048
    arrays = {"w_nk": synth.bf16_weights(rng, (n, k)), "w_f32": synth.f32_weights(rng, (256, 512)),
              "big": synth.bf16_weights(rng, (5000, 4096))}            # 41 MB: several trips round the staging ring
    d = tmp_path_factory.mktemp("npz")
    np.savez(d / "stored.npz", **arrays)
    np.savez_compressed(d / "deflated.npz", **arrays)
    return d, arrays


@pytest.mark.parametrize("fname", ["stored.npz", "deflated.npz"])
def test_bytes_arrive_unchanged(archive, fname):
    d, arrays = archive
    for key, wdtype in (("w_nk", backend.W_BF16), ("big", backend.W_BF16), ("w_f32", backend.W_F32)):
        a = arrays[key]
        buf, rows = backend.load_npz(d / fname, key, a.shape[0], a.shape[1], wdtype)
        assert rows == a.shape[0]
        got = buf.download(a.dtype, a.size).reshape(a.shape)
        assert np.array_equal(got, a), f"{fname}:{key}"
        buf.free()


def test_gemv_on_an_ingested_weight_matches_the_oracle(archive):
    d, arrays = archive
    w = arrays["w_nk"]
    n, k = w.shape
    x = synth.activations(np.random.default_rng(3), (1, k))
    buf, _ = backend.load_npz(d / "stored.npz", "w_nk", n, k)
    dx, dy = backend.DeviceBuffer.from_host(x), backend.DeviceBuffer(4 * n)
    backend.gemv_dev(buf, dx, dy, 1, k, n, backend.LAYOUT_NK, backend.W_BF16)
    backend.sync()
    ref = oracle.gemm_bf16_nt(x, w)
    assert_parity(dy.download(F, n).reshape(1, n), ref, TOL_BF16, "ingested weight")


@pytest.mark.parametrize("world", [2, 3, 8])
def test_each_rank_reads_only_its_rows(archive, world):
    d, arrays = archive
    a = arrays["big"]
    lib = _lib.load()
    seen = 0
    for rank in range(world):
        r0, r1 = sharded.shard_range(a.shape[0], rank, world)
        buf, rows = backend.load_npz(d / "deflated.npz" if rank == 1 else d / "stored.npz", "big", a.shape[0], a.shape[1],
                                     backend.W_BF16, rank, world)
        assert rows == r1 - r0
        assert np.array_equal(buf.download(np.uint16, rows * a.shape[1]).reshape(rows, -1), a[r0:r1])
        seen += rows
        buf.free()
    assert seen == a.shape[0]


def test_host_copy_is_registered_as_resident(archive):
    d, arrays = archive
    w = arrays["w_nk"]
    n, k = w.shape
    lib = _lib.load()
    host = np.zeros_like(w)                                   # the Forge buffer the JIT would hand around
    before = lib.dmc_cuda_resident_count()
    buf, _ = backend.load_npz(d / "stored.npz", "w_nk", n, k, host_dst=host)
    assert np.array_equal(host, w)
    assert lib.dmc_cuda_resident_count() == before + 1
    x = synth.activations(np.random.default_rng(5), (1, k))
    out = np.full((1, n), np.nan, F)
    dmc.matmul_bf16_gpu_nt(x, host, out, 1, k, n)             # by host pointer: hits the registered range
    assert lib.dmc_cuda_resident_count() == before + 1        # nothing was uploaded again
    assert_parity(out, oracle.gemm_bf16_nt(x, w), TOL_BF16, "registered ingest")
    assert lib.dmc_cuda_unregister_weight(host.ctypes.data) == 0


def test_refusals(archive, tmp_path):
    d, arrays = archive
    lib = _lib.load()
    a = arrays["w_nk"]
    cases = [("w_nk", a.shape[0] + 1, a.shape[1], backend.W_BF16),   # entry shorter than the tensor: no partial load
             ("w_nk", a.shape[0], a.shape[1], backend.W_F32),        # item size of the entry is 2, not 4
             ("absent", 4, 4, backend.W_BF16)]
    for key, rows, cols, wdtype in cases:
        with pytest.raises(_lib.DmcCudaError) as e:
            backend.load_npz(d / "stored.npz", key, rows, cols, wdtype)
        assert e.value.code == 8, str(e.value)                        # DMC_CUDA_ERR_IO
        lib.dmc_cuda_clear_error()
    with pytest.raises(_lib.DmcCudaError):
        backend.load_npz(tmp_path / "missing.npz", "w", 4, 4)
    lib.dmc_cuda_clear_error()
