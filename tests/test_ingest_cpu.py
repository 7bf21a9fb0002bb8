"""The `.npz` reader behind `dmc_cuda_load_npz`, on the host only: it must find the bytes
`vault.load_npz` would copy (dmc_vault_load_npz, compiler/src/jit.rs:29836-29927 -- zip entry
`<key>.npy` or `<key>`, NPY v1/v2 header, raw little-endian data)."""
import io
import zipfile

import numpy as np
import pytest

from demonic_b200 import backend, synth


def payload(path, info):
    with open(path, "rb") as f:
        f.seek(info["data_offset"])
        return f.read(info["data_bytes"])


@pytest.fixture
def arrays():
    rng = np.random.default_rng(7)
    return {"w": synth.bf16_weights(rng, (96, 200)), "b": rng.standard_normal((5, 3)).astype(np.float32),
            "v": np.arange(17, dtype=np.uint16)}


def test_stored_entries_of_numpy_savez(tmp_path, arrays):
    p = tmp_path / "m.npz"
    np.savez(p, **arrays)                      # stored entries, zip64 local headers
    for key, a in arrays.items():
        info = backend.npz_locate(p, key)
        assert info["method"] == 0 and info["shape"] == a.shape and info["itemsize"] == a.itemsize
        assert not info["fortran_order"] and info["data_bytes"] == a.nbytes
        assert payload(p, info) == a.tobytes()


def test_deflated_entries_are_described(tmp_path, arrays):
    p = tmp_path / "c.npz"
    np.savez_compressed(p, **arrays)
    info = backend.npz_locate(p, "w")
    assert info["method"] == 8 and info["data_offset"] == -1
    assert info["shape"] == (96, 200) and info["data_bytes"] == arrays["w"].nbytes and info["descr"] == "<u2"


def test_npy_v2_header_and_key_without_extension(tmp_path, arrays):
    p = tmp_path / "v2.npz"
    with zipfile.ZipFile(p, "w") as z:
        buf = io.BytesIO()
        np.lib.format.write_array(buf, arrays["w"], version=(2, 0))     # 4-byte header length
        z.writestr("w.npy", buf.getvalue())
        buf = io.BytesIO()
        np.lib.format.write_array(buf, arrays["b"], version=(1, 0))
        z.writestr("bare", buf.getvalue())                              # some savers omit `.npy`
    info = backend.npz_locate(p, "w")
    assert payload(p, info) == arrays["w"].tobytes()
    info = backend.npz_locate(p, "bare")
    assert info["shape"] == (5, 3) and payload(p, info) == arrays["b"].tobytes()


def test_fortran_order_and_item_size_are_reported(tmp_path):
    p = tmp_path / "f.npz"
    np.savez(p, f=np.asfortranarray(np.arange(12, dtype=np.float64).reshape(3, 4)))
    info = backend.npz_locate(p, "f")
    assert info["fortran_order"] and info["itemsize"] == 8 and info["shape"] == (3, 4)


def test_many_entries_and_archive_comment(tmp_path):
    p = tmp_path / "many.npz"
    with zipfile.ZipFile(p, "w") as z:
        for i in range(300):
            buf = io.BytesIO()
            np.lib.format.write_array(buf, np.full(3, i, np.uint16))
            z.writestr(f"k{i}.npy", buf.getvalue())
        z.comment = b"x" * 1000
    info = backend.npz_locate(p, "k257")
    assert payload(p, info) == np.full(3, 257, np.uint16).tobytes()


def test_errors(tmp_path, arrays):
    p = tmp_path / "m.npz"
    np.savez(p, **arrays)
    with pytest.raises(OSError):
        backend.npz_locate(p, "missing")
    with pytest.raises(OSError):
        backend.npz_locate(tmp_path / "nope.npz", "w")
    junk = tmp_path / "junk.npz"
    junk.write_bytes(b"this is not a zip archive" * 10)
    with pytest.raises(OSError):
        backend.npz_locate(junk, "w")
    notnpy = tmp_path / "notnpy.npz"
    with zipfile.ZipFile(notnpy, "w") as z:
        z.writestr("w.npy", b"0123456789abcdef")
    with pytest.raises(OSError):
        backend.npz_locate(notnpy, "w")
