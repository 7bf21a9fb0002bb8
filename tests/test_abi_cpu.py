"""CPU-side checks of the boundary: the library loads, exports every symbol the
header declares, the selection predicate follows the reference's `--blas` rule,
and calls fail loudly (no CPU fallback) when there is no device."""
import re
from pathlib import Path

import numpy as np
import pytest

import demonic_b200 as dmc
from demonic_b200 import _lib
from demonic_b200.lowering import (CPU_BF16, CPU_F32, SYM_BATCHED, SYM_BATCHED_DEFERRED, SYM_F32, SYM_SINGLE,
                                   Lowering)

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "dmc_cuda.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dmc_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 30
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/dmc_cuda.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"


def test_selection_predicate():
    # modelled on `jit_blas_selection_predicate`, compiler/src/jit.rs:39087-39103
    sel = dmc.matmul_selected
    assert sel(True, 0, 1, 2048, 2048), "eligible GEMV refused"
    assert not sel(False, 0, 1, 2048, 2048), "selected with the flag off"
    assert not sel(True, 1, 1, 2048, 2048), "selected inside @deterministic"
    assert not sel(True, 2, 1, 2048, 2048), "selected inside nested @deterministic"
    assert not sel(True, 0, 1, 1024, 1024), "selected below the 4e6 single-GEMV gate"
    assert sel(True, 0, 1, 2000, 2000) and not sel(True, 0, 1, 1999, 2000), "k*n boundary, both sides"
    # batched projection: total MACs gate 1e6, batch <= 65536 (compiler/src/jit.rs:19912-19915)
    assert sel(True, 0, 1, 2560, 128, batch=32)
    assert not sel(True, 0, 1, 16, 16, batch=32)
    assert not sel(True, 0, 1, 64, 64, batch=65537)
    # f32 site: the BLAS_MIN_MACS threshold, both sides (compiler/src/jit.rs:39100-39102)
    assert sel(True, 0, 1, 1, 131_072, rhs_bf16=False)
    assert not sel(True, 0, 1, 1, 131_071, rhs_bf16=False)
    assert sel(True, 0, 64, 64, 64, rhs_bf16=False) and not sel(True, 0, 32, 32, 32, rhs_bf16=False)
    assert not sel(True, 1, 64, 64, 64, rhs_bf16=False)


def test_flag_defaults_off_and_changes_nothing():
    # `jit_blas_defaults_off`, compiler/src/jit.rs:39105-39113: with the flag unset every
    # matmul lowers as before (to the reference's own CPU builtins)
    low = Lowering()
    assert low.cuda is False
    plan = low.lower((1, 4096), (4096, 4096))
    assert [c.symbol for c in plan.calls] == [CPU_BF16]
    assert [c.symbol for c in low.lower((96, 96), (96, 96), rhs_bf16=False).calls] == [CPU_F32]


def test_flag_is_unreachable_inside_deterministic():
    # `jit_blas_fast_path_is_unreachable_inside_deterministic`, compiler/src/jit.rs:39056-39085:
    # inside the block the flag makes no difference at all; outside, the same shape is eligible
    on, off = Lowering(cuda=True), Lowering(cuda=False)
    with on.deterministic(), off.deterministic():
        with on.deterministic():
            pass                                        # an inner block ending must not clear the outer
        a = on.lower((1, 4096), (4096, 4096))
        b = off.lower((1, 4096), (4096, 4096))
        assert [c.symbol for c in a.calls] == [c.symbol for c in b.calls] == [CPU_BF16]
        assert [c.symbol for c in on.lower((96, 96), (96, 96), rhs_bf16=False).calls] == [CPU_F32]
    assert [c.symbol for c in on.lower((1, 4096), (4096, 4096)).calls] == [SYM_BATCHED]
    assert [c.symbol for c in on.lower((96, 96), (96, 96), rhs_bf16=False).calls] == [SYM_F32]


def test_batched_lowering_is_affine_for_decode_projections():
    # compiler/src/jit.rs:19897-19957 and the shapes of compiler/src/gpu.rs:784-790
    low = Lowering(cuda=True)
    q = low.lower((1, 1, 1, 2560), (32, 2560, 128)).calls          # [B,1,S,K] @ [H,K,N]
    assert len(q) == 1 and q[0].symbol == SYM_BATCHED
    assert (q[0].batch, q[0].ls, q[0].rs) == (32, 0, 2560 * 128)
    wo = low.lower((1, 32, 1, 128), (32, 128, 2560)).calls
    assert (wo[0].batch, wo[0].ls, wo[0].rs) == (32, 128, 128 * 2560)
    ffn = low.lower((1, 2560), (2560, 9728)).calls
    assert (ffn[0].symbol, ffn[0].batch, ffn[0].ls, ffn[0].rs) == (SYM_BATCHED, 1, 0, 0)
    # non-affine broadcast ([2,1] x [1,3] batch dims) falls back to per-slice calls
    per = low.lower((2, 1, 1, 2048), (1, 3, 2048, 2048)).calls
    assert len(per) == 6 and all(c.symbol == SYM_SINGLE for c in per)
    assert [c.l_off for c in per] == [0, 0, 0, 2048, 2048, 2048]
    assert [c.r_off for c in per] == [0, 2048 * 2048, 2 * 2048 * 2048] * 2
    # too small for the GPU stays on the CPU builtin
    assert [c.symbol for c in low.lower((1, 64), (64, 64)).calls] == [CPU_BF16]
    # prefill (m > 1) uses the single entry when the weight is big enough
    assert [c.symbol for c in low.lower((4, 4096), (4096, 4096)).calls] == [SYM_SINGLE]


def test_deferred_lowering_emits_flush_before_direct_reads():
    # compiler/src/jit.rs:19935-19961, 20903-20914
    low = Lowering(cuda=True)
    low.defer_hint = True
    a = low.lower((1, 4096), (4096, 4096))
    assert a.calls[0].symbol == SYM_BATCHED_DEFERRED and low.defer_pending
    low.defer_hint = False
    b = low.lower((1, 64), (64, 64))                    # per-slice CPU path: must flush first
    assert b.flush_first and not low.defer_pending
    assert not low.lower((1, 64), (64, 64)).flush_first


def test_shape_errors():
    # compiler/src/check_tests.rs:115-185 / compiler/src/jit.rs:19864-19882
    low = Lowering(cuda=True)
    with pytest.raises(ValueError, match="rank >= 2"):
        low.lower((4,), (4, 4))
    with pytest.raises(ValueError, match="inner dim mismatch"):
        low.lower((1, 4), (5, 4))
    with pytest.raises(ValueError, match="not broadcastable"):
        low.lower((2, 1, 4), (3, 4, 4))


def test_no_device_fails_loudly_without_touching_out():
    lib = _lib.load()
    if lib.dmc_cuda_device_count() > 0:
        pytest.skip("a CUDA device is present")
    x = np.ones((1, 8), np.float32)
    w = np.full((8, 8), 0x3F80, np.uint16)
    out = np.full((1, 8), 123.0, np.float32)
    with pytest.raises(dmc.DmcCudaError) as ei:
        dmc.matmul_bf16_gpu(x, w, out, 1, 8, 8)
    assert ei.value.code == 1 and "no CUDA device" in str(ei.value)
    assert np.all(out == 123.0), "a failed call must not write `out` (and must not compute on the CPU)"
    lib.dmc_cuda_clear_error()
    assert lib.dmc_cuda_status() == 0
    # empty shapes return before touching the device, like compiler/src/gpu.rs:402
    dmc.matmul_bf16_gpu(x, w, out, 0, 8, 8)
    dmc.matmul_bf16_gpu(x, w, out, 1, 8, 0)
    assert lib.dmc_cuda_status() == 0


def test_product_package_never_imports_the_oracle():
    for p in (ROOT / "demonic_b200").rglob("*"):
        if p.suffix in (".py", ".cu", ".cuh", ".h"):
            text = p.read_text()
            assert not re.search(r"import\s+oracle|from\s+oracle|dmc_oracle|oracle/|orc_", text), \
                f"{p} reaches for the CPU oracle"
