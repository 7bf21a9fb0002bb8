"""The reference-side integration files, as far as they can be checked without cargo or a GPU: the
Rust glue declares every builtin the library exports under the reference's names, and the number
comparison of the program-level differential does what it says."""
import importlib.util
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_rust_glue_declares_the_reference_builtins_with_their_arity():
    src = (ROOT / "integration" / "rust" / "gpu_cuda.rs").read_text()
    header = (ROOT / "include" / "dmc_cuda.h").read_text()
    for name, arity in (("dmc_matmul_bf16_gpu", 6), ("dmc_matmul_bf16_gpu_batched", 9),
                        ("dmc_matmul_bf16_gpu_batched_deferred", 9), ("dmc_matmul_bf16_gpu_flush", 0)):
        m = re.search(r"pub extern \"C\" fn " + name + r"\(([^)]*)\)", src, re.S)
        assert m, f"{name}: no exported wrapper"
        params = [p for p in m.group(1).replace("\n", " ").split(",") if p.strip()]
        assert len(params) == arity and all(p.strip().endswith("i64") for p in params), name
        assert re.search(r"\b" + name + r"\(", header), f"{name}: not in the C header"
    patch = (ROOT / "integration" / "rust" / "dmc_cuda_flag.patch").read_text()
    for needle in ('"--cuda"', "cuda-unavailable", "gpu_allowed_here", "cuda_matmul_selected", "jit_cuda_defaults_off"):
        assert needle in patch, needle


def test_program_differential_compares_numbers_not_bytes():
    spec = importlib.util.spec_from_file_location("diff_backends_cuda", ROOT / "integration" / "tools" / "diff_backends_cuda.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.compare_numbers("sum = 1.00000 [2.5, 3.0]", "sum = 1.00001 [2.5, 3.0]") is None
    assert "numbers differ" in mod.compare_numbers("sum = 1.0", "sum = 1.1")
    assert "text" in mod.compare_numbers("sum = 1.0", "total = 1.0")
