"""The reference's two external gates, extended to the CUDA path (integration/tools/): both run
against the built library on a GPU and must pass, and the oracle's meta-test must show that a wrong
reference is caught."""
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
TOOLS = Path(__file__).resolve().parent.parent / "integration" / "tools"


def run(script, *args):
    return subprocess.run([sys.executable, str(TOOLS / script), *args], capture_output=True, text=True, timeout=600)


def test_numpy_oracle_on_the_cuda_path():
    p = run("numpy_oracle_cuda.py", "--verbose", "--meta-test")
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "meta-test: ok" in p.stdout and "8/8 matmul cases match numpy" in p.stdout


def test_backend_differential_at_the_matmul_sites():
    p = run("diff_backends_cuda.py", "--verbose")
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "0 diverged" in p.stdout and "not-selected" in p.stdout
