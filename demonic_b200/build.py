"""Builds libdmc_cuda.so in-tree for sm_100a with nvcc (no GPU needed).

Every ``csrc/*.cu`` is compiled to an object of its own (in parallel) and the objects are linked
into one shared library; an object is rebuilt only when its source, a header or the flags changed.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libdmc_cuda.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [PKG.parent / "include" / "dmc_cuda.h"]


def _stamp() -> str:
    """Digest of everything every object depends on besides its own source."""
    h = hashlib.sha256(" ".join(FLAGS).encode())
    for p in headers():
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    return any(p.stat().st_mtime > t for p in sources() + headers())


def _compile(src: Path, stamp: str, verbose: bool) -> tuple[Path, str]:
    obj = OBJ / (src.stem + ".o")
    tag = OBJ / (src.stem + ".tag")
    want = stamp + ":" + hashlib.sha256(src.read_bytes()).hexdigest()[:16]
    if obj.exists() and tag.exists() and tag.read_text() == want:
        return obj, ""
    cmd = [NVCC, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", "-o", str(obj), str(src)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{proc.stdout}{proc.stderr}")
    tag.write_text(want)
    return obj, proc.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    OBJ.mkdir(exist_ok=True)
    if force:
        for p in OBJ.glob("*.tag"):
            p.unlink()
    stamp = _stamp()
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        results = list(pool.map(lambda s: _compile(s, stamp, verbose), sources()))
    if verbose:
        sys.stderr.write("".join(log for _, log in results))
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", str(LIB),
           *[str(o) for o, _ in results], "-ldl"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed linking libdmc_cuda.so:\n{proc.stdout}{proc.stderr}")
    return LIB


if __name__ == "__main__":
    build(force="-f" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
