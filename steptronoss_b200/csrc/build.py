"""Build the native library in-tree: every ``*.cu`` beside this file is compiled for sm_100a with
nvcc and linked into ``steptronoss_b200/_native/libstb200.so``.

    python -m steptronoss_b200.csrc.build [--force] [--verbose]

The kernels have no PyTorch dependency (raw pointers + stream in, status out), so the build is a
handful of nvcc invocations that cross-compile on a machine without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE.parent / "_native"
LIB = OUT_DIR / "libstb200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
              "--expt-relaxed-constexpr"]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def sources() -> list[Path]:
    return sorted(HERE.glob("*.cu"))


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for hdr in sorted(HERE.glob("*.cuh")) + sorted(HERE.glob("*.h")):
        h.update(hdr.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile(src: Path, force: bool, verbose: bool) -> tuple[Path, bool, str]:
    obj = OUT_DIR / (src.stem + ".o")
    stamp = OUT_DIR / (src.stem + ".sha")
    dig = _digest(src)
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj, False, ""
    cmd = [nvcc_path(), *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(HERE), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(dig)
    (OUT_DIR / (src.stem + ".ptxas.txt")).write_text(r.stderr)
    return obj, True, r.stderr if verbose else ""


def build(force: bool = False, verbose: bool = False) -> Path:
    OUT_DIR.mkdir(exist_ok=True)
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, force, verbose), srcs))
    objs = [r[0] for r in results]
    if verbose:
        for r in results:
            if r[2]:
                print(r[2])
    if any(r[1] for r in results) or not LIB.exists():
        cmd = [nvcc_path(), "-shared", *ARCH_FLAGS, "-o", str(LIB), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    build_expstore(force)
    return LIB


EXPSTORE_SRC = HERE / "expstore" / "expstore_server.cpp"
EXPSTORE_BIN = OUT_DIR / "stb_expstore"


def build_expstore(force: bool = False) -> Path:
    """The experiment store server (plain C++, no CUDA): ``_native/stb_expstore``."""
    OUT_DIR.mkdir(exist_ok=True)
    stamp = OUT_DIR / "stb_expstore.sha"
    dig = hashlib.sha256(EXPSTORE_SRC.read_bytes()).hexdigest()
    if not force and EXPSTORE_BIN.exists() and stamp.exists() and stamp.read_text() == dig:
        return EXPSTORE_BIN
    cxx = os.environ.get("CXX", "g++")
    r = subprocess.run([cxx, "-O2", "-std=c++17", "-o", str(EXPSTORE_BIN), str(EXPSTORE_SRC)],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building the experiment store failed:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(dig)
    return EXPSTORE_BIN


if __name__ == "__main__":
    lib = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(lib)
