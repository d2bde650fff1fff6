"""Builds and loads the native library (``bux_b200/_ext/libbux_b200.so``).

The library is built in-tree with plain ``nvcc`` / ``g++`` commands for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``); nvcc cross-compiles without a GPU.
`load()` loads a library whose recorded source hash matches the sources, and rebuilds
otherwise. On a machine with a GPU the ops refuse to run without the library.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
EXT_DIR = Path(__file__).resolve().parent.parent / "_ext"
LIB = EXT_DIR / "libbux_b200.so"
STAMP = EXT_DIR / "libbux_b200.hash"
CUDA_SOURCES = ("gemm_sm100.cu", "elementwise.cu", "attention_sm100.cu", "attention_bwd_sm100.cu",
                "comm_sm100.cu", "no_alloc.cu", "scan_sm100.cu", "conv_sm100.cu")
CPP_SOURCES = ("bindings.cpp",)
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-diag-suppress", "177"]
_lock = threading.Lock()
_loaded = False


def _existing(names) -> list:
    return [CSRC / n for n in names if (CSRC / n).exists()]


def source_hash() -> str:
    h = hashlib.sha256()
    for path in sorted(CSRC.glob("*")):
        if path.suffix in (".cu", ".cuh", ".h", ".cpp"):
            h.update(path.name.encode())
            h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _run(cmd: list) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"native build failed: {' '.join(map(str, cmd))}\n{proc.stdout}\n{proc.stderr}")


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA/C++ source for sm_100a and link the shared library."""
    with _lock:
        digest = source_hash()
        if not force and LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == digest:
            return LIB
        EXT_DIR.mkdir(exist_ok=True)
        # one builder per folder: other processes (ranks that start together) wait here and
        # then find the library fresh
        import fcntl

        with open(EXT_DIR / ".lock", "w") as turn:
            fcntl.flock(turn, fcntl.LOCK_EX)
            if not force and LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == digest:
                return LIB
            return _build_locked(digest, verbose)


def _build_locked(digest: str, verbose: bool) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    obj_dir = EXT_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    includes = [f"-I{p}" for p in ce.include_paths(device_type="cuda")] + [f"-I{CSRC}"]
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    jobs = []
    for src in _existing(CUDA_SOURCES):
        obj = obj_dir / (src.stem + ".o")
        jobs.append(([nvcc, *NVCC_FLAGS, f"-I{CSRC}", "-c", str(src), "-o", str(obj)], obj))
    for src in _existing(CPP_SOURCES):
        obj = obj_dir / (src.stem + ".o")
        jobs.append((["g++", "-O2", "-std=c++17", "-fPIC", abi, *includes, "-DTORCH_API_INCLUDE_EXTENSION_H",
                      "-c", str(src), "-o", str(obj)], obj))
    if verbose:
        print(f"[bux_b200] building {len(jobs)} objects for sm_100a", file=sys.stderr)
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
        list(pool.map(lambda j: _run(j[0]), jobs))
    lib_dirs = ce.library_paths(device_type="cuda")
    link = ["g++", "-shared", "-o", str(LIB), *[str(o) for _, o in jobs],
            *[f"-L{d}" for d in lib_dirs], *[f"-Wl,-rpath,{d}" for d in lib_dirs],
            "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda", "-lcudart"]
    _run(link)
    STAMP.write_text(digest)
    return LIB


def available() -> bool:
    return LIB.exists()


def load(required: bool = False) -> bool:
    """Load the library into this process (registers ``torch.ops.bux_b200``). Builds
    it first when it is missing or stale. Returns whether the ops are usable."""
    global _loaded
    if _loaded:
        return True
    import torch

    try:
        path = build()
        torch.ops.load_library(str(path))
        _loaded = True
    except Exception as err:  # noqa: BLE001
        if required:
            raise RuntimeError(
                "bux_b200's native sm_100a library could not be built or loaded; the CUDA "
                f"path refuses to fall back to eager PyTorch: {err}") from err
        return False
    return True


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
