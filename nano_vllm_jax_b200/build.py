"""In-tree nvcc build of the sm_100a kernel library.

`build()` compiles every `.cu` file under `csrc/` (one object each, in parallel) and links them into
`nano_vllm_jax_b200/libnvj_b200.so` (next to this file, so the built library
travels with a snapshot of the source tree) and is a no-op when the library is
newer than every source.  The pattern follows the reference's build-on-import of
its own CUDA FFI library (nanovllm_jax/kernels/cuda_fp32_ffi.py:121-178) with the
architecture fixed to sm_100a.
"""

from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_PATH = PKG_DIR / "libnvj_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]
OBJ_DIR = PKG_DIR / "build"


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > built for p in sources() + _headers())


def nvcc_path() -> str | None:
    return shutil.which("nvcc") or (
        "/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else None
    )


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if needed and return its path.

    Every `.cu` file becomes one object under `build/` (compiled in parallel, recompiled when the
    file or any header is newer than its object); the objects are then linked into the library.
    """
    if not force and not _stale():
        return LIB_PATH
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libnvj_b200.so")
    OBJ_DIR.mkdir(exist_ok=True)
    newest_header = max((p.stat().st_mtime for p in _headers()), default=0.0)

    def compile_one(src: Path):
        obj = OBJ_DIR / (src.stem + ".o")
        if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, newest_header):
            return obj, ""
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-c", "-o", str(obj), str(src)]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n" + proc.stdout + proc.stderr)
        return obj, proc.stderr

    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as pool:
        results = list(pool.map(compile_one, sources()))
    if verbose:
        for obj, log in results:
            if log:
                print(f"---- {obj.name}\n{log}")
    link = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "-o", str(LIB_PATH)]
    link += [str(obj) for obj, _ in results]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("link failed:\n" + proc.stdout + proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
