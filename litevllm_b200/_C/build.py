"""In-tree native build: every ``csrc/**/*.cu`` is compiled for sm_100a with nvcc and linked into
``libfi_kernels.so``; every ``csrc/host/*.cpp`` is compiled with g++ into ``libfi_host.so``.

The libraries expose ``extern "C"`` entry points taking raw device pointers and a stream, so they
are bound with ``ctypes`` and never allocate device memory themselves.  Object files are cached by a
hash of the source, every header under ``csrc/`` and the flags, so repeated builds are cheap.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_ROOT = PKG_DIR.parent.parent
CSRC = REPO_ROOT / "csrc"
BUILD_DIR = PKG_DIR / "build"
KERNEL_LIB = PKG_DIR / "libfi_kernels.so"
HOST_LIB = PKG_DIR / "libfi_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--expt-extended-lambda", "-Xcompiler", "-fPIC",
    "-Xptxas", "-v", "--use_fast_math",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc() -> str:
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _stamp(src: Path, flags: list[str]) -> str:
    h = hashlib.sha1()
    h.update(src.read_bytes())
    # every header of the tree: a .cu file may include headers from any directory (the shared GEMM
    # epilogue, the collective descriptor, codebook tables), and a stale object would silently keep the
    # old struct layouts
    for inc in sorted(p for p in CSRC.rglob("*") if p.suffix in (".h", ".cuh", ".hpp", ".inc")):
        h.update(str(inc.relative_to(CSRC)).encode())
        h.update(inc.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _compile_one(src: Path, cmd_prefix: list[str], flags: list[str], verbose: bool) -> Path:
    rel = src.relative_to(CSRC)
    obj = BUILD_DIR / (str(rel).replace("/", "_") + "." + _stamp(src, flags) + ".o")
    if obj.exists():
        return obj
    for old in BUILD_DIR.glob(str(rel).replace("/", "_") + ".*.o"):
        old.unlink()
    cmd = cmd_prefix + flags + ["-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = BUILD_DIR / (str(rel).replace("/", "_") + ".log")
    log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(f"[build] {rel}")
    return obj


def build_all(verbose: bool = True, force: bool = False) -> dict[str, Path]:
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    if force:
        for f in BUILD_DIR.glob("*.o"):
            f.unlink()
    cu = sorted(p for p in CSRC.rglob("*.cu"))
    cpp = sorted(p for p in (CSRC / "host").glob("*.cpp"))
    with cf.ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as ex:
        cu_objs = list(ex.map(lambda s: _compile_one(s, [_nvcc()], NVCC_FLAGS, verbose), cu))
        cpp_objs = list(ex.map(lambda s: _compile_one(s, ["g++"], CXX_FLAGS, verbose), cpp))
    out = {}
    if cu_objs:
        newest = max(o.stat().st_mtime for o in cu_objs)
        if force or not KERNEL_LIB.exists() or KERNEL_LIB.stat().st_mtime < newest:
            cmd = [_nvcc(), "-shared", "-o", str(KERNEL_LIB)] + [str(o) for o in cu_objs] + \
                ["-gencode", "arch=compute_100a,code=sm_100a"]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"link failed: {res.stdout}\n{res.stderr}")
        out["kernels"] = KERNEL_LIB
    if cpp_objs:
        newest = max(o.stat().st_mtime for o in cpp_objs)
        if force or not HOST_LIB.exists() or HOST_LIB.stat().st_mtime < newest:
            cmd = ["g++", "-shared", "-o", str(HOST_LIB)] + [str(o) for o in cpp_objs] + ["-pthread", "-ldl"]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"link failed: {res.stdout}\n{res.stderr}")
        out["host"] = HOST_LIB
    return out


if __name__ == "__main__":
    libs = build_all(verbose=True, force="--force" in sys.argv)
    for k, v in libs.items():
        print(k, v)
