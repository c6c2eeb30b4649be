"""ctypes binding of the in-tree native libraries.

``kernels()`` returns the sm_100a kernel library, ``host()`` the C++ host-runtime library.  Both are
built by ``litevllm_b200._C.build`` and live next to it.  On a machine with a GPU a missing kernel
library is an error (there is no silent eager fallback for CUDA tensors).
"""
from __future__ import annotations

import ctypes
import re
from functools import lru_cache
from pathlib import Path

_C_DIR = Path(__file__).resolve().parent.parent / "_C"

_CODES = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_long, "f": ctypes.c_float,
          "d": ctypes.c_double, "u": ctypes.c_uint64}

_CSRC = Path(__file__).resolve().parent.parent.parent / "csrc"
_PROTO = re.compile(r'extern "C" (int|void|long|float|double|const char\*|void\*|uint64_t) (\w+)\((.*?)\)\s*\{', re.S)
_RET = {"int": ctypes.c_int, "void": None, "long": ctypes.c_long, "float": ctypes.c_float,
        "double": ctypes.c_double, "const char*": ctypes.c_char_p, "void*": ctypes.c_void_p,
        "uint64_t": ctypes.c_uint64}


def _arg_code(arg: str) -> str:
    arg = arg.strip()
    if "*" in arg:
        return "p"
    for prefix, code in (("long", "l"), ("int64_t", "l"), ("uint64_t", "u"), ("size_t", "u"),
                         ("float", "f"), ("double", "d"), ("int", "i"), ("unsigned", "i"),
                         ("uint32_t", "i"), ("bool", "i")):
        if arg.startswith(prefix):
            return code
    raise ValueError(f"unsupported C argument type: {arg!r}")


@lru_cache(maxsize=None)
def _signatures(kind: str) -> dict:
    """Parse the ``extern "C"`` prototypes of the native sources so the ctypes argument types
    can never drift from the C side."""
    pattern = "*.cu" if kind == "kernels" else "*.cpp"
    root = _CSRC if kind == "kernels" else _CSRC / "host"
    sigs = {}
    for f in sorted(root.rglob(pattern)):
        for m in _PROTO.finditer(f.read_text()):
            args = [a for a in m.group(3).replace("\n", " ").split(",") if a.strip() and a.strip() != "void"]
            sigs[m.group(2)] = ("".join(_arg_code(a) for a in args), _RET[m.group(1)])
    return sigs


class NativeLibraryMissing(RuntimeError):
    pass


def _declare(lib, sigs):
    for name, (codes, ret) in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.argtypes = [_CODES[c] for c in codes]
        fn.restype = ret
    return lib


def declare(lib, name: str, codes: str, restype=ctypes.c_int):
    fn = getattr(lib, name)
    fn.argtypes = [_CODES[c] for c in codes]
    fn.restype = restype
    return fn


@lru_cache(maxsize=None)
def kernels():
    path = _C_DIR / "libfi_kernels.so"
    if not path.exists():
        raise NativeLibraryMissing(
            f"{path} not found: run `python -m litevllm_b200._C.build` (or __graft_entry__.build())")
    lib = ctypes.CDLL(str(path))
    return _declare(lib, _signatures("kernels"))


@lru_cache(maxsize=None)
def host():
    path = _C_DIR / "libfi_host.so"
    if not path.exists():
        raise NativeLibraryMissing(f"{path} not found: run `python -m litevllm_b200._C.build`")
    return _declare(ctypes.CDLL(str(path)), _signatures("host"))


def have_kernels() -> bool:
    return (_C_DIR / "libfi_kernels.so").exists()


def have_host() -> bool:
    return (_C_DIR / "libfi_host.so").exists()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"native call {what} failed with code {rc}")
