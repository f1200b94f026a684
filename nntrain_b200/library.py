"""ctypes loader for libnntrain_grad_b200.so.

Signatures are read from include/nntrain_grad_abi.h, so the header is the
single source of truth for the boundary.  A missing library is an error (the
product has no CPU path); build it with `python -m nntrain_b200.build`.
"""
from __future__ import annotations

import ctypes
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_HERE, "libnntrain_grad_b200.so")
HEADER_PATH = os.path.join(_HERE, "..", "include", "nntrain_grad_abi.h")
HEADER_PATHS = (HEADER_PATH, os.path.join(_HERE, "..", "include", "nntrain_host_plan.h"))


class LibraryMissingError(ImportError):
    pass


class NativeCudaError(RuntimeError):
    """A native entry point returned a non-zero cudaError_t.

    Mirrors NativeCudaException (NNtrain.Core/Tensors/NativeCudaRuntime.cs:9-22)."""

    def __init__(self, operation: str, status: int):
        super().__init__(f"CUDA {operation} failed with status {status}")
        self.operation = operation
        self.status = status


class ErrorInfo(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_uint32), ("abi_version", ctypes.c_uint32),
                ("sequence", ctypes.c_uint64), ("status", ctypes.c_int32),
                ("device", ctypes.c_int32), ("operation", ctypes.c_uint32),
                ("reserved", ctypes.c_uint32)]


_SCALARS = {
    "int": ctypes.c_int, "float": ctypes.c_float, "double": ctypes.c_double,
    "long long": ctypes.c_longlong, "unsigned long long": ctypes.c_ulonglong,
    "size_t": ctypes.c_size_t, "uint32_t": ctypes.c_uint32, "uint64_t": ctypes.c_uint64,
    "int32_t": ctypes.c_int32, "nntrain_stream_t": ctypes.c_void_p,
    "nntrain_event_t": ctypes.c_void_p, "unsigned short": ctypes.c_ushort, "unsigned": ctypes.c_uint,
}


def _ctype(decl: str):
    decl = decl.strip()
    if decl in ("void", ""):
        return None
    if "*" in decl:
        return ctypes.c_void_p
    words = [w for w in decl.replace("const", " ").split()]
    # drop the parameter name (last word) when a type precedes it
    for take in (len(words) - 1, len(words)):
        name = " ".join(words[:take])
        if name in _SCALARS:
            return _SCALARS[name]
    raise ValueError(f"cannot map C declaration {decl!r}")


def declared_functions(header_path: str | None = None) -> dict[str, tuple]:
    """{name: (restype, [argtypes])} for every function the headers declare."""
    if header_path is None:
        merged = {}
        for path in HEADER_PATHS:
            merged.update(declared_functions(path))
        return merged
    text = open(header_path).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"^\s*#.*$", " ", text, flags=re.M)
    text = re.sub(r"typedef\s+struct\s+\w+\s*\{.*?\}\s*\w+\s*;", " ", text, flags=re.S)
    text = re.sub(r"typedef[^;]*;", " ", text)
    text = text.replace('extern "C" {', " ")
    out = {}
    for match in re.finditer(r"([\w\s\*]+?)\b(nntrain_\w+)\s*\(([^)]*)\)\s*;", text):
        restype, name, args = match.group(1), match.group(2), match.group(3)
        argtypes = [] if args.strip() in ("void", "") else [_ctype(a) for a in args.split(",")]
        out[name] = (_ctype(restype + " x") if restype.strip() != "void" else None, argtypes)
    return out


_lib = None


def load() -> ctypes.CDLL:
    """Loads the library once and attaches the header's signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIBRARY_PATH):
        raise LibraryMissingError(
            f"{LIBRARY_PATH} is missing: the CUDA library has not been built "
            "(python -m nntrain_b200.build).  There is no CPU fallback.")
    import torch  # noqa: F401  (loads the CUDA runtime and NCCL the process will share)
    lib = ctypes.CDLL(LIBRARY_PATH)
    for name, (restype, argtypes) in declared_functions().items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(operation: str, status: int) -> None:
    if status != 0:
        raise NativeCudaError(operation, status)


def last_error() -> ErrorInfo:
    info = ErrorInfo()
    check("last_error", load().nntrain_last_error(ctypes.addressof(info), ctypes.sizeof(info)))
    return info
