"""ctypes binding of ``libflashrt_b200.so`` (the C-ABI CUDA library).

The prototypes are read from ``include/flashrt_b200.h`` so the header stays the
single statement of the ABI.  There is no fallback: if the shared object is
missing or a call returns a non-zero status, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflashrt_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "flashrt_b200.h")

_CTYPE = {
    "int": C.c_int,
    "long long": C.c_longlong,
    "float": C.c_float,
    "unsigned": C.c_uint,
    "unsigned long long": C.c_ulonglong,
}


class KernelLibraryMissing(RuntimeError):
    """The sm_100a CUDA library has not been built (run ``python -m flashrt_b200._build``)."""


class KernelError(RuntimeError):
    """A C-ABI entry point returned a non-zero status."""


def parse_header(path: str = HEADER_PATH) -> dict[str, list[str]]:
    """Return ``{function name: [argument C types]}`` for every ``int frt_b200_*(...)`` prototype."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos: dict[str, list[str]] = {}
    for m in re.finditer(r"\bint\s+(frt_b200_\w+)\s*\(([^)]*)\)\s*;", text):
        name, args = m.group(1), m.group(2).strip()
        types: list[str] = []
        if args and args != "void":
            for a in args.split(","):
                a = " ".join(a.split())
                if "*" in a:
                    types.append("ptr")
                else:
                    types.append(" ".join(a.split(" ")[:-1]).replace("const ", "").strip())
        protos[name] = types
    return protos


_lib = None
_protos: dict[str, list[str]] | None = None


def load() -> C.CDLL:
    global _lib, _protos
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise KernelLibraryMissing(
            f"{LIB_PATH} not found: build it with `python -m flashrt_b200._build` "
            "(needs nvcc; there is no CPU or PyTorch fallback for these kernels)")
    lib = C.CDLL(LIB_PATH)
    _protos = parse_header()
    for name, types in _protos.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:  # header and library out of step
            raise KernelLibraryMissing(f"{LIB_PATH} does not export {name}; rebuild it") from e
        fn.restype = C.c_int
        fn.argtypes = [C.c_void_p if t == "ptr" else _CTYPE[t] for t in types]
    _lib = lib
    return lib


def exported_names() -> list[str]:
    load()
    return sorted(_protos or {})


_ERRORS = {-1: "invalid argument", -2: "unsupported shape or feature", -3: "bounded device wait gave up",
           -4: "request larger than the library's built-in fixed-size scratch"}


def call(name: str, *args) -> int:
    """Call entry point ``name``; raise :class:`KernelError` on a non-zero status."""
    rc = getattr(load(), name)(*args)
    if rc != 0:
        why = _ERRORS.get(rc, f"CUDA error {-rc - 1000}" if rc <= -1000 else "error")
        raise KernelError(f"{name} failed: status {rc} ({why})")
    return rc


def call_status(name: str, *args) -> int:
    """Call an entry point whose return value is data or a status the caller inspects."""
    return getattr(load(), name)(*args)
