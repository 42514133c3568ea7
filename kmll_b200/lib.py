"""ctypes binding of libkmll_b200.so.

Prototypes are read from the public headers (include/*.h), so the Python side can never drift
from the C ABI.  There is no CPU fallback: importing works anywhere (the library only needs the
CUDA runtime it links statically), but every operator call needs a CUDA device and raises
KmllError otherwise.
"""
from __future__ import annotations

import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
LIB_PATH = os.path.join(_HERE, "libkmll_b200.so")
HEADERS = [os.path.join(_ROOT, "include", n) for n in ("kmll_b200.h", "kmll_b200_runtime.h")]


class KmllError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"kmll_b200 error {code}: {message}")
        self.code = code
        self.message = message


_SCALARS = {
    "int": C.c_int, "float": C.c_float, "size_t": C.c_size_t, "uint32_t": C.c_uint32, "uint64_t": C.c_uint64,
    "int32_t": C.c_int32, "int64_t": C.c_int64, "double": C.c_double, "kmll_stream_t": C.c_void_p,
    "kmll_decoder_t": C.c_void_p, "kmll_batch_t": C.c_void_p,
}


def _ctype(decl: str):
    decl = decl.strip()
    if "*" in decl or "[" in decl:
        return C.c_void_p
    decl = decl.replace("const ", "").strip()
    base = decl.rsplit(" ", 1)[0] if " " in decl else decl
    if base not in _SCALARS:
        raise ValueError(f"unsupported parameter type in header: {decl!r}")
    return _SCALARS[base]


def parse_prototypes(path: str) -> dict[str, tuple[object, list[object]]]:
    """{name: (restype, [argtypes])} for every `kmll_*` function declared in a header."""
    if not os.path.exists(path):
        return {}
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    text = re.sub(r"^\s*#.*$", " ", text, flags=re.M)
    protos = {}
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(kmll_\w+)\s*\(([^;{}]*?)\)\s*;", text, flags=re.S):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        if ret.startswith("typedef"):
            continue
        if "*" in ret:
            restype = C.c_char_p if "char" in ret else C.c_void_p
        elif ret == "void":
            restype = None
        else:
            restype = _SCALARS[ret.replace("const ", "").strip()]
        argtypes = [] if args in ("", "void") else [_ctype(a) for a in args.split(",")]
        protos[name] = (restype, argtypes)
    return protos


def declared_symbols() -> dict[str, tuple[object, list[object]]]:
    out = {}
    for h in HEADERS:
        out.update(parse_prototypes(h))
    return out


_lib = None


def load() -> C.CDLL:
    """Load the shared library (built in-tree by kmll_b200/build.py) and attach prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise KmllError(-100, f"{LIB_PATH} is missing: run `python -m kmll_b200.build` (no CPU fallback exists)")
    lib = C.CDLL(LIB_PATH)
    for name, (restype, argtypes) in declared_symbols().items():
        fn = getattr(lib, name)  # AttributeError here = header declares a symbol the library lacks
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != 0:
        msg = load().kmll_last_error()
        raise KmllError(rc, msg.decode() if msg else "")
