"""Argument types of the native libraries, read from ``include/kestrel.h``.

The header is the one declaration of every exported function: the C and CUDA sources include
it (a definition that differs does not compile) and the ctypes bindings are made from it here,
so there is no hand-typed table that could drift.  The header keeps to one declaration per
statement in a small set of plain types, which is all this reader understands.
"""
from __future__ import annotations

import ctypes
import os
import re
from typing import Dict, List, Tuple

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "kestrel.h")

_BASE = {"void": None, "int": ctypes.c_int, "float": ctypes.c_float, "long long": ctypes.c_longlong,
         "char": ctypes.c_char, "kestrel_stream_t": ctypes.c_void_p}

_DECL = re.compile(r"KESTREL_API\s+([^;()]+?)\s*\b(\w+)\s*\(([^;]*?)\)\s*;", re.S)
_DEFINE = re.compile(r"^#define\s+(\w+)\s+(-?\d+)\s*(?:/\*.*)?$", re.M)


def _ctype(text: str, what: str):
    """ctypes type of a C type written as in the header; every pointer is an address."""
    t = " ".join(text.replace("*", " * ").split())
    t = t.replace("const ", "").strip()
    if t.endswith("*"):
        if t == "char *":
            return ctypes.c_char_p
        return ctypes.c_void_p
    if t not in _BASE:
        raise ValueError(f"kestrel.h: type '{text}' of {what} is not one the bindings know")
    return _BASE[t]


def parse(path: str = HEADER) -> Tuple[Dict[str, Tuple[object, List[object], List[str]]], Dict[str, int]]:
    """(functions, constants): name -> (result type, argument types, argument names); #define name -> int."""
    with open(path) as f:
        src = f.read()
    src_nc = re.sub(r"/\*.*?\*/", " ", src, flags=re.S)
    funcs: Dict[str, Tuple[object, List[object], List[str]]] = {}
    for m in _DECL.finditer(src_nc):
        ret, name, params = m.group(1), m.group(2), m.group(3).strip()
        args, names = [], []
        if params and params != "void":
            for p in params.split(","):
                p = p.strip()
                pm = re.match(r"(.*?)(\w+)$", p, re.S)
                if not pm or not pm.group(1).strip():
                    raise ValueError(f"kestrel.h: parameter '{p}' of {name} needs a type and a name")
                args.append(_ctype(pm.group(1), f"{name}({pm.group(2)})"))
                names.append(pm.group(2))
        funcs[name] = (_ctype(ret, name), args, names)
    consts = {m.group(1): int(m.group(2)) for m in _DEFINE.finditer(src)}
    return funcs, consts


_parsed = None


def declarations():
    global _parsed
    if _parsed is None:
        _parsed = parse()
    return _parsed


def constants() -> Dict[str, int]:
    return declarations()[1]


def declare(lib: ctypes.CDLL, prefixes: Tuple[str, ...]) -> List[str]:
    """Sets restype and argtypes of every function of the header whose name starts with one of
    ``prefixes``; a function the library does not export is an error.  Returns the names."""
    funcs, _ = declarations()
    done = []
    for name, (res, args, _names) in funcs.items():
        if not name.startswith(prefixes):
            continue
        try:
            fn = getattr(lib, name)
        except AttributeError:
            raise RuntimeError(f"{getattr(lib, '_name', 'library')} does not export {name}, which kestrel.h declares") from None
        fn.restype = res
        fn.argtypes = args
        done.append(name)
    return done
