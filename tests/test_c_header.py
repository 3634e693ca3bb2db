"""The C header of the kernel library against the table the Python package loads it with.

csrc/tinyllama_c_b200.h (and no_alloc.h, which it includes) declares every exported function; every
.cu file includes it, so the compiler has held the definitions to it.  Here the prototypes are parsed
and compared with ops._SIGNATURES: same names, same number of arguments, same kind of each argument
(pointer, int, float, long long) and of the result.  A wrong entry in that table would be a bad pointer
on the GPU."""
import ctypes
import os
import re

from tinyllama_c_b200 import ops

CSRC = os.path.join(os.path.dirname(os.path.abspath(ops.__file__)), "..", "csrc")


def _kind(decl: str) -> str:
    decl = decl.strip()
    if "*" in decl or re.search(r"\bcudaStream_t\b", decl):
        return "pointer"
    if re.search(r"\blong long\b", decl):
        return "long long"
    if re.search(r"\bfloat\b", decl):
        return "float"
    if re.search(r"\b(int|unsigned)\b", decl):
        return "int"
    if decl == "void":
        return "void"
    raise AssertionError(f"unknown C type in '{decl}'")


_CTYPES_KIND = {ctypes.c_void_p: "pointer", ctypes.c_char_p: "pointer", ctypes.c_int: "int", ctypes.c_float: "float",
                ctypes.c_longlong: "long long", None: "void"}


def parse_header():
    text = ""
    for name in ("tinyllama_c_b200.h", "no_alloc.h"):
        with open(os.path.join(CSRC, name)) as f:
            text += f.read() + "\n"
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    text = re.sub(r"^\s*#[^\n]*", " ", text, flags=re.M)
    protos = {}
    for m in re.finditer(r"(?:extern\s+\"C\"\s+)?([A-Za-z_][\w\s\*]*?)\b(tlc_\w+)\s*\(([^)]*)\)\s*;", text):
        result, name, args = m.group(1), m.group(2), m.group(3).strip()
        arg_kinds = [] if args in ("", "void") else [_kind(a) for a in args.split(",")]
        res = "pointer" if "*" in result else _kind(result)
        assert name not in protos, f"{name} is declared twice"
        protos[name] = (res, arg_kinds)
    return protos


def test_every_declared_function_is_loaded_with_matching_types():
    protos = parse_header()
    assert len(protos) >= 40
    assert sorted(protos) == sorted(ops._SIGNATURES), (
        f"only in the header: {sorted(set(protos) - set(ops._SIGNATURES))}; "
        f"only in the table: {sorted(set(ops._SIGNATURES) - set(protos))}")
    for name, (res, kinds) in protos.items():
        restype, argtypes = ops._SIGNATURES[name]
        assert _CTYPES_KIND[restype] == res, f"{name}: result {res} in the header, {restype} in the table"
        got = [_CTYPES_KIND[a] for a in argtypes]
        assert got == kinds, f"{name}: header {kinds}\n table {got}"


def test_every_definition_is_declared():
    """No .cu file exports a tlc_ function that the header does not declare."""
    protos = parse_header()
    for fn in sorted(os.listdir(CSRC)):
        if not fn.endswith(".cu"):
            continue
        src = open(os.path.join(CSRC, fn)).read()
        for m in re.finditer(r'^extern "C"[^\n(]*?\b(tlc_\w+)\s*\(', src, flags=re.M):
            assert m.group(1) in protos, f"{fn} exports {m.group(1)}, which the header does not declare"
