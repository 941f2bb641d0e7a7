"""The C-ABI library: loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    src = open(os.path.join(ROOT, "include", "faith_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(fb_[a-z0-9_]+)\s*\(", src)))


def test_library_builds_and_exports_header_symbols():
    from faith_b200 import build
    lib_path = build.build()
    lib = ctypes.CDLL(lib_path)
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), "symbol %s declared in include/faith_b200.h is not exported" % n


def test_ctypes_prototypes_cover_header():
    from faith_b200 import _lib
    assert set(declared_symbols()) == set(_lib.SIGNATURES)
    lib = _lib.load()
    assert lib.fb_version() >= 100
    assert lib.fb_status_string(0) == b"ok"


def test_argument_validation_without_gpu():
    """Bad arguments are rejected before any CUDA call is made."""
    from faith_b200 import _lib
    lib = _lib.load()
    assert lib.fb_relax_f32(0, None, None, None, None, None, None, None, None, 1, 4, 4, 1, 2, 0.1, 0, None, None) == 1
    assert lib.fb_concretize_f32(1, 1, 1, 1, 1, 1, 1, 4, 4, 1, 7, 0.1, 0, None) == 1  # unknown norm
    assert lib.fb_concretize_f32(1, 1, 1, 1, 1, 1, 1, 6, 4, 4, 2, 0.1, 0, None) == 2  # Di % words != 0


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch
    import faith_b200
    x = torch.zeros(1, 2, 4, 4)
    b = torch.zeros(1, 2, 4)
    with pytest.raises(faith_b200.FaithError):
        faith_b200.BoundsLite(2, 0.1, x, b, x, b).relu()


def declared_prototypes():
    """name -> list of parameter kinds ('p' pointer, 'i' int, 'l' 64-bit integer, 'f' float, 'd' double) read from the header."""
    src = open(os.path.join(ROOT, "include", "faith_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    src = re.sub(r"//[^\n]*", "", src)
    out = {}
    for name, args in re.findall(r"\b(fb_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", src):
        kinds = []
        for a in (s.strip() for s in args.split(",")):
            if a in ("", "void"):
                continue
            if "*" in a:
                kinds.append("p")
            elif re.search(r"\b(u?int64_t|size_t)\b", a):
                kinds.append("l")
            elif re.search(r"\bdouble\b", a):
                kinds.append("d")
            elif re.search(r"\bfloat\b", a):
                kinds.append("f")
            else:
                kinds.append("i")
        out[name] = kinds
    return out


def test_ctypes_prototypes_match_the_header_parameter_by_parameter():
    """Every ctypes signature has the header's parameter count and, per parameter, the header's kind of type; a
    mismatch would otherwise only show as a TypeError (or a shifted argument) on the first call on a GPU."""
    from faith_b200 import _lib

    def kind(t):
        if t in (ctypes.c_int, ctypes.c_uint):
            return "i"
        if t in (ctypes.c_int64, ctypes.c_uint64, ctypes.c_size_t):
            return "l"
        if t is ctypes.c_float:
            return "f"
        if t is ctypes.c_double:
            return "d"
        return "p"

    protos = declared_prototypes()
    for name, argtypes in _lib.SIGNATURES.items():
        assert [kind(t) for t in argtypes] == protos[name], name
