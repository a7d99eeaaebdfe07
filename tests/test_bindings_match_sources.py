"""The ctypes signatures in ``prism_b200.ops`` against the ``extern "C"`` declarations in the CUDA sources
(CPU, by reading the sources): same functions, same number of arguments, same kind of each argument.
A mismatch would not fail at load time; it would pass garbage to a kernel."""

import ctypes
import glob
import os
import re

from prism_b200 import ops

CSRC = os.path.join(os.path.dirname(os.path.abspath(ops.__file__)), "..", "csrc")


def _kind(decl: str):
    decl = decl.strip()
    if "*" in decl or decl.startswith("cudaStream_t"):
        return ctypes.c_void_p
    t = " ".join(decl.split()[:-1])
    t = t.replace("const ", "").strip()
    return {"int": ctypes.c_int, "float": ctypes.c_float, "long long": ctypes.c_longlong}[t]


def _declared():
    out = {}
    for path in sorted(glob.glob(os.path.join(CSRC, "*.cu"))):
        src = re.sub(r"//[^\n]*", "", open(path).read())
        for m in re.finditer(r"PRISM_EXPORT\s+int\s+(prism_\w+)\s*\(([^)]*)\)", src):
            args = [a for a in m.group(2).replace("\n", " ").split(",") if a.strip() and a.strip() != "void"]
            out[m.group(1)] = [_kind(a) for a in args]
    return out


def test_every_binding_matches_its_declaration():
    declared = _declared()
    bound = {n: getattr(ops._Sig, n) for n in dir(ops._Sig) if n.startswith("prism_")}
    assert bound, "no bindings found"
    missing = sorted(set(bound) - set(declared))
    assert not missing, f"bound but not declared in csrc: {missing}"
    for name, sig in bound.items():
        want = declared[name]
        assert len(sig) == len(want), (name, len(sig), len(want))
        bad = [i for i, (a, b) in enumerate(zip(sig, want)) if a is not b]
        assert not bad, (name, "argument kinds differ at", bad)
