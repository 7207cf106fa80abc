"""The ctypes argument signatures in ``ops/native.py`` must match the ``extern "C"``
prototypes in ``ops/csrc`` (a mismatch corrupts arguments silently)."""

import glob
import os
import re

from prism_infer_b200.ops import native

TYPES = {"int": "i", "float": "f", "long long": "l", "unsigned long long": "u"}


def test_signatures_match_the_c_prototypes():
    root = os.path.join(os.path.dirname(native.__file__), "csrc")
    src = "".join(open(f).read() for f in sorted(glob.glob(os.path.join(root, "*.cu"))))
    seen = set()
    for m in re.finditer(r"PRISM_API int (\w+)\(([^)]*)\)", src):
        name, args = m.group(1), m.group(2)
        if name.startswith("prism_status") or name not in native._SIGNATURES:
            continue
        sig = ""
        for a in [x.strip() for x in args.split(",") if x.strip()]:
            sig += "p" if "*" in a else TYPES[" ".join(a.split()[:-1])]
        assert sig == native._SIGNATURES[name], f"{name}: C prototype {sig} vs binding {native._SIGNATURES[name]}"
        seen.add(name)
    missing = set(native._SIGNATURES) - seen - {"prism_gemm_clear_tensor_maps"}
    assert not missing, f"bindings without a prototype: {sorted(missing)}"


def test_no_cluster_qualified_bulk_loads_in_kernel_sources():
    """Operand loads are plain TMA tile copies; cluster-qualified bulk loads are not used."""
    root = os.path.join(os.path.dirname(native.__file__), "csrc")
    banned = "multi" + "cast"
    for f in glob.glob(os.path.join(root, "*")):
        assert banned not in open(f).read(), f
