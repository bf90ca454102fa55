"""The C-ABI shared object builds, loads and exports every function that
include/dsv4_attn.h declares.  No compute calls: runs without a GPU."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include" / "dsv4_attn.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"^\s*(?:int64_t|int|void)\s+(\w+)\s*\(", text, flags=re.M)))


def test_header_declares_expected_surface():
    names = declared_functions()
    for must in ("hca_decode_fwd", "dsv4_csa_sparse_decode_fwd", "dsv4_hca_dense_decode_fwd",
                 "dsv4_attn_combine", "dsv4_attn_plan_splits", "dsv4_attn_workspace_bytes"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from dsv4_attn_b200 import build
    so = build.build(quiet=True)
    lib = ctypes.CDLL(str(so))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


STRUCTS = {
    # C struct name -> ctypes mirror
    "Dsv4CsaSparseDecodeParams": "CsaSparseDecodeParams",
    "Dsv4HcaDenseDecodeParams": "HcaDenseDecodeParams",
    "Dsv4CombineParams": "CombineParams",
    "Dsv4PlanParams": "PlanParams",
    "Dsv4CsaCompressReduceParams": "CsaCompressReduceParams",
    "Dsv4IndexerTopkParams": "IndexerTopkParams",
    "Dsv4RopeNormParams": "RopeNormParams",
    "Dsv4HcaPackedDecodeParams": "HcaPackedDecodeParams",
    "Dsv4CacheDest": "CacheDest",
    "Dsv4HcaCompressParams": "HcaCompressParams",
    "Dsv4KvQuantizeInsertParams": "KvQuantizeInsertParams",
}


def test_struct_layouts_match_header():
    """Every ctypes mirror of a parameter struct has the C layout: size and the offset of
    every field, printed by a tiny C program compiled against the header."""
    import subprocess, tempfile
    from dsv4_attn_b200 import _lib
    header = (ROOT / "include" / "dsv4_attn.h").read_text()
    declared = set(re.findall(r"typedef struct (Dsv4\w+)", header))
    assert declared == set(STRUCTS), f"structs without a layout check: {declared ^ set(STRUCTS)}"
    lines, want = [], []
    for cname, pyname in STRUCTS.items():
        mirror = getattr(_lib, pyname)
        lines.append(f'printf("%zu\\n", sizeof({cname}));')
        want.append(ctypes.sizeof(mirror))
        for fname, _ in mirror._fields_:
            lines.append(f'printf("%zu\\n", offsetof({cname}, {fname}));')
            want.append(getattr(mirror, fname).offset)
    src = '#include <stdio.h>\n#include <stddef.h>\n#include "dsv4_attn.h"\nint main(void) {\n' + "\n".join(lines) + "\nreturn 0; }\n"
    with tempfile.TemporaryDirectory() as td:
        c = Path(td) / "s.c"
        c.write_text(src)
        exe = Path(td) / "s"
        subprocess.run(["gcc", "-I", str(ROOT / "include"), str(c), "-o", str(exe)], check=True)
        got = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    assert got == want


def test_planner_is_host_only_and_sane():
    from dsv4_attn_b200 import _lib
    f = _lib.LIB.dsv4_attn_plan_splits
    assert f(64, 128, 910, 148) == 1          # 128 blocks already fill most of 148 SMs
    assert f(1, 128, 64, 148) == 1            # a single tile cannot be split
    s = f(1, 128, 25000, 148)
    assert 8 <= s <= 64
    assert f(0, 128, 100, 148) < 0
    off = ctypes.c_int64()
    n = _lib.LIB.dsv4_attn_workspace_bytes(256, 128, 8, ctypes.byref(off))
    assert off.value == 8 * 256 * 128 * 512 * 4 and n >= off.value + 8 * 256 * 128 * 4
    assert _lib.LIB.dsv4_attn_workspace_bytes(256, 128, 1, None) == 0
