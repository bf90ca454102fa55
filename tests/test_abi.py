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


def test_struct_sizes_match_header():
    """ctypes mirrors of the parameter structs have the C layout (checked by
    compiling a tiny C program against the header)."""
    import subprocess, tempfile, sys
    from dsv4_attn_b200 import _lib
    src = r'''
#include <stdio.h>
#include <stddef.h>
#include "dsv4_attn.h"
int main(void) {
  printf("%zu %zu %zu %zu %zu %zu\n", sizeof(Dsv4CsaSparseDecodeParams), offsetof(Dsv4CsaSparseDecodeParams, status),
         sizeof(Dsv4HcaDenseDecodeParams), offsetof(Dsv4HcaDenseDecodeParams, status),
         sizeof(Dsv4CombineParams), offsetof(Dsv4CombineParams, stride_lse_n));
  return 0; }
'''
    with tempfile.TemporaryDirectory() as td:
        c = Path(td) / "s.c"
        c.write_text(src)
        exe = Path(td) / "s"
        subprocess.run(["gcc", "-I", str(ROOT / "include"), str(c), "-o", str(exe)], check=True)
        got = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    want = [ctypes.sizeof(_lib.CsaSparseDecodeParams), _lib.CsaSparseDecodeParams.status.offset,
            ctypes.sizeof(_lib.HcaDenseDecodeParams), _lib.HcaDenseDecodeParams.status.offset,
            ctypes.sizeof(_lib.CombineParams), _lib.CombineParams.stride_lse_n.offset]
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
