"""The C-ABI shared library: it loads, exports every symbol include/fdma.h declares, and rejects bad
arguments with status codes before touching a device (no GPU needed for any of this)."""
import ctypes
import os
import re

import pytest

from flash_sparse_attn import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "fdma.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fdma_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_list_the_same_symbols():
    assert _declared_functions() == sorted(_lib.EXPORTED_SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    for name in _declared_functions():
        assert hasattr(lib, name), name
    assert lib.fdma_version() == 10100


def test_strerror_covers_every_status():
    lib = _lib.load()
    for code in (0, -1, -2, -3, -4, -5, -6, -7, 1, 700, -99):
        msg = lib.fdma_strerror(code)
        assert msg is not None and len(msg) > 0


def test_null_and_invalid_arguments_are_rejected_without_a_device():
    lib = _lib.load()
    assert lib.fdma_fwd(None, None) == -1
    assert lib.fdma_bwd(None, None) == -1
    assert lib.fdma_create_mask(None, None) == -1
    p = _lib.FwdParams()  # all-zero: null pointers
    assert lib.fdma_fwd(ctypes.byref(p), None) == -1
    assert lib.fdma_fwd_workspace_bytes(ctypes.byref(p)) == 0
    buf = ctypes.create_string_buffer(64)
    addr = ctypes.addressof(buf)
    for f in ("q", "k", "v", "out", "lse"):
        setattr(p, f, addr)
    p.b, p.seqlen_q, p.seqlen_k, p.h, p.h_k, p.d = 1, 1, 1, 3, 2, 64
    assert lib.fdma_fwd(ctypes.byref(p), None) == -1  # 3 query heads over 2 kv heads
    p.h = 2
    p.d = 260
    assert lib.fdma_fwd(ctypes.byref(p), None) == -2  # head dim > 256
    p.d = 60
    assert lib.fdma_fwd(ctypes.byref(p), None) == -2  # not a multiple of 8
    p.d = 64
    p.dtype = _lib.FDMA_FP32
    assert lib.fdma_fwd(ctypes.byref(p), None) == -2  # fp32 attention is not built
    m = _lib.MaskParams()
    m.bias, m.out = addr, addr
    m.kind = 7
    assert lib.fdma_create_mask(ctypes.byref(m), None) == -1


def test_struct_layout_matches_the_header(tmp_path):
    """Every ctypes mirror has the size, and every field the offset, that gcc gives the C struct of include/fdma.h
    (a small C program prints them; a change on either side shows up here)."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    pairs = (("fdma_fwd_params", _lib.FwdParams), ("fdma_bwd_params", _lib.BwdParams),
             ("fdma_mask_params", _lib.MaskParams), ("fdma_compact_params", _lib.CompactParams),
             ("fdma_rows_params", _lib.RowsParams), ("fdma_merge_params", _lib.MergeParams))
    lines = ["#include <stdio.h>", "#include <stddef.h>", '#include "fdma.h"', "int main(void) {"]
    for cname, cls in pairs:
        lines.append(f'  printf("{cname} %zu\\n", sizeof({cname}));')
        for fname, _ in cls._fields_:
            if fname == "f":
                continue
            lines.append(f'  printf("{cname}.{fname} %zu\\n", offsetof({cname}, {fname}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([gcc, "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    want = dict(ln.split() for ln in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for cname, cls in pairs:
        assert ctypes.sizeof(cls) == int(want[cname]), cname
        for fname, _ in cls._fields_:
            if fname == "f":
                continue
            assert getattr(cls, fname).offset == int(want[f"{cname}.{fname}"]), f"{cname}.{fname}"
    assert ctypes.sizeof(_lib.FwdParams) == 312  # fdma_bwd_params embeds it first: growing it moves every later field
