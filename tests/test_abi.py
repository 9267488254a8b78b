"""CPU checks of the drop-in boundary: the shared library loads, exports every symbol
include/kq.h declares (and nothing is declared that the Python binding does not
bind), and refuses to work without a GPU instead of falling back."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "kq.h")).read()
    return sorted(set(re.findall(r"KQ_API\s+[\w\s\*]+?\b(kq_\w+)\s*\(", text)))


def test_header_declares_the_entry_points():
    names = declared_symbols()
    for required in ("kq_init", "kq_weight_upload", "kq_weight_dequant", "kq_linear", "kq_linear_multi",
                     "kq_linear_host", "kq_graph_begin", "kq_sync", "kq_last_error"):
        assert required in names


def test_library_exports_every_declared_symbol():
    from karume_b200 import _lib
    exported = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True,
                              check=True).stdout
    exported = set(re.findall(r"\bT\s+(kq_\w+)", exported))
    declared = set(declared_symbols())
    assert declared <= exported, f"declared but not exported: {sorted(declared - exported)}"
    assert exported <= declared, f"exported but not declared: {sorted(exported - declared)}"
    assert set(_lib.SYMBOLS) == declared


def test_no_torch_types_in_the_abi():
    text = open(os.path.join(ROOT, "include", "kq.h")).read()
    assert "torch" not in text and "at::" not in text and "#include <cuda" not in text


def test_version_string():
    from karume_b200 import lib
    assert lib.kq_version().decode().endswith("sm_100a")


def test_product_path_never_touches_the_oracle():
    pkg = os.path.join(ROOT, "karume_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(base, f)).read()
                assert "import oracle" not in text and "kq_oracle" not in text and "kqo_" not in text, f


def test_without_a_gpu_the_library_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import karume_b200 as kb
    with pytest.raises(kb.KqError):
        kb.acquire_gpu()
    import ctypes
    ctx = ctypes.c_void_p()
    rc = kb.lib.kq_init(0, 0, ctypes.byref(ctx))
    assert rc != 0 and ctx.value is None
    assert kb.lib.kq_last_error(None)


def test_the_deno_binding_table_lists_every_export():
    """INTEGRATION.md shows the Deno.dlopen symbol table a karume maintainer would paste: it has
    to name every entry point of the header."""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    table = set(re.findall(r"^\s*(kq_\w+):\s*\{\s*parameters", text, flags=re.M))
    declared = set(declared_symbols())
    assert declared <= table, f"missing from the dlopen table: {sorted(declared - table)}"
    assert table <= declared, f"in the table but not in the header: {sorted(table - declared)}"
