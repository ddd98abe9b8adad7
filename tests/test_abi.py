"""The C ABI library loads and exports every symbol that include/bitnet_b200.h declares
(no GPU needed, no compute calls)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not fn.endswith(".h"):
            continue
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"//[^\n]*", "", text)
        text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
        for m in re.finditer(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{}]*\)\s*;", text):
            names.append(m.group(1))
    return sorted(set(names))


def test_library_builds_and_exports_declared_symbols():
    from bitnet_b200 import build

    path = build.build()
    lib = ctypes.CDLL(path)
    declared = _declared_symbols()
    assert "bitlinear_int8xint2" in declared and "quantize_i2_s" in declared
    missing = [n for n in declared if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_binding_table_covers_header():
    from bitnet_b200 import _lib

    assert sorted(_lib.SIGNATURES) == [n for n in _declared_symbols() if n in _lib.SIGNATURES]
    assert set(_declared_symbols()) <= set(_lib.SIGNATURES), set(_declared_symbols()) - set(_lib.SIGNATURES)


def test_argument_checks_need_no_gpu():
    from bitnet_b200 import _lib

    L = _lib.lib
    assert L.bitnet_w2t_bytes(2560, 2560) == 2560 * 2560 // 4
    assert L.bitnet_w2t_bytes(20, 200) == 32 * 256 // 4
    assert L.bitnet_pack_ternary(None, None, 16, 128, None) == 1
    assert L.bitnet_last_status() == 1
    assert L.bitnet_status_string(1) == b"bad argument"
    L.bitlinear_int8xint2(None, None, None, None, None, 1, 16, 128, None)
    assert L.bitnet_last_status() == 1
