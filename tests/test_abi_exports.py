"""CPU: the C-ABI library loads and exports every entry point include/flamia_b200.h declares (no compute calls)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    src = open(os.path.join(ROOT, "include", "flamia_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\bint\s+(fl_\w+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    from flamia_blackwell_attention_b200 import _lib, build
    build.build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = declared()
    assert len(names) >= 9
    for n in names:
        assert hasattr(lib, n), n
    assert set(_lib.EXPORTS) == set(names)
    assert _lib.load().fl_abi_version() == _lib.ABI_VERSION == 8


def test_bad_arguments_are_refused_without_a_device():
    from flamia_blackwell_attention_b200 import _lib
    lib = _lib.load()
    a = _lib.QuantArgs()
    assert lib.fl_quant_blocks(ctypes.byref(a), None) == _lib.FL_ERR_BAD_ARG
    f = _lib.AttnArgs()
    assert lib.fl_fwd(ctypes.byref(f), None) == _lib.FL_ERR_BAD_ARG
