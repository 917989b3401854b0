"""The C-ABI library loads without a GPU and exports every symbol include/coresets_b200.h declares."""
import ctypes
import re
from pathlib import Path

from coresets_b200 import _native, build

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "coresets_b200.h").read_text()
    return sorted(set(re.findall(r"CS_API\s+[\w\s\*]+?\b(cs_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(_native.EXPORTS)


def test_library_exports_every_declared_symbol():
    build.build()
    lib = ctypes.CDLL(str(build.LIB))
    for name in declared_symbols():
        assert hasattr(lib, name), name
    lib.cs_version.restype = ctypes.c_int
    assert lib.cs_version() == _native.CS_ABI_VERSION
    lib.cs_error_string.restype = ctypes.c_char_p
    for code in range(0, -7, -1):
        assert lib.cs_error_string(code)


def test_struct_layouts_match_the_header():
    assert ctypes.sizeof(_native.CtlView) == 256
    assert ctypes.sizeof(_native.CsState) == 128 + 8 + 64 + 8  # + rank/xchg, 8 peer windows, timeout
    assert _native.CsState.D.offset == 48 and _native.CsState.world_size.offset == 52
    assert _native.CtlView.live_rows.offset == 40 and _native.CtlView.last_idx.offset == 52
