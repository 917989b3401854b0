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


def test_decode_key_round_trip():
    """The Python decoder of the 64-bit arg-max key against the encoder of the test stand-in."""
    from tests.fake_native import make_key
    import numpy as np
    assert _native.decode_key(0) == (float("-inf"), -1)
    for h in (0.0, 1e-30, 3.25, 1e9, float("inf"), -1.0):
        for idx in (0, 1, 12345, 2**31 - 1):
            val, i = _native.decode_key(make_key(np.float32(h), idx))
            assert i == idx and np.float32(val) == np.float32(h)
    # order: larger value first, then the smaller index
    assert make_key(np.float32(2.0), 9) > make_key(np.float32(1.0), 3)
    assert make_key(np.float32(2.0), 3) > make_key(np.float32(2.0), 9)
    # a key read back as a signed 64-bit integer decodes the same
    k = make_key(np.float32(5.0), 77)
    assert _native.decode_key(k - (1 << 64)) == (5.0, 77)


def test_typed_wrapper_binds_every_entry_point():
    """`_native.Native()` loads the library, checks the ABI version and sets the argument types of
    every entry point it wraps (no GPU needed: nothing is called)."""
    n = _native.Native()
    assert n.lib.cs_version() == _native.CS_ABI_VERSION
    for name in _native.EXPORTS:
        assert hasattr(n.lib, name), name
