"""The C-ABI library builds, loads and exports every symbol the public header declares (no GPU needed)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "worldattention_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from worldattention_b200 import _lib
    handle = _lib.lib()
    names = _declared_functions()
    assert len(names) >= 15
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert handle.wa_abi_version() == 3


def test_struct_layouts_match_the_header():
    from worldattention_b200 import _lib
    assert ctypes.sizeof(_lib.Tensor4) == 40
    assert ctypes.sizeof(_lib.PageCopy) == 40
    assert ctypes.sizeof(_lib.HsaParams) == 14 * 4 + 2 * 8 + 6 * 40 + 9 * 8 + 8 + 6 * 8 + 8 + 2 * 4 + 8 + 3 * 8 + 2 * 4 + 8 * 8
    assert ctypes.sizeof(_lib.HsaParams) == _lib.lib().wa_hsa_params_size()       # what the compiler laid out
    assert _lib.HsaParams.tau_min.offset == 56 and _lib.HsaParams.q.offset == 72


def test_argument_errors_are_reported_without_a_device():
    from worldattention_b200 import _lib
    handle = _lib.lib()
    rc = handle.wa_route_scores(None, None, 1, 1, 1, 1, 1, None, None)
    assert rc == _lib.WA_ERR_ARG
    assert b"null" in handle.wa_last_error()
    params = _lib.HsaParams()
    assert handle.wa_hsa_workspace_bytes(ctypes.byref(params)) == 0
    assert handle.wa_hsa_forward(ctypes.byref(params), None, None) == _lib.WA_ERR_ARG
