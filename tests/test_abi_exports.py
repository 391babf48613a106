"""CPU: the C-ABI library builds, loads and exports every symbol include/weftmoe_b200.h declares.
No compute call is made (no GPU here)."""
import ctypes
import re
from pathlib import Path

from weftmoe_b200 import _lib, build

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "weftmoe_b200.h").read_text()
    return sorted(set(re.findall(r"WM_API\s+[\w\s\*]+?\b(wm_\w+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    for must in ("wm_runtime_create", "wm_forward", "wm_backward", "wm_runtime_export_handle",
                 "wm_runtime_import_peers", "wm_route_plan", "wm_status_poll", "wm_last_error"):
        assert must in names


def test_library_builds_and_exports_every_declared_symbol():
    so = build.build()
    lib = ctypes.CDLL(str(so))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared but not exported"


def test_ctypes_table_covers_the_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    _lib.load()


def test_contract_errors_without_a_gpu():
    lib = _lib.load()
    cfg = _lib.WmConfig(rank=0, world=3, experts=8, top_k=2, hidden=256, intermediate=128,
                        max_tokens=4, max_rows=8, training=0, reserved=0)
    handle = ctypes.c_void_p()
    assert lib.wm_runtime_create(ctypes.byref(cfg), ctypes.byref(handle)) == _lib.WM_ERR_INVALID
    assert "world" in _lib.last_error()
    cfg.world, cfg.hidden = 1, 100
    assert lib.wm_runtime_create(ctypes.byref(cfg), ctypes.byref(handle)) == _lib.WM_ERR_INVALID
