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


def test_route_plan_refuses_oversized_expert_shards_before_any_device_work():
    """The planning kernel keeps one shared-memory word per local expert (at most 512).  The stand-alone
    entry points must refuse a larger shard, and top_k > experts, from the host-side argument check:
    no CUDA call is made (this test runs without a GPU)."""
    lib = _lib.load()
    out = _lib.WmRouteOut()
    counts = (ctypes.c_int32 * 4096)()
    routes = (ctypes.c_int32 * 8)()
    for entry in (lib.wm_route_plan, lib.wm_route_plan_noalloc):
        rc = entry(1, 1, 0, 1024, 2, 4, 4, 1024 * 128, routes, counts, ctypes.byref(out), None)
        assert rc in (_lib.WM_ERR_INVALID, _lib.WM_ERR_CAPACITY), rc
        rc = entry(1, 1, 0, 4, 8, 1, 1, 1024, routes, counts, ctypes.byref(out), None)
        assert rc == _lib.WM_ERR_INVALID, rc
    rc = lib.wm_route_plan(1, 2, 0, 2048, 2, 4, 4, 1024 * 128, routes, counts, ctypes.byref(out), None)
    assert rc == _lib.WM_ERR_INVALID and "512" in _lib.last_error()


def test_wait_budget_setter_is_exported_and_restores_its_default():
    lib = _lib.load()
    assert lib.wm_debug_set_wait_budget(1000) == _lib.WM_OK
    assert lib.wm_debug_set_wait_budget(0) == _lib.WM_OK   # back to the default


def test_ctypes_structures_match_the_header_layout(tmp_path):
    """The Python mirrors of the header's structs have the C compiler's sizes and field offsets (gcc on the
    header itself: a field added on one side only would shift every pointer behind it)."""
    import ctypes
    import subprocess
    structs = {"wm_config": _lib.WmConfig, "wm_sizes": _lib.WmSizes, "wm_quant_weights": _lib.WmQuantWeights,
               "wm_route_out": _lib.WmRouteOut}
    header = ROOT / "include" / "weftmoe_b200.h"
    lines = ["#include <stdio.h>", "#include <stddef.h>", f'#include "{header}"', "int main(void) {"]
    for name, mirror in structs.items():
        lines.append(f'  printf("{name} %zu\\n", sizeof({name}));')
        for field, _ in mirror._fields_:
            lines.append(f'  printf("{name}.{field} %zu\\n", offsetof({name}, {field}));')
    lines += ["  return 0;", "}"]
    source = tmp_path / "layout.c"
    source.write_text("\n".join(lines))
    binary = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c11", "-o", str(binary), str(source)], check=True)
    found = dict(line.split() for line in subprocess.run([str(binary)], check=True, capture_output=True,
                                                         text=True).stdout.splitlines())
    for name, mirror in structs.items():
        assert int(found[name]) == ctypes.sizeof(mirror), name
        for field, _ in mirror._fields_:
            assert int(found[f"{name}.{field}"]) == getattr(mirror, field).offset, (name, field)
