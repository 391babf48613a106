"""ctypes binding of libweftmoe_b200.so (the C ABI declared in include/weftmoe_b200.h).

There is no fallback: if the shared library is missing or a symbol cannot be resolved the import
of the operator fails with instructions to build it.  The reference resolves its native module in
`weftmoe/jit.py:220-246` (`jit.load`); this is the equivalent step.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path

LIBRARY = Path(__file__).resolve().parent / "libweftmoe_b200.so"

WM_OK, WM_ERR_INVALID, WM_ERR_CUDA, WM_ERR_TIMEOUT, WM_ERR_ROUTE, WM_ERR_CAPACITY, WM_ERR_STATE = 0, 2, 3, 4, 5, 6, 7


class WmConfig(Structure):
    _fields_ = [(name, c_int32) for name in (
        "rank", "world", "experts", "top_k", "hidden", "intermediate", "max_tokens", "max_rows",
        "training", "reserved")]  # reserved = precision: 0 BF16, 1 FP8, 2 NVFP4


class WmSizes(Structure):
    _fields_ = [("arena_bytes", c_int64), ("scratch_bytes", c_int64), ("tape_bytes", c_int64),
                ("row_capacity", c_int32), ("ipc_handle_bytes", c_int32)]


class WmQuantWeights(Structure):
    _fields_ = [("w1", c_void_p), ("w1_sf", c_void_p), ("w2", c_void_p), ("w2_sf", c_void_p),
                ("x_scale", c_float), ("w1_scale", c_float), ("u_scale", c_float), ("w2_scale", c_float),
                ("dy_scale", c_float), ("dab_scale", c_float),
                ("source_q", c_void_p), ("source_scales", c_void_p),
                ("w1_scales", c_void_p), ("w2_scales", c_void_p), ("wgrad_f32", c_int32)]


class WmRouteOut(Structure):
    _fields_ = [(name, c_void_p) for name in (
        "sorted_slot", "sorted_expert", "local_offset", "dst_rank", "dst_row", "dst_prow",
        "expert_total", "expert_base", "expert_pbase", "padded_start", "tile_group", "num_tiles",
        "padded_rows", "dst_primary")]


# name -> (restype, argtypes); every entry is declared in include/weftmoe_b200.h
SIGNATURES = {
    "wm_last_error": (c_char_p, []),
    "wm_runtime_create": (c_int, [POINTER(WmConfig), POINTER(c_void_p)]),
    "wm_runtime_sizes": (c_int, [c_void_p, POINTER(WmSizes)]),
    "wm_runtime_export_handle": (c_int, [c_void_p, c_void_p, c_size_t]),
    "wm_runtime_import_peers": (c_int, [c_void_p, c_void_p, c_size_t]),
    "wm_runtime_retire_peers": (c_int, [c_void_p]),
    "wm_runtime_destroy": (c_int, [c_void_p]),
    "wm_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32,
                           c_void_p, c_void_p, c_void_p]),
    "wm_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_void_p,
                            c_void_p, c_void_p, c_void_p, c_void_p]),
    "wm_forward_quantized": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, POINTER(WmQuantWeights), c_int32,
                                     c_void_p, c_void_p, c_void_p]),
    "wm_backward_quantized": (c_int, [c_void_p, c_void_p, c_void_p, POINTER(WmQuantWeights), c_int32, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p]),
    "wm_fp8_pack_weight_scales": (c_int, [c_void_p, c_int32, c_int32, c_void_p, c_void_p]),
    "wm_status_poll": (c_int, [c_void_p, POINTER(c_int32), c_void_p]),
    "wm_launch_count": (ctypes.c_longlong, []),
    "wm_stage_count": (c_int, []),
    "wm_stage_name": (c_char_p, [c_int]),
    "wm_runtime_enable_timing": (c_int, [c_void_p, c_int]),
    "wm_runtime_read_timing": (c_int, [c_void_p, POINTER(ctypes.c_double), POINTER(ctypes.c_longlong), c_int]),
    "wm_route_plan": (c_int, [c_int32] * 8 + [c_void_p, c_void_p, POINTER(WmRouteOut), c_void_p]),
    "wm_fp8_quantize": (c_int, [c_void_p] + [c_int32] * 6 + [c_void_p, c_void_p, c_void_p]),
    "wm_fp8_quantize_weight": (c_int, [c_void_p] + [c_int32] * 4 + [c_void_p] * 5),
    "wm_fp8_transpose_weight": (c_int, [c_void_p, c_void_p] + [c_int32] * 3 + [c_void_p] * 3),
    "wm_fp8_gemm": (c_int, [c_void_p] * 5 + [c_int32] * 7 + [c_void_p]),
    "wm_nvfp4_quantize": (c_int, [c_void_p, c_int32, c_int32, c_float, c_void_p, c_void_p, c_int32, c_void_p]),
    "wm_nvfp4_gemm": (c_int, [c_void_p] * 5 + [c_int32] * 3 + [c_float, c_int32, c_void_p]),
    "wm_route_plan_noalloc": (c_int, [c_int32] * 8 + [c_void_p, c_void_p, POINTER(WmRouteOut), c_void_p]),
    "wm_stage_inputs": (c_int, [c_void_p, c_int64, c_void_p, c_int32, c_int64, c_void_p, c_int64] + [c_int32] * 5
                        + [c_void_p, c_void_p, c_void_p, c_void_p]),
    "wm_scatter_output": (c_int, [c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p]),
    "wm_debug_force_gemm_pairs": (None, [c_int]),
    "wm_debug_set_wait_budget": (c_int, [ctypes.c_longlong]),
    "wm_debug_wait_flag": (c_int, [c_void_p, c_void_p, c_int32, c_void_p]),
    "wm_debug_grouped_gemm": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      POINTER(c_int), c_int, c_int, c_int, c_void_p, c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it is absent (no CPU or eager fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIBRARY.is_file():
        raise RuntimeError(
            f"{LIBRARY} is missing: build it with `python -m weftmoe_b200.build` "
            "(nvcc, sm_100a). weftmoe_b200 has no fallback path.")
    lib = ctypes.CDLL(str(LIBRARY))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means a stale build
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    message = load().wm_last_error()
    return message.decode() if message else ""


def check(code: int) -> None:
    """Map a C status to the exception type the reference raises for the same condition
    (ValueError for contract violations, RuntimeError otherwise; weftmoe/runtime.py:245-275)."""
    if code == WM_OK:
        return
    message = last_error() or f"weftmoe_b200 status {code}"
    if code in (WM_ERR_INVALID, WM_ERR_CAPACITY, WM_ERR_ROUTE):
        raise ValueError(message)
    raise RuntimeError(message)


def ptr(tensor) -> c_void_p:
    return c_void_p(0 if tensor is None else tensor.data_ptr())
