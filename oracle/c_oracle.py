"""TEST INFRASTRUCTURE ONLY — ctypes access to oracle/liboracle.so (route_oracle.c, quant_oracle.c)
and, when it was built, to the reference's own host planner oracle/_ref/libref_route.so.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_lib = None


def build():
    """Compile the C restatement (gcc) if it is missing or stale."""
    so = HERE / "liboracle.so"
    sources = [HERE / "route_oracle.c", HERE / "quant_oracle.c"]
    if not so.is_file() or any(s.stat().st_mtime_ns > so.stat().st_mtime_ns for s in sources):
        subprocess.run(["make", "-C", str(HERE)], check=True, capture_output=True)
    return so


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        _lib.wm_oracle_owner_tiles.restype = ctypes.c_int
        _lib.wm_oracle_e4m3.restype = ctypes.c_uint8
        _lib.wm_oracle_e4m3.argtypes = [ctypes.c_float]
        _lib.wm_oracle_fp8_block_scale.restype = ctypes.c_float
        _lib.wm_oracle_fp8_block_scale.argtypes = [ctypes.c_float, ctypes.c_int]
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def route_plan(world: int, experts: int, top_k: int, routes_per_rank: list[np.ndarray]):
    """Full plan for every rank.  routes_per_rank[r]: int32 [T_r, K].  Returns a list of dicts."""
    L = lib()
    e_local = experts // world
    locals_ = []
    cm = np.zeros((world, experts), np.int32)
    for r, routes in enumerate(routes_per_rank):
        routes = np.ascontiguousarray(routes, np.int32).reshape(-1, top_k)
        t = routes.shape[0]
        ss, se, lo = (np.zeros((t, top_k), np.int32) for _ in range(3))
        cnt = np.zeros(experts, np.int32)
        L.wm_oracle_local_plan(experts, top_k, ctypes.c_int64(t), _p(routes), _p(ss), _p(se), _p(lo), _p(cnt))
        cm[r] = cnt
        locals_.append((routes, ss, se, lo))
    total, base, pbase = (np.zeros(experts, np.int32) for _ in range(3))
    padded_rows = np.zeros(world, np.int32)
    L.wm_oracle_global_plan(world, experts, _p(cm), _p(total), _p(base), _p(pbase), _p(padded_rows))
    out = []
    for r, (routes, ss, se, lo) in enumerate(locals_):
        t = routes.shape[0]
        drank, drow, dprow = (np.zeros((t, top_k), np.int32) for _ in range(3))
        L.wm_oracle_route_rows(world, experts, top_k, r, ctypes.c_int64(t), _p(routes), _p(lo), _p(cm),
                               _p(base), _p(pbase), _p(drank), _p(drow), _p(dprow))
        dprimary = np.zeros((t, top_k), np.int32)
        L.wm_oracle_route_primary(experts, top_k, ctypes.c_int64(t), _p(routes), _p(drank), _p(dprow), _p(dprimary))
        pstart = np.zeros(e_local + 1, np.int32)
        tiles = np.zeros(max(1, int(padded_rows[r]) // 128), np.int32)
        n_tiles = L.wm_oracle_owner_tiles(world, experts, r, _p(total), _p(pstart), _p(tiles))
        out.append(dict(sorted_slot=ss, sorted_expert=se, local_offset=lo, count_matrix=cm.copy(),
                        dst_rank=drank, dst_row=drow, dst_prow=dprow, dst_primary=dprimary,
                        expert_total=total.copy(),
                        expert_base=base.copy(), expert_pbase=pbase.copy(), padded_start=pstart,
                        tile_group=tiles[:n_tiles].copy(), num_tiles=n_tiles,
                        padded_rows=int(padded_rows[r])))
    return out


def fp8_quantize(x: np.ndarray, block_rows: int, transpose: bool):
    """x: float32 [..., rows, cols].  Returns (q uint8 [..., m, k_padded], scales float32)."""
    x = np.ascontiguousarray(x, np.float32)
    rows, cols = x.shape[-2:]
    batch = int(np.prod(x.shape[:-2])) if x.ndim > 2 else 1
    m, k = (cols, rows) if transpose else (rows, cols)
    kb = (k + 127) // 128
    mb = (m + block_rows - 1) // block_rows
    q = np.zeros((batch, m, kb * 128), np.uint8)
    s = np.zeros((batch, mb, kb), np.float32)
    lib().wm_oracle_fp8_quantize(_p(x), batch, rows, cols, block_rows, int(transpose), _p(q), _p(s))
    lead = x.shape[:-2]
    return q.reshape(*lead, m, kb * 128), s.reshape(*lead, mb, kb)


def nvfp4_quantize(x: np.ndarray, layer_scale: float):
    """x: float32 [rows, cols].  Returns (packed uint8 [rows, cols/2], sf uint8 [rows, cols/16],
    rounded float32 [rows, cols])."""
    x = np.ascontiguousarray(x, np.float32)
    rows, cols = x.shape
    packed = np.zeros((rows, cols // 2), np.uint8)
    sf = np.zeros((rows, cols // 16), np.uint8)
    rounded = np.zeros((rows, cols), np.float32)
    lib().wm_oracle_nvfp4_quantize(_p(x), rows, cols, ctypes.c_double(layer_scale), _p(packed), _p(sf),
                                   _p(rounded))
    return packed, sf, rounded


def reference_route_lib():
    """The reference's own host planner, if oracle/_ref was built in this checkout (else None)."""
    so = HERE / "_ref" / "libref_route.so"
    if not so.is_file():
        return None
    ref = ctypes.CDLL(str(so))
    ref.ref_route_error.restype = ctypes.c_char_p
    return ref


def reference_route_plan(ref, world, experts, top_k, routes_per_rank, rank):
    tokens = np.asarray([len(r) for r in routes_per_rank], np.uint64)
    flat = np.concatenate([np.asarray(r, np.int32).reshape(-1) for r in routes_per_rank]).astype(np.int32) \
        if sum(len(r) for r in routes_per_rank) else np.zeros(1, np.int32)
    n = int(tokens[rank]) * top_k
    e_local = experts // world
    cm = np.zeros(world * experts, np.uint64)
    lo, row = np.zeros(max(n, 1), np.uint64), np.zeros(max(n, 1), np.uint64)
    drank, order = np.zeros(max(n, 1), np.uint32), np.zeros(max(n, 1), np.uint32)
    cnt, pre = np.zeros(e_local, np.uint64), np.zeros(e_local, np.uint64)
    rc = ref.ref_route_plan(world, experts, top_k, 128, _p(tokens), _p(flat), rank, _p(cm), _p(lo), _p(row),
                            _p(drank), _p(order), _p(cnt), _p(pre))
    if rc:
        raise RuntimeError(ref.ref_route_error().decode())
    return dict(count_matrix=cm.reshape(world, experts), local_offset=lo[:n], route_dst_row=row[:n],
                route_dst_rank=drank[:n], combine_order=order[:n], expert_row_count=cnt,
                expert_row_prefix=pre)
