"""Helpers for the GPU parity tests: thin callers of the C ABI on torch CUDA tensors."""
import ctypes

import numpy as np
import torch

from weftmoe_b200 import _lib


def device_route_plan(world, experts, top_k, routes_per_rank, cap=None, row_capacity=None):
    """One GPU plays every rank in turn (phase 0 fills the count matrix, phase 1 the rest).
    Returns a list of dicts of numpy arrays shaped like oracle.c_oracle.route_plan's."""
    lib = _lib.load()
    dev = torch.device("cuda")
    e_local = experts // world
    cap = cap or max(1, max(len(r) for r in routes_per_rank))
    total_rows = sum(len(r) for r in routes_per_rank) * top_k
    row_capacity = row_capacity or ((total_rows + 127) // 128 * 128 + 128 * e_local)
    cm = torch.zeros(world * experts, dtype=torch.int32, device=dev)
    i32 = lambda *shape: torch.full(shape, -7, dtype=torch.int32, device=dev)
    outs = []
    for phase in (0, 1):
        outs = []
        for rank, routes in enumerate(routes_per_rank):
            r = torch.as_tensor(np.ascontiguousarray(routes, np.int32)).reshape(-1, top_k).to(dev)
            t = r.shape[0]
            bufs = dict(sorted_slot=i32(t, top_k), sorted_expert=i32(t, top_k), local_offset=i32(t, top_k),
                        dst_rank=i32(t, top_k), dst_row=i32(t, top_k), dst_prow=i32(t, top_k),
                        expert_total=i32(experts), expert_base=i32(experts), expert_pbase=i32(experts),
                        padded_start=i32(e_local + 1), tile_group=i32(row_capacity // 128 + 1),
                        num_tiles=i32(1), padded_rows=i32(1), dst_primary=i32(t, top_k))
            out = _lib.WmRouteOut(**{k: v.data_ptr() for k, v in bufs.items()})
            rc = lib.wm_route_plan(phase, world, rank, experts, top_k, t, cap, row_capacity,
                                   _lib.ptr(r) if t else None, _lib.ptr(cm), ctypes.byref(out), None)
            _lib.check(rc)
            outs.append(bufs)
    torch.cuda.synchronize()
    result = []
    for bufs in outs:
        d = {k: v.cpu().numpy() for k, v in bufs.items()}
        d["num_tiles"] = int(d["num_tiles"][0])
        d["padded_rows"] = int(d["padded_rows"][0])
        d["tile_group"] = d["tile_group"][: d["num_tiles"]]
        d["count_matrix"] = cm.cpu().numpy().reshape(world, experts)
        result.append(d)
    return result


def grouped_gemm(kind, a, b, out, rows_per_group, n, k_or_m, aux=None, prob=None):
    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device=a.device)
    arr = (ctypes.c_int * len(rows_per_group))(*rows_per_group)
    rc = lib.wm_debug_grouped_gemm(kind, _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(aux), _lib.ptr(prob),
                                   arr, len(rows_per_group), n, k_or_m, _lib.ptr(status), None)
    _lib.check(rc)
    assert status.item() == 0, f"device status {status.item()}"


def rel_l2(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()
