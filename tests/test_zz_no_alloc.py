"""GPU: wm_route_plan_noalloc, the route planner for callers that cannot allocate device memory
(a server whose own pool holds all free HBM, or a latency-critical path that cannot afford
cudaMalloc's device-wide synchronisation).  It keeps its temporaries in a fixed 1 MiB device array
inside the library, so this file checks, through the C ABI, that two calls in a row (which share
that array and see each other's leftovers) each give exactly the output of wm_route_plan and of the
CPU oracle (every field, the per-owner primary rows included), and that requests beyond the fixed size
are refused with a message.  Collected last on purpose."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import c_oracle
from weftmoe_b200 import _lib

pytestmark = pytest.mark.gpu

FIELDS = ("sorted_slot", "sorted_expert", "local_offset", "dst_rank", "dst_row", "dst_prow", "dst_primary",
          "expert_total", "expert_base", "expert_pbase", "padded_start", "tile_group", "num_tiles", "padded_rows")
# Fields the CPU oracle (oracle/route_oracle.c) also produces, compared bit for bit below.
ORACLE_FIELDS = ("sorted_slot", "sorted_expert", "local_offset", "dst_rank", "dst_row", "dst_prow", "dst_primary",
                 "expert_total", "expert_base", "expert_pbase", "padded_start", "tile_group")


def plan(entry, world, experts, top_k, routes_per_rank, row_capacity):
    """Both phases for every rank on one GPU through `entry`; returns per-rank dicts of numpy arrays."""
    lib = _lib.load()
    fn = getattr(lib, entry)
    dev = torch.device("cuda")
    e_local = experts // world
    cap = max(1, max(len(r) for r in routes_per_rank))
    cm = torch.zeros(world * experts, dtype=torch.int32, device=dev)
    result = []
    for phase in (0, 1):
        result = []
        for rank, routes in enumerate(routes_per_rank):
            r = torch.as_tensor(np.ascontiguousarray(routes, np.int32)).reshape(-1, top_k).to(dev)
            t = r.shape[0]
            i32 = lambda *shape: torch.full(shape, -7, dtype=torch.int32, device=dev)
            bufs = dict(sorted_slot=i32(t, top_k), sorted_expert=i32(t, top_k), local_offset=i32(t, top_k),
                        dst_rank=i32(t, top_k), dst_row=i32(t, top_k), dst_prow=i32(t, top_k),
                        expert_total=i32(experts), expert_base=i32(experts), expert_pbase=i32(experts),
                        padded_start=i32(e_local + 1), tile_group=i32(row_capacity // 128 + 1),
                        num_tiles=i32(1), padded_rows=i32(1), dst_primary=i32(t, top_k))
            out = _lib.WmRouteOut(**{k: v.data_ptr() for k, v in bufs.items()})
            _lib.check(fn(phase, world, rank, experts, top_k, t, cap, row_capacity,
                          _lib.ptr(r) if t else None, _lib.ptr(cm), ctypes.byref(out), None))
            result.append(bufs)
    torch.cuda.synchronize()
    out = []
    for bufs in result:
        d = {k: v.cpu().numpy() for k, v in bufs.items()}
        d["tile_group"] = d["tile_group"][: int(d["num_tiles"][0])]
        d["count_matrix"] = cm.cpu().numpy()
        out.append(d)
    return out


def random_routes(seed, world, experts, top_k, max_tokens):
    rng = np.random.default_rng(seed)
    return [rng.integers(-1, experts, size=(int(rng.integers(0, max_tokens)), top_k)).astype(np.int32)
            for _ in range(world)]


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    # Two different problems back to back: the second call finds the first call's data in the
    # shared scratch array and must not be affected by it.
    for seed, (world, experts, top_k, max_tokens) in enumerate([(4, 64, 8, 3000), (2, 16, 4, 500)]):
        routes = random_routes(seed, world, experts, top_k, max_tokens)
        rows = sum(len(r) for r in routes) * top_k
        row_capacity = (rows + 127) // 128 * 128 + 128 * (experts // world)
        mine = plan("wm_route_plan_noalloc", world, experts, top_k, routes, row_capacity)
        ref = plan("wm_route_plan", world, experts, top_k, routes, row_capacity)
        oracle = c_oracle.route_plan(world, experts, top_k, routes)
        for rank in range(world):
            for k in FIELDS + ("count_matrix",):
                assert np.array_equal(mine[rank][k], ref[rank][k]), (seed, rank, k)  # integers: bit-exact
            for k in ORACLE_FIELDS:  # and against the CPU restatement of the reference's planner
                assert np.array_equal(mine[rank][k].reshape(-1), np.asarray(oracle[rank][k]).reshape(-1)), (seed, rank, k)
            assert int(mine[rank]["num_tiles"][0]) == oracle[rank]["num_tiles"]
            assert int(mine[rank]["padded_rows"][0]) == oracle[rank]["padded_rows"]


def test_sizes_beyond_the_fixed_scratch_are_refused():
    lib = _lib.load()
    dev = torch.device("cuda")
    cm = torch.zeros(1024, dtype=torch.int32, device=dev)
    out = _lib.WmRouteOut()
    routes = torch.zeros(8, dtype=torch.int32, device=dev)
    # experts above the limit
    rc = lib.wm_route_plan_noalloc(0, 1, 0, 1024, 2, 4, 4, 1024, _lib.ptr(routes), _lib.ptr(cm), ctypes.byref(out), None)
    assert rc == _lib.WM_ERR_CAPACITY and "512 experts" in _lib.last_error()
    # routes above the limit (nothing is read before the check)
    rc = lib.wm_route_plan_noalloc(0, 1, 0, 64, 32, 8192, 8192, 1024, _lib.ptr(routes), _lib.ptr(cm), ctypes.byref(out), None)
    assert rc == _lib.WM_ERR_CAPACITY and "131072 routes" in _lib.last_error()
