"""GPU: route planning through the C ABI is bit-exact against the CPU oracle and the reference
planner's golden vectors; full-size cases are checked through structural properties."""
import json

import numpy as np
import pytest
import torch

from oracle import c_oracle
from tests.gpu_util import device_route_plan

pytestmark = pytest.mark.gpu

KEYS = ("sorted_slot", "sorted_expert", "local_offset", "dst_rank", "dst_row", "dst_prow", "dst_primary")
OWNER_KEYS = ("expert_total", "expert_base", "expert_pbase", "padded_start", "tile_group")


def assert_same(dev, cpu):
    for rank, (d, c) in enumerate(zip(dev, cpu)):
        assert np.array_equal(d["count_matrix"], c["count_matrix"])
        for k in KEYS + OWNER_KEYS:
            assert np.array_equal(d[k].reshape(-1), np.asarray(c[k]).reshape(-1)), (rank, k)
        assert d["num_tiles"] == c["num_tiles"] and d["padded_rows"] == c["padded_rows"]


def test_reference_golden_cases(golden):
    for case in json.loads((golden / "route_cases.json").read_text()):
        world, experts, top_k = case["world"], case["experts"], case["top_k"]
        routes = [np.asarray(r, np.int32).reshape(-1, top_k) for r in case["routes"]]
        dev = device_route_plan(world, experts, top_k, routes)
        for rank, ref in enumerate(case["ranks"]):
            assert dev[rank]["count_matrix"].tolist() == ref["count_matrix"]
            assert dev[rank]["local_offset"].reshape(-1).tolist() == ref["local_offset"]
            assert dev[rank]["dst_row"].reshape(-1).tolist() == ref["route_dst_row"]
            assert dev[rank]["dst_rank"].reshape(-1).tolist() == ref["route_dst_rank"]
            assert dev[rank]["sorted_slot"].reshape(-1).tolist() == ref["combine_order"]


@pytest.mark.parametrize("world,experts,top_k,max_tokens", [
    (1, 8, 2, 300), (2, 16, 4, 700), (4, 64, 8, 1500), (8, 256, 8, 400), (8, 64, 6, 2100), (1, 512, 32, 77)])
def test_matches_cpu_oracle_with_invalid_and_duplicate_routes(world, experts, top_k, max_tokens):
    rng = np.random.default_rng(world * 1000 + experts)
    routes = []
    for r in range(world):
        t = 0 if (world > 1 and r == 1) else int(rng.integers(1, max_tokens))
        x = rng.integers(-1, experts, size=(t, top_k)).astype(np.int32)  # duplicates and -1 occur
        if t > 2:
            x[0] = 3
            x[1] = -1
            x[2, -1] = experts + 5  # out of range means "no route"
        routes.append(x)
    assert_same(device_route_plan(world, experts, top_k, routes), c_oracle.route_plan(world, experts, top_k, routes))


def test_empty_everywhere():
    routes = [np.zeros((0, 4), np.int32) for _ in range(4)]
    dev = device_route_plan(4, 16, 4, routes)
    assert all(d["num_tiles"] == 0 and d["padded_rows"] == 0 for d in dev)


@pytest.mark.parametrize("tokens", [8192, 20480])
def test_full_size_properties(tokens):
    """Benchmark shapes (E=256, K=8, 8 ranks): rows are a permutation, ordinals are stable."""
    world, experts, top_k = 8, 256, 8
    g = torch.Generator().manual_seed(tokens)
    bias = torch.randn(experts, generator=g) * 0.5
    routes = [(torch.randn(tokens, experts, generator=g) + bias).topk(top_k).indices.int().numpy() for _ in range(world)]
    dev = device_route_plan(world, experts, top_k, routes)
    e_local = experts // world
    for owner in range(world):
        rows = np.concatenate([d["dst_prow"][d["dst_rank"] == owner] for d in dev])
        assert len(np.unique(rows)) == len(rows) == dev[owner]["expert_total"][owner * e_local:(owner + 1) * e_local].sum()
        assert rows.max() < dev[owner]["padded_rows"]
    # stability: within (source, expert) the physical row grows with (token, slot)
    d = dev[3]
    flat_e, flat_row = routes[3].reshape(-1), d["dst_prow"].reshape(-1)
    for e in (0, 17, 255):
        r = flat_row[flat_e == e]
        assert (np.diff(r) == 1).all()
    assert np.array_equal(np.bincount(flat_e, minlength=experts), d["count_matrix"][3])
    # a checksum of checksums against the CPU oracle
    cpu = c_oracle.route_plan(world, experts, top_k, routes)
    assert sum(int(x["dst_prow"].astype(np.int64).sum()) for x in dev) == sum(int(x["dst_prow"].astype(np.int64).sum()) for x in cpu)
    assert_same(dev, cpu)


def test_row_capacity_overflow_is_reported():
    routes = [np.zeros((600, 2), np.int32)]
    routes[0][:, 1] = 1
    with pytest.raises(ValueError):
        device_route_plan(1, 8, 2, routes, row_capacity=256)
