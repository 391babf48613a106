"""CPU: the C route oracle against the reference planner's golden vectors (and the planner itself
when oracle/_ref was built in this checkout)."""
import json

import numpy as np
import pytest

from oracle import c_oracle


def _cases(golden):
    return json.loads((golden / "route_cases.json").read_text())


def test_route_oracle_matches_reference_golden(golden):
    for case in _cases(golden):
        world, experts, top_k = case["world"], case["experts"], case["top_k"]
        routes = [np.asarray(r, np.int32).reshape(-1, top_k) for r in case["routes"]]
        plan = c_oracle.route_plan(world, experts, top_k, routes)
        for rank, ref in enumerate(case["ranks"]):
            mine = plan[rank]
            e_local = experts // world
            assert mine["count_matrix"].tolist() == ref["count_matrix"]
            assert mine["local_offset"].reshape(-1).tolist() == ref["local_offset"]
            assert mine["dst_row"].reshape(-1).tolist() == ref["route_dst_row"]
            assert mine["dst_rank"].reshape(-1).tolist() == ref["route_dst_rank"]
            assert mine["sorted_slot"].reshape(-1).tolist() == ref["combine_order"]
            own = slice(rank * e_local, (rank + 1) * e_local)
            assert mine["expert_total"][own].tolist() == ref["expert_row_count"]
            assert mine["expert_base"][own].tolist() == ref["expert_row_prefix"]


def test_route_oracle_matches_reference_planner_live():
    ref = c_oracle.reference_route_lib()
    if ref is None:
        pytest.skip("oracle/_ref not built in this checkout")
    rng = np.random.default_rng(11)
    for world, experts, top_k in ((2, 16, 4), (8, 64, 6), (4, 32, 8)):
        routes = [np.stack([rng.permutation(experts)[:top_k] for _ in range(int(rng.integers(1, 50)))]).astype(np.int32)
                  for _ in range(world)]
        plan = c_oracle.route_plan(world, experts, top_k, routes)
        for rank in range(world):
            r = c_oracle.reference_route_plan(ref, world, experts, top_k, routes, rank)
            assert (plan[rank]["count_matrix"] == r["count_matrix"]).all()
            assert (plan[rank]["dst_row"].reshape(-1) == r["route_dst_row"]).all()
            assert (plan[rank]["sorted_slot"].reshape(-1) == r["combine_order"]).all()


def test_padded_layout_properties():
    rng = np.random.default_rng(3)
    world, experts, top_k = 4, 32, 4
    routes = [rng.integers(-1, experts, size=(int(rng.integers(0, 300)), top_k)).astype(np.int32) for _ in range(world)]
    plan = c_oracle.route_plan(world, experts, top_k, routes)
    e_local = experts // world
    for owner in range(world):
        seen = set()
        for src in range(world):
            m = plan[src]["dst_rank"] == owner
            rows = plan[src]["dst_prow"][m]
            assert not (set(rows.tolist()) & seen), "two routes share a physical row"
            seen |= set(rows.tolist())
        p = plan[owner]
        assert p["padded_start"][-1] == p["padded_rows"] == p["num_tiles"] * 128
        assert all(s % 128 == 0 for s in p["padded_start"])
        live = sum(int(p["expert_total"][owner * e_local + l]) for l in range(e_local))
        assert len(seen) == live
        # invalid routes never get a row, duplicates inside a token get distinct rows
        for src in range(world):
            bad = (routes[src] < 0) | (routes[src] >= experts)
            assert (plan[src]["dst_prow"][bad] == -1).all()


def test_primary_rows_hand_made_case_and_properties():
    """One NVLink pull per (token, owner): dst_primary names the owner row that is pulled; the token's other
    rows in that owner are copied from it.  Hand-made case: 2 ranks x 2 experts each, top-4."""
    routes = [np.array([[3, 0, 1, 2],      # experts 0, 1 -> rank 0 (head = slot 1); 3, 2 -> rank 1 (head = slot 3)
                        [1, 1, -1, 0],     # rank 0 three times: head = expert 0 (slot 3); duplicates of expert 1 copy
                        [2, 2, 2, 2]],     # one expert four times: head = slot 0
                       np.int32), np.zeros((0, 4), np.int32)]
    p = c_oracle.route_plan(2, 4, 4, routes)[0]
    prow, primary = p["dst_prow"], p["dst_primary"]
    assert primary[0].tolist() == [prow[0, 3], prow[0, 1], prow[0, 1], prow[0, 3]]
    assert primary[1].tolist() == [prow[1, 3], prow[1, 3], -1, prow[1, 3]]
    assert primary[2].tolist() == [prow[2, 0]] * 4
    # properties on random routes: the primary is a row of the same token and owner, never above the row
    # itself (so the first pipelined half never waits for the second), and every (token, owner) has one
    rng = np.random.default_rng(11)
    world, experts, top_k = 4, 32, 8
    routes = [rng.integers(-1, experts, size=(int(rng.integers(1, 200)), top_k)).astype(np.int32) for _ in range(world)]
    for p in c_oracle.route_plan(world, experts, top_k, routes):
        valid = p["dst_rank"] >= 0
        assert ((p["dst_primary"] == -1) == ~valid).all()
        assert (p["dst_primary"][valid] <= p["dst_prow"][valid]).all()
        for t in range(p["dst_rank"].shape[0]):
            for owner in set(p["dst_rank"][t][valid[t]].tolist()):
                mine = p["dst_rank"][t] == owner
                heads = p["dst_prow"][t][mine & (p["dst_primary"][t] == p["dst_prow"][t])]
                assert len(heads) == 1 and (p["dst_primary"][t][mine] == heads[0]).all()
