"""CPU: the layer oracle against (a) golden outputs of the reference's torch MoE and (b) the
reference's own `verify_step` acceptance when the reference checkout is present."""
import importlib.util
import os
import sys
from pathlib import Path

import pytest
import torch

from oracle import moe_oracle as O

REFERENCE = Path(os.environ.get("WEFTMOE_REFERENCE", "/root/reference"))


def rel_l2(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()


@pytest.mark.parametrize("tag,limit", [("fp32", 2e-6), ("bf16", 6e-3)])
def test_layer_oracle_matches_reference_golden(golden, tag, limit):
    g = torch.load(golden / "moe_small.pt")[tag]
    y, dx, dg, dw1, dw2 = O.moe_layer(g["x"], g["routes"], g["gates"], g["w1"], g["w2"], g["dy"], precision=tag)
    for name, mine, ref in (("y", y, g["y"]), ("dx", dx, g["dx"]), ("dgates", dg, g["dgates"]),
                            ("dw1", dw1, g["dw1"]), ("dw2", dw2, g["dw2"])):
        # BF16: the reference rounds at fewer points than the device path (autograd keeps FP32
        # intermediates), so the bound is the reference's own acceptance scale, not bit equality.
        assert rel_l2(mine, ref) < limit, (tag, name, rel_l2(mine, ref))


def test_multi_rank_oracle_equals_single_rank():
    cfg = dict(experts=8, top_k=2, hidden=256, intermediate=128, tokens=40)
    d = O.make_inputs(cfg, seed=4)
    y, dx, dg, dw1, dw2 = O.moe_layer(d["x"], d["routes"], d["gates"], d["w1"], d["w2"], d["dy"])
    world = 4
    xs, rs, gs, dys = (list(t.chunk(world)) for t in (d["x"], d["routes"], d["gates"], d["dy"]))
    ys, dxs, dgs, dw1s, dw2s = O.moe_layer_ep(xs, rs, gs, list(d["w1"].chunk(world)), list(d["w2"].chunk(world)), dys)
    assert torch.equal(torch.cat(ys), y) and torch.equal(torch.cat(dxs), dx) and torch.equal(torch.cat(dgs), dg)
    # weight gradients: the row order inside an expert is (source rank, token, slot) either way
    assert torch.equal(torch.cat(dw1s), dw1) and torch.equal(torch.cat(dw2s), dw2)


def test_invalid_and_duplicate_routes():
    cfg = dict(experts=8, top_k=4, hidden=256, intermediate=128, tokens=12)
    d = O.make_inputs(cfg, seed=9)
    d["routes"][0] = 3
    d["routes"][1] = -1
    y, dx, dg, _, _ = O.moe_layer(d["x"], d["routes"], d["gates"], d["w1"], d["w2"], d["dy"])
    assert (y[1] == 0).all() and (dx[1] == 0).all() and (dg[1] == 0).all()
    assert y[0].abs().sum() > 0


@pytest.mark.skipif(not (REFERENCE / "benchmarks/training_reference.py").is_file(),
                    reason="reference checkout not present")
def test_reference_verify_step_accepts_the_oracle():
    """The CPU-runnable FP32 configuration through the reference's verify_step (benchmarks/training_reference.py:15-79),
    gloo world 1, with a stub runtime that returns this oracle's tensors."""
    import torch.distributed as dist
    spec = importlib.util.spec_from_file_location("ref_training_reference", REFERENCE / "benchmarks/training_reference.py")
    ref = importlib.util.module_from_spec(spec)
    sys.path.insert(0, str(REFERENCE))
    spec.loader.exec_module(ref)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29613")
        dist.init_process_group("gloo", rank=0, world_size=1)
    cfg = dict(experts=8, top_k=2, hidden=512, intermediate=512, tokens=256)
    d = O.make_inputs(cfg, seed=0, dtype=torch.float32)
    y, dx, dg, dw1, dw2 = O.moe_layer(d["x"], d["routes"], d["gates"], d["w1"], d["w2"], d["dy"], precision="fp32")

    class Tape:
        output = y

    class Stub:
        def forward(self, *a):
            return Tape()

        def backward(self, tape, dy):
            return dx, dg, dw1, dw2

    errors = ref.verify_step(Stub(), d["x"], d["routes"], d["gates"], d["w1"], d["w2"], d["dy"])
    assert all(e["relative_l2"] < 1e-5 for e in errors.values()), errors


def test_nvfp4_training_oracle_is_consistent_with_the_forward_oracle_and_the_unquantised_layer():
    """The NVFP4 training restatement (weftmoe/nvfp4_backward.py:59-112) gives the forward oracle's output
    bit for bit, and its gradients stay within 4-bit distance of the unquantised layer's."""
    cfg = dict(experts=4, top_k=2, hidden=128, intermediate=64, tokens=24)
    d = O.make_inputs(cfg, seed=5, x_std=0.2, w_std=0.025)
    d["routes"][0] = 1
    d["routes"][1] = -1
    dy = (d["dy"].float() * 0.2).to(torch.bfloat16)
    scales = (1 / 32, 1 / 64, 1 / 512, 1 / 64, 1 / 32, 1 / 512)
    y, dx, dg, dw1, dw2 = O.nvfp4_training_layer(d["x"], d["routes"], d["gates"], d["w1"], d["w2"], dy, scales=scales)
    fwd = O.quantized_layer(d["x"], d["routes"], d["gates"], d["w1"], d["w2"], kind="nvfp4", scales=scales[:4])
    assert torch.equal(y, fwd)
    ref = O.moe_layer(d["x"], d["routes"], d["gates"], d["w1"], d["w2"], dy)
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert rel(dx, ref[1]) < 0.3 and rel(dw1, ref[3]) < 0.3 and rel(dw2, ref[4]) < 0.3 and rel(dg, ref[2]) < 0.3
    assert (dx[1] == 0).all() and (dg[1] == 0).all()
