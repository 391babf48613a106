"""Generate the golden fixtures in this folder by RUNNING THE REFERENCE's own code.

Run in a container that has the reference checkout (path given with --reference) — the fixtures are
committed because the GPU box has no reference.  Nothing here is imported by the product.

    python tests/golden/make_golden.py [--reference <checkout>]

Outputs
  moe_small.pt        inputs + outputs of the reference's torch MoE layer
                      (tests/torchrun_tensor_runtime.py:13-27 `reference_moe`, gradients by autograd
                      exactly as benchmarks/training_reference.py:36-51 takes them), BF16 and FP32
  route_cases.json    inputs + outputs of the reference's host route planner
                      (src/metadata/notify_dispatch.cpp through oracle/_ref/libref_route.so)
  fp8_quant.pt        inputs + (bytes, scales) of tests/test_fp8.py:20-36 `quant_reference`, plus the
                      zero / tiny / non-finite known answers of tests/test_fp8.py:53-63
  nvfp4_round.pt      inputs + outputs of tests/torchrun_sm100_nvfp4.py:13-27 `round_nvfp4_blocks`,
                      plus the byte-exact midpoint case of tests/torchrun_sm100_nvfp4_backward.py:29-45
"""
from __future__ import annotations

import argparse
import ctypes
import importlib.util
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def moe_fixture(reference):
    ref = load(reference / "tests/torchrun_tensor_runtime.py", "ref_tensor_runtime")
    out = {}
    for tag, dtype in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        g = torch.Generator().manual_seed(20241)
        E, K, H, I, T = (4, 2, 256, 128, 48) if dtype == torch.bfloat16 else (2, 2, 256, 128, 24)
        x = torch.randn(T, H, generator=g).to(dtype)
        w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(dtype)
        w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(dtype)
        dy = torch.randn(T, H, generator=g).to(dtype)
        scores, routes = torch.randn(T, E, generator=g).topk(K, dim=-1)
        gates = scores.softmax(-1).float()
        routes = routes.int()
        leaves = [t.clone().requires_grad_() for t in (x, gates, w1, w2)]
        if dtype == torch.float32:
            # reference_moe hard-codes a BF16 cast of U; the FP32 variant of the same math is
            # benchmarks/training_reference.py:41-45 (`.to(x.dtype)`), evaluated here expert by expert.
            y = torch.zeros(T, H)
            for e in range(E):
                rows, slots = torch.where(routes == e)
                a, b = (leaves[0][rows] @ leaves[2][e].T).chunk(2, dim=-1)
                u = (torch.nn.functional.silu(a.float()) * b.float() * leaves[1][rows, slots, None]).to(dtype)
                y = y.index_add(0, rows, u @ leaves[3][e].T)
        else:
            y = ref.reference_moe(leaves[0], routes, leaves[1], leaves[2], leaves[3])
        grads = torch.autograd.grad(y, leaves, dy)
        out[tag] = dict(x=x, routes=routes, gates=gates, w1=w1, w2=w2, dy=dy, y=y.detach(),
                        dx=grads[0], dgates=grads[1], dw1=grads[2], dw2=grads[3])
    torch.save(out, HERE / "moe_small.pt")
    print("moe_small.pt", {k: tuple(v["y"].shape) for k, v in out.items()})


def route_fixture(reference):
    subprocess.run(["make", "-C", str(ROOT / "oracle"), "ref", f"REFERENCE={reference}"], check=True)
    lib = ctypes.CDLL(str(ROOT / "oracle/_ref/libref_route.so"))
    lib.ref_route_error.restype = ctypes.c_char_p
    rng = np.random.default_rng(7)
    cases = []
    specs = [  # world, experts, top_k, tokens per rank
        (1, 8, 2, [16]), (1, 8, 2, [0]), (2, 8, 2, [5, 9]), (4, 16, 4, [0, 7, 3, 11]),
        (8, 64, 8, [3, 0, 9, 17, 1, 5, 12, 8]), (2, 16, 1, [33, 2]), (8, 256, 8, [40] * 8),
        (4, 8, 2, [130, 1, 0, 64]),
    ]
    for world, experts, top_k, tokens in specs:
        routes = []
        for t in tokens:
            if t == 130:  # skew: everything to the first two experts of rank 0
                r = np.tile(np.arange(top_k, dtype=np.int32), (t, 1))
            else:
                r = np.stack([rng.permutation(experts)[:top_k] for _ in range(t)]).astype(np.int32) \
                    if t else np.zeros((0, top_k), np.int32)
            routes.append(r)
        flat = np.concatenate([r.reshape(-1) for r in routes]).astype(np.int32)
        tok = np.asarray(tokens, dtype=np.uint64)
        per_rank = []
        for rank in range(world):
            n = tokens[rank] * top_k
            e_local = experts // world
            cm = np.zeros(world * experts, np.uint64)
            lo, row = np.zeros(n, np.uint64), np.zeros(n, np.uint64)
            drank, order = np.zeros(n, np.uint32), np.zeros(n, np.uint32)
            cnt, pre = np.zeros(e_local, np.uint64), np.zeros(e_local, np.uint64)
            p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
            rc = lib.ref_route_plan(world, experts, top_k, 128, p(tok), p(flat), rank, p(cm), p(lo),
                                    p(row), p(drank), p(order), p(cnt), p(pre))
            assert rc == 0, lib.ref_route_error()
            per_rank.append(dict(count_matrix=cm.reshape(world, experts).tolist(), local_offset=lo.tolist(),
                                 route_dst_row=row.tolist(), route_dst_rank=drank.tolist(),
                                 combine_order=order.tolist(), expert_row_count=cnt.tolist(),
                                 expert_row_prefix=pre.tolist()))
        cases.append(dict(world=world, experts=experts, top_k=top_k, tokens=tokens,
                          routes=[r.tolist() for r in routes], ranks=per_rank))
    (HERE / "route_cases.json").write_text(json.dumps(cases, separators=(",", ":")))
    print("route_cases.json", len(cases), "cases")


def fp8_fixture(reference):
    sys.path.insert(0, str(reference))
    ref = load(reference / "tests/test_fp8.py", "ref_test_fp8")
    cases = []
    for dtype in (torch.bfloat16, torch.float32):
        for shape in ((1, 1), (67, 259), (2, 129, 257), (4, 256)) if dtype == torch.bfloat16 else ((1, 1), (67, 259)):
            for block_rows, transpose in ((1, False), (1, True), (128, False)):
                torch.manual_seed(12)
                x = torch.randn(shape, dtype=dtype)
                x[..., 0, 0] = 0
                x[..., -1, -1] = 87
                q, scales = ref.quant_reference(x, block_rows, transpose)
                cases.append(dict(x=x, block_rows=block_rows, transpose=transpose,
                                  q=q.view(torch.uint8).clone(), scales=scales.clone()))
    x = torch.zeros(4, 256, dtype=torch.float32)
    x[1, :128] = 2.0 ** -135
    x[2, :128] = float("inf")
    x[3, 0] = float("nan")
    special = dict(x=x, tiny=float(torch.finfo(torch.float32).tiny))
    torch.save(dict(cases=cases, special=special), HERE / "fp8_quant.pt")
    print("fp8_quant.pt", len(cases), "cases")


def nvfp4_fixture(reference):
    sys.path.insert(0, str(reference))
    ref = load(reference / "tests/torchrun_sm100_nvfp4.py", "ref_nvfp4")
    cases = []
    g = torch.Generator().manual_seed(5)
    for scale, std in ((1 / 32, 0.16), (1 / 64, 0.023), (0.025, 0.1), (1 / 4, 1.0)):
        x = (torch.randn(24, 128, generator=g) * std).bfloat16()
        x[0, :16] = 0
        x[1, 3] = 1000.0
        cases.append(dict(x=x, scale=scale, rounded=ref.round_nvfp4_blocks(x, scale)))
    # Exact ties of the E2M1 grid: value / (sf * scale) in {0.25, 0.75, ..., 5.0} with sf = 1.
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5,
                         -3.5, -5.0, -6.0]).bfloat16()[None]
    cases.append(dict(x=ties, scale=1.0, rounded=ref.round_nvfp4_blocks(ties, 1.0)))
    # Byte-exact known answer (tests/torchrun_sm100_nvfp4_backward.py:29-45): a block of 0.1171875
    # with every fourth row holding 0.016845703125 at odd columns, layer scale 0.025 ->
    # scale byte E4M3(0.75), codes 7 (6.0) and 2 (1.0).
    x = torch.full((128, 128), 0.1171875, dtype=torch.bfloat16)
    x[::4, 1::2] = 0.016845703125
    codes = torch.full((128, 128), 7, dtype=torch.uint8)
    codes[::4, 1::2] = 2
    midpoint = dict(x=x, scale=0.025,
                    sf_byte=int(torch.tensor(0.75).to(torch.float8_e4m3fn).view(torch.uint8)),
                    packed=(codes[:, ::2] | (codes[:, 1::2] << 4)))
    torch.save(dict(cases=cases, midpoint=midpoint), HERE / "nvfp4_round.pt")
    print("nvfp4_round.pt", len(cases), "cases")


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default="/root/reference")
    reference = Path(parser.parse_args().reference)
    sys.path.insert(0, str(reference))
    moe_fixture(reference)
    route_fixture(reference)
    fp8_fixture(reference)
    nvfp4_fixture(reference)
