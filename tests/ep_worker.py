"""Multi-rank parity worker: run with `python -m torch.distributed.run --nproc-per-node N tests/ep_worker.py`.

Mirrors the reference's torchrun tests (tests/torchrun_sm100_invariant.py,
tests/torchrun_tensor_runtime.py): every rank runs forward + backward through the Tensor API over
a real EP group, compares with the CPU oracle, checks that EPn equals EP1 bit for bit on the
forward output, that repeated interleaved tapes repeat bit for bit, and that a rank with zero
tokens and an idle expert are handled.  Backend nccl on GPUs (bootstrap collectives only).
"""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from oracle import moe_oracle as O  # noqa: E402
from weftmoe_b200 import SingleRankGroup, TensorRuntime  # noqa: E402


def rel_l2(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()


def bits(t):
    return t.contiguous().view(torch.int16 if t.dtype == torch.bfloat16 else torch.int32)


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    E, K, H, I = 16 * world // 2 if world > 2 else 16, 4, 512, 256
    E = max(E, 2 * world)
    e_local = E // world
    # ---- per-rank inputs; rank 1 holds no tokens in the second scenario
    # "mixed planners": rank 0 holds more than 4096 routes and plans with the general kernels, the other
    # ranks stay below and plan in one launch with the hand-shakes inside; both must speak one protocol
    for scenario, counts in (("mixed planners", [1200 if r == 0 else 90 + 7 * r for r in range(world)]),
                             ("ragged", [37 + 11 * r for r in range(world)]),
                             ("zero-token rank", [0 if r == 1 else 20 + r for r in range(world)])):
        g = torch.Generator().manual_seed(1234)
        w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.03).bfloat16()
        w2 = (torch.randn(E, H, I, generator=g) * 0.03).bfloat16()
        xs, rs, gs, dys = [], [], [], []
        for r in range(world):
            t = counts[r]
            xs.append((torch.randn(t, H, generator=g)).bfloat16())
            dys.append((torch.randn(t, H, generator=g)).bfloat16())
            ids = torch.rand(t, E, generator=g).topk(K).indices.int()
            ids.clamp_(max=E - 2)  # the last expert stays idle (and duplicates appear)
            if t > 2:
                ids[0] = 3
                ids[1] = -1
            rs.append(ids)
            gs.append(torch.rand(t, K, generator=g))
        cap = max(max(counts), 1)
        rt = TensorRuntime(group=dist.group.WORLD, experts=E, top_k=K, hidden=H, intermediate=I,
                           max_tokens=cap, max_rows=sum(counts) * K, training=True, max_saved=2)
        dev = lambda t: t.cuda()
        lw1, lw2 = dev(w1.chunk(world)[rank]), dev(w2.chunk(world)[rank])
        x, routes, gates, dy = dev(xs[rank]), dev(rs[rank]), dev(gs[rank]), dev(dys[rank])
        expected = None
        for _ in range(2):
            t = rt.forward_async(x, routes, gates, lw1, lw2)
            other = rt.forward_async(x, routes.roll(1, dims=1).contiguous(), gates, lw1, lw2)
            rt.backward_async(other, dy)
            result = (t.output, *rt.backward_async(t, dy))
            rt.drain()
            if expected is None:
                expected = tuple(v.clone() for v in result)
            else:
                for a, b in zip(result, expected):
                    assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), (scenario, "repeat differs")
        ys, dxs, dgs, dw1s, dw2s = O.moe_layer_ep(xs, rs, gs, list(w1.chunk(world)), list(w2.chunk(world)), dys)
        for name, mine, ref in zip(("y", "dx", "dgates", "dw1", "dw2"), expected,
                                   (ys[rank], dxs[rank], dgs[rank], dw1s[rank], dw2s[rank])):
            if ref.numel():
                err = rel_l2(mine, ref)
                assert err < 2e-3, (scenario, rank, name, err)
        assert (expected[3][-1] == 0).all() if rank == world - 1 else True  # idle expert: zero dW
        rt.close()
        # ---- EPn forward bits == EP1 forward bits on the same tokens
        ep1 = TensorRuntime(group=SingleRankGroup(), experts=E, top_k=K, hidden=H, intermediate=I,
                            max_tokens=max(sum(counts), 1), max_rows=sum(counts) * K, training=False)
        y1 = ep1.inference_eager(dev(torch.cat(xs)), dev(torch.cat(rs)), dev(torch.cat(gs)), dev(w1), dev(w2))
        begin = sum(counts[:rank])
        assert torch.equal(bits(y1[begin:begin + counts[rank]]), bits(expected[0])), (scenario, "EP1 != EPn bits")
        ep1.close()
        if rank == 0:
            print(f"EP{world} {scenario}: oracle parity, bitwise repeat and EP1 == EP{world} bits passed", flush=True)
    # ---- decode under a CUDA graph across ranks (DT contract, docs/usage.md:104-112): the multi-stream
    #      forward is captured by the caller's graph; every replay advances the device-side generation
    #      of the cross-rank flags, reads fresh inputs from the same addresses and gives the eager bits
    inf = TensorRuntime(group=dist.group.WORLD, experts=E, top_k=K, hidden=H, intermediate=I,
                        max_tokens=cap, max_rows=sum(counts) * K, training=False)
    eager = inf.inference_eager(x, routes, gates, lw1, lw2).clone()
    x2 = (x * 0.5).contiguous()
    eager2 = inf.inference_eager(x2, routes, gates, lw1, lw2).clone()
    xg = x.clone()
    inf.inference(0, xg, routes, gates, lw1, lw2)             # warm-up of this layer outside capture
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_graph = inf.inference(0, xg, routes, gates, lw1, lw2)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(bits(y_graph), bits(eager)), "graph replay differs from eager"
    xg.copy_(x2)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(bits(y_graph), bits(eager2)), "graph replay with new inputs differs from eager"
    # eager calls still line up with the peers after the replays (generations stayed in step)
    assert torch.equal(bits(inf.inference_eager(x, routes, gates, lw1, lw2)), bits(eager))
    del graph
    inf.close()
    if rank == 0:
        print(f"EP{world} decode under a CUDA graph: replays == eager bits passed", flush=True)
    # ---- quantised inference (NVFP4 and blockwise FP8) over the EP group: EPn bits == EP1 bits
    from weftmoe_b200.fp8 import prepare_fp8_weights
    from weftmoe_b200.nvfp4 import prepare_nvfp4_weights
    counts = [29 + 5 * r for r in range(world)]
    g = torch.Generator().manual_seed(77)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.023).bfloat16()
    w2 = (torch.randn(E, H, I, generator=g) * 0.023).bfloat16()
    xs = [(torch.randn(t, H, generator=g) * 0.16).bfloat16() for t in counts]
    rs = [torch.rand(t, E, generator=g).topk(K).indices.int() for t in counts]
    gs = [torch.rand(t, K, generator=g) for t in counts]
    for precision in ("nvfp4", "fp8"):
        outs = []
        for group, n, sl in ((dist.group.WORLD, max(counts), slice(rank * e_local, (rank + 1) * e_local)),
                             (SingleRankGroup(), sum(counts), slice(0, E))):
            rt = TensorRuntime(group=group, experts=E, top_k=K, hidden=H, intermediate=I, max_tokens=max(n, 1),
                               max_rows=sum(counts) * K, training=False, precision=precision)
            lw1, lw2 = w1[sl].contiguous().cuda(), w2[sl].contiguous().cuda()
            single = isinstance(group, SingleRankGroup)
            x = (torch.cat(xs) if single else xs[rank]).cuda()
            r = (torch.cat(rs) if single else rs[rank]).cuda()
            gt = (torch.cat(gs) if single else gs[rank]).cuda()
            if precision == "nvfp4":
                y = rt.inference_nvfp4(0, x, r, gt, prepare_nvfp4_weights(lw1, lw2))
            else:
                y = rt.inference_fp8(0, x, r, gt, prepare_fp8_weights(lw1, lw2, training=False))
            outs.append(y.clone())
            rt.close()
        begin = sum(counts[:rank])
        assert torch.equal(bits(outs[1][begin:begin + counts[rank]]), bits(outs[0])), (precision, "EP1 != EPn bits")
        ref = O.quantized_layer(torch.cat(xs), torch.cat(rs), torch.cat(gs), w1, w2, kind=precision)
        err = rel_l2(outs[0], ref[begin:begin + counts[rank]])
        assert err < 5e-3, (precision, err)
    if rank == 0:
        print(f"EP{world} quantised inference (nvfp4, fp8): oracle parity and EP1 == EP{world} bits passed", flush=True)
    # ---- NVFP4 training over the EP group: output and all gradients, EPn bits == EP1 bits
    dys = [(torch.randn(t, H, generator=g) * 0.2).bfloat16() for t in counts]
    grads = []
    for group, n, sl in ((dist.group.WORLD, max(counts), slice(rank * e_local, (rank + 1) * e_local)),
                         (SingleRankGroup(), sum(counts), slice(0, E))):
        rt = TensorRuntime(group=group, experts=E, top_k=K, hidden=H, intermediate=I, max_tokens=max(n, 1),
                           max_rows=sum(counts) * K, training=True, precision="nvfp4", max_saved=1)
        single = isinstance(group, SingleRankGroup)
        pick = (lambda parts: torch.cat(parts).cuda()) if single else (lambda parts: parts[rank].cuda())
        lw1, lw2 = w1[sl].contiguous().cuda(), w2[sl].contiguous().cuda()
        tape = rt.forward_async(pick(xs), pick(rs), pick(gs), lw1, lw2)
        grads.append((tape.output, *rt.backward(tape, pick(dys))))
        rt.close()
    begin = sum(counts[:rank])
    mine = slice(begin, begin + counts[rank])
    for name, part, whole in zip(("y", "dx", "dgates"), grads[0][:3], grads[1][:3]):
        assert torch.equal(bits(whole[mine]), bits(part)), ("nvfp4 training", name, "EP1 != EPn bits")
    for name, part, whole in zip(("dw1", "dw2"), grads[0][3:], grads[1][3:]):
        assert torch.equal(bits(whole[rank * e_local:(rank + 1) * e_local]), bits(part)), ("nvfp4 training", name)
    if rank == 0:
        print(f"EP{world} NVFP4 training: EP1 == EP{world} bits for y, dx, dgates, dw1, dw2 passed", flush=True)
    # ---- received rows beyond max_rows: a collective, reported error, runtime stays usable
    small = TensorRuntime(group=dist.group.WORLD, experts=E, top_k=K, hidden=H, intermediate=I,
                          max_tokens=512, max_rows=128, training=False)
    g = torch.Generator().manual_seed(5 + rank)
    x = torch.randn(512, H, generator=g).bfloat16().cuda()
    routes = torch.zeros(512, K, dtype=torch.int32).cuda() + torch.arange(K, dtype=torch.int32).cuda()  # all to rank 0
    gates = torch.rand(512, K, generator=g).cuda()
    lw1, lw2 = w1.chunk(world)[rank].cuda(), w2.chunk(world)[rank].cuda()
    failed = False
    try:
        small.inference_eager(x, routes, gates, lw1, lw2)
    except ValueError:
        failed = True
    flags = [None] * world
    dist.all_gather_object(flags, failed)
    # every rank holds the same count matrix, so every rank reports the owner's overflow
    # (the reference fails collectively too: src/metadata/notify_dispatch.cpp:2003-2035)
    assert all(flags), f"all ranks must report the overflow, got {flags}"
    y = small.inference_eager(x[:4], routes[:4], gates[:4], lw1, lw2)
    assert torch.isfinite(y.float()).all()
    small.close()
    if rank == 0:
        print(f"EP{world} overflow reporting passed", flush=True)
    if os.environ.get("WM_EP_HEADLINE", "1") != "0":
        headline_scenario(rank, world)
    absent_rank_scenario(rank, world, w1, w2, E, K, H, I)
    dist.destroy_process_group()


def headline_scenario(rank, world):
    """The headline training shape over the EP group (E=256, K=8, H=2048, I=512, 8192 tokens per rank, router
    bias shared by all ranks so that owners are unevenly loaded).  The whole-layer oracle would take minutes
    per rank, so parity is sampled the way tests/test_gpu_layer.py does at EP1:
      * forward + backward twice: all five tensors repeat bit for bit;
      * y / dX / dprob of a few of this rank's tokens against the oracle (they depend only on the token's
        row and the weights of the experts it is routed to, wherever those live);
      * dW1 / dW2 of this rank's most and least loaded expert against the oracle (they depend only on the
        rows routed to that expert, from every rank);
      * this rank's first 256 tokens through an EP1 runtime holding all experts: same forward bits.
    Every rank regenerates the other ranks' seeded inputs on its own GPU (same seed, same Philox stream)."""
    E, K, H, I, T = 256, 8, 2048, 512, 8192
    e_local = E // world
    dev = torch.device("cuda", torch.cuda.current_device())

    def rank_inputs(r):
        g = torch.Generator(device=dev).manual_seed(9000 + r)
        x = torch.randn(T, H, device=dev, generator=g).bfloat16()
        dy = torch.randn(T, H, device=dev, generator=g).bfloat16()
        logits = torch.randn(T, E, device=dev, generator=g)
        bias = torch.randn(E, device=dev, generator=torch.Generator(device=dev).manual_seed(77)) * 0.5
        scores, routes = (logits + bias).topk(K, dim=-1)
        return x, dy, routes.int().contiguous(), scores.softmax(-1).float().contiguous()

    def rank_weights(r):
        g = torch.Generator(device=dev).manual_seed(500 + r)
        w1 = (torch.randn(e_local, 2 * I, H, device=dev, generator=g) * 0.02).bfloat16()
        w2 = (torch.randn(e_local, H, I, device=dev, generator=g) * 0.02).bfloat16()
        return w1, w2

    x, dy, routes, gates = rank_inputs(rank)
    w1, w2 = rank_weights(rank)
    rt = TensorRuntime(group=dist.group.WORLD, experts=E, top_k=K, hidden=H, intermediate=I, max_tokens=T,
                       max_rows=2 * T * K, training=True, max_saved=1)
    runs = []
    for _ in range(2):
        tape = rt.forward_async(x, routes, gates, w1, w2)
        runs.append((tape.output, *rt.backward_async(tape, dy)))
        rt.drain()
    for a, b in zip(*runs):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), "headline shape: repeat differs"
    y, dx, dg, dw1, dw2 = runs[0]
    rt.close()

    weights = {}

    def expert_weights(ids):
        out1, out2 = [], []
        for e in ids:
            owner = e // e_local
            if owner not in weights:
                weights[owner] = tuple(t.cpu() for t in rank_weights(owner))
            out1.append(weights[owner][0][e % e_local])
            out2.append(weights[owner][1][e % e_local])
        return torch.stack(out1), torch.stack(out2)

    def compact(xs, routes_, gates_, dys):
        """The oracle on a few tokens with only the experts they touch (ids renumbered)."""
        used = routes_[routes_ >= 0].unique()
        remap = torch.full((E,), -1, dtype=torch.int32)
        remap[used.long()] = torch.arange(len(used), dtype=torch.int32)
        local = torch.where(routes_ >= 0, remap[routes_.clamp_min(0).long()], routes_)
        ow1, ow2 = expert_weights(used.tolist())
        return used, O.moe_layer(xs, local, gates_, ow1, ow2, dys)

    sample = torch.tensor([0, 1, 4097, 8191])
    cs = lambda t: t[sample.to(dev)].cpu()
    _, (ys, dxs, dgs, _, _) = compact(cs(x), cs(routes), cs(gates), cs(dy))
    for name, mine, ref in (("y", y, ys), ("dx", dx, dxs), ("dgates", dg, dgs)):
        err = rel_l2(cs(mine), ref)
        assert err < 2e-3, ("headline shape", rank, name, err)
    everyone = [rank_inputs(r) for r in range(world)]
    all_routes = torch.cat([v[2] for v in everyone])
    counts = torch.bincount(all_routes.flatten().long(), minlength=E)[rank * e_local:(rank + 1) * e_local]
    for local_e in (int(counts.argmax()), int(counts.argmin())):
        expert = rank * e_local + local_e
        hit = (all_routes == expert).any(dim=1).nonzero().flatten()
        pick = lambda i: torch.cat([v[i] for v in everyone])[hit].cpu()
        only = torch.where(pick(2) == expert, pick(2), torch.full_like(pick(2), -1))
        used, (_, _, _, w1g, w2g) = compact(pick(0), only, pick(3), pick(1))
        assert used.tolist() == [expert]
        for name, mine, ref in (("dw1", dw1[local_e], w1g[0]), ("dw2", dw2[local_e], w2g[0])):
            err = rel_l2(mine, ref)
            assert err < 2e-3, ("headline shape", rank, name, expert, err)
    del everyone
    # EP1 with every expert on this GPU: the same tokens give the same forward bits
    full = [rank_weights(r) for r in range(world)]
    fw1, fw2 = torch.cat([f[0] for f in full]), torch.cat([f[1] for f in full])
    del full
    ep1 = TensorRuntime(group=SingleRankGroup(), experts=E, top_k=K, hidden=H, intermediate=I, max_tokens=256,
                        max_rows=256 * K, training=False)
    y1 = ep1.inference_eager(x[:256].contiguous(), routes[:256].contiguous(), gates[:256].contiguous(), fw1, fw2)
    assert torch.equal(bits(y1), bits(y[:256])), "headline shape: EP1 != EPn forward bits"
    ep1.close()
    ok = [None] * world
    dist.all_gather_object(ok, True)
    if rank == 0:
        print(f"EP{world} headline shape (E=256 K=8 H=2048 I=512, 8192 tokens/rank): sampled oracle parity "
              f"(y, dx, dgates, dw1, dw2), bitwise repeat and EP1 == EP{world} forward bits passed", flush=True)


def absent_rank_scenario(rank, world, w1, w2, E, K, H, I):
    """One rank leaves between steps (it simply makes no further call; nothing of it is in flight): the
    other ranks' next call must end by itself with a RuntimeError from the bounded flag wait instead of
    waiting for ever, and the group must still close cleanly.  The wait budget is shortened to about
    50 ms through the diagnostic setter; the failure is made on the host only."""
    from weftmoe_b200 import _lib
    lib = _lib.load()
    rt = TensorRuntime(group=dist.group.WORLD, experts=E, top_k=K, hidden=H, intermediate=I, max_tokens=32,
                       max_rows=32 * K * world, training=False)
    g = torch.Generator().manual_seed(900 + rank)
    x = torch.randn(32, H, generator=g).bfloat16().cuda()
    routes = torch.rand(32, E, generator=g).topk(K).indices.int().cuda()
    gates = torch.rand(32, K, generator=g).cuda()
    lw1, lw2 = w1.chunk(world)[rank].cuda(), w2.chunk(world)[rank].cuda()
    good = rt.inference_eager(x, routes, gates, lw1, lw2).clone()        # every rank takes part
    torch.cuda.synchronize()
    dist.barrier()
    raised = None
    if rank != world - 1:
        lib.wm_debug_set_wait_budget(100_000_000)
        try:
            rt.inference_eager(x, routes, gates, lw1, lw2)
            raised = False
        except RuntimeError as exc:
            raised = "wait" in str(exc)
        finally:
            lib.wm_debug_set_wait_budget(0)
    torch.cuda.synchronize()
    seen = [None] * world
    dist.all_gather_object(seen, raised)
    assert all(v is True for v in seen[:-1]) and seen[-1] is None, seen
    assert torch.isfinite(good.float()).all()
    rt.close()
    if rank == 0:
        print(f"EP{world} absent rank: the others' bounded waits ran out with RuntimeError, clean close passed",
              flush=True)


if __name__ == "__main__":
    main()
