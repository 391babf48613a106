"""GPU: the Megatron adapter end to end on a stand-in MoE layer (EP1): patched forward, per-expert
Parameter gradients through `_Routed`, no-grad (checkpoint first pass) path, FP8 mode, suspend/close."""
import types

import pytest
import torch

from oracle import moe_oracle as O
from tests.gpu_util import rel_l2
from weftmoe_b200 import SingleRankGroup, megatron

pytestmark = pytest.mark.gpu


class MoELayer(torch.nn.Module):
    def __init__(self, experts, hidden, inter, top_k, w1, w2, router):
        super().__init__()
        fc1, fc2 = torch.nn.Module(), torch.nn.Module()
        for i in range(experts):
            fc1.register_parameter(f"weight{i}", torch.nn.Parameter(w1[i].clone()))
            fc2.register_parameter(f"weight{i}", torch.nn.Parameter(w2[i].clone()))
        self.experts = torch.nn.Module()
        self.experts.linear_fc1, self.experts.linear_fc2 = fc1, fc2
        self.num_local_experts = experts
        self.ep_group = SingleRankGroup()
        self.router = torch.nn.Parameter(router.clone())
        self.config = types.SimpleNamespace(num_moe_experts=experts, moe_router_topk=top_k, hidden_size=hidden,
                                            moe_ffn_hidden_size=inter)

    def shared_experts_compute(self, hidden_states):
        return None

    def route(self, hidden_states, padding_mask):
        logits = hidden_states.reshape(-1, hidden_states.shape[-1]).float() @ self.router.float()
        return logits.softmax(-1), None


@pytest.mark.parametrize("fp8", [False, True])
def test_megatron_adapter_forward_backward(fp8):
    torch.manual_seed(3)
    E, H, I, K, T = 8, 256, 128, 2, 48
    w1 = (torch.randn(E, 2 * I, H) * 0.05).bfloat16().cuda()
    w2 = (torch.randn(E, H, I) * 0.05).bfloat16().cuda()
    router = (torch.randn(H, E) * 0.1).cuda()
    layer = MoELayer(E, H, I, K, w1, w2, router).cuda()
    adapter = megatron.MegatronAdapter([layer], max_tokens=T, fp8=fp8)
    x = torch.randn(6, 8, H, device="cuda").bfloat16().requires_grad_()   # [seq, batch, hidden]
    out, bias = layer(x)
    assert bias is None and out.shape == x.shape
    dy = torch.randn_like(out)
    out.backward(dy)
    probs = (x.detach().reshape(-1, H).float() @ router).softmax(-1)
    gates, routes = probs.topk(K, dim=-1)
    ref = O.moe_layer(x.detach().reshape(-1, H).cpu(), routes.int().cpu(), gates.cpu(), w1.cpu(), w2.cpu(),
                      dy.reshape(-1, H).cpu(), precision="bf16")
    tol = 0.08 if fp8 else 3e-3
    assert rel_l2(out.detach().reshape(-1, H), ref[0]) < tol
    grads1 = torch.stack([getattr(layer.experts.linear_fc1, f"weight{i}").grad for i in range(E)])
    grads2 = torch.stack([getattr(layer.experts.linear_fc2, f"weight{i}").grad for i in range(E)])
    assert rel_l2(grads1, ref[3]) < tol and rel_l2(grads2, ref[4]) < tol
    assert layer.router.grad is not None and torch.isfinite(layer.router.grad).all()   # dprob reached the router
    with torch.no_grad():                                                               # checkpoint's first pass
        again, _ = layer(x)
    assert torch.equal(again.view(torch.int16), out.detach().view(torch.int16))
    assert adapter.runtime.native.usage()["notify_slots_in_use"] == 0
    adapter.suspend()
    assert adapter.runtime is None
    adapter.close()


def test_sglang_staging_and_scatter_kernels_match_their_torch_definitions():
    """wm_stage_inputs / wm_scatter_output (the jobs of the reference's Triton staging kernels,
    weftmoe/_sglang_kernels.py:21-99) against the torch expressions that define them, bit for bit, for int32
    and int64 ids, masked (-1) entries, a strided input, every rank's slice incl. an empty one."""
    from weftmoe_b200 import sglang
    torch.manual_seed(11)
    tokens, hidden, k, world = 37, 512, 6, 4
    wide = torch.randn(tokens, hidden + 64, device="cuda").bfloat16()
    hidden_states = wide[:, :hidden]                                  # row stride hidden + 64 elements
    weights = torch.rand(tokens, k, device="cuda")
    for dtype in (torch.int32, torch.int64):
        ids = torch.randint(-1, 16, (tokens, k), device="cuda", dtype=dtype)
        for rank in range(world + 1):                                 # the last one is past the end: valid = 0
            local, start, valid = sglang.row_shard(tokens, world, min(rank, world - 1) if rank < world else world - 1)
            if rank == world:
                start, valid = tokens, 0
            mine = sglang.stage_inputs(hidden_states, ids, weights, start, valid, local)
            ref = sglang.stage_inputs(hidden_states.cpu(), ids.cpu(), weights.cpu(), start, valid, local)
            for a, b in zip(mine, ref):
                assert a.dtype == b.dtype and torch.equal(a.cpu().view(torch.uint8), b.view(torch.uint8)), (dtype, rank)
            out = torch.randn(local, hidden, device="cuda").bfloat16()
            scattered = sglang.scatter_output(out, tokens, min(start, tokens), valid)
            expect = sglang.scatter_output(out.cpu(), tokens, min(start, tokens), valid)
            assert torch.equal(scattered.cpu().view(torch.int16), expect.view(torch.int16))
