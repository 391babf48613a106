"""CPU: the framework-independent parts of the Megatron and SGLang adapters (parameter stacking,
layer validation, row sharding, route sanitisation, staging and scatter)."""
import types

import pytest
import torch

from weftmoe_b200 import megatron, sglang


class MoELayer(torch.nn.Module):
    """Stand-in with the attributes the adapter reads from Megatron-Core's MoELayer."""

    def __init__(self, experts=3, hidden=8, inter=4, **config):
        super().__init__()
        fc1, fc2 = torch.nn.Module(), torch.nn.Module()
        for i in range(experts):
            fc1.register_parameter(f"weight{i}", torch.nn.Parameter(torch.randn(2 * inter, hidden)))
            fc2.register_parameter(f"weight{i}", torch.nn.Parameter(torch.randn(hidden, inter)))
        self.experts = torch.nn.Module()
        self.experts.linear_fc1, self.experts.linear_fc2 = fc1, fc2
        self.num_local_experts = experts
        self.config = types.SimpleNamespace(**config)


def test_megatron_pack_stacks_parameters_and_reuses_the_workspace():
    layer = MoELayer()
    adapter = megatron.MegatronAdapter([layer], max_tokens=16)
    parameters = adapter._parameters(layer)
    w1, w2 = adapter.pack(parameters)
    assert w1.shape == (3, 8, 8) and w2.shape == (3, 8, 4)
    assert all(torch.equal(w1[i], parameters[i]) and torch.equal(w2[i], parameters[3 + i]) for i in range(3))
    again = adapter.pack(parameters)
    assert again[0].data_ptr() == w1.data_ptr() and len(adapter.packed) == 1
    version = adapter.weight_version
    adapter.weights_updated()
    assert adapter.weight_version == version + 1


def test_megatron_rejects_unsupported_layers():
    with pytest.raises(ValueError, match="ETP1"):
        megatron.MegatronAdapter([MoELayer(add_bias_linear=True)], max_tokens=4)
    with pytest.raises(ValueError, match="ETP1"):
        megatron.MegatronAdapter([MoELayer(expert_tensor_parallel_size=2)], max_tokens=4)
    with pytest.raises(ValueError, match="No Megatron MoE layers"):
        megatron.MegatronAdapter([torch.nn.Linear(2, 2)], max_tokens=4)


def test_sglang_row_sharding_staging_and_scatter():
    assert sglang.row_shard(10, 4, 0) == (3, 0, 3) and sglang.row_shard(10, 4, 3) == (3, 9, 1)
    assert sglang.row_shard(2, 4, 3) == (1, 3, 0)
    hidden = torch.arange(40, dtype=torch.float32).view(10, 4)
    ids = torch.tensor([[0, 1], [2, -1], [3, 4], [-1, -1], [5, 6], [7, 0], [1, 2], [3, 4], [5, 6], [7, 1]])
    weights = torch.full((10, 2), 0.5)
    local, start, valid = sglang.row_shard(10, 4, 3)
    x, routes, gates = sglang.stage_inputs(hidden, ids, weights, start, valid, local)
    assert x.shape == (3, 4) and torch.equal(x[0], hidden[9]) and (x[1:] == 0).all()
    assert routes.tolist() == [[7, 1], [-1, -1], [-1, -1]] and gates[1:].sum() == 0
    r, g = sglang.sanitize_routes(ids[1:2], weights[1:2])
    assert r.dtype == torch.int32 and r.tolist() == [[2, -1]] and g.tolist() == [[0.5, 0.0]]
    out = sglang.scatter_output(torch.ones(3, 4), 10, start, valid)
    assert out.shape == (10, 4) and out.sum() == 4 and out[9].sum() == 4
    with pytest.raises(ImportError):
        sglang.install()
