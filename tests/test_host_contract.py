"""CPU: argument contract of the Tensor API for the quantised precisions, with a fake native object
(the checks run before anything reaches the device; reference: weftmoe/runtime.py:100-147,243-275)."""
import pytest
import torch

from weftmoe_b200 import SingleRankGroup
from weftmoe_b200.runtime import TensorRuntime


class FakeNative:
    def __init__(self, col, *args):
        self.args, self.stream, self.scales = args, args[6], None
        self.seen = []

    def forward_async(self, *tensors, **kw):
        self.seen.append("forward_async")
        return "tape"


def make(precision, training, intermediate=256, **kw):
    return TensorRuntime(group=SingleRankGroup(), experts=8, top_k=2, hidden=256, intermediate=intermediate,
                         max_tokens=16, max_rows=64, training=training, stream=object(), precision=precision,
                         _native_factory=FakeNative, **kw)


def test_nvfp4_runtimes_may_train_and_carry_six_layer_scales():
    rt = make("nvfp4", True, nvfp4_scales=(1 / 4, 1 / 64, 1 / 64, 1 / 64, 1 / 4, 1 / 64))
    assert rt.native.args[-1] == "nvfp4" and rt.native.scales.dy == 1 / 4 and rt.native.scales.dgate_up == 1 / 64
    assert make("nvfp4", True).native.scales.x == 1 / 32            # the reference's defaults
    with pytest.raises(ValueError, match="finite and positive"):
        make("nvfp4", True, nvfp4_scales=(1, 1, 0, 1, 1, 1))
    with pytest.raises(ValueError, match="divisible by 256"):
        make("nvfp4", True, intermediate=128)
    with pytest.raises(ValueError, match="requires NVFP4"):
        make("bf16", True, nvfp4_scales=(1, 1, 1, 1, 1, 1))


def test_forward_is_refused_where_the_precision_has_its_own_entry_point(monkeypatch):
    x = torch.zeros(4, 256, dtype=torch.bfloat16)
    args = (x, torch.zeros(4, 2, dtype=torch.int32), torch.zeros(4, 2), torch.zeros(8, 512, 256, dtype=torch.bfloat16),
            torch.zeros(8, 256, 256, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="forward_fp8"):
        make("fp8", True, intermediate=256).forward_async(*args)
    with pytest.raises(ValueError, match="inference_nvfp4"):
        make("nvfp4", False).forward_async(*args)


def test_decode_only_runtimes_are_inference_only_and_bounded():
    """decode_only is honoured, not ignored: a decode runtime (reference: the DT runtime, docs/usage.md:104-112)
    refuses training and keeps every call within the single-launch route planner."""
    assert make("bf16", False, decode_only=True).decode_only
    with pytest.raises(ValueError, match="inference-only"):
        make("bf16", True, decode_only=True)
    with pytest.raises(ValueError, match="at most 4096 routes"):
        TensorRuntime(group=SingleRankGroup(), experts=8, top_k=2, hidden=256, intermediate=256, max_tokens=4096,
                      max_rows=64, training=False, stream=object(), decode_only=True, _native_factory=FakeNative)
