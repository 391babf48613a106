"""CPU: host-side logic of the FP8 / NVFP4 Python boundary (no kernel runs here)."""
import pytest
import torch

from weftmoe_b200 import fp8, nvfp4


def test_nvfp4_block_stats_boundaries_known_answer():
    """The reference's known answer for the default dY scale (tests/test_nvfp4_scales.py:10-17): block
    maxima for zero input, underflow, the half-ulp tie, the smallest subnormal scale, a normal scale, the
    largest scale and overflow."""
    scale = 1 / 32
    maxima = torch.tensor([0, 2 ** -16, 6 * scale * 2 ** -10, 6 * scale * 2 ** -9, 0.1, 84, 100])
    stats = nvfp4.nvfp4_block_stats(maxima[:, None].expand(-1, 16), scale)
    assert {k: int(v) for k, v in stats.items()} == {
        "blocks": 7, "nonzero_to_zero": 2, "subnormal_scale": 1, "above_range": 1}


def test_nvfp4_block_stats_rejects_bad_input():
    with pytest.raises(ValueError):
        nvfp4.nvfp4_block_stats(torch.zeros(4, 15), 1 / 32)
    with pytest.raises(ValueError):
        nvfp4.nvfp4_block_stats(torch.zeros(4, 16, dtype=torch.int32), 1 / 32)
    for bad in (0.0, -1.0, float("inf"), float("nan")):
        with pytest.raises(ValueError):
            nvfp4.nvfp4_block_stats(torch.zeros(4, 16), bad)


def test_fp8_storage_geometry():
    assert fp8._storage_shapes((300, 200), 1) == ((300, 256), (300, 2))
    assert fp8._storage_shapes((4, 300, 200), 128) == ((4, 300, 256), (4, 3, 2))
    assert fp8._storage_shapes((0, 128), 128) == ((0, 128), (0, 1))


def test_fp8_argument_contract_without_a_gpu():
    cpu = torch.zeros(4, 128)
    with pytest.raises(ValueError):
        fp8.quantize_fp8(cpu)                       # not a CUDA tensor
    with pytest.raises(ValueError):
        fp8.FP8Tensor(cpu.to(torch.float8_e4m3fn), torch.ones(4, 1), (4, 128))
    for bad in (-1, 2 ** 64, True, 1.5):
        with pytest.raises(ValueError):
            fp8.prepare_fp8_weights(cpu, cpu, version=bad)
