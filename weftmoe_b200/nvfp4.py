"""NVFP4 block-16 E2M1 operands with E4M3 block scales.

Mirror of the reference's `weftmoe/nvfp4.py` public names (NVFP4Scales :79-87, NVFP4Weights :90-94,
nvfp4_block_stats :102-119, prepare_nvfp4_weights :122-142) over the C ABI (`wm_nvfp4_quantize`).
Weights keep the canonical row order ([gate rows, up rows]); their scale bytes are stored in the 512-byte
tensor-core chunks this library's block-scaled kernel reads: int32 [E, N/128, K/64, 128] (word
(n%32)*4 + (n%128)/32 of a chunk holds the four scales of row n for one 64-column group).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import NamedTuple

import torch

from . import _lib


class NVFP4Scales(NamedTuple):
    """Layer-wide dequantization factors, independent of the token batch."""
    x: float = 1 / 32
    w1: float = 1 / 64
    intermediate: float = 1 / 512
    w2: float = 1 / 64
    dy: float = 1 / 32
    dgate_up: float = 1 / 512


@dataclass(frozen=True)
class NVFP4Weights:
    fc1: tuple
    fc2: tuple
    tensor_scales: tuple


def _validate_scales(scales):
    """Layer scales divide and multiply values on the device: each must be a finite positive number."""
    for value in scales:
        if not (math.isfinite(value) and value > 0):
            raise ValueError("NVFP4 tensor scales must be finite and positive")


_E4M3_MAX = 448.0            # largest finite E4M3 value: the block scale saturates here
_E2M1_MAX = 6.0              # largest E2M1 magnitude
_E4M3_MIN_NORMAL = 2.0 ** -6


def nvfp4_block_stats(tensor, scale):
    """How the block-16 scales of `tensor` (blocks along its last axis) would fare with layer scale
    `scale`: the number of blocks, and how many of them lose a non-zero block to a zero scale, land on a
    subnormal E4M3 scale, or exceed the E4M3 range.  Used to calibrate layer scales before quantising
    (same report as the reference's nvfp4_block_stats, weftmoe/nvfp4.py:102-119).  The counts are device
    tensors: nothing is synchronised here."""
    _validate_scales((scale,))
    usable = tensor.is_floating_point() and tensor.ndim >= 1 and tensor.shape[-1] % 16 == 0
    if not usable:
        raise ValueError("Expected floating-point data with a last dimension divisible by 16")
    blocks = tensor.detach().reshape(*tensor.shape[:-1], tensor.shape[-1] // 16, 16)
    block_amax = blocks.abs().amax(dim=-1).float()
    wanted = block_amax / (_E2M1_MAX * scale)                       # the scale each block asks for
    stored = wanted.clamp(max=_E4M3_MAX).to(torch.float8_e4m3fn).float()
    lost = (stored == 0) & (block_amax > 0)
    tiny = (stored > 0) & (stored < _E4M3_MIN_NORMAL)
    return {"blocks": block_amax.numel(), "nonzero_to_zero": lost.sum(), "subnormal_scale": tiny.sum(),
            "above_range": (wanted > _E4M3_MAX).sum()}


def quantize_nvfp4(x: torch.Tensor, scale: float, *, chunked: bool = False):
    """BF16 [rows, cols] -> (packed uint8 [rows, cols/2], scale bytes).  Row-major scale bytes
    [rows, cols/16], or int32 chunks [ceil(rows/128), cols/64, 128] when `chunked`."""
    if x.ndim != 2 or x.dtype != torch.bfloat16 or not x.is_cuda or not x.is_contiguous() or x.shape[1] % 16:
        raise ValueError("Expected contiguous CUDA BF16 [rows, cols] with cols divisible by 16")
    _validate_scales((scale,))
    rows, cols = x.shape
    with torch.cuda.device(x.device):
        data = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
        if chunked:
            sf = torch.empty((rows + 127) // 128, cols // 64, 128, dtype=torch.int32, device=x.device)
        else:
            sf = torch.empty(rows, cols // 16, dtype=torch.uint8, device=x.device)
        _lib.check(_lib.load().wm_nvfp4_quantize(_lib.ptr(x), rows, cols, scale, _lib.ptr(data), _lib.ptr(sf),
                                                 int(chunked), torch.cuda.current_stream().cuda_stream))
    return data, sf


def _is_device_bf16(t):
    return isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()


def prepare_nvfp4_weights(w1, w2, *, weight_scales=(1 / 64, 1 / 64)):
    """Quantise BF16 expert weights w1 [E, 2I, H] (gate rows, then up rows) and w2 [E, H, I] once:
    packed E2M1 [E, N, K/2] (int8 storage) plus the scale chunks the block-scaled kernel reads,
    [E, N/128, K/64, 128] int32.  `weight_scales` are the two layer-wide dequantisation factors."""
    if w1.ndim != 3 or w2.ndim != 3:
        raise ValueError("Expected canonical expert weights [E,2I,H] and [E,H,I]")
    experts, hidden, inter = w2.shape
    if tuple(w1.shape) != (experts, 2 * inter, hidden):
        raise ValueError("Expected canonical expert weights [E,2I,H] and [E,H,I]")
    if not (_is_device_bf16(w1) and _is_device_bf16(w2) and w1.device == w2.device):
        raise ValueError("Expected contiguous CUDA BF16 weights on the same device")
    if experts == 0 or hidden % 128 or inter % 128 or hidden == 0 or inter == 0 or len(weight_scales) != 2:
        raise ValueError("NVFP4 requires H and I divisible by 128 and two weight scales")
    _validate_scales(weight_scales)

    def pack(weight, scale):
        e, n, k = weight.shape
        data, chunks = quantize_nvfp4(weight.view(e * n, k), scale, chunked=True)
        return data.view(torch.int8).view(e, n, k // 2), chunks.view(e, n // 128, k // 64, 128)

    return NVFP4Weights(pack(w1, weight_scales[0]), pack(w2, weight_scales[1]), tuple(weight_scales))
