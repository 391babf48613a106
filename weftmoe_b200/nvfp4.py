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
    if any(not math.isfinite(s) or s <= 0 for s in scales):
        raise ValueError("NVFP4 tensor scales must be finite and positive")


def nvfp4_block_stats(tensor, scale):
    """Count finite-input block-16 scale range events along the last (reduction) axis."""
    _validate_scales((scale,))
    if not tensor.is_floating_point() or tensor.ndim == 0 or tensor.shape[-1] % 16:
        raise ValueError("Expected floating-point data with a last dimension divisible by 16")
    amax = tensor.detach().unflatten(-1, (-1, 16)).abs().amax(dim=-1).float()
    unrounded = amax / (6.0 * scale)
    encoded = unrounded.clamp(max=448).to(torch.float8_e4m3fn).float()
    return {
        "blocks": amax.numel(),
        "nonzero_to_zero": ((amax > 0) & (encoded == 0)).sum(),
        "subnormal_scale": ((encoded > 0) & (encoded < 2 ** -6)).sum(),
        "above_range": (unrounded > 448).sum(),
    }


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


def prepare_nvfp4_weights(w1, w2, *, weight_scales=(1 / 64, 1 / 64)):
    """Quantize canonical BF16 expert weights. Scales are layer-wide dequantization factors."""
    if w1.ndim != 3 or w2.ndim != 3 or w1.shape != (w2.shape[0], 2 * w2.shape[2], w2.shape[1]):
        raise ValueError("Expected canonical expert weights [E,2I,H] and [E,H,I]")
    if w1.device != w2.device or any(not w.is_cuda or w.dtype != torch.bfloat16 or not w.is_contiguous()
                                     for w in (w1, w2)):
        raise ValueError("Expected contiguous CUDA BF16 weights on the same device")
    if min(w1.shape) <= 0 or len(weight_scales) != 2 or w1.shape[1] % 256 or w1.shape[2] % 128:
        raise ValueError("NVFP4 requires H and I divisible by 128 and two weight scales")
    _validate_scales(weight_scales)
    matrices = []
    for w, scale in zip((w1, w2), weight_scales):
        e, n, k = w.shape
        data, sf = quantize_nvfp4(w.view(e * n, k), scale, chunked=True)
        matrices.append((data.view(torch.int8).view(e, n, k // 2), sf.view(e, n // 128, k // 64, 128)))
    return NVFP4Weights(*matrices, tuple(weight_scales))
