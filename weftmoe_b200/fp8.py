"""Blockwise E4M3 tensors and prepared (pre-quantised) expert weights for the FP8 path.

Public names, fields and error types follow the reference's FP8 module so that its callers and tests
read the same here (`FP8Tensor`, `quantize_fp8`, `transpose_fp8_weight`, `fp8_gemm`,
`PreparedFP8Weights`, `prepare_fp8_weights`: weftmoe/fp8.py:31-277); the numerics contract is the
reference's quantiser (src/cuda/fp8/quantization.cuh:35-81).  All arithmetic runs in libweftmoe_b200.so
through the `wm_fp8_*` entry points of include/weftmoe_b200.h; this file only lays out storage, checks
arguments and tracks weight versions.

Storage rules:
  * a logical matrix [M, K] is stored K-contiguous with K padded up to a multiple of 128;
  * one FP32 scale per [block_rows x 128] block (block_rows 1 for activations, 128 for weights); a
    stored byte times its block's scale is the represented value;
  * a leading batch axis (experts) separates independent quantisation domains.
"""
from __future__ import annotations

import weakref
from dataclasses import dataclass

import torch

from . import _lib

_BLOCK_K = 128
_SOURCE_DTYPES = (torch.bfloat16, torch.float32)


def _ceil_to(n: int, step: int) -> int:
    return -(-n // step) * step


def _storage_shapes(shape, block_rows):
    """(data shape, scale shape) of a logical [..., M, K] matrix."""
    *lead, m, k = shape
    return (*lead, m, _ceil_to(k, _BLOCK_K)), (*lead, -(-m // block_rows), -(-k // _BLOCK_K))


def _require_cuda(tensor, dtypes, what):
    ok = (isinstance(tensor, torch.Tensor) and tensor.is_cuda and tensor.is_contiguous()
          and tensor.dtype in dtypes and tensor.ndim in (2, 3))
    if not ok:
        names = " or ".join(str(d).replace("torch.", "") for d in dtypes)
        raise ValueError(f"{what}: expected a contiguous CUDA {names} tensor of rank 2 or 3")


@dataclass(frozen=True)
class FP8Tensor:
    """E4M3 bytes + FP32 block scales + the logical (unpadded) shape they describe."""
    data: torch.Tensor
    scales: torch.Tensor
    shape: tuple[int, ...]
    block_rows: int = 1

    def __post_init__(self):
        _require_cuda(self.data, (torch.float8_e4m3fn,), "FP8Tensor.data")
        _require_cuda(self.scales, (torch.float32,), "FP8Tensor.scales")
        dims_ok = len(self.shape) in (2, 3) and all(isinstance(n, int) and n >= 0 for n in self.shape)
        if not dims_ok or self.block_rows not in (1, 128):
            raise ValueError("Invalid FP8 logical shape or block_rows")
        want_data, want_scales = _storage_shapes(self.shape, self.block_rows)
        if tuple(self.data.shape) != want_data or tuple(self.scales.shape) != want_scales:
            raise ValueError("FP8 storage/scales do not match the logical matrix")
        if self.scales.device != self.data.device:
            raise ValueError("FP8 storage/scales do not match the logical matrix")

    @property
    def batches(self) -> int:
        return self.shape[0] if len(self.shape) == 3 else 1

    def matrix(self, expert: int) -> "FP8Tensor":
        """One expert's matrix of a batched tensor (a view, nothing is copied)."""
        if len(self.shape) != 3:
            raise ValueError("Only batched FP8 tensors have expert matrices")
        return FP8Tensor(self.data[expert], self.scales[expert], tuple(self.shape[1:]), self.block_rows)

    def dequantize(self) -> torch.Tensor:
        """FP32 values the tensor represents.  For tests and diagnostics only."""
        m, k = self.shape[-2:]
        per_row = self.scales.repeat_interleave(self.block_rows, dim=-2)[..., :m, :]
        per_elem = per_row.repeat_interleave(_BLOCK_K, dim=-1)
        return (self.data.float() * per_elem)[..., :k]


def _allocate(shape, block_rows, device) -> FP8Tensor:
    data_shape, scale_shape = _storage_shapes(shape, block_rows)
    return FP8Tensor(torch.empty(data_shape, dtype=torch.float8_e4m3fn, device=device),
                     torch.empty(scale_shape, dtype=torch.float32, device=device), tuple(shape), block_rows)


def _swap_last_two(shape):
    return (*shape[:-2], shape[-1], shape[-2])


def _source_args(tensor):
    """(pointer, is_fp32, batches, rows, cols) of a BF16/FP32 source for the C ABI."""
    batches = tensor.shape[0] if tensor.ndim == 3 else 1
    return _lib.ptr(tensor), int(tensor.dtype == torch.float32), batches, tensor.shape[-2], tensor.shape[-1]


def quantize_fp8(tensor: torch.Tensor, *, block_rows: int = 1, transpose: bool = False) -> FP8Tensor:
    """Quantise BF16/FP32 values.  With transpose=True the result is the K-contiguous TRANSPOSE, its
    blocks taken along the source's rows (the source itself is read once; an already quantised tensor
    is never re-quantised)."""
    _require_cuda(tensor, _SOURCE_DTYPES, "quantize_fp8")
    if block_rows not in (1, 128):
        raise ValueError("block_rows must be 1 or 128")
    logical = _swap_last_two(tuple(tensor.shape)) if transpose else tuple(tensor.shape)
    with torch.cuda.device(tensor.device):
        out = _allocate(logical, block_rows, tensor.device)
        stream = torch.cuda.current_stream()
        _lib.check(_lib.load().wm_fp8_quantize(*_source_args(tensor), block_rows, int(transpose),
                                               _lib.ptr(out.data), _lib.ptr(out.scales), stream.cuda_stream))
        tensor.record_stream(stream)
    return out


def _quantize_fp8_weight_pair(tensor: torch.Tensor) -> tuple[FP8Tensor, FP8Tensor]:
    """W and W^T with 128 x 128 blocks from one pass over the source: both orientations hold the same
    bytes and the same block scales (reference kernel: src/cuda/fp8/quantization.cuh:157-237)."""
    _require_cuda(tensor, _SOURCE_DTYPES, "weight quantisation")
    with torch.cuda.device(tensor.device):
        straight = _allocate(tuple(tensor.shape), 128, tensor.device)
        flipped = _allocate(_swap_last_two(tuple(tensor.shape)), 128, tensor.device)
        stream = torch.cuda.current_stream()
        _lib.check(_lib.load().wm_fp8_quantize_weight(
            *_source_args(tensor), _lib.ptr(straight.data), _lib.ptr(straight.scales),
            _lib.ptr(flipped.data), _lib.ptr(flipped.scales), stream.cuda_stream))
        tensor.record_stream(stream)
    return straight, flipped


def transpose_fp8_weight(weight: FP8Tensor) -> FP8Tensor:
    """Transpose a 128 x 128-block weight: bytes and scales move, no value changes."""
    if weight.block_rows != 128:
        raise ValueError("Rowwise activations require a new columnwise quantization")
    device = weight.data.device
    with torch.cuda.device(device):
        out = _allocate(_swap_last_two(tuple(weight.shape)), 128, device)
        stream = torch.cuda.current_stream()
        _lib.check(_lib.load().wm_fp8_transpose_weight(
            _lib.ptr(weight.data), _lib.ptr(weight.scales), weight.batches, weight.shape[-2], weight.shape[-1],
            _lib.ptr(out.data), _lib.ptr(out.scales), stream.cuda_stream))
        for t in (weight.data, weight.scales):
            t.record_stream(stream)
    return out


def fp8_gemm(a: FP8Tensor, b: FP8Tensor, *, dtype=torch.bfloat16, out: torch.Tensor | None = None,
             accumulate: bool = False) -> torch.Tensor:
    """Diagnostic A @ B^T (A [M,K], B [N,K]) on the block-scaled tensor cores; the layer itself uses the
    grouped kernels.  `accumulate` adds into an existing FP32 `out`."""
    two_d = len(a.shape) == 2 and len(b.shape) == 2
    if not two_d or a.shape[1] != b.shape[1] or a.data.device != b.data.device:
        raise ValueError("FP8 GEMM requires [M,K], [N,K] on the same device")
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("FP8 GEMM output dtype must be BF16 or FP32")
    if accumulate and (out is None or out.dtype != torch.float32):
        raise ValueError("FP8 accumulation requires an existing FP32 output")
    m, n, k = a.shape[0], b.shape[0], a.shape[1]
    device = a.data.device
    with torch.cuda.device(device):
        if out is None:
            out = torch.empty((m, n), dtype=dtype, device=device)
        else:
            fits = (tuple(out.shape) == (m, n) and out.dtype == dtype and out.device == device
                    and out.is_contiguous())
            if not fits:
                raise ValueError("FP8 output shape, dtype, device or layout mismatch")
        _lib.check(_lib.load().wm_fp8_gemm(
            _lib.ptr(a.data), _lib.ptr(a.scales), _lib.ptr(b.data), _lib.ptr(b.scales), _lib.ptr(out),
            m, n, k, a.block_rows, b.block_rows, int(dtype == torch.float32), int(accumulate),
            torch.cuda.current_stream().cuda_stream))
    return out


class _ParameterStamp:
    """Identity and in-place version of the parameter tensor a weight was prepared from."""
    __slots__ = ("ref", "version")

    def __init__(self, tensor):
        self.ref = weakref.ref(tensor)
        # inference tensors carry no version counter
        self.version = None if tensor.is_inference() else tensor._version

    def check(self, tensor):
        if self.ref() is not tensor:
            raise ValueError("FP8 cache was prepared from different parameters")
        if self.version is not None and tensor._version != self.version:
            raise RuntimeError("FP8 cache is stale after a parameter update; prepare new weights")


class PreparedFP8Weights:
    """One immutable version of the expert weights in every layout the layer reads: `w1`, `w2` for the
    forward GEMMs and, when prepared for training, `w1_t`, `w2_t` (same bytes, transposed) for dU / dX.

    After an optimizer step prepare a NEW object; tapes of earlier forwards keep the object they were
    made with.  Writing into any of the tensors afterwards is detected (`_validate_version`)."""

    __slots__ = ("w1", "w2", "w1_t", "w2_t", "version", "scale_mantissas", "_ready", "_stamps", "_origin",
                 "_wm_chunks", "_wm_chunks_t", "__weakref__")

    def __init__(self, w1, w2, w1_t, w2_t, version, origin=(), scale_mantissas=False):
        self.w1, self.w2, self.w1_t, self.w2_t = w1, w2, w1_t, w2_t
        self.version = version
        # True: some block scale is not a power of two (an imported checkpoint); the kernels then take
        # the FP32 scales beside the packed exponents and promote every K128 block in FP32.
        self.scale_mantissas = bool(scale_mantissas)
        self._origin = tuple(origin)            # _ParameterStamp or None per weight
        self._wm_chunks = self._wm_chunks_t = None   # packed scale chunks, filled lazily by the runtime
        with torch.cuda.device(w1.data.device):
            self._ready = torch.cuda.Event()
            self._ready.record()                # preparation kernels were enqueued on this stream
        self._stamps = tuple(t._version for t in self.tensors())

    def __setattr__(self, name, value):
        if name in ("w1", "w2", "w1_t", "w2_t", "version", "scale_mantissas") and hasattr(self, "_stamps"):
            raise AttributeError("PreparedFP8Weights is immutable; prepare a new weight version")
        object.__setattr__(self, name, value)

    def tensors(self):
        """Every device tensor held, data before scales, forward layouts first."""
        held = [w for w in (self.w1, self.w2, self.w1_t, self.w2_t) if w is not None]
        return tuple(t for w in held for t in (w.data, w.scales))

    _tensors = tensors

    def _validate_version(self, *, training: bool = False):
        if tuple(t._version for t in self.tensors()) != self._stamps:
            raise RuntimeError("Prepared FP8 weights were modified; prepare a new weight version")
        if training and (self.w1_t is None or self.w2_t is None):
            raise ValueError("Backward requires weights prepared with training=True")

    def wait(self, *, training: bool = False):
        """Order the current stream after the preparation kernels and keep the storage alive for it."""
        self._validate_version(training=training)
        with torch.cuda.device(self.w1.data.device):
            stream = torch.cuda.current_stream()
            stream.wait_event(self._ready)
            for t in self.tensors():
                t.record_stream(stream)

    def validate_parameters(self, w1, w2):
        """When prepared from trainable parameters: those must be the same, unmodified tensors."""
        for stamp, parameter in zip(self._origin, (w1, w2)):
            if stamp is not None:
                stamp.check(parameter)


def _import_quantised(weight: FP8Tensor) -> FP8Tensor:
    """Private copy of an already quantised weight (a checkpoint): bytes and scales are kept as they are."""
    if weight.block_rows != 128:
        raise ValueError("Expert weights require 128x128 quantization")
    with torch.cuda.device(weight.data.device):
        return FP8Tensor(weight.data.clone(), weight.scales.clone(), tuple(weight.shape), 128)


def _check_imported(weights) -> bool:
    """Imported bytes must be finite E4M3 and their scales finite and positive (one host sync).  Returns whether
    any scale carries a mantissa (is not a power of two).

    The block-scaled tensor-core kernels apply a scale's exponent INSIDE the MMA (UE8M0).  Weights whose
    scales have mantissas, as some checkpoints carry, are neither rounded nor quantised again: their FP32
    scales go to the kernels as well, which then promote every K128 block in FP32 by the mantissas (the
    reference's Hopper kernel promotes by the whole scale, src/cuda/fp8/gemm.cuh:68-70)."""
    if not weights:
        return False
    healthy, pow2 = [], []
    for w in weights:
        healthy.append((w.scales > 0).logical_and(torch.isfinite(w.scales)).all())
        healthy.append((w.data.view(torch.uint8).bitwise_and(0x7F) != 0x7F).all())   # 0x7f / 0xff = NaN
        pow2.append((w.scales.view(torch.int32).bitwise_and(0x007FFFFF) == 0).all())  # FP32 mantissa field empty
    findings = torch.stack([torch.stack(healthy).all(), torch.stack(pow2).all()]).tolist()
    if not findings[0]:
        raise ValueError("FP8 weights must be finite and scales finite and positive")
    return not findings[1]


@torch.inference_mode(False)
@torch.no_grad()
def prepare_fp8_weights(w1, w2, *, training: bool = True, version: int = 0) -> PreparedFP8Weights:
    """Quantise (or import) the expert weights once, outside forward/backward.

    w1 [E, 2I, H] (gate rows then up rows) and w2 [E, H, I] are BF16/FP32 tensors or FP8Tensors with
    128 x 128 blocks.  training=True also keeps W^T of each (same bytes and scales) for the backward
    data gradients."""
    if not isinstance(version, int) or isinstance(version, bool) or not 0 <= version < 1 << 64:
        raise ValueError("weight version must be an unsigned 64-bit integer")
    forward, backward, imported, origin = [], [], [], []
    for source in (w1, w2):
        if isinstance(source, FP8Tensor):
            q = _import_quantised(source)
            imported.append(q)
            qt = None
            origin.append(None)
        else:
            if training:
                q, qt = _quantize_fp8_weight_pair(source)
            else:
                q, qt = quantize_fp8(source, block_rows=128), None
            origin.append(_ParameterStamp(source))
        forward.append(q)
        backward.append(qt)
    a, b = forward
    consistent = (len(a.shape) == 3 and len(b.shape) == 3 and a.shape[0] == b.shape[0]
                  and a.shape[1] == 2 * b.shape[2] and a.shape[2] == b.shape[1]
                  and a.data.device == b.data.device and 0 not in (*a.shape, *b.shape)
                  and a.shape[2] % 128 == 0 and b.shape[2] % 128 == 0)
    if not consistent:
        raise ValueError("Expected W1 [E,2I,H], W2 [E,H,I], H/I multiples of 128")
    with torch.cuda.device(a.data.device):
        mantissas = _check_imported(imported)
        if training:
            backward = [qt if qt is not None else transpose_fp8_weight(q) for q, qt in zip(forward, backward)]
        else:
            backward = [None, None]
        return PreparedFP8Weights(a, b, backward[0], backward[1], version, origin, mantissas)
