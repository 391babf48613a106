"""GPU: blockwise FP8 quantisers through the C ABI — exact bytes and scales against the golden vectors
the reference's quant_reference produced (tests/test_fp8.py:20-36) and against the CPU oracle; the
zero / tiny / non-finite known answers (:53-63); weight pair == two independent quantisations (:80-95);
transpose preserves bits (:66-76)."""
import numpy as np
import pytest
import torch

from oracle import c_oracle
from weftmoe_b200 import _lib
from weftmoe_b200.fp8 import (FP8Tensor, _quantize_fp8_weight_pair, prepare_fp8_weights, quantize_fp8,
                              transpose_fp8_weight)

pytestmark = pytest.mark.gpu


def same(actual: FP8Tensor, q_ref, s_ref):
    assert torch.equal(actual.data.view(torch.uint8).cpu(), torch.as_tensor(q_ref))
    assert torch.equal(actual.scales.cpu(), torch.as_tensor(s_ref))


def test_reference_golden_bytes_and_scales(golden):
    for case in torch.load(golden / "fp8_quant.pt")["cases"]:
        actual = quantize_fp8(case["x"].cuda(), block_rows=case["block_rows"], transpose=case["transpose"])
        same(actual, case["q"], case["scales"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 1), (67, 259), (2, 129, 257), (3, 256, 384), (1000, 2048)])
@pytest.mark.parametrize("block_rows,transpose", [(1, False), (1, True), (128, False), (128, True)])
def test_matches_cpu_oracle(dtype, shape, block_rows, transpose):
    torch.manual_seed(12)
    x = torch.randn(shape, dtype=dtype)
    x[..., 0, 0] = 0
    x[..., -1, -1] = 87
    q, s = c_oracle.fp8_quantize(x.float().numpy(), block_rows, transpose)
    same(quantize_fp8(x.cuda(), block_rows=block_rows, transpose=transpose), q, s)


def test_zero_small_and_nonfinite(golden):
    x = torch.load(golden / "fp8_quant.pt")["special"]["x"].cuda()
    actual = quantize_fp8(x)
    assert torch.equal(actual.scales[0], torch.ones_like(actual.scales[0]))
    assert actual.scales[1, 0] == torch.finfo(torch.float32).tiny
    torch.testing.assert_close(actual.dequantize()[1], x[1], rtol=0, atol=0)
    assert actual.scales[2:, 0].isnan().all()
    assert torch.equal(actual.scales[2:, 1], torch.ones_like(actual.scales[2:, 1]))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 3), (129, 257), (2, 131, 270), (2, 256, 384), (0, 128), (128, 0), (0, 128, 256)])
def test_weight_pair_matches_independent_quantization(dtype, shape):
    torch.manual_seed(42)
    x = torch.randn(shape, dtype=dtype)
    if x.numel():
        x[..., :128, :128] *= 16
        x[..., -1, -1] = -87
    row, column = _quantize_fp8_weight_pair(x.cuda())
    if not x.numel():
        assert row.data.numel() == column.data.numel() == 0
        return
    for actual, transpose in ((row, False), (column, True)):
        q, s = c_oracle.fp8_quantize(x.float().numpy(), 128, transpose)
        same(actual, q, s)


@pytest.mark.parametrize("shape", [(1, 3), (129, 257), (2, 131, 270)])
def test_weight_transpose_preserves_quantization(shape):
    x = torch.randn(shape, device="cuda", dtype=torch.bfloat16)
    q = quantize_fp8(x, block_rows=128)
    qt = transpose_fp8_weight(q)
    torch.testing.assert_close(qt.dequantize(), q.dequantize().transpose(-1, -2), rtol=0, atol=0)
    back = transpose_fp8_weight(qt)
    assert torch.equal(back.data.view(torch.uint8), q.data.view(torch.uint8)) and torch.equal(back.scales, q.scales)


def test_columnwise_quantization_is_not_a_transposed_rowwise_cast():
    x = torch.randn(129, 128, device="cuda")
    x[0] *= 1000
    row, col = quantize_fp8(x), quantize_fp8(x, transpose=True)
    assert col.shape == (128, 129) and col.scales.shape == (128, 2)
    assert not torch.equal(col.dequantize(), row.dequantize().T)


def test_native_validation_and_prepared_weights():
    x = torch.randn(128, 128, device="cuda", dtype=torch.bfloat16)
    row, column = _quantize_fp8_weight_pair(x)
    lib = _lib.load()
    rc = lib.wm_fp8_quantize_weight(_lib.ptr(x), 0, 1, 128, 128, _lib.ptr(row.data), _lib.ptr(row.scales),
                                    _lib.ptr(row.data), _lib.ptr(column.scales), None)
    assert rc == _lib.WM_ERR_INVALID and "alias" in _lib.last_error()
    unaligned = torch.empty(128 * 128 + 1, device="cuda", dtype=torch.uint8)[1:]
    rc = lib.wm_fp8_quantize_weight(_lib.ptr(x), 0, 1, 128, 128, _lib.ptr(unaligned), _lib.ptr(row.scales),
                                    _lib.ptr(column.data), _lib.ptr(column.scales), None)
    assert rc == _lib.WM_ERR_INVALID and "aligned" in _lib.last_error()
    w1 = torch.randn(4, 512, 256, device="cuda", dtype=torch.bfloat16) * 0.02
    w2 = torch.randn(4, 256, 256, device="cuda", dtype=torch.bfloat16) * 0.02
    prepared = prepare_fp8_weights(w1, w2)
    assert prepared.w1.shape == (4, 512, 256) and prepared.w1_t.shape == (4, 256, 512)
    torch.testing.assert_close(prepared.w1_t.dequantize(), prepared.w1.dequantize().transpose(-1, -2), rtol=0, atol=0)
    prepared.validate_parameters(w1, w2)
    w1.add_(1)
    with pytest.raises(RuntimeError, match="stale"):
        prepared.validate_parameters(w1, w2)
    prepared.w2.scales.mul_(2)
    with pytest.raises(RuntimeError, match="modified"):
        prepared.wait()
    with pytest.raises(ValueError):
        prepare_fp8_weights(w1[:, :, :100].contiguous(), w2)


def global_diff(actual, expected):
    """The reference's FP8 acceptance metric (benchmarks/fp8_validation.py:23-35)."""
    a, b = actual.double(), expected.double()
    den = (a.square() + b.square()).sum().item()
    return ((a - b).square().sum().item() / den) if den else 0.0


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (65, 137, 259), (128, 256, 4096), (300, 640, 1024),
                                   (0, 64, 128), (64, 0, 128), (3, 9, 0)])
@pytest.mark.parametrize("b_block_rows", [1, 128])
def test_gemm(m, n, k, b_block_rows):
    """tests/test_fp8.py:146-168 of the reference: different scales per K block, M/N/K tails,
    diff < 1e-6 against the dequantised FP64 product and < 5e-3 against the original operands."""
    from weftmoe_b200.fp8 import fp8_gemm
    torch.manual_seed(1234)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    if k:
        a[:, :min(128, k)] *= 4
        b[:, :min(128, k)] *= 0.0625
    aq, bq = quantize_fp8(a), quantize_fp8(b, block_rows=b_block_rows)
    expected = aq.dequantize().double() @ bq.dequantize().double().T
    original = a.double() @ b.double().T
    actual = fp8_gemm(aq, bq, dtype=torch.float32)
    assert global_diff(actual, expected) < 1e-6 and global_diff(actual, original) < 5e-3
    out = torch.full((m, n), 0.5, device="cuda", dtype=torch.float32)
    fp8_gemm(aq, bq, dtype=torch.float32, out=out, accumulate=True)
    assert global_diff(out, expected + 0.5) < 1e-6
    assert torch.equal(fp8_gemm(aq, bq), actual.bfloat16())


@pytest.mark.parametrize("m,n,k", [(65, 137, 259), (128, 256, 4096), (300, 640, 1024)])
@pytest.mark.parametrize("a_block_rows", [1, 128])
def test_gemm_with_scales_that_are_not_powers_of_two(m, n, k, a_block_rows):
    """Scales with mantissas (imported checkpoints: the reference multiplies them by 1.125 / 0.875,
    tests/torchrun_fp8.py:235-255) are neither rounded nor re-quantised: the product equals the dequantised
    FP64 product of the same bytes and the scaled scales, and differs from the power-of-two result."""
    from weftmoe_b200.fp8 import fp8_gemm
    torch.manual_seed(4321)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    aq, bq = quantize_fp8(a, block_rows=a_block_rows), quantize_fp8(b, block_rows=128)
    # a different mantissa per block, so that a wrong (row, K block) index shows
    fa = 1.0 + torch.rand_like(aq.scales) * 0.9
    fb = 1.0 + torch.rand_like(bq.scales) * 0.9
    aq2 = FP8Tensor(aq.data, (aq.scales * fa).contiguous(), tuple(aq.shape), a_block_rows)
    bq2 = FP8Tensor(bq.data, (bq.scales * fb).contiguous(), tuple(bq.shape), 128)
    for left, right in ((aq, bq2), (aq2, bq2), (aq2, bq)):
        expected = left.dequantize().double() @ right.dequantize().double().T
        actual = fp8_gemm(left, right, dtype=torch.float32)
        assert global_diff(actual, expected) < 1e-6
        out = torch.full((m, n), 0.5, device="cuda", dtype=torch.float32)
        fp8_gemm(left, right, dtype=torch.float32, out=out, accumulate=True)
        assert global_diff(out, expected + 0.5) < 1e-6
    assert global_diff(fp8_gemm(aq, bq2, dtype=torch.float32), fp8_gemm(aq, bq, dtype=torch.float32)) > 1e-3
    with pytest.raises(ValueError, match="128 x 128"):
        fp8_gemm(aq, FP8Tensor(quantize_fp8(b).data, quantize_fp8(b).scales * 1.125, tuple(b.shape), 1))
