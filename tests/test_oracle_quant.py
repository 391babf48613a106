"""CPU: the C quantiser oracle against golden vectors produced by the reference's own
quant_reference (tests/test_fp8.py:20-36) and round_nvfp4_blocks (tests/torchrun_sm100_nvfp4.py:13-27)."""
import ctypes

import numpy as np
import torch

from oracle import c_oracle


def test_fp8_quantiser_bytes_and_scales(golden):
    data = torch.load(golden / "fp8_quant.pt")
    for case in data["cases"]:
        x = case["x"].float().numpy()
        q, s = c_oracle.fp8_quantize(x, case["block_rows"], case["transpose"])
        ref_q = case["q"].numpy()
        assert q.shape[-2] == ref_q.shape[-2]
        assert np.array_equal(q[..., : ref_q.shape[-1]], ref_q), (x.shape, case["block_rows"], case["transpose"])
        assert np.array_equal(s, case["scales"].numpy())


def test_fp8_zero_tiny_nonfinite(golden):
    """Known answers of tests/test_fp8.py:53-63."""
    special = torch.load(golden / "fp8_quant.pt")["special"]
    x = special["x"].numpy()
    q, s = c_oracle.fp8_quantize(x, 1, False)
    assert (s[0] == 1.0).all()
    assert s[1, 0] == np.float32(special["tiny"])
    lib = c_oracle.lib()
    lib.wm_oracle_e4m3_to_f32.restype = ctypes.c_float
    row = np.array([lib.wm_oracle_e4m3_to_f32(int(b)) for b in q[1, :256]], np.float32)
    scale = np.repeat(s[1], 128)
    assert np.array_equal(row * scale, x[1])
    assert np.isnan(s[2:, 0]).all()
    assert (s[2:, 1] == 1.0).all()


def test_e4m3_matches_torch_cast():
    vals = torch.cat([torch.linspace(-448, 448, 20001), torch.randn(20000) * 3, torch.randn(5000) * 0.01,
                      torch.tensor([0.0, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -9, 447.9, 448.0])])
    ref = vals.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    lib = c_oracle.lib()
    mine = np.array([lib.wm_oracle_e4m3(float(v)) for v in vals.numpy()], np.uint8)
    assert np.array_equal(mine & 0x7f, ref & 0x7f)  # sign of zero is not compared
    nz = vals.numpy() != 0
    assert np.array_equal(mine[nz], ref[nz])


def test_nvfp4_rounding_matches_reference(golden):
    data = torch.load(golden / "nvfp4_round.pt")
    for case in data["cases"]:
        x = case["x"].float().numpy()
        _, _, rounded = c_oracle.nvfp4_quantize(x, case["scale"])
        assert np.array_equal(rounded, case["rounded"].numpy()), case["scale"]


def test_nvfp4_midpoint_known_answer(golden):
    """Byte-exact case of tests/torchrun_sm100_nvfp4_backward.py:29-45."""
    mid = torch.load(golden / "nvfp4_round.pt")["midpoint"]
    packed, sf, _ = c_oracle.nvfp4_quantize(mid["x"].float().numpy(), mid["scale"])
    assert (sf == mid["sf_byte"]).all()
    assert np.array_equal(packed, mid["packed"].numpy())


def test_nvfp4_midpoint_known_answer_holds_in_both_orientations(golden):
    """tests/torchrun_sm100_nvfp4_backward.py:29-45 checks the same block both along the columns and along
    the rows (the weight-gradient operands are quantised along the rows): in the transposed matrix every
    16-block again holds the maximum 0.1171875, so the scale byte is E4M3(0.75) and the codes are the
    transpose of the row-wise codes (7 = 6.0 everywhere, 2 = 1.0 at rows 0 mod 4 x odd columns)."""
    mid = torch.load(golden / "nvfp4_round.pt")["midpoint"]
    x = mid["x"].float()
    assert x.shape == (128, 128)
    packed_t, sf_t, _ = c_oracle.nvfp4_quantize(x.T.contiguous().numpy(), mid["scale"])
    assert (sf_t == mid["sf_byte"]).all()
    codes = torch.full((128, 128), 7, dtype=torch.uint8)
    codes[::4, 1::2] = 2
    expected = codes.T.contiguous()
    assert np.array_equal(packed_t, (expected[:, ::2] | (expected[:, 1::2] << 4)).numpy())
