"""GPU: NVFP4 quantiser and block-scaled GEMM through the C ABI against the golden vectors produced by
the reference's round_nvfp4_blocks (tests/torchrun_sm100_nvfp4.py:13-27), the byte-exact midpoint case
(tests/torchrun_sm100_nvfp4_backward.py:29-45) and the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import c_oracle
from weftmoe_b200 import _lib

pytestmark = pytest.mark.gpu
MAG = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def quantize(x, scale, chunked=False):
    rows, cols = x.shape
    data = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
    n_sf = ((rows + 127) // 128) * (cols // 64) * 512 if chunked else rows * (cols // 16)
    sf = torch.empty(n_sf, dtype=torch.uint8, device=x.device)
    _lib.check(_lib.load().wm_nvfp4_quantize(_lib.ptr(x), rows, cols, scale, _lib.ptr(data), _lib.ptr(sf),
                                             int(chunked), None))
    return data, sf if chunked else sf.view(rows, cols // 16)


def decode(data, sf):
    """value * block scale (without the layer scale), like round_nvfp4_blocks returns."""
    d = data.cpu().long()
    nib = torch.stack([d & 15, d >> 4], dim=-1).flatten(-2)
    val = MAG[nib & 7] * torch.where((nib & 8) > 0, -1.0, 1.0)
    scale = sf.cpu().view(torch.float8_e4m3fn).float().repeat_interleave(16, -1)
    return val * scale


def test_rounding_matches_reference_golden(golden):
    data = torch.load(golden / "nvfp4_round.pt")
    for case in data["cases"]:
        x = case["x"]
        if x.shape[1] % 16:
            continue
        q, sf = quantize(x.cuda().contiguous(), case["scale"])
        assert torch.equal(decode(q, sf), case["rounded"]), case["scale"]


def test_midpoint_known_answer_bytes(golden):
    mid = torch.load(golden / "nvfp4_round.pt")["midpoint"]
    q, sf = quantize(mid["x"].cuda(), mid["scale"])
    assert (sf.cpu() == mid["sf_byte"]).all()
    assert torch.equal(q.cpu(), mid["packed"])


@pytest.mark.parametrize("rows,cols,scale", [(1, 64, 1 / 32), (200, 512, 1 / 64), (384, 3072, 1 / 4), (130, 1024, 0.025)])
def test_matches_cpu_oracle_and_chunked_layout(rows, cols, scale):
    torch.manual_seed(rows)
    x = (torch.randn(rows, cols) * (scale * 8)).bfloat16()
    x[0, :16] = 0
    packed, sf, _ = c_oracle.nvfp4_quantize(x.float().numpy(), scale)
    q, s = quantize(x.cuda(), scale)
    assert np.array_equal(q.cpu().numpy(), packed) and np.array_equal(s.cpu().numpy(), sf)
    q2, chunks = quantize(x.cuda(), scale, chunked=True)
    assert torch.equal(q2, q)
    chunks = chunks.cpu().numpy()
    k64 = cols // 64
    r = np.arange(rows)[:, None]
    g = np.arange(cols // 16)[None, :]
    off = (((r // 128) * k64 + g // 4) * 128 + (r % 32) * 4 + (r % 128) // 32) * 4 + g % 4
    assert np.array_equal(chunks[off], sf)


@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (200, 384, 1024), (64, 1024, 3072), (130, 256, 320)])
def test_gemm_against_reference_formula(m, n, k):
    """reference_gemm (tests/torchrun_sm100_nvfp4.py:30-33): (round(a) @ round(b).T) * (sa * sb)."""
    torch.manual_seed(m + k)
    sa, sb = 1 / 32, 1 / 64
    a = (torch.randn(m, k) * 0.16).bfloat16()
    b = (torch.randn(n, k) * 0.023).bfloat16()
    ra = c_oracle.nvfp4_quantize(a.float().numpy(), sa)[2]
    rb = c_oracle.nvfp4_quantize(b.float().numpy(), sb)[2]
    expected = torch.from_numpy(ra).double() @ torch.from_numpy(rb).double().T * (sa * sb)
    aq, asf = quantize(a.cuda(), sa)
    bq, bsf = quantize(b.cuda(), sb)
    out = torch.empty(m, n, dtype=torch.float32, device="cuda")
    _lib.check(_lib.load().wm_nvfp4_gemm(_lib.ptr(aq), _lib.ptr(asf), _lib.ptr(bq), _lib.ptr(bsf), _lib.ptr(out),
                                         m, n, k, sa * sb, 1, None))
    err = ((out.cpu().double() - expected).norm() / expected.norm()).item()
    assert err < 1e-5, err
