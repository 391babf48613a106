"""GPU: each tcgen05 grouped GEMM form against a torch FP32 matmul of the same operands."""
import pytest
import torch

from tests.gpu_util import grouped_gemm, rel_l2
from weftmoe_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 1], ids=["one_cta", "cta_pair"], autouse=True)
def kernel_choice(request):
    """Every case runs on the one-CTA kernel and on the CTA-pair (cta_group::2) kernel."""
    lib = _lib.load()
    lib.wm_debug_force_gemm_pairs(request.param)
    yield request.param
    lib.wm_debug_force_gemm_pairs(-1)


TOL = 4e-3  # one BF16 rounding of an FP32-accumulated result (2^-9 relative) plus slack


def starts(rows):
    s = [0]
    for r in rows:
        s.append(s[-1] + r)
    return s


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("n,k,rows", [(512, 256, [256, 128, 384]), (384, 1024, [128, 0, 256]), (2048, 512, [128] * 5)])
def test_m_grouped(kind, n, k, rows):
    torch.manual_seed(kind + n)
    dev = torch.device("cuda")
    groups, total, st = len(rows), sum(rows), starts(rows)
    a = torch.randn(total, k, device=dev).bfloat16()
    b = (torch.randn(groups, n, k, device=dev) if kind == 0 else torch.randn(groups, k, n, device=dev)).bfloat16()
    out = torch.full((total, n), 7.0, device=dev).bfloat16()
    grouped_gemm(kind, a, b, out, rows, n, k)
    for g in range(groups):
        if rows[g] == 0:
            continue
        sl = slice(st[g], st[g + 1])
        ref = a[sl].float() @ (b[g].float().T if kind == 0 else b[g].float())
        assert rel_l2(out[sl], ref) < TOL


@pytest.mark.parametrize("m,n,rows", [(256, 512, [256, 128, 384]), (1024, 2048, [128, 0, 256]), (128, 384, [0, 0, 128])])
def test_k_grouped_weight_gradient_form(m, n, rows):
    torch.manual_seed(m)
    dev = torch.device("cuda")
    groups, total, st = len(rows), sum(rows), starts(rows)
    a = torch.randn(total, m, device=dev).bfloat16()
    b = torch.randn(total, n, device=dev).bfloat16()
    out = torch.full((groups, m, n), 7.0, device=dev).bfloat16()
    grouped_gemm(2, a, b, out, rows, n, m)
    for g in range(groups):
        sl = slice(st[g], st[g + 1])
        if rows[g] == 0:
            assert (out[g] == 0).all()  # an idle expert gets an exactly zero gradient
        else:
            assert rel_l2(out[g], a[sl].float().T @ b[sl].float()) < TOL


def test_fc1_swiglu_epilogue():
    torch.manual_seed(5)
    dev = torch.device("cuda")
    rows, inter, hidden = [256, 128, 384], 256, 512
    total, st = sum(rows), starts(rows)
    a = torch.randn(total, hidden, device=dev).bfloat16()
    b = (torch.randn(len(rows), 2 * inter, hidden, device=dev) * 0.05).bfloat16()
    prob = torch.rand(total, device=dev)
    u = torch.empty(total, inter, device=dev, dtype=torch.bfloat16)
    ab = torch.empty(total, 2 * inter, device=dev, dtype=torch.bfloat16)
    grouped_gemm(3, a, b, u, rows, inter, hidden, aux=ab, prob=prob)
    for g in range(len(rows)):
        sl = slice(st[g], st[g + 1])
        full = (a[sl].float() @ b[g].float().T).bfloat16().float()
        assert rel_l2(ab[sl], full) < TOL
        ref = torch.nn.functional.silu(full[:, :inter]) * full[:, inter:] * prob[sl, None]
        assert rel_l2(u[sl], ref) < 2 * TOL


def test_row_bits_do_not_depend_on_position_or_neighbours():
    """Batch invariance of the contraction: the same A row gives the same output bits wherever it sits."""
    torch.manual_seed(9)
    dev = torch.device("cuda")
    n, k = 512, 1024
    a = torch.randn(384, k, device=dev).bfloat16()
    b = torch.randn(1, n, k, device=dev).bfloat16()
    out = torch.empty(384, n, device=dev, dtype=torch.bfloat16)
    grouped_gemm(0, a, b, out, [384], n, k)
    perm = torch.randperm(384, device=dev)
    out2 = torch.empty_like(out)
    grouped_gemm(0, a[perm].contiguous(), b, out2, [384], n, k)
    assert torch.equal(out[perm].view(torch.int16), out2.view(torch.int16))
    out3 = torch.empty(128, n, device=dev, dtype=torch.bfloat16)
    grouped_gemm(0, a[:128].contiguous(), b, out3, [128], n, k)
    assert torch.equal(out[:128].view(torch.int16), out3.view(torch.int16))


def test_device_timeline_diagnostic_prints_the_stamps(kernel_choice):
    """WM_DEBUG_TIMELINE=<launcher> makes the one-CTA kernel stamp %globaltimer per tile and the
    launcher print them; the GEMM result is unaffected.  Run in a child process to read its stderr."""
    if kernel_choice:
        pytest.skip("the timeline covers the one-CTA kernel")
    import os
    import subprocess
    import sys
    code = (
        "import torch\n"
        "from tests.gpu_util import grouped_gemm\n"
        "from weftmoe_b200 import _lib\n"
        "_lib.load().wm_debug_force_gemm_pairs(0)\n"
        "a = torch.randn(256, 256, device='cuda').bfloat16()\n"
        "b = torch.randn(1, 512, 256, device='cuda').bfloat16()\n"
        "out = torch.empty(256, 512, device='cuda', dtype=torch.bfloat16)\n"
        "grouped_gemm(0, a, b, out, [256], 512, 256)\n"
        "ref = a.float() @ b[0].float().T\n"
        "print('rel', ((out.float() - ref).norm() / ref.norm()).item())\n")
    env = dict(os.environ, WM_DEBUG_TIMELINE="nt", WM_DEBUG_TIMELINE_CTA="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True,
                         timeout=300)
    assert run.returncode == 0, run.stderr
    assert float(run.stdout.split("rel")[1]) < TOL
    assert "[nt] CTA starts within" in run.stderr
    rows = [l for l in run.stderr.splitlines() if l.strip().startswith("0 |")]
    assert rows, run.stderr   # CTA 1 handled one tile (4 tiles over the grid) and stamped it
    stamps = [int(v) for v in rows[0].replace("|", " ").split()[1:]]
    assert len(stamps) == 12 and stamps[3] >= stamps[2] >= 0   # producer: last stage after first stage


def test_cta_pair_and_one_cta_kernels_give_the_same_bits():
    """The kernel choice depends on the batch (pairs where experts average many rows), so the two kernels
    must agree bit for bit for the forward contractions: same K order, same UMMA_K, a row's accumulator only
    sees that row, whichever way the tile is split over CTAs."""
    lib = _lib.load()
    torch.manual_seed(5)
    dev = torch.device("cuda")
    rows, n, k = [384, 128, 256], 512, 1024
    total = sum(rows)
    a = torch.randn(total, k, device=dev).bfloat16()
    results = {}
    try:
        for mode in (0, 1):
            lib.wm_debug_force_gemm_pairs(mode)
            b = torch.randn(len(rows), n, k, device=dev, generator=torch.Generator(device=dev).manual_seed(1)).bfloat16()
            out = torch.empty(total, n, device=dev, dtype=torch.bfloat16)
            grouped_gemm(0, a, b, out, rows, n, k)                                  # FC2 form
            w1 = torch.randn(len(rows), 2 * 256, k, device=dev, generator=torch.Generator(device=dev).manual_seed(2)).bfloat16()
            u = torch.empty(total, 256, device=dev, dtype=torch.bfloat16)
            ab = torch.empty(total, 512, device=dev, dtype=torch.bfloat16)
            prob = torch.rand(total, device=dev, generator=torch.Generator(device=dev).manual_seed(3))
            grouped_gemm(3, a, w1, u, rows, 256, k, aux=ab, prob=prob)              # FC1 + SwiGLU form
            results[mode] = (out, u, ab)
    finally:
        lib.wm_debug_force_gemm_pairs(-1)
    for single, pair in zip(results[0], results[1]):
        assert torch.equal(single.view(torch.int16), pair.view(torch.int16))
