"""tcgen05 NVFP4 GEMM on a B200 against the fp32 oracle."""
import pytest
import torch

from tilerl_b200 import formats as F
from tilerl_b200.ops import ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from tilerl_b200.ops.cuda import CudaOps
    return CudaOps(DEV)


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9))


def _w(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    return F.quantize_nvfp4(torch.randn(n, k, generator=g) * 0.02).to(DEV)


def test_scale_tiling_layout():
    from tilerl_b200.ops.gemm_tc import tile_scales
    r, k = 130, 512
    s = torch.arange(r * (k // 16), dtype=torch.int32).remainder(251).to(torch.uint8).view(r, k // 16)
    t = tile_scales(s.view(torch.float8_e4m3fn), k).flatten()
    kt4 = 2 * 4
    for row, kb in ((0, 0), (5, 3), (33, 4), (127, 31), (129, 17)):
        off = ((row // 128) * kt4 + kb // 4) * 512 + (row % 32) * 16 + ((row % 128) // 32) * 4 + kb % 4
        assert int(t[off]) == int(s[row, kb])


def test_quant_act_matches_dequant_sum(ops):
    """The J quantised terms, dequantised and summed, reproduce the activation."""
    from tilerl_b200.ops.gemm_tc import quant_act
    g = torch.Generator().manual_seed(0)
    t, k = 3, 1024
    x = (torch.randn(t, k, generator=g) * 3).to(DEV, torch.bfloat16)
    for terms, tol in ((1, 0.12), (2, 0.02), (4, 1.5e-3)):
        xq, sfx, rs = quant_act(ops, x, k, terms)
        torch.cuda.synchronize()
        cols = t * terms
        kt4 = (k // 256) * 4
        sf = torch.empty(cols, k // 16, dtype=torch.uint8)
        flat = sfx.cpu()
        for c in range(cols):
            for kb in range(k // 16):
                off = ((c // 128) * kt4 + kb // 4) * 512 + (c % 32) * 16 + ((c % 128) // 32) * 4 + kb % 4
                sf[c, kb] = flat[off]
        deq = F.dequantize_act_nvfp4(xq.cpu(), sf.view(torch.float8_e4m3fn), rs.cpu())
        rec = deq.view(t, terms, k).sum(1)
        assert _rel(rec, x.cpu()) < tol, (terms, _rel(rec, x.cpu()))


@pytest.mark.parametrize("t,n,k,terms", [
    (1, 256, 512, 4), (1, 5120, 6144, 4), (3, 384, 2176, 4), (8, 1024, 5120, 2),
    (16, 200, 1024, 1), (100, 640, 1536, 1), (300, 512, 768, 1), (512, 1024, 5120, 1),
])
def test_gemm_nvfp4_plain(ops, t, n, k, terms):
    from tilerl_b200.ops.gemm_tc import gemm_nvfp4
    from tilerl_b200.ops import native
    w = _w(n, k, n + k)
    x = (torch.randn(t, k, generator=torch.Generator().manual_seed(t)) * 2).to(DEV, torch.bfloat16)
    y = torch.zeros(t, n, dtype=torch.bfloat16, device=DEV)
    gemm_nvfp4(ops, x, w, y, terms=terms)
    torch.cuda.synchronize()
    assert native.read_error()[0] == 0
    want = ref.linear(x, w)
    tol = {1: 0.14, 2: 0.03, 4: 7e-3}[terms]
    assert _rel(y, want) < tol, _rel(y, want)
    # second launch on the same scratch: the kernel must have left it zeroed
    y2 = torch.zeros_like(y)
    gemm_nvfp4(ops, x, w, y2, terms=terms)
    torch.cuda.synchronize()
    assert torch.equal(y, y2)


def test_gemm_nvfp4_exact_against_dequantised_operands(ops):
    """With J = 1 the kernel must equal deq(xq) @ deq(w)^T up to fp32 summation order:
    this pins every layout (nibbles, scale tiling, swizzle, TMEM mapping)."""
    from tilerl_b200.ops.gemm_tc import gemm_nvfp4, quant_act
    t, n, k = 40, 384, 1024
    w = _w(n, k, 7)
    x = (torch.randn(t, k, generator=torch.Generator().manual_seed(3)) * 2).to(DEV, torch.bfloat16)
    y = torch.zeros(t, n, dtype=torch.float32, device=DEV)
    gemm_nvfp4(ops, x, w, y, terms=1, epi=3)
    xq, sfx, rs = quant_act(ops, x, k, 1)
    torch.cuda.synchronize()
    kt4 = (k // 256) * 4
    flat = sfx.cpu()
    sf = torch.empty(t, k // 16, dtype=torch.uint8)
    for c in range(t):
        for kb in range(k // 16):
            sf[c, kb] = flat[((c // 128) * kt4 + kb // 4) * 512 + (c % 32) * 16 + ((c % 128) // 32) * 4 + kb % 4]
    xd = F.dequantize_act_nvfp4(xq.cpu(), sf.view(torch.float8_e4m3fn), rs.cpu())
    want = xd.double() @ w.dequant().cpu().double().t()
    assert _rel(y.cpu().double(), want) < 2e-5


def test_gemm_nvfp4_epilogues_and_fused_norm(ops):
    from tilerl_b200.ops.gemm_tc import gemm_nvfp4
    g = torch.Generator().manual_seed(11)
    t, n, k = 5, 1024, 2048
    w = _w(n, k, 3)
    x = (torch.randn(t, k, generator=g) * 4).to(DEV, torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(k, generator=g)).to(DEV)
    h = ref.rmsnorm(x, nw, 1e-6).to(torch.bfloat16)
    y = torch.zeros(t, n, dtype=torch.bfloat16, device=DEV)
    gemm_nvfp4(ops, x, w, y, terms=4, norm_w=nw, eps=1e-6)
    assert _rel(y, ref.linear(h, w)) < 7e-3
    res = torch.randn(t, n, generator=g).to(DEV, torch.bfloat16)
    out = res.clone()
    gemm_nvfp4(ops, x, w, out, terms=4, residual=out, epi=1)
    assert _rel(out, ref.linear(x, w, res)) < 7e-3
    act = torch.zeros(t, n // 2, dtype=torch.bfloat16, device=DEV)
    gemm_nvfp4(ops, x, w, act, terms=4, norm_w=nw, eps=1e-6, epi=2)
    assert _rel(act, ref.swiglu(ref.linear(h, w))) < 1.2e-2
    # SwiGLU folded into the quantiser of the next projection
    w2 = _w(256, n // 2, 5)
    gu = ref.linear(h, w).to(torch.bfloat16)
    y2 = torch.zeros(t, 256, dtype=torch.bfloat16, device=DEV)
    gemm_nvfp4(ops, gu, w2, y2, terms=4, swiglu_in=True)
    assert _rel(y2, ref.linear(ref.swiglu(gu).to(torch.bfloat16), w2)) < 7e-3
    # forced split-K (few CTAs -> partial tiles reduced through the scratch buffer)
    y3 = torch.zeros(t, n, dtype=torch.bfloat16, device=DEV)
    gemm_nvfp4(ops, x, w, y3, terms=4, norm_w=nw, eps=1e-6, max_ctas=3)
    assert _rel(y3, ref.linear(h, w)) < 7e-3
    from tilerl_b200.ops import native
    torch.cuda.synchronize()
    assert native.read_error()[0] == 0


@pytest.mark.parametrize("outliers", [False, True])
def test_two_residual_terms_are_at_least_as_accurate_as_e4m3_1x128_activations(ops, outliers):
    """The M > 1 path quantises an activation row into two NVFP4 residual terms.  Its error against
    the exact product (bf16 activations x dequantised weights) must not exceed what the same GEMM
    gives with the activations quantised to e4m3 with one scale per 1 x 128 block -- the FP8
    activation format this path stands in for -- on plain and on outlier-heavy rows."""
    from tilerl_b200.ops.gemm_tc import gemm_nvfp4
    t, n, k = 96, 1024, 5120
    g = torch.Generator().manual_seed(21)
    w = _w(n, k, 17)
    x = torch.randn(t, k, generator=g)
    if outliers:                                  # a few channels 30x larger, as residual streams have
        idx = torch.randint(0, k, (24,), generator=g)
        x[:, idx] *= 30.0
    x = x.to(DEV, torch.bfloat16)
    wd = w.dequant().float()
    exact = x.float() @ wd.t()
    # e4m3 with a scale per 1 x 128 block (amax / 448), in torch
    xb = x.float().view(t, k // 128, 128)
    s = xb.abs().amax(-1, keepdim=True).clamp_min(1e-12) / 448.0
    x8 = ((xb / s).to(torch.float8_e4m3fn).float() * s).view(t, k)
    err_fp8 = _rel(x8 @ wd.t(), exact)
    y = torch.zeros(t, n, dtype=torch.float32, device=DEV)
    gemm_nvfp4(ops, x, w, y, terms=2, epi=3)
    torch.cuda.synchronize()
    err_j2 = _rel(y, exact)
    assert err_j2 <= err_fp8 * 1.05 + 1e-4, (err_j2, err_fp8)
