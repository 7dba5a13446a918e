import torch

from tilerl_b200 import formats as F


def test_e2m1_roundtrip_all_codes():
    codes = torch.arange(16, dtype=torch.uint8)
    vals = F.e2m1_decode(codes)
    back = F.e2m1_encode(vals)
    # -0 encodes as code 8; everything else is exact
    assert torch.equal(back[1:8], codes[1:8]) and torch.equal(back[9:], codes[9:])


def test_e2m1_ties_round_to_even():
    x = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -2.5])
    got = F.e2m1_decode(F.e2m1_encode(x))
    assert got.tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -2.0]


def test_nibble_order_low_is_even_k():
    code = torch.tensor([[1, 2, 3, 4]], dtype=torch.uint8)
    p = F.pack_nibbles(code)
    assert p.tolist() == [[1 | (2 << 4), 3 | (4 << 4)]]
    assert torch.equal(F.unpack_nibbles(p), code)


def test_nvfp4_quant_error_and_idempotence():
    torch.manual_seed(0)
    w = torch.randn(64, 128) * 0.02
    q = F.quantize_nvfp4(w)
    assert q.wq.shape == (64, 64) and q.scale.shape == (64, 8) and q.scale.dtype == torch.float8_e4m3fn
    d = q.dequant()
    rel = (d - w).norm() / w.norm()
    assert rel < 0.12
    # values already on the grid survive a second quantisation with the same tensor scale
    q2 = F.quantize_nvfp4(d, tscale=q.tscale)
    assert torch.allclose(q2.dequant(), d, rtol=0, atol=1e-7)


def test_fp8_block_and_act_quant():
    torch.manual_seed(1)
    w = torch.randn(200, 384)
    q = F.quantize_fp8_block(w)
    assert q.wscale.shape == (2, 3)
    assert (q.dequant() - w).abs().max() < 0.08 * w.abs().max()
    x = torch.randn(5, 256) * 3
    x8, s = F.quantize_act_fp8_1x128(x)
    assert s.shape == (5, 2)
    assert (F.dequantize_act_fp8_1x128(x8, s) - x).abs().max() < 0.07 * x.abs().max()
    xq, sf, rs = F.quantize_act_nvfp4(x)
    assert (F.dequantize_act_nvfp4(xq, sf, rs) - x).norm() / x.norm() < 0.15


def test_format_nbytes_and_weight_specs():
    assert F.nbytes("nvfp4", (128, 256)) == 128 * 256 // 2 + 128 * 256 // 16 + 4
    assert F.nbytes("bf16", (3, 5)) == 30
    from tilerl_b200.config import qwen38_27b
    cfg = qwen38_27b()
    total = F.served_weight_bytes(cfg)
    # NVFP4 projections + bf16 embed/lm_head: between 18 and 20 GB
    assert 18e9 < total < 20e9
    assert 26e9 < cfg.n_params() < 28.5e9
