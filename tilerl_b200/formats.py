"""Numeric formats: NVFP4 (e2m1 + e4m3 block scales + fp32 tensor scale) and
block-scaled FP8, as torch reference code plus a byte-accounting registry.

The packed layouts here are exactly what the CUDA kernels consume:

* ``wq``    uint8 ``[N, K/2]``: two e2m1 codes per byte, low nibble = even k.
* ``scale`` float8_e4m3fn ``[N, K/16]``: one scale per 16 consecutive k.
* ``tscale`` fp32 scalar: tensor-level scale.  ``w ~= e2m1(wq) * scale * tscale``.

This is the on-disk NVFP4 checkpoint layout, kept as is on the device so the
tcgen05 block-scaled MMA can read it without repacking.

Parity: reference ``packages/tilerl-kernels/src/tilerl_kernels/reference.py:189-419``
(format maths) and ``src/tilerl/precision.py:34-181`` (format registry).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, Tuple

import torch

FP4_BLOCK = 16
FP8_BLOCK = 128
E2M1_MAX = 6.0
E4M3_MAX = 448.0

# magnitude of each 3-bit e2m1 code
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# midpoints between neighbouring magnitudes and whether a tie rounds up
# (round-to-nearest-even on the code's mantissa bit, as cvt.rn does)
_E2M1_MID = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
_E2M1_TIE_UP = (False, True, False, True, False, True, False)


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit e2m1 code (uint8 in 0..15), round-to-nearest-even, saturating."""
    a = x.abs()
    code = torch.zeros_like(a, dtype=torch.uint8)
    for mid, up in zip(_E2M1_MID, _E2M1_TIE_UP):
        code += ((a >= mid) if up else (a > mid)).to(torch.uint8)
    sign = (x < 0) | ((x == 0) & torch.signbit(x))
    return code | (sign.to(torch.uint8) << 3)


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    lut = torch.tensor(E2M1_VALUES + tuple(-v for v in E2M1_VALUES), dtype=torch.float32,
                       device=code.device)
    return lut[code.long()]


def pack_nibbles(code: torch.Tensor) -> torch.Tensor:
    """[..., K] codes -> [..., K/2] bytes, low nibble = even k."""
    lo, hi = code[..., 0::2], code[..., 1::2]
    return (lo | (hi << 4)).contiguous()


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    lo, hi = packed & 0xF, packed >> 4
    return torch.stack([lo, hi], dim=-1).flatten(-2)


@dataclass
class NVFP4Tensor:
    """A quantised 2-D weight.  ``shape`` is the logical ``[N, K]``."""
    wq: torch.Tensor       # uint8 [N, K/2]
    scale: torch.Tensor    # float8_e4m3fn [N, K/16]
    tscale: torch.Tensor   # fp32 [1]

    @property
    def shape(self) -> Tuple[int, int]:
        return (self.wq.shape[0], self.wq.shape[1] * 2)

    def to(self, device) -> "NVFP4Tensor":
        return NVFP4Tensor(self.wq.to(device), self.scale.to(device), self.tscale.to(device))

    def nbytes(self) -> int:
        return self.wq.numel() + self.scale.numel() + 4

    def dequant(self) -> torch.Tensor:
        return dequantize_nvfp4(self)


def quantize_nvfp4(w: torch.Tensor, tscale: torch.Tensor | None = None) -> NVFP4Tensor:
    """Quantise ``[N, K]`` (K multiple of 16) to NVFP4.

    tensor scale = amax / (6 * 448) so the largest block scale lands on the e4m3
    maximum; block scale = blockmax / 6 / tscale rounded to e4m3; elements are
    rounded to the nearest e2m1 of ``w / (scale * tscale)``."""
    if w.dim() != 2 or w.shape[1] % FP4_BLOCK:
        raise ValueError(f"NVFP4 needs [N, K] with K % 16 == 0, got {tuple(w.shape)}")
    w = w.float()
    n, k = w.shape
    if tscale is None:
        amax = w.abs().max().clamp_min(1e-30)
        # tensor / tensor: a true IEEE division (tensor / python-scalar may be lowered
        # to a multiply by the reciprocal, which differs in the last bit)
        tscale = (amax / torch.tensor(E2M1_MAX * E4M3_MAX, device=w.device)).reshape(1)
    tscale = tscale.float().reshape(1)
    blocks = w.view(n, k // FP4_BLOCK, FP4_BLOCK)
    bmax = blocks.abs().amax(-1)
    s = (bmax / torch.tensor(E2M1_MAX, device=w.device) / tscale).clamp(max=E4M3_MAX)
    s8 = s.to(torch.float8_e4m3fn)
    sf = s8.float()
    denom = (sf * tscale).unsqueeze(-1)
    q = torch.where(denom > 0, blocks / denom.clamp_min(1e-30), torch.zeros_like(blocks))
    code = e2m1_encode(q).view(n, k)
    return NVFP4Tensor(pack_nibbles(code), s8, tscale.clone())


def dequantize_nvfp4(t: NVFP4Tensor) -> torch.Tensor:
    n, k = t.shape
    vals = e2m1_decode(unpack_nibbles(t.wq)).view(n, k // FP4_BLOCK, FP4_BLOCK)
    return (vals * t.scale.float().unsqueeze(-1) * t.tscale.float()).view(n, k)


def nvfp4_roundtrip(w: torch.Tensor) -> torch.Tensor:
    return dequantize_nvfp4(quantize_nvfp4(w)).to(w.dtype)


def quantize_act_nvfp4(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Activation quantisation used by the M>1 NVFP4 GEMM: one fp32 scale per row
    (token) and e4m3 scales per 16 k.  Returns (xq uint8 [M,K/2], sf e4m3 [M,K/16],
    row_scale fp32 [M])."""
    x = x.float()
    m, k = x.shape
    amax = x.abs().amax(-1).clamp_min(1e-30)
    rs = amax / (E2M1_MAX * E4M3_MAX)
    blocks = x.view(m, k // FP4_BLOCK, FP4_BLOCK)
    s = (blocks.abs().amax(-1) / E2M1_MAX / rs.unsqueeze(-1)).clamp(max=E4M3_MAX)
    s8 = s.to(torch.float8_e4m3fn)
    denom = (s8.float() * rs.unsqueeze(-1)).unsqueeze(-1)
    q = torch.where(denom > 0, blocks / denom.clamp_min(1e-30), torch.zeros_like(blocks))
    return pack_nibbles(e2m1_encode(q).view(m, k)), s8, rs


def dequantize_act_nvfp4(xq, sf, rs) -> torch.Tensor:
    m, k = xq.shape[0], xq.shape[1] * 2
    v = e2m1_decode(unpack_nibbles(xq)).view(m, k // FP4_BLOCK, FP4_BLOCK)
    return (v * sf.float().unsqueeze(-1) * rs.view(m, 1, 1)).view(m, k)


# ---- FP8 ---------------------------------------------------------------------
@dataclass
class FP8BlockTensor:
    """e4m3 weight ``[N, K]`` with one fp32 scale per 128x128 block."""
    w8: torch.Tensor      # float8_e4m3fn [N, K]
    wscale: torch.Tensor  # fp32 [ceil(N/128), ceil(K/128)]

    @property
    def shape(self) -> Tuple[int, int]:
        return tuple(self.w8.shape)

    def nbytes(self) -> int:
        return self.w8.numel() + self.wscale.numel() * 4

    def to(self, device) -> "FP8BlockTensor":
        return FP8BlockTensor(self.w8.to(device), self.wscale.to(device))

    def dequant(self) -> torch.Tensor:
        return dequantize_fp8_block(self)


def _block_view(w: torch.Tensor, b: int):
    n, k = w.shape
    pn, pk = (-n) % b, (-k) % b
    wp = torch.nn.functional.pad(w, (0, pk, 0, pn))
    return wp.view((n + pn) // b, b, (k + pk) // b, b).permute(0, 2, 1, 3), n, k


def quantize_fp8_block(w: torch.Tensor) -> FP8BlockTensor:
    blocks, n, k = _block_view(w.float(), FP8_BLOCK)
    amax = blocks.abs().amax((-1, -2)).clamp_min(1e-30)
    scale = amax / E4M3_MAX
    q = (blocks / scale[..., None, None]).permute(0, 2, 1, 3).reshape(
        blocks.shape[0] * FP8_BLOCK, blocks.shape[1] * FP8_BLOCK)[:n, :k]
    return FP8BlockTensor(q.contiguous().to(torch.float8_e4m3fn), scale.contiguous())


def dequantize_fp8_block(t: FP8BlockTensor) -> torch.Tensor:
    n, k = t.shape
    s = t.wscale.repeat_interleave(FP8_BLOCK, 0).repeat_interleave(FP8_BLOCK, 1)[:n, :k]
    return t.w8.float() * s


def quantize_act_fp8_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Activation quant for the block-scaled FP8 GEMM: one fp32 scale per
    (row, 128 consecutive k).  Returns (x8 e4m3 [M,K], scale fp32 [M, K/128])."""
    x = x.float()
    m, k = x.shape
    if k % FP8_BLOCK:
        raise ValueError("K must be a multiple of 128")
    b = x.view(m, k // FP8_BLOCK, FP8_BLOCK)
    s = b.abs().amax(-1).clamp_min(1e-30) / E4M3_MAX
    return (b / s.unsqueeze(-1)).view(m, k).to(torch.float8_e4m3fn), s


def dequantize_act_fp8_1x128(x8: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    m, k = x8.shape
    return (x8.float().view(m, k // FP8_BLOCK, FP8_BLOCK) * s.unsqueeze(-1)).view(m, k)


def quantize_kv_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """KV-cache fp8: one scale per (token, head) = amax/448 over the head dim.
    Reference ``reference.py:382-402``."""
    s = x.float().abs().amax(-1).clamp_min(1e-30) / E4M3_MAX
    return (x.float() / s.unsqueeze(-1)).to(torch.float8_e4m3fn), s


# ---- byte accounting ------------------------------------------------------------
@dataclass(frozen=True)
class Format:
    """Prices a tensor: ``bits`` per element plus scale planes given as
    (elements-per-scale, bytes-per-scale)."""
    name: str
    bits: int
    scales: Tuple[Tuple[int, int], ...] = ()
    per_tensor_bytes: int = 0

    def nbytes(self, shape: Iterable[int]) -> int:
        n = 1
        for d in shape:
            n *= int(d)
        total = (n * self.bits + 7) // 8 + self.per_tensor_bytes
        for per, b in self.scales:
            total += (n + per - 1) // per * b
        return total


FORMATS: Dict[str, Format] = {
    "bf16": Format("bf16", 16),
    "f32": Format("f32", 32),
    "nvfp4": Format("nvfp4", 4, ((FP4_BLOCK, 1),), 4),
    "fp8_block": Format("fp8_block", 8, ((FP8_BLOCK * FP8_BLOCK, 4),)),
    "fp8": Format("fp8", 8, (), 4),
    "kv_bf16": Format("kv_bf16", 16),
    "kv_fp8": Format("kv_fp8", 8, ((1 << 30, 0),)),
}


def kv_format(fp8: bool, head_dim: int) -> Format:
    """fp8 KV stores one fp32 scale per (token, head)."""
    return Format("kv_fp8", 8, ((head_dim, 4),)) if fp8 else FORMATS["kv_bf16"]


def nbytes(fmt: str | Format, shape: Iterable[int]) -> int:
    f = FORMATS[fmt] if isinstance(fmt, str) else fmt
    return f.nbytes(shape)


def weight_specs(cfg) -> Dict[str, Tuple[Tuple[int, ...], str]]:
    """Every served tensor -> (shape, format name).  The cost model, the memory
    planner and the dry-run ledger all read this one table.
    Reference ``precision.py:103`` (``weight_specs``)."""
    from .config import ATTN
    q = cfg.quant
    lin = {"nvfp4": "nvfp4", "fp8": "fp8_block", "bf16": "bf16"}[q]
    h = cfg.hidden
    out: Dict[str, Tuple[Tuple[int, ...], str]] = {
        "embed": ((cfg.vocab, h), "bf16"),
        "final_norm": ((h,), "bf16"),
    }
    if not cfg.tie_embeddings:
        out["lm_head"] = ((cfg.vocab, h), {"nvfp4": "nvfp4", "bf16": "bf16"}.get(cfg.lm_head_quant, "bf16"))
    for i, t in enumerate(cfg.layer_types):
        p = f"L{i}."
        out[p + "norm1"] = ((h,), "bf16")
        out[p + "norm2"] = ((h,), "bf16")
        if t == ATTN:
            out[p + "qkv"] = ((cfg.qkv_rows, h), lin)
            out[p + "o"] = ((h, cfg.attn_out_dim), lin)
            out[p + "q_norm"] = ((cfg.head_dim,), "bf16")
            out[p + "k_norm"] = ((cfg.head_dim,), "bf16")
        else:
            out[p + "in"] = ((cfg.gdn_in_rows, h), lin)
            out[p + "out"] = ((h, cfg.gdn_v_dim), lin)
            out[p + "conv"] = ((cfg.gdn_conv_dim, cfg.gdn_conv), "f32")
            out[p + "dt_bias"] = ((cfg.gdn_v_heads,), "f32")
            out[p + "a_log"] = ((cfg.gdn_v_heads,), "f32")
            out[p + "gdn_norm"] = ((cfg.gdn_head_dim,), "f32")
        out[p + "gate_up"] = ((2 * cfg.ffn, h), lin)
        out[p + "down"] = ((h, cfg.ffn), lin)
    return out


def served_weight_bytes(cfg) -> int:
    return sum(nbytes(f, s) for s, f in weight_specs(cfg).values())
