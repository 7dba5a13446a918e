"""Model configuration for the hybrid (gated-GQA attention + Gated-DeltaNet) decoder.

One frozen dataclass describes every shape the kernels, the KV pools, the
tensor-parallel shard tables and the cost model derive from.  Layer kinds are
spelled out per layer (``"attn"`` / ``"gdn"``) rather than as an index set so a
checkpoint's ``layer_types`` list maps onto it one to one.

Parity: reference ``src/tilerl/config.py:11`` (``ModelConfig``), ``:114``
(``qwen38_27b``), ``:153`` (``tiny``).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Tuple

ATTN = "attn"
GDN = "gdn"


@dataclass(frozen=True)
class ModelConfig:
    name: str
    hidden: int
    ffn: int
    vocab: int
    layer_types: Tuple[str, ...]
    # gated GQA attention
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    rotary_dim: int
    rope_theta: float
    attn_gated: bool = True
    # Gated DeltaNet
    gdn_k_heads: int = 0
    gdn_v_heads: int = 0
    gdn_head_dim: int = 0
    gdn_conv: int = 4
    # misc
    rms_eps: float = 1e-6
    max_ctx: int = 262144
    tie_embeddings: bool = False
    quant: str = "nvfp4"  # "nvfp4" | "fp8" | "bf16": format of the served linears
    lm_head_quant: str = "bf16"

    def __post_init__(self) -> None:
        object.__setattr__(self, "layer_types", tuple(self.layer_types))
        for t in self.layer_types:
            if t not in (ATTN, GDN):
                raise ValueError(f"unknown layer type {t!r}")
        if self.n_q_heads % self.n_kv_heads:
            raise ValueError("n_q_heads must be a multiple of n_kv_heads (GQA)")
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError("rotary_dim must be even and <= head_dim")
        if self.n_gdn_layers:
            if self.gdn_k_heads <= 0 or self.gdn_v_heads <= 0 or self.gdn_head_dim <= 0:
                raise ValueError("GDN layers need gdn_k_heads/gdn_v_heads/gdn_head_dim")
            if self.gdn_v_heads % self.gdn_k_heads:
                raise ValueError("gdn_v_heads must be a multiple of gdn_k_heads")

    # ---- derived ---------------------------------------------------------
    @property
    def n_layers(self) -> int:
        return len(self.layer_types)

    @property
    def attn_layers(self) -> Tuple[int, ...]:
        return tuple(i for i, t in enumerate(self.layer_types) if t == ATTN)

    @property
    def gdn_layers(self) -> Tuple[int, ...]:
        return tuple(i for i, t in enumerate(self.layer_types) if t == GDN)

    @property
    def n_attn_layers(self) -> int:
        return len(self.attn_layers)

    @property
    def n_gdn_layers(self) -> int:
        return len(self.gdn_layers)

    @property
    def gqa_group(self) -> int:
        return self.n_q_heads // self.n_kv_heads

    @property
    def q_rows(self) -> int:
        """Rows of the q projection: per head [query(D); gate(D)] when gated."""
        return self.n_q_heads * self.head_dim * (2 if self.attn_gated else 1)

    @property
    def kv_rows(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def qkv_rows(self) -> int:
        return self.q_rows + 2 * self.kv_rows

    @property
    def attn_out_dim(self) -> int:
        return self.n_q_heads * self.head_dim

    @property
    def gdn_qk_dim(self) -> int:
        return self.gdn_k_heads * self.gdn_head_dim

    @property
    def gdn_v_dim(self) -> int:
        return self.gdn_v_heads * self.gdn_head_dim

    @property
    def gdn_conv_dim(self) -> int:
        """Channels that go through the depthwise conv: q, k, v."""
        return 2 * self.gdn_qk_dim + self.gdn_v_dim

    @property
    def gdn_in_rows(self) -> int:
        """Rows of the fused GDN input projection: [q; k; v; z; a; b]."""
        return self.gdn_conv_dim + self.gdn_v_dim + 2 * self.gdn_v_heads

    def attn_index(self, layer: int) -> int:
        return self.attn_layers.index(layer)

    def gdn_index(self, layer: int) -> int:
        return self.gdn_layers.index(layer)

    def n_params(self) -> int:
        h = self.hidden
        n = self.vocab * h * (1 if self.tie_embeddings else 2) + h
        for t in self.layer_types:
            n += 2 * h + 3 * h * self.ffn
            if t == ATTN:
                n += self.qkv_rows * h + h * self.attn_out_dim + 2 * self.head_dim
            else:
                n += self.gdn_in_rows * h + h * self.gdn_v_dim
                n += self.gdn_conv_dim * self.gdn_conv + 2 * self.gdn_v_heads + self.gdn_head_dim
        return n


def qwen38_27b() -> ModelConfig:
    """The 27B hybrid: 64 layers, every 4th (3, 7, ..., 63) gated GQA attention
    (24 q / 4 kv heads x 256, partial RoPE 64, theta 1e7), the rest Gated DeltaNet
    (16 key / 48 value heads x 128, conv width 4); SwiGLU FFN 17408; vocab 248320.
    Reference ``src/tilerl/config.py:114-140``."""
    types = tuple(ATTN if i % 4 == 3 else GDN for i in range(64))
    return ModelConfig(
        name="qwen38-27b", hidden=5120, ffn=17408, vocab=248320, layer_types=types,
        n_q_heads=24, n_kv_heads=4, head_dim=256, rotary_dim=64, rope_theta=1e7,
        gdn_k_heads=16, gdn_v_heads=48, gdn_head_dim=128, gdn_conv=4,
        rms_eps=1e-6, max_ctx=262144, tie_embeddings=False, quant="nvfp4",
    )


def qwen36_27b() -> ModelConfig:
    """Same shapes as :func:`qwen38_27b` (reference ``config.py:143``)."""
    return replace(qwen38_27b(), name="qwen36-27b")


def tiny_hybrid() -> ModelConfig:
    """Two-layer CPU gate model: layer 0 GDN (4 heads x 64, conv 4), layer 1
    gated GQA (4 q / 2 kv heads x 64, theta 1e6), d_model 256, FFN 768,
    vocab 1024, eps 1e-6."""
    return ModelConfig(
        name="tiny-hybrid", hidden=256, ffn=768, vocab=1024, layer_types=(GDN, ATTN),
        n_q_heads=4, n_kv_heads=2, head_dim=64, rotary_dim=64, rope_theta=1e6,
        gdn_k_heads=4, gdn_v_heads=4, gdn_head_dim=64, gdn_conv=4,
        rms_eps=1e-6, max_ctx=4096, tie_embeddings=False, quant="nvfp4",
    )


def tiny(max_ctx: int = 512) -> ModelConfig:
    """Smallest smoke model (attention layer first, then GDN), tied embeddings,
    byte vocabulary of 320.  Reference ``config.py:153``."""
    return ModelConfig(
        name="tiny" if max_ctx == 512 else "tiny-agent",
        hidden=64, ffn=128, vocab=320, layer_types=(ATTN, GDN),
        n_q_heads=4, n_kv_heads=2, head_dim=16, rotary_dim=16, rope_theta=1e7,
        gdn_k_heads=2, gdn_v_heads=2, gdn_head_dim=16, gdn_conv=4,
        rms_eps=1e-6, max_ctx=max_ctx, tie_embeddings=True, quant="bf16",
    )


def small_gpu() -> ModelConfig:
    """A 4-layer model with the 27B's head geometry (D=256, GDN 128) but narrow
    width; used by GPU kernel/engine tests and profiler captures so every kernel
    template instantiated for the 27B is exercised on a few hundred MB."""
    types = (GDN, GDN, GDN, ATTN)
    return ModelConfig(
        name="small-gpu", hidden=1024, ffn=3072, vocab=32768, layer_types=types,
        n_q_heads=8, n_kv_heads=2, head_dim=256, rotary_dim=64, rope_theta=1e7,
        gdn_k_heads=4, gdn_v_heads=8, gdn_head_dim=128, gdn_conv=4,
        rms_eps=1e-6, max_ctx=65536, tie_embeddings=False, quant="nvfp4",
    )


def small_gpu_tp() -> ModelConfig:
    """:func:`small_gpu` with head counts and widths that divide 2, 4 and 8 ways (8 q / 2 kv
    heads -- kv heads replicated from 4 ranks on, as the 27B's 4 kv heads are at 8 --, 8 key /
    16 value GDN heads, FFN 4096): the model of the tensor-parallel GPU gates."""
    types = (GDN, GDN, GDN, ATTN)
    return ModelConfig(
        name="small-gpu-tp", hidden=1024, ffn=4096, vocab=32768, layer_types=types,
        n_q_heads=8, n_kv_heads=2, head_dim=256, rotary_dim=64, rope_theta=1e7,
        gdn_k_heads=8, gdn_v_heads=16, gdn_head_dim=128, gdn_conv=4,
        rms_eps=1e-6, max_ctx=65536, tie_embeddings=False, quant="nvfp4",
    )


_REGISTRY = {
    "qwen38-27b": qwen38_27b, "qwen36-27b": qwen36_27b, "tiny": tiny,
    "tiny-hybrid": tiny_hybrid, "small-gpu": small_gpu, "small-gpu-tp": small_gpu_tp,
    "tiny-agent": lambda: tiny(65536),
}


def get_config(name: str) -> ModelConfig:
    try:
        return _REGISTRY[name]()
    except KeyError:
        raise ValueError(f"unknown model {name!r}; known: {sorted(_REGISTRY)}") from None
