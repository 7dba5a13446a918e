"""Named flag sets for ``cli train``: a recipe expands to defaults that explicit flags override.

Parity: reference ``src/tilerl/recipes.py:6-86`` (``RECIPES``).
"""
from __future__ import annotations

from typing import Any, Dict

RECIPES: Dict[str, Dict[str, Any]] = {
    "grpo-tiny-smoke": dict(model="tiny-hybrid", rl=True, group=4, prompts_per_step=2, steps=2, max_tokens=8,
                            lr=1e-5, lora_rank=0, reward="even", optim="adamw", allow_short_rollouts=True),
    "indexer-warmup": dict(model="qwen38-27b", indexer_warmup=True, steps=200, lr=1e-3, ctx=8192),
    "grpo-gsm8k-27b": dict(model="qwen38-27b", rl=True, group=8, prompts_per_step=8, steps=100, max_tokens=1024,
                           lr=1e-6, lora_rank=16, reward="gsm8k", optim="adamw", micro=1, eval_every=10,
                           patience=3),
    "grpo-math-27b": dict(model="qwen38-27b", rl=True, group=8, prompts_per_step=8, steps=200, max_tokens=2048,
                          lr=1e-6, lora_rank=16, reward="boxed", optim="adamw", micro=1),
    "opd-gsm8k-27b": dict(model="qwen38-27b", opd=True, prompts_per_step=8, steps=100, max_tokens=1024, lr=1e-6,
                          lora_rank=16, ema=0.99),
    "sft-iso-27b": dict(model="qwen38-27b", rl=False, steps=500, lr=2e-5, optim="iso", served_fp4=True, micro=2),
    "grpo-27b-zero3-tp8": dict(model="qwen38-27b", rl=True, group=8, prompts_per_step=8, steps=10, max_tokens=512,
                               lr=1e-6, lora_rank=0, zero=8, tp=8, optim="adamw", reward="mod7"),
}


def expand(name: str, overrides: Dict[str, Any]) -> Dict[str, Any]:
    if name not in RECIPES:
        raise KeyError(f"unknown recipe {name!r}; known: {sorted(RECIPES)}")
    out = dict(RECIPES[name])
    out.update({k: v for k, v in overrides.items() if v is not None})
    return out
