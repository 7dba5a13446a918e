"""Large-M projections.

``linear(ops, x, w, y)`` computes ``y = x @ W^T`` (bf16 out) for ``M > 8`` tokens:

* NVFP4 weights: the tcgen05 block-scaled GEMM (``csrc/gemm_nvfp4.cu``): the
  activation is quantised on the fly to NVFP4 (e2m1, e4m3 scale per 16, fp32 scale
  per token), both operands are streamed by TMA and multiplied by
  ``tcgen05.mma.kind::mxf4nvf4.block_scale`` with the accumulator in TMEM.
* FP8 block weights: ``ops/gemm_fp8.py`` (``tcgen05.mma.kind::f8f6f4`` with per-128-k
  promotion; ``csrc/gemm_fp8.cu``).
* bf16 weights: the tcgen05 ``kind::f16`` GEMM (``csrc/gemm_bf16.cu``).

``TRL_GEMM=dequant`` selects a debugging path (dequantise to bf16 into scratch,
then a library matmul) used to bisect numerics; it is never the default.
"""
from __future__ import annotations

import os

import torch

from ..formats import FP8BlockTensor, NVFP4Tensor
from . import native as N

_MODE = os.environ.get("TRL_GEMM", "tc")


def has_tc(ops) -> bool:
    return hasattr(ops.lib, "trl_gemm_nvfp4") and _MODE == "tc" and ops.use_tc_gemm


def linear(ops, x: torch.Tensor, w, y: torch.Tensor) -> None:
    if isinstance(w, NVFP4Tensor):
        if has_tc(ops):
            from .gemm_tc import gemm_nvfp4
            return gemm_nvfp4(ops, x, w, y, terms=ops.terms_large)
        n, k = w.shape
        wd = ops.ws.get("dequant_w", (n, k), torch.bfloat16)
        ops.dequantize_nvfp4(w, wd)
        torch.matmul(x, wd.t(), out=y)
        return
    if isinstance(w, FP8BlockTensor):
        if hasattr(ops.lib, "trl_gemm_fp8") and _MODE == "tc" and w.shape[1] % 128 == 0:
            from . import gemm_fp8
            return gemm_fp8.linear(ops, x, w, y)
        wd = w.dequant().to(torch.bfloat16)
        torch.matmul(x, wd.t(), out=y)
        return
    if hasattr(ops.lib, "trl_gemm_bf16") and _MODE == "tc" and ops.use_tc_gemm:
        from .gemm_tc import gemm_bf16
        return gemm_bf16(ops, x, w, y)
    torch.matmul(x, w.t(), out=y)
