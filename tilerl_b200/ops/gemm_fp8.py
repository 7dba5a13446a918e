"""Projections over block-scaled FP8 weights (``formats.FP8BlockTensor``).

* more than ``GEMV_ROWS`` tokens: ``trl_quant_act_fp8`` (RMSNorm folded in, e4m3 with one
  fp32 scale per token and 128 k) then ``trl_gemm_fp8``: TMA-fed ``tcgen05.mma.kind::f8f6f4``
  with per-128-k promotion of the TMEM accumulator by ``wscale * ascale`` (``csrc/gemm_fp8.cu``);
* up to ``GEMV_ROWS`` tokens: ``trl_gemv_fp8`` streams the e4m3 rows once and multiplies them
  with the bf16-rounded activation in fp32 (no activation quantisation on the decode path).

Reference parity: ``linear_fp8`` / ``linear_fp8_gemv`` / ``quant_fp8``
(packages/tilerl-kernels/src/tilerl_kernels/kernels_linear.py:1442-1813).
"""
from __future__ import annotations

import torch

from . import native as N

GEMV_ROWS = 2     # measured on the 27B gate_up shape: GEMV 43 us at 1 row, 116 us at 4; quantiser + GEMM 83 us
EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU, EPI_STORE_F32 = 0, 1, 2, 3


def available(ops) -> bool:
    return hasattr(ops.lib, "trl_gemm_fp8")


def quant_act(ops, x: torch.Tensor, norm_w=None, eps: float = 0.0, swiglu_in: bool = False):
    """bf16 ``[T, K]`` (``[T, 2K]`` interleaved gate/up with ``swiglu_in``) -> (e4m3 ``[T, K]``,
    fp32 ``[T, K/128]``) in workspace buffers."""
    t = x.shape[0]
    k = x.shape[1] // 2 if swiglu_in else x.shape[1]
    if k % 128:
        raise ValueError("FP8 projections need K % 128 == 0")
    x8 = ops.ws.get("fp8_x8", (t, k), torch.uint8)
    sc = ops.ws.get("fp8_xs", (t, k // 128), torch.float32)
    N.check(ops.lib.trl_quant_act_fp8(x.data_ptr(), x.stride(0), N.ptr(norm_w), eps, x8.data_ptr(), sc.data_ptr(),
                                      t, k, int(swiglu_in), N.stream()), "quant_act_fp8")
    N.count()
    return x8, sc


def gemm(ops, x, w, y, *, norm_w=None, eps=0.0, residual=None, epi=EPI_STORE) -> None:
    t = x.shape[0]
    n, k = w.shape
    x8, sc = quant_act(ops, x, norm_w, eps)
    N.check(ops.lib.trl_gemm_fp8(w.w8.data_ptr(), w.wscale.data_ptr(), x8.data_ptr(), sc.data_ptr(),
                                 N.ptr(residual), residual.stride(0) if residual is not None else 0,
                                 y.data_ptr(), y.stride(0), t, n, k, epi, N.stream()), "gemm_fp8")
    N.count()


def gemv(ops, x, w, y, *, norm_w=None, eps=0.0, residual=None, epi=EPI_STORE) -> None:
    m = x.shape[0]
    n, k = w.shape
    if epi == EPI_SWIGLU:
        tmp = ops.ws.get("fp8_gu", (m, n), torch.bfloat16)
        gemv(ops, x, w, tmp, norm_w=norm_w, eps=eps)
        N.check(ops.lib.trl_swiglu(tmp.data_ptr(), y.data_ptr(), y.numel(), N.stream()), "swiglu")
        N.count()
        return
    N.check(ops.lib.trl_gemv_fp8(x.data_ptr(), x.stride(0), w.w8.data_ptr(), w.wscale.data_ptr(), N.ptr(norm_w), eps,
                                 N.ptr(residual), residual.stride(0) if residual is not None else 0,
                                 y.data_ptr(), y.stride(0), m, n, k, epi, N.stream()), "gemv_fp8")
    N.count((m + 3) // 4)


def linear(ops, x, w, y, *, norm_w=None, eps=0.0, residual=None, epi=EPI_STORE) -> None:
    if x.shape[0] <= GEMV_ROWS:
        gemv(ops, x, w, y, norm_w=norm_w, eps=eps, residual=residual, epi=epi)
    else:
        gemm(ops, x, w, y, norm_w=norm_w, eps=eps, residual=residual, epi=epi)
