"""Python side of the tcgen05 NVFP4 GEMM: scale-factor tiling, scratch buffers, launch.

``gemm_nvfp4(ops, x, w, y, ...)`` runs ``y = epi(x' @ W^T)`` for any token count:

* ``terms`` (J) NVFP4 residual terms per token decide the activation precision
  (1 = W4A4, 2 ~ FP8-class, 4 ~ bf16); ``norm_w`` folds RMSNorm and ``swiglu_in``
  folds SwiGLU of an interleaved gate/up row into the quantiser.
* the weight's e4m3 scales are re-tiled once into the 128x4 layout the tensor core
  reads (``w.sf_tiled``), next to the checkpoint-layout scales the GEMV uses.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..formats import NVFP4Tensor
from . import native as N

N.register("trl_quant_act_nvfp4", [N.P, N.I, N.P, N.F, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.P])
N.register("trl_gemm_nvfp4", [N.P, N.P, N.P, N.P, N.P, N.P, N.P, N.I, N.P, N.I, N.P, N.P, N.L,
                              N.I, N.I, N.I, N.I, N.I, N.I, N.I, N.I, N.P])
N.register("trl_gemm_nvfp4_scratch_bytes", [N.I, N.I, N.I, N.I, N.I])
N.register("trl_gemv_stream_bytes", [N.I, N.I])
N.register("trl_gemv_stream_pack", [N.P, N.P, N.P, N.I, N.I, N.P])
N.register("trl_gemv2_nvfp4", [N.P, N.I, N.P, N.P, N.P, N.F, N.P, N.I, N.P, N.I, N.I, N.I, N.I, N.I, N.P])
N.register("trl_gemv2_nvfp4_push", [N.P, N.I, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.I, N.I, N.P])

KT = 256  # K elements per k-tile


def tile_scales(scale: torch.Tensor, K: int) -> torch.Tensor:
    """``[R, K/16]`` e4m3 (any device) -> tiled bytes ``[ceil(R/128), nk*4, 32, 4, 4]`` with
    byte (r, k16) at ``((r//128)*kt4 + k16//4)*512 + (r%32)*16 + ((r%128)//32)*4 + k16%4``;
    padding rows / k-blocks are zero."""
    r, kb = scale.shape
    nk = (K + KT - 1) // KT
    rp, kp = (r + 127) // 128 * 128, nk * 16
    s = torch.zeros(rp, kp, dtype=torch.uint8, device=scale.device)
    s[:r, :kb] = scale.view(torch.uint8)
    s = s.view(rp // 128, 4, 32, kp // 4, 4)        # [atom, r/32, r%32, k64, k16%4]
    return s.permute(0, 3, 2, 1, 4).contiguous()      # [atom, k64, r%32, r/32, k16%4]


def tile_weight(wq: torch.Tensor, K: int) -> torch.Tensor:
    """Packed nibbles ``[N, K/2]`` -> tile-contiguous ``[ceil(N/128), nk, 128, 128]`` bytes:
    every (128 rows x 256 k) operand tile is one contiguous 16 KB run, so a TMA box is a
    single DRAM burst instead of 128 strided 128-byte reads.  Tails are zero-padded."""
    n, kb = wq.shape
    nk = (K + KT - 1) // KT
    np_, kp = (n + 127) // 128 * 128, nk * 128
    if (np_, kp) != (n, kb):
        t = torch.zeros(np_, kp, dtype=torch.uint8, device=wq.device)
        t[:n, :kb] = wq
    else:
        t = wq
    return t.view(np_ // 128, 128, nk, 128).permute(0, 2, 1, 3).contiguous()


def wq_tiled(w: NVFP4Tensor) -> torch.Tensor:
    t = getattr(w, "wq_tiled", None)
    if t is None:
        t = tile_weight(w.wq, w.shape[1])
        w.wq_tiled = t
        w.wq_version = w.wq._version
    elif getattr(w, "wq_version", None) != w.wq._version:
        # the weight was rewritten in place (re-quantisation, resync): refresh the copy in place
        # too, so kernels captured in CUDA graphs keep reading the right address
        t.copy_(tile_weight(w.wq, w.shape[1]))
        w.wq_version = w.wq._version
    return t


def sf_tiled(w: NVFP4Tensor) -> torch.Tensor:
    t = getattr(w, "sf_tiled", None)
    if t is None:
        t = tile_scales(w.scale, w.shape[1])
        w.sf_tiled = t
        w.sf_version = w.scale._version
    elif getattr(w, "sf_version", None) != w.scale._version:
        t.copy_(tile_scales(w.scale, w.shape[1]))
        w.sf_version = w.scale._version
    return t


def stream_layout(wq: torch.Tensor, scale: torch.Tensor, K: int) -> torch.Tensor:
    """Torch statement of the GEMV stream layout (``csrc/gemv2.cu``): rows in pairs, K in steps of
    32 chunks of 32 weights; unit (pair, step) = ``[n x 16 B row 0][n x 16 B row 1][n x 2 B scales
    row 0][n x 2 B scales row 1]`` with n = 32 (fewer in a row's last step), units back to back."""
    n_rows, kb = wq.shape
    nchunks = K // 32
    w = wq.view(n_rows // 2, 2, nchunks, 16)
    s = scale.view(torch.uint8).view(n_rows // 2, 2, nchunks, 2)
    parts = []
    for c0 in range(0, nchunks, 32):
        c1 = min(nchunks, c0 + 32)
        parts.append(w[:, :, c0:c1].reshape(n_rows // 2, -1))
        parts.append(s[:, :, c0:c1].reshape(n_rows // 2, -1))
    return torch.cat(parts, dim=1).contiguous().view(-1)


def stream_ok(w: NVFP4Tensor) -> bool:
    n, k = w.shape
    return n % 2 == 0 and k % 128 == 0


def w_stream(w: NVFP4Tensor) -> torch.Tensor:
    """The weight's stream-layout copy for the decode GEMV (built on the device, refreshed in place
    when the weight was rewritten so captured graphs keep their address)."""
    t = getattr(w, "w_stream", None)
    fresh = t is None
    ver = (w.wq._version, w.scale._version)
    if fresh:
        n, k = w.shape
        t = torch.empty((n // 2) * (k // 32) * 36, dtype=torch.uint8, device=w.wq.device)
        w.w_stream = t
    if fresh or getattr(w, "stream_version", None) != ver:
        n, k = w.shape
        N.check(N.lib().trl_gemv_stream_pack(w.wq.data_ptr(), w.scale.data_ptr(), t.data_ptr(), n, k, N.stream()),
                "gemv_stream_pack")
        w.stream_version = ver
    return t


def quant_act(ops, x: torch.Tensor, K: int, terms: int, *, norm_w=None, eps: float = 0.0,
              swiglu_in: bool = False):
    """Quantise ``x [T, K]`` (or ``[T, 2K]`` interleaved gate/up when ``swiglu_in``).
    Returns (xq, sfx, rs) workspace views."""
    t = x.shape[0]
    cols = t * terms
    nk = (K + KT - 1) // KT
    atoms = (cols + 255) // 256 * 2
    xq = ops.ws.get("tc_xq", (cols, K // 2), torch.uint8)
    sfx = ops.ws.get("tc_sfx", (atoms * nk * 4 * 512,), torch.uint8)
    rs = ops.ws.get("tc_rs", (cols,), torch.float32)
    N.check(ops.lib.trl_quant_act_nvfp4(x.data_ptr(), x.stride(0), N.ptr(norm_w), eps, xq.data_ptr(),
                                        sfx.data_ptr(), rs.data_ptr(), t, K, terms, int(swiglu_in), N.stream()),
            "quant_act_nvfp4")
    N.count()
    return xq, sfx, rs


def _scratch(ops, nbytes: int, tiles: int):
    """Split-K slot buffer (contents irrelevant) and the zero-initialised tile counters
    (the kernel resets each counter it used)."""
    buf = ops.ws.get("tc_partial", (max(nbytes // 4, 1),), torch.float32)
    cnt = ops.ws.bufs.get("tc_counters")
    if cnt is None or cnt.numel() < tiles:
        if cnt is not None and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("tile counters would be reallocated during graph capture")
        ops.ws.bufs["tc_counters"] = torch.zeros(max(tiles, 8192), dtype=torch.int32, device=ops.device)
    return buf, ops.ws.bufs["tc_counters"]


def _want_split(ops, n: int, k: int, cols: int) -> bool:
    """Split tiles along K only when whole tiles cannot occupy the SMs."""
    import os
    mode = os.environ.get("TRL_SPLITK", "auto")
    if mode in ("0", "1"):
        return mode == "1"
    tiles = ((n + 127) // 128) * ((cols + 255) // 256 if cols > 256 else 1)
    return tiles < ops.sms


def gemm_nvfp4(ops, x: torch.Tensor, w: NVFP4Tensor, y: torch.Tensor, *, terms: int = 1, norm_w=None,
               eps: float = 0.0, residual: Optional[torch.Tensor] = None, epi: int = 0,
               swiglu_in: bool = False, max_ctas: int = 0, split: Optional[bool] = None) -> None:
    n, k = w.shape
    t = x.shape[0]
    xq, sfx, rs = quant_act(ops, x, k, terms, norm_w=norm_w, eps=eps, swiglu_in=swiglu_in)
    cols = t * terms
    bn = 16
    while bn < cols and bn < 256:
        bn *= 2
    c_tiles = (cols + bn - 1) // bn
    n_tiles = (n + 127) // 128
    ops.lib.trl_gemm_nvfp4_scratch_bytes.restype = __import__("ctypes").c_long
    nbytes = ops.lib.trl_gemm_nvfp4_scratch_bytes(t, terms, n, k, max_ctas)
    partial, counters = _scratch(ops, nbytes, n_tiles * c_tiles)
    tiled = getattr(ops, "tile_weights", True)
    N.check(ops.lib.trl_gemm_nvfp4(
        (wq_tiled(w) if tiled else w.wq).data_ptr(), sf_tiled(w).data_ptr(), w.tscale.data_ptr(), xq.data_ptr(), sfx.data_ptr(),
        rs.data_ptr(), N.ptr(residual), residual.stride(0) if residual is not None else 0,
        y.data_ptr(), y.stride(0), partial.data_ptr(), counters.data_ptr(), partial.numel() * 4, t, terms, n, k,
        epi, max_ctas, int(_want_split(ops, n, k, cols) if split is None else split), int(tiled),
        N.stream()), "gemm_nvfp4")
    N.count()


def gemm_bf16(ops, x, w, y):
    torch.matmul(x, w.t(), out=y)
