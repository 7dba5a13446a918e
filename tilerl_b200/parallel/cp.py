"""Context parallelism for the training forward: the sequence is cut in ``2 * cp`` chunks and
rank ``r`` owns chunks ``r`` and ``2 * cp - 1 - r`` (zigzag: causal work is balanced).

* Full attention: K / V (after RoPE) and their absolute positions are all-gathered along the
  token axis; the causal mask is ``kpos <= qpos`` on absolute positions, so no chunk ordering
  is assumed.  Backward reduce-scatters dK / dV to their owners.
* Gated DeltaNet: a chunk acts on the state as an affine map ``S_out = A S_in + B``
  (``A = prod_t (I - beta_t k_t k_t^T) e^{g_t}``, ``B`` = the state reached from zero).  Every
  rank summarises its two chunks as (A, B), one all-gather exchanges the 2*cp pairs, each rank
  folds the pairs of the chunks before its own (in sequence order) to get the entry state,
  then runs its chunks from there.  The depthwise conv needs the last ``K - 1`` raw rows of
  the preceding chunk: one all-gather of chunk tails (the *halo*).
* Every collective is an autograd function (all-gather forward, sum-and-keep-own backward),
  so the hand-written tape can differentiate the block locally with ``torch.autograd`` and
  the cross-rank gradient of the entry state flows back to the ranks that produced it.

Parity: reference ``tilerl_kernels/reference.py`` -- ``affine_prefix_scan:704-766``,
``gdn_span_ab`` / ``gdn_cp:590-999``, halo backward ``:859-902``; ``backend.py:283-364``
(``cp_gather``, ``cp_reduce_scatter``, ``cp_prefix_scan``, ``cp_halo``);
zigzag ``src/tilerl/tensor_parallel.py:115-150``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .mesh import zigzag_chunks, zigzag_positions


@dataclass
class CPContext:
    group: object
    world: int
    rank: int
    halo: bool = True          # False = negative control of the gates: no conv halo exchange

    @classmethod
    def from_group(cls, group=None) -> "CPContext":
        return cls(group, dist.get_world_size(group), dist.get_rank(group))


class _AllGather(torch.autograd.Function):
    """``[...] -> [world, ...]``; the gradient of a rank's piece is the sum over ranks."""

    @staticmethod
    def forward(ctx, x, cp: CPContext):
        ctx.cp = cp
        x = x.contiguous()
        out = [torch.empty_like(x) for _ in range(cp.world)]
        dist.all_gather(out, x, group=cp.group)
        return torch.stack(out)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.cp.group)
        return g[ctx.cp.rank], None


def all_gather(x: torch.Tensor, cp: CPContext) -> torch.Tensor:
    return _AllGather.apply(x, cp)


def split_zigzag(x: torch.Tensor, cp: int, rank: int, dim: int = 1) -> torch.Tensor:
    """This rank's tokens of a full-sequence tensor (two chunks, concatenated)."""
    t = x.shape[dim]
    return torch.cat([x.narrow(dim, a, b - a) for a, b in zigzag_chunks(t, cp, rank)], dim)


def merge_zigzag(parts: List[torch.Tensor], dim: int = 1) -> torch.Tensor:
    """Inverse of :func:`split_zigzag` given every rank's slice (rank order)."""
    cp = len(parts)
    c = parts[0].shape[dim] // 2
    chunks = [None] * (2 * cp)
    for r, p in enumerate(parts):
        chunks[r] = p.narrow(dim, 0, c)
        chunks[2 * cp - 1 - r] = p.narrow(dim, c, c)
    return torch.cat(chunks, dim)


def chunk_order(cp: int) -> List[Tuple[int, int]]:
    """(rank, which) of chunks 0 .. 2cp-1 in sequence order; which = 0 / 1 = first / second local chunk."""
    out = [None] * (2 * cp)
    for r in range(cp):
        out[r] = (r, 0)
        out[2 * cp - 1 - r] = (r, 1)
    return out


def gather_kv(k: torch.Tensor, v: torch.Tensor, pos: torch.Tensor, cp: CPContext):
    """``k, v [B, t, H, D]``, ``pos [t]`` (absolute) -> the same over all ranks' tokens ``[B, t*W, ...]``."""
    ka = all_gather(k, cp)                      # [W, B, t, H, D]
    va = all_gather(v, cp)
    w, b, t = ka.shape[0], ka.shape[1], ka.shape[2]
    ka = ka.permute(1, 0, 2, 3, 4).reshape(b, w * t, *ka.shape[3:])
    va = va.permute(1, 0, 2, 3, 4).reshape(b, w * t, *va.shape[3:])
    pa = [torch.empty_like(pos) for _ in range(cp.world)]
    dist.all_gather(pa, pos.contiguous(), group=cp.group)
    return ka, va, torch.cat(pa)


def conv_halo(raw: torch.Tensor, kw: int, cp: CPContext) -> torch.Tensor:
    """``raw [B, 2c, C]`` (this rank's two chunks of pre-conv rows) -> ``[B, 2, kw-1, C]``: for each
    local chunk the last ``kw - 1`` rows of the chunk that precedes it in the sequence (zeros
    before chunk 0)."""
    b, t2, ch = raw.shape
    c = t2 // 2
    tails = torch.stack([raw[:, c - (kw - 1):c], raw[:, 2 * c - (kw - 1):]], 1)   # [B, 2, kw-1, C]
    allt = all_gather(tails, cp)                                                    # [W, B, 2, kw-1, C]
    order = chunk_order(cp.world)
    mine = [cp.rank, 2 * cp.world - 1 - cp.rank]
    out = []
    for gidx in mine:
        if gidx == 0 or not cp.halo:
            out.append(torch.zeros_like(tails[:, 0]))
        else:
            r, which = order[gidx - 1]
            out.append(allt[r, :, which])
    return torch.stack(out, 1)


def fold_entry_states(a_loc: torch.Tensor, b_loc: torch.Tensor, cp: CPContext) -> torch.Tensor:
    """``a_loc [2, B, H, dk, dk]``, ``b_loc [2, B, H, dk, dv]`` (this rank's two chunk summaries)
    -> entry states ``[2, B, H, dk, dv]`` of its two chunks: the fold ``S <- A_j S + B_j`` over
    every chunk ``j`` before it in sequence order (float64 payload, as the products of decays
    span many orders of magnitude)."""
    aa = all_gather(a_loc.double(), cp)         # [W, 2, ...]
    ba = all_gather(b_loc.double(), cp)
    order = chunk_order(cp.world)
    mine = [cp.rank, 2 * cp.world - 1 - cp.rank]
    s = torch.zeros_like(ba[0, 0])
    entry = {}
    for gidx, (r, which) in enumerate(order):
        if gidx in mine:
            entry[gidx] = s
        s = aa[r, which] @ s + ba[r, which]
    return torch.stack([entry[g] for g in mine]).to(b_loc.dtype)


def positions_for(seq_len: int, cp: CPContext) -> torch.Tensor:
    return zigzag_positions(seq_len, cp.world, cp.rank)
