"""The op surface the model calls, and its fp32 torch implementation.

The model never touches a kernel directly: it calls the few *fused* entry
points below, each of which corresponds to one (or a short chain of) sm_100a
kernels in :mod:`tilerl_b200.ops.cuda`.  :class:`RefOps` implements the same
surface with the fp32 oracle of :mod:`tilerl_b200.ops.ref`; it is the CPU test
backend and the correctness twin of the CUDA path, and under a process group it
uses ``torch.distributed`` (gloo on CPU) for the tensor-parallel reductions.

Parity: reference ``src/tilerl/testing.py:37-296`` (``RefBackend``) and the
``Backend`` op surface ``packages/tilerl-kernels/src/tilerl_kernels/backend.py:559-1797``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import ref


class TPContext:
    """Tensor-parallel group handle; ``world == 1`` means no collectives."""

    def __init__(self, rank: int = 0, world: int = 1, group=None):
        self.rank, self.world, self.group = rank, world, group


class RefOps:
    name = "ref"

    def __init__(self, tp: Optional[TPContext] = None, act_dtype=torch.float32):
        self.tp = tp or TPContext()
        self.act_dtype = act_dtype

    # -- collectives -----------------------------------------------------------
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp.world > 1:
            import torch.distributed as dist
            dist.all_reduce(x, group=self.tp.group)
        return x

    def all_gather_last(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp.world == 1:
            return x
        import torch.distributed as dist
        parts = [torch.empty_like(x) for _ in range(self.tp.world)]
        dist.all_gather(parts, x.contiguous(), group=self.tp.group)
        return torch.cat(parts, dim=-1)

    # -- fused entry points --------------------------------------------------------
    def embed(self, table, ids):
        return ref.embedding(table, ids).to(self.act_dtype)

    def _lora(self, y, x, lora):
        if lora is not None:
            a, b, s = lora
            y = y + (x.float() @ a.float().t()) @ b.float().t() * s
        return y

    def norm_linear(self, x, norm_w, w, eps, lora=None):
        h = ref.rmsnorm(x, norm_w, eps)
        return self._lora(ref.linear(h, w), h, lora).to(self.act_dtype)

    def norm_linear_swiglu(self, x, norm_w, w, eps, lora=None):
        h = ref.rmsnorm(x, norm_w, eps)
        return ref.swiglu(self._lora(ref.linear(h, w), h, lora)).to(self.act_dtype)

    def device_alive(self) -> bool:
        return True

    def linear_residual(self, a, w, residual, lora=None):
        """Row-parallel linear: partial product, all-reduce over TP, residual add."""
        y = self._lora(ref.linear(a, w), a, lora)
        y = self.all_reduce(y)
        return (y + residual.float()).to(self.act_dtype)

    def attention(self, qkv, lp, batch, pool, attn_idx, cfg, n_q, n_kv):
        q, gate, k, v = ref.attn_prep(
            qkv, lp["q_norm"], lp["k_norm"], batch.positions, n_q=n_q, n_kv=n_kv,
            head_dim=cfg.head_dim, rotary_dim=cfg.rotary_dim, theta=cfg.rope_theta,
            eps=cfg.rms_eps, gated=cfg.attn_gated)
        kc, vc = pool.layer(attn_idx)
        if getattr(pool, "fp8", False):
            ref.kv_write_fp8(kc, vc, pool.k_scale[attn_idx], pool.v_scale[attn_idx], k, v, batch.slot_mapping)
            kc = ref.kv_dequant_fp8(kc, pool.k_scale[attn_idx])
            vc = ref.kv_dequant_fp8(vc, pool.v_scale[attn_idx])
        else:
            ref.kv_write(kc, vc, k, v, batch.slot_mapping)
        scale = 1.0 / math.sqrt(cfg.head_dim)
        table, pos = batch.block_table, batch.positions
        sp = batch.sparse
        if sp is not None and sp.active(attn_idx):
            table, pos = sp.packed(attn_idx, q, kc)    # [selected pages ; trailing window]
        out = ref.paged_attention(q, gate, kc, vc, table, batch.seq_ids, pos, scale)
        return out.to(self.act_dtype)

    def gdn(self, inp, lp, batch, spool, gdn_idx, cfg, nk, nv):
        d = cfg.gdn_head_dim
        out = torch.zeros(inp.shape[0], nv * d, dtype=torch.float32, device=inp.device)
        for r in range(batch.n_seqs):
            s0, n = int(batch.q_start[r]), int(batch.q_len[r])
            if n == 0:
                continue
            slot = int(batch.state_slots[r])
            cur = int(spool.cur[slot])
            state = spool.states[slot, gdn_idx, cur].clone()
            steps = None
            keep = bool(batch.keep_steps) and batch.keep_rows[r]
            if keep:
                steps = torch.zeros(n, nv, d, d, dtype=torch.float32, device=inp.device)
            ring = spool.ring[slot, gdn_idx]
            ring_f = ring.float()
            out[s0:s0 + n] = ref.gdn_sequence(
                inp[s0:s0 + n], batch.positions[s0:s0 + n], state, ring_f,
                conv_w=lp["conv"], dt_bias=lp["dt_bias"], a_log=lp["a_log"],
                norm_w=lp["gdn_norm"], nk=nk, nv=nv, dk=d, dv=d, eps=cfg.rms_eps,
                step_states=steps)
            ring.copy_(ring_f.to(ring.dtype))
            if keep:
                spool.states[slot, gdn_idx, :n].copy_(steps)
            else:
                spool.states[slot, gdn_idx, cur].copy_(state)
        return out.to(self.act_dtype)

    def lm_head(self, x, norm_w, w, eps):
        """Final norm + vocab(-parallel) head; returns full-vocab fp32 logits."""
        h = ref.rmsnorm(x, norm_w, eps)
        return self.all_gather_last(ref.linear(h, w))

    def full_logits(self, logits):
        return logits

    def argmax(self, logits):
        return torch.argmax(logits, dim=-1)
