"""Optimizers for the hand-written tape: AdamW, Adafactor, ISO, schedule, clipping.

All state is fp32 and keyed by parameter name; updates are written back with
``copy_`` so parameter storage addresses never change (captured CUDA graphs and
the in-place requantiser rely on that).  ``step_param`` updates one tensor, so
the tape's streaming ``on_grad`` hook can run the optimizer during backward and
drop each gradient immediately.  On B200 the AdamW update is one fused kernel
(:func:`tilerl_b200.ops.cuda.adamw_step`); the torch form below is its oracle.

Parity: reference ``src/tilerl/autograd.py`` -- ``AdamW:466``, ``Adafactor:511``,
``cosine_warmup:648``, ``clip_grad_norm:661-709``; ``src/tilerl/iso.py`` (ISO).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Iterable, Optional, Tuple

import torch


def cosine_warmup(step: int, total: int, warmup: int, lr: float, min_ratio: float = 0.1) -> float:
    if warmup and step < warmup:
        return lr * (step + 1) / warmup
    if total <= warmup:
        return lr
    p = min(1.0, (step - warmup) / max(1, total - warmup))
    return lr * (min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * p)))


def clip_grad_norm(grads: Dict[str, torch.Tensor], max_norm: float, *, sharded: Optional[Callable[[str], bool]] = None,
                   tp_group=None, tp_world: int = 1) -> float:
    """Global-norm clip in place.  Under TP the squared norms of sharded tensors are
    summed across ranks while replicated tensors are counted once: one all-reduce
    of two numbers in fp64."""
    dev = next(iter(grads.values())).device if grads else torch.device("cpu")
    sh = torch.zeros((), dtype=torch.float64, device=dev)
    rep = torch.zeros((), dtype=torch.float64, device=dev)
    for k, g in grads.items():
        s = g.double().pow(2).sum()
        if sharded is not None and sharded(k):
            sh += s
        else:
            rep += s
    if tp_world > 1:
        import torch.distributed as dist
        # every rank contributes its shard's squares and its (identical) copy of the replicated ones:
        # after the sum the replicated part is tp_world times too large, the sharded part is whole.
        # The buffer lives on the gradients' device (NCCL reduces device tensors only).
        buf = torch.stack([sh, rep])
        dist.all_reduce(buf, group=tp_group)
        total = float(buf[0] + buf[1] / tp_world)
    else:
        total = float(sh + rep)
    norm = math.sqrt(total)
    if max_norm > 0 and norm > max_norm:
        c = max_norm / (norm + 1e-6)
        for g in grads.values():
            g.mul_(c)
    return norm


class AdamW:
    def __init__(self, params: Dict[str, torch.Tensor], lr: float = 1e-5, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.0):
        self.params = params
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.m: Dict[str, torch.Tensor] = {}
        self.v: Dict[str, torch.Tensor] = {}
        self.t: Dict[str, int] = {}

    def step_param(self, name: str, grad: torch.Tensor, lr: Optional[float] = None) -> None:
        p = self.params[name]
        if name not in self.m:
            self.m[name] = torch.zeros_like(p, dtype=torch.float32)
            self.v[name] = torch.zeros_like(p, dtype=torch.float32)
            self.t[name] = 0
        self.t[name] += 1
        t, (b1, b2) = self.t[name], self.betas
        lr = self.lr if lr is None else lr
        g = grad.float()
        m, v = self.m[name], self.v[name]
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        mhat = m / (1 - b1 ** t)
        vhat = v / (1 - b2 ** t)
        w = p.float()
        if self.wd and p.dim() >= 2:
            w = w * (1 - lr * self.wd)
        w = w - lr * mhat / (vhat.sqrt() + self.eps)
        p.copy_(w.to(p.dtype))

    def step(self, grads: Dict[str, torch.Tensor], lr: Optional[float] = None) -> None:
        for k, g in grads.items():
            self.step_param(k, g, lr)

    def state_dict(self) -> Dict[str, object]:
        return dict(m=self.m, v=self.v, t=self.t, lr=self.lr)

    def load_state_dict(self, sd) -> None:
        self.m, self.v, self.t = sd["m"], sd["v"], dict(sd["t"])
        self.lr = sd.get("lr", self.lr)


class Adafactor:
    """Factored second moment for 2-D tensors (row and column statistics), full
    second moment for vectors; no first moment; update clipping by RMS."""

    def __init__(self, params: Dict[str, torch.Tensor], lr: float = 1e-4, decay: float = 0.8,
                 eps: float = 1e-30, clip: float = 1.0, tp_reduce: Optional[Callable] = None):
        self.params, self.lr, self.decay, self.eps, self.clip = params, lr, decay, eps, clip
        self.tp_reduce = tp_reduce  # (name, row_stats, col_stats) -> reduced stats under TP
        self.r: Dict[str, torch.Tensor] = {}
        self.c: Dict[str, torch.Tensor] = {}
        self.v: Dict[str, torch.Tensor] = {}
        self.t: Dict[str, int] = {}

    def step_param(self, name: str, grad: torch.Tensor, lr: Optional[float] = None) -> None:
        p = self.params[name]
        g = grad.float()
        self.t[name] = t = self.t.get(name, 0) + 1
        beta = 1.0 - t ** (-self.decay)
        g2 = g * g + self.eps
        if g.dim() == 2:
            r, c = g2.mean(1), g2.mean(0)
            if self.tp_reduce is not None:
                r, c = self.tp_reduce(name, r, c)
            if name not in self.r:
                self.r[name], self.c[name] = torch.zeros_like(r), torch.zeros_like(c)
            self.r[name].mul_(beta).add_(r, alpha=1 - beta)
            self.c[name].mul_(beta).add_(c, alpha=1 - beta)
            rr, cc = self.r[name], self.c[name]
            vhat = torch.outer(rr / rr.mean().clamp_min(self.eps), cc)
        else:
            if name not in self.v:
                self.v[name] = torch.zeros_like(g2)
            self.v[name].mul_(beta).add_(g2, alpha=1 - beta)
            vhat = self.v[name]
        u = g / vhat.sqrt().clamp_min(1e-30)
        u = u / max(1.0, float(u.pow(2).mean().sqrt()) / self.clip)
        p.copy_((p.float() - (self.lr if lr is None else lr) * u).to(p.dtype))

    def step(self, grads, lr=None):
        for k, g in grads.items():
            self.step_param(k, g, lr)


def newton_schulz_polar(g: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Approximate polar factor U V^T of ``g`` by the quintic Newton-Schulz iteration."""
    a, b, c = 3.4445, -4.7750, 2.0315
    x = g / (g.norm() + 1e-7)
    tr = x.shape[0] > x.shape[1]
    if tr:
        x = x.t()
    for _ in range(steps):
        xx = x @ x.t()
        x = a * x + (b * xx + c * xx @ xx) @ x
    return x.t() if tr else x


class ISO:
    """Orthogonalised update for matrices (polar factor of the momentum, scaled to
    the RMS an Adafactor step would have), Adafactor for everything else."""

    def __init__(self, params: Dict[str, torch.Tensor], lr: float = 1e-4, momentum: float = 0.9,
                 ns_steps: int = 5):
        self.params, self.lr, self.mu, self.ns_steps = params, lr, momentum, ns_steps
        self.buf: Dict[str, torch.Tensor] = {}
        self.fallback = Adafactor(params, lr)

    def step_param(self, name: str, grad: torch.Tensor, lr: Optional[float] = None) -> None:
        p = self.params[name]
        if grad.dim() != 2 or min(grad.shape) < 2:
            return self.fallback.step_param(name, grad, lr)
        g = grad.float()
        b = self.buf.setdefault(name, torch.zeros_like(g))
        b.mul_(self.mu).add_(g)
        u = newton_schulz_polar(b, self.ns_steps)
        scale = math.sqrt(max(1.0, g.shape[0] / g.shape[1]))
        p.copy_((p.float() - (self.lr if lr is None else lr) * scale * u).to(p.dtype))

    def step(self, grads, lr=None):
        for k, g in grads.items():
            self.step_param(k, g, lr)


def make_optimizer(kind: str, params: Dict[str, torch.Tensor], lr: float, **kw):
    kind = kind.lower()
    if kind == "adamw":
        return AdamW(params, lr, **kw)
    if kind == "adafactor":
        return Adafactor(params, lr, **kw)
    if kind == "iso":
        return ISO(params, lr, **kw)
    raise ValueError(f"unknown optimizer {kind!r}")
