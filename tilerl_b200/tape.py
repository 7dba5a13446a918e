"""Hand-written reverse-mode tape.

No ``torch.autograd`` graph is built for the model: every op below runs its
forward under ``no_grad`` and pushes a node ``(inputs, outputs, backward)`` on the
tape; ``Tape.backward`` walks the nodes in reverse, keeps gradients in a dict
keyed by tensor identity, and hands each leaf gradient to ``on_grad`` as soon as
the last node that can contribute to it has run, so an optimizer (or a ZeRO
reduce-scatter) can consume and free it while the rest of backward proceeds.
``checkpoint`` stores only a segment's inputs and replays the segment on a
private tape during backward.

The collectives are ops on the same tape (``tp_fork``: identity forward /
all-reduce backward; ``all_reduce``: the converse), so tensor-parallel training
needs no special casing.

Parity: reference ``src/tilerl/autograd.py`` -- ``RecordingBackend:65``, handler
table ``_BWD:275-301``, ``Tape:304``, ``backward:360``, streaming release
``_release:441``, ``checkpoint:34``; collectives on the tape ``:229-255``.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .ops import ref


class _Node:
    __slots__ = ("inputs", "outputs", "bwd", "name")

    def __init__(self, name, inputs, outputs, bwd):
        self.name, self.inputs, self.outputs, self.bwd = name, inputs, outputs, bwd


class Tape:
    def __init__(self, tp_group=None, tp_world: int = 1):
        self.nodes: List[_Node] = []
        self.leaves: Dict[int, torch.Tensor] = {}
        self.tp_group, self.tp_world = tp_group, tp_world
        self.enabled = True

    # ---- recording -------------------------------------------------------------
    def watch(self, *tensors: torch.Tensor) -> None:
        for t in tensors:
            self.leaves[id(t)] = t

    def record(self, name: str, inputs: Sequence[torch.Tensor], outputs: Sequence[torch.Tensor],
               bwd: Callable) -> None:
        if self.enabled:
            self.nodes.append(_Node(name, tuple(inputs), tuple(outputs), bwd))

    # ---- backward ----------------------------------------------------------------
    def backward(self, root: torch.Tensor, grad: Optional[torch.Tensor] = None,
                 on_grad: Optional[Callable[[torch.Tensor, torch.Tensor], None]] = None
                 ) -> Dict[int, torch.Tensor]:
        grads: Dict[int, torch.Tensor] = {id(root): torch.ones_like(root) if grad is None else grad}
        # first node (in forward order) that reads each leaf = last to contribute in reverse
        first_use: Dict[int, int] = {}
        for idx, n in enumerate(self.nodes):
            for t in n.inputs:
                if id(t) in self.leaves and id(t) not in first_use:
                    first_use[id(t)] = idx
        for idx in range(len(self.nodes) - 1, -1, -1):
            n = self.nodes[idx]
            gouts = [grads.pop(id(o), None) for o in n.outputs]
            if all(g is None for g in gouts):
                continue
            gins = n.bwd(*gouts)
            if not isinstance(gins, (tuple, list)):
                gins = (gins,)
            for t, g in zip(n.inputs, gins):
                if g is None:
                    continue
                k = id(t)
                grads[k] = g if k not in grads else grads[k] + g
            if on_grad is not None:
                for t in n.inputs:
                    k = id(t)
                    if first_use.get(k) == idx and k in grads:
                        on_grad(t, grads.pop(k))
        self.nodes.clear()
        return {k: g for k, g in grads.items() if k in self.leaves}

    def grad_of(self, grads: Dict[int, torch.Tensor], t: torch.Tensor) -> Optional[torch.Tensor]:
        return grads.get(id(t))

    # ---- checkpoint -----------------------------------------------------------------
    def checkpoint(self, fn: Callable, *inputs: torch.Tensor,
                   params: Sequence[torch.Tensor] = ()) -> torch.Tensor:
        """Run ``fn(tape, *inputs)`` without recording and keep only its inputs;
        backward replays it on a private tape.  ``params`` lists the watched leaves
        ``fn`` reads through its closure so their gradients flow out of the segment."""
        was = self.enabled
        self.enabled = False
        try:
            out = fn(self, *inputs)
        finally:
            self.enabled = was
        params = tuple(params)

        def bwd(g):
            sub = Tape(self.tp_group, self.tp_world)
            for t in inputs + params:
                sub.leaves[id(t)] = t
            y = fn(sub, *inputs)
            gs = sub.backward(y, g)
            return tuple(gs.get(id(t)) for t in inputs + params)

        self.record("checkpoint", inputs + params, (out,), bwd)
        return out


# ---- ops ---------------------------------------------------------------------------------
def _nograd(fn):
    def wrapped(*a, **k):
        with torch.no_grad():
            return fn(*a, **k)
    wrapped.__name__ = fn.__name__
    wrapped.__doc__ = fn.__doc__
    return wrapped


@_nograd
def embedding(tape: Tape, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    out = table[ids.long()].float()

    def bwd(g):
        gt = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        gt.index_add_(0, ids.reshape(-1).long(), g.reshape(-1, g.shape[-1]).float())
        return (gt,)

    if id(table) in tape.leaves:        # a frozen table needs no [vocab, hidden] gradient buffer
        tape.record("embedding", (table,), (out,), bwd)
    return out


@_nograd
def rmsnorm(tape: Tape, x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    xn = xf * rstd
    out = xn * w.float()

    def bwd(g):
        g = g.float()
        gw = (g * xn).reshape(-1, x.shape[-1]).sum(0)
        gx = g * w.float()
        dx = rstd * (gx - xn * (gx * xn).mean(-1, keepdim=True))
        return dx, gw

    tape.record("rmsnorm", (x, w), (out,), bwd)
    return out


# Device hook: a CUDA backend installs its NVFP4 -> bf16 dequantisation kernel here so the
# frozen-base linears of the training forward do not run the torch decoder.
DEQUANT_BF16: Optional[Callable] = None


def set_dequant(fn: Optional[Callable]) -> None:
    global DEQUANT_BF16
    DEQUANT_BF16 = fn


@_nograd
def linear(tape: Tape, x: torch.Tensor, w, frozen: bool = False) -> torch.Tensor:
    """``y = x @ W^T``.  ``w`` is a dense master tensor (dX and dW) or a quantised
    weight / ``frozen=True`` dense tensor (dX only, the LoRA-on-frozen-base mode).
    On CUDA the three GEMMs run in bf16 with fp32 accumulation; on CPU everything is fp32
    (the oracle path)."""
    dense = isinstance(w, torch.Tensor)
    if x.is_cuda:
        if dense:
            wf = w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)
        elif DEQUANT_BF16 is not None and hasattr(w, "wq"):
            wf = DEQUANT_BF16(w)
        else:
            wf = w.dequant().to(x.device, torch.bfloat16)
        xb = x.to(torch.bfloat16)
        out = (xb @ wf.t()).float()

        def bwd(g):
            gb = g.to(torch.bfloat16)
            dx = (gb @ wf).float()
            if dense and not frozen:
                dw = (gb.reshape(-1, gb.shape[-1]).t() @ xb.reshape(-1, xb.shape[-1])).float()
                return dx, dw
            return (dx,)

        tape.record("linear", (x, w) if dense and not frozen else (x,), (out,), bwd)
        return out
    wf = w.float() if dense else w.dequant().to(x.device)
    out = x.float() @ wf.t()

    def bwd(g):
        g = g.float()
        dx = g @ wf
        if dense and not frozen:
            dw = g.reshape(-1, g.shape[-1]).t() @ x.float().reshape(-1, x.shape[-1])
            return dx, dw
        return (dx,)

    tape.record("linear", (x, w) if dense and not frozen else (x,), (out,), bwd)
    return out


@_nograd
def add(tape: Tape, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    out = a + b
    tape.record("add", (a, b), (out,), lambda g: (g, g))
    return out


@_nograd
def scale(tape: Tape, a: torch.Tensor, s: float) -> torch.Tensor:
    out = a * s
    tape.record("scale", (a,), (out,), lambda g: (g * s,))
    return out


@_nograd
def swiglu(tape: Tape, gu: torch.Tensor) -> torch.Tensor:
    g_, u_ = gu[..., 0::2].float(), gu[..., 1::2].float()
    sig = torch.sigmoid(g_)
    out = g_ * sig * u_

    def bwd(g):
        dg = g * u_ * sig * (1 + g_ * (1 - sig))
        du = g * g_ * sig
        return (torch.stack([dg, du], -1).flatten(-2),)

    tape.record("swiglu", (gu,), (out,), bwd)
    return out


@_nograd
def attention_block(tape: Tape, qkv: torch.Tensor, q_norm_w: torch.Tensor, k_norm_w: torch.Tensor,
                    positions: torch.Tensor, *, n_q, n_kv, head_dim, rotary_dim, theta, eps,
                    gated=True, cp=None) -> torch.Tensor:
    """Dense causal gated-GQA attention on ``qkv [B, T, rows]``: split, per-head q/k
    RMSNorm, partial RoPE, softmax(QK^T)V, sigmoid gate.  Backward is derived by
    hand (softmax Jacobian, RoPE transpose rotation, RMSNorm).  With a context-parallel
    ``cp`` the rotated K, V and their absolute positions are all-gathered over the ranks
    (the mask compares absolute positions) and dK / dV are reduce-scattered in backward."""
    b, t, _ = qkv.shape
    d, g = head_dim, n_q // n_kv
    x = qkv.float()
    q_rows = n_q * d * (2 if gated else 1)
    if gated:
        qg = x[..., :q_rows].view(b, t, n_q, 2, d)
        q_raw, gate = qg[..., 0, :], qg[..., 1, :]
    else:
        q_raw, gate = x[..., :q_rows].view(b, t, n_q, d), None
    k_raw = x[..., q_rows:q_rows + n_kv * d].view(b, t, n_kv, d)
    v = x[..., q_rows + n_kv * d:].view(b, t, n_kv, d)

    def norm(z, w):
        rstd = torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + eps)
        return z * rstd, rstd

    qn, q_rstd = norm(q_raw, q_norm_w)
    kn, k_rstd = norm(k_raw, k_norm_w)
    half = rotary_dim // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float64, device=x.device) * 2.0 / rotary_dim)
    ang = positions.to(torch.float64)[..., None] * inv
    cos, sin = ang.cos().float(), ang.sin().float()
    if cos.dim() == 2:
        cos, sin = cos[None], sin[None]
    cos, sin = cos[:, :, None, :], sin[:, :, None, :]

    def rope(z, sgn=1.0):
        o = z.clone()
        z1, z2 = z[..., :half], z[..., half:rotary_dim]
        o[..., :half] = z1 * cos - sgn * z2 * sin
        o[..., half:rotary_dim] = z2 * cos + sgn * z1 * sin
        return o

    q = rope(qn * q_norm_w.float())
    k = rope(kn * k_norm_w.float())
    sc = 1.0 / math.sqrt(d)
    qq = q.view(b, t, n_kv, g, d)
    pos = positions if positions.dim() == 2 else positions[None].expand(b, -1)
    k_loc, v_loc = k, v
    if cp is not None:
        from .parallel.cp import gather_kv
        k, v, pos_all = gather_kv(k_loc, v_loc, positions.reshape(-1)[:t].contiguous(), cp)
        kpos = pos_all[None].expand(b, -1)
    else:
        kpos = pos
    s = torch.einsum("bthgd,bshd->bhgts", qq, k) * sc
    mask = kpos[:, None, :] <= pos[:, :, None]                    # [b, t, s]
    s = s.masked_fill(~mask[:, None, None], float("-inf"))
    p = torch.softmax(s, -1)
    o = torch.einsum("bhgts,bshd->bthgd", p, v).reshape(b, t, n_q, d)
    sig = torch.sigmoid(gate) if gated else None
    out = (o * sig if gated else o).reshape(b, t, n_q * d)

    def bwd(gout):
        go = gout.float().view(b, t, n_q, d)
        if gated:
            dgate = go * o * sig * (1 - sig)
            go = go * sig
        gog = go.view(b, t, n_kv, g, d)
        dv = torch.einsum("bhgts,bthgd->bshd", p, gog)
        dp = torch.einsum("bthgd,bshd->bhgts", gog, v)
        ds = p * (dp - (dp * p).sum(-1, keepdim=True))
        dq = torch.einsum("bhgts,bshd->bthgd", ds, k).reshape(b, t, n_q, d) * sc
        dk = torch.einsum("bhgts,bthgd->bshd", ds, qq) * sc
        if cp is not None:
            # reduce-scatter: every rank holds gradients for all ranks' keys / values
            import torch.distributed as dist
            both = torch.stack([dk, dv]).contiguous()
            dist.all_reduce(both, group=cp.group)
            dk, dv = both[0][:, cp.rank * t:(cp.rank + 1) * t], both[1][:, cp.rank * t:(cp.rank + 1) * t]
        dq, dk = rope(dq, -1.0), rope(dk, -1.0)   # transpose of a rotation = inverse rotation

        def norm_bwd(gz, zn, rstd, w):
            gw = (gz * zn).reshape(-1, d).sum(0)
            gx = gz * w.float()
            return rstd * (gx - zn * (gx * zn).mean(-1, keepdim=True)), gw

        dq_raw, gqw = norm_bwd(dq, qn, q_rstd, q_norm_w)
        dk_raw, gkw = norm_bwd(dk, kn, k_rstd, k_norm_w)
        parts = []
        if gated:
            parts.append(torch.stack([dq_raw, dgate], 3).reshape(b, t, q_rows))
        else:
            parts.append(dq_raw.reshape(b, t, q_rows))
        parts += [dk_raw.reshape(b, t, -1), dv.reshape(b, t, -1)]
        return torch.cat(parts, -1), gqw, gkw

    tape.record("attention", (qkv, q_norm_w, k_norm_w), (out,), bwd)
    return out


def _gdn_block_cp(inp, conv_w, dt_bias, a_log, norm_w, *, nk, nv, dk, dv, eps, chunk, cp):
    """Context-parallel GDN block on this rank's two zigzag chunks ``inp [B, 2c, rows]``."""
    from .parallel import cp as CP
    b, t2, _ = inp.shape
    c = t2 // 2
    q_raw, k_raw, v_raw, z, a, bb = ref.gdn_split(inp.float(), nk=nk, nv=nv, dk=dk, dv=dv)
    qkv = torch.cat([q_raw, k_raw, v_raw], -1)
    kw = conv_w.shape[1]
    halo = CP.conv_halo(qkv, kw, cp)                                  # [B, 2, kw-1, C]
    outs = []
    prepped = []
    for i in range(2):
        xp = torch.cat([halo[:, i], qkv[:, i * c:(i + 1) * c]], 1)
        conv = sum(xp[:, j:j + c] * conv_w.float()[:, j] for j in range(kw))
        cc = F.silu(conv)
        qc = cc[..., :nk * dk].view(b, c, nk, dk)
        kc = cc[..., nk * dk:2 * nk * dk].view(b, c, nk, dk)
        vc = cc[..., 2 * nk * dk:].view(b, c, nv, dv)
        rep = nv // nk
        qn = (ref.l2norm(qc) / math.sqrt(dk)).repeat_interleave(rep, 2)
        kn = ref.l2norm(kc).repeat_interleave(rep, 2)
        g, beta = ref.gdn_gates(a[:, i * c:(i + 1) * c], bb[:, i * c:(i + 1) * c], a_log, dt_bias)
        prepped.append((qn, kn, vc, g, beta))
    # chunk summaries: B = state reached from zero, A = the map applied to an identity "state"
    a_loc, b_loc = [], []
    eye = torch.eye(dk, dtype=torch.float32, device=inp.device).expand(b, nv, dk, dk)
    for qn, kn, vc, g, beta in prepped:
        ck = min(chunk, c) if chunk else c
        _, bs = ref.gdn_chunked(qn, kn, vc, g, beta, torch.zeros(b, nv, dk, dv, device=inp.device), chunk=ck)
        _, as_ = ref.gdn_chunked(qn, kn, torch.zeros(b, c, nv, dk, device=inp.device), g, beta, eye, chunk=ck)
        a_loc.append(as_)
        b_loc.append(bs)
    entry = CP.fold_entry_states(torch.stack(a_loc), torch.stack(b_loc), cp)
    for i, (qn, kn, vc, g, beta) in enumerate(prepped):
        ck = min(chunk, c) if chunk else c
        o, _ = ref.gdn_chunked(qn, kn, vc, g, beta, entry[i], chunk=ck)
        outs.append(ref.gdn_gated_norm(o, z[:, i * c:(i + 1) * c].reshape(b, c, nv, dv), norm_w, eps))
    return torch.cat(outs, 1).reshape(b, t2, nv * dv)


def gdn_block_torch(inp, conv_w, dt_bias, a_log, norm_w, *, nk, nv, dk, dv, eps, chunk=64,
                    state=None, cp=None):
    """Differentiable dense GDN block on ``inp [B, T, rows]`` (zero initial state
    and zero conv history): the autograd twin of the serving kernels."""
    if cp is not None:
        return _gdn_block_cp(inp, conv_w, dt_bias, a_log, norm_w, nk=nk, nv=nv, dk=dk, dv=dv, eps=eps,
                             chunk=chunk, cp=cp)
    b, t, _ = inp.shape
    q_raw, k_raw, v_raw, z, a, bb = ref.gdn_split(inp.float(), nk=nk, nv=nv, dk=dk, dv=dv)
    qkv = torch.cat([q_raw, k_raw, v_raw], -1)
    kw = conv_w.shape[1]
    xp = F.pad(qkv, (0, 0, kw - 1, 0))
    conv = sum(xp[:, j:j + t] * conv_w.float()[:, j] for j in range(kw))
    c = F.silu(conv)
    qc = c[..., :nk * dk].view(b, t, nk, dk)
    kc = c[..., nk * dk:2 * nk * dk].view(b, t, nk, dk)
    vc = c[..., 2 * nk * dk:].view(b, t, nv, dv)
    rep = nv // nk
    qn = (ref.l2norm(qc) / math.sqrt(dk)).repeat_interleave(rep, 2)
    kn = ref.l2norm(kc).repeat_interleave(rep, 2)
    g, beta = ref.gdn_gates(a, bb, a_log, dt_bias)
    s0 = torch.zeros(b, nv, dk, dv, dtype=torch.float32, device=inp.device) if state is None else state
    if chunk and t > 1:
        o, _ = ref.gdn_chunked(qn, kn, vc, g, beta, s0, chunk=min(chunk, max(1, t)))
    else:
        o, _ = ref.gdn_recurrent_batched(qn, kn, vc, g, beta, s0)
    out = ref.gdn_gated_norm(o, z.reshape(b, t, nv, dv), norm_w, eps)
    return out.reshape(b, t, nv * dv)


def gdn_block(tape: Tape, inp: torch.Tensor, conv_w, dt_bias, a_log, norm_w, **kw) -> torch.Tensor:
    """GDN block as one tape op.  Forward runs without a graph; backward recomputes
    the block (activation checkpointing at block granularity) and differentiates
    the chunked form locally."""
    with torch.no_grad():
        out = gdn_block_torch(inp, conv_w, dt_bias, a_log, norm_w, **kw)
    params = (conv_w, dt_bias, a_log, norm_w)

    def bwd(g):
        with torch.enable_grad():
            leaves = [t.detach().float().requires_grad_(True) for t in (inp,) + params]
            y = gdn_block_torch(*leaves, **kw)
            gs = torch.autograd.grad(y, leaves, g.float(), allow_unused=True)
        return tuple(gs)

    tape.record("gdn", (inp,) + params, (out,), bwd)
    return out


@_nograd
def cross_entropy(tape: Tape, logits: torch.Tensor, targets: torch.Tensor,
                  weights: torch.Tensor) -> torch.Tensor:
    """``sum_i w_i * nll_i`` over flattened rows; the gradient is produced together
    with the loss (the form used by SFT and by the policy-gradient step)."""
    lg = logits.reshape(-1, logits.shape[-1])
    loss, grad = ref.cross_entropy_grad(lg, targets.reshape(-1), weights.reshape(-1).float())
    grad = grad.view_as(logits)
    tape.record("cross_entropy", (logits,), (loss,), lambda g: (grad * g,))
    return loss


@_nograd
def cross_entropy_tp(tape: Tape, logits: torch.Tensor, targets: torch.Tensor, lp_weights_fn: Callable):
    """Vocab-parallel weighted cross-entropy: ``logits [.., V / tp]`` is this rank's shard.  Three
    all-reduces of per-token scalars (max, sum-exp, picked logit) give every rank the target
    log-probabilities; ``lp_weights_fn(logprobs) -> weights`` and the local gradient shard follow,
    so the full ``[T, V]`` logits are never gathered.  Returns ``(loss, logprobs)``.
    Parity: reference ``tilerl_kernels/reference.py:1541-1603`` (sharded CE)."""
    import torch.distributed as dist
    lg = logits.reshape(-1, logits.shape[-1]).float()
    tg = targets.reshape(-1).long()
    v_local = lg.shape[-1]
    rank = dist.get_rank(tape.tp_group) if tape.tp_world > 1 else 0
    m = lg.amax(-1)
    if tape.tp_world > 1:
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=tape.tp_group)
    se = torch.exp(lg - m[:, None]).sum(-1)
    loc = tg - rank * v_local
    ok = (loc >= 0) & (loc < v_local)
    picked = torch.where(ok, lg.gather(-1, loc.clamp(0, v_local - 1)[:, None]).squeeze(-1), torch.zeros_like(m))
    if tape.tp_world > 1:
        dist.all_reduce(se, group=tape.tp_group)
        dist.all_reduce(picked, group=tape.tp_group)
    lse = m + torch.log(se)
    lp = (picked - lse).view(logits.shape[:-1])
    wts = lp_weights_fn(lp).reshape(-1).float().to(lg.device)
    loss = -(wts * lp.reshape(-1)).sum()
    grad = torch.exp(lg - lse[:, None])
    rows = torch.nonzero(ok).squeeze(-1)
    grad[rows, loc[rows]] -= 1.0
    grad = (grad * wts[:, None]).view_as(logits)
    tape.record("cross_entropy_tp", (logits,), (loss,), lambda g: (grad * g,))
    return loss, lp


@_nograd
def linear_cross_entropy(tape: Tape, h: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, weights_fn: Callable,
                         *, frozen: bool = True, chunk: int = 1024):
    """lm_head + weighted cross-entropy without ever holding ``[T, V]``: the head GEMM runs in
    token chunks twice -- pass 1 collects the log-probability of every target token, the caller's
    ``weights_fn(logprobs [T]) -> weights [T]`` (SFT mask / N, or the PPO-clip weight times the
    advantage) turns them into per-token weights, pass 2 recomputes each chunk's logits and
    immediately folds ``w_i (softmax - onehot)`` into dH (and dW when the head is trainable).
    Returns ``(loss, logprobs)``; the gradients are final, backward only scales them.

    Parity: the reference forms the full logits and overwrites them with the gradient
    (``tilerl_kernels/backend.py:1651-1672``, ``reference.py:1511-1603``)."""
    t_shape = h.shape[:-1]
    hf = h.reshape(-1, h.shape[-1])
    tg = targets.reshape(-1).long()
    n = hf.shape[0]
    cd = torch.bfloat16 if h.is_cuda else torch.float32
    wc = w if w.dtype == cd else w.to(cd)
    lp = torch.empty(n, dtype=torch.float32, device=h.device)
    for a in range(0, n, chunk):
        lg = (hf[a:a + chunk].to(cd) @ wc.t()).float()
        lp[a:a + chunk] = lg.gather(-1, tg[a:a + chunk, None]).squeeze(-1) - torch.logsumexp(lg, -1)
    wts = weights_fn(lp.view(t_shape)).reshape(-1).float().to(h.device)
    loss = -(wts * lp).sum()
    dh = torch.empty(n, hf.shape[-1], dtype=torch.float32, device=h.device)
    dw = None if frozen else torch.zeros(w.shape, dtype=torch.float32, device=h.device)
    for a in range(0, n, chunk):
        hc = hf[a:a + chunk].to(cd)
        lg = (hc @ wc.t()).float()
        g = torch.softmax(lg, -1)
        g[torch.arange(g.shape[0], device=g.device), tg[a:a + chunk]] -= 1.0
        g = (g * wts[a:a + chunk, None]).to(cd)
        dh[a:a + chunk] = (g @ wc).float()
        if dw is not None:
            dw += (g.t() @ hc).float()
    dh = dh.view(h.shape)

    def bwd(g):
        return (dh * g, dw * g) if dw is not None else (dh * g,)

    tape.record("linear_cross_entropy", (h, w) if dw is not None else (h,), (loss,), bwd)
    return loss, lp.view(t_shape)


@_nograd
def tp_fork(tape: Tape, x: torch.Tensor) -> torch.Tensor:
    """Identity forward; all-reduce of the gradient in backward (entry of a
    column-parallel region)."""
    out = x.view_as(x)

    def bwd(g):
        if tape.tp_world > 1:
            import torch.distributed as dist
            g = g.contiguous()
            dist.all_reduce(g, group=tape.tp_group)
        return (g,)

    tape.record("tp_fork", (x,), (out,), bwd)
    return out


@_nograd
def all_reduce(tape: Tape, x: torch.Tensor) -> torch.Tensor:
    """All-reduce forward (exit of a row-parallel region); identity backward."""
    out = x.clone()
    if tape.tp_world > 1:
        import torch.distributed as dist
        dist.all_reduce(out, group=tape.tp_group)
    tape.record("all_reduce", (x,), (out,), lambda g: (g,))
    return out


@_nograd
def lora(tape: Tape, y: torch.Tensor, x: torch.Tensor, a: torch.Tensor, b: torch.Tensor,
         s: float) -> torch.Tensor:
    """``y + s * (x A^T) B^T`` with gradients for x, A and B."""
    xa = x.float() @ a.float().t()
    out = y + (xa @ b.float().t()) * s

    def bwd(g):
        g = g.float()
        g2 = g.reshape(-1, g.shape[-1])
        db = (g2.t() @ xa.reshape(-1, xa.shape[-1])) * s
        dxa = (g @ b.float()) * s
        da = dxa.reshape(-1, dxa.shape[-1]).t() @ x.float().reshape(-1, x.shape[-1])
        return g, dxa @ a.float(), da, db

    tape.record("lora", (y, x, a, b), (out,), bwd)
    return out
