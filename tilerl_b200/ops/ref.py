"""fp32 torch oracle for every op of the hybrid model.

These functions are the executable specification: each CUDA kernel in
``csrc/`` is tested against the function of the same name here, and the CPU
engine / training tests run the whole model through them.

Activations are *flat over tokens* (``[T, ...]``): a tick's tokens from all
sequences are concatenated, and per-token ``positions`` / ``seq_ids`` say where
each belongs.  There is no padding row anywhere in the serving path.

Row layouts of the fused projections (shared with the kernels and the
checkpoint loader):

* attention ``qkv``: ``[hq x (query D ; gate D)] ++ [hkv x D] ++ [hkv x D]``
* GDN ``in``:  ``[q nk*dk ; k nk*dk ; v nv*dv ; z nv*dv ; a nv ; b nv]``
* MLP ``gate_up``: rows interleaved, ``2j`` = gate_j, ``2j+1`` = up_j

Parity: the maths follows reference
``packages/tilerl-kernels/src/tilerl_kernels/reference.py`` -- partial RoPE
``:84-97``, attention prelude ``:99-134``, GDN prep ``:1142-1200`` and the
decay-first delta rule ``:1202-1277``, sharded cross-entropy ``:1541-1603``,
sampling ``:1656-1720``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

KV_BLOCK = 16  # tokens per KV page


def _f(x: torch.Tensor) -> torch.Tensor:
    return x.float()


# ---- elementwise / norm ---------------------------------------------------------
def rmsnorm(x, w, eps: float):
    x = _f(x)
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * _f(w)


def swiglu(gate_up):
    gu = _f(gate_up)
    return F.silu(gu[..., 0::2]) * gu[..., 1::2]


def embedding(table, ids):
    return _f(table)[ids.long()]


def rope_partial(x, positions, theta: float, rotary_dim: int):
    """rotate-half RoPE on the leading ``rotary_dim`` dims of ``x [T, heads, D]``."""
    x = _f(x)
    half = rotary_dim // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float64, device=x.device) * 2.0 / rotary_dim)
    ang = positions.to(torch.float64)[:, None] * inv[None, :]
    cos, sin = ang.cos().float()[:, None, :], ang.sin().float()[:, None, :]
    x1, x2 = x[..., :half], x[..., half:rotary_dim]
    out = x.clone()
    out[..., :half] = x1 * cos - x2 * sin
    out[..., half:rotary_dim] = x2 * cos + x1 * sin
    return out


# ---- attention ---------------------------------------------------------------------
def attn_prep(qkv, q_norm_w, k_norm_w, positions, *, n_q, n_kv, head_dim, rotary_dim,
              theta, eps, gated=True):
    """Split the fused qkv rows, per-head RMSNorm q and k (fp32), partial RoPE.
    Returns q, gate (or None), k, v as ``[T, heads, D]`` fp32."""
    qkv = _f(qkv)
    t = qkv.shape[0]
    d = head_dim
    q_rows = n_q * d * (2 if gated else 1)
    qg = qkv[:, :q_rows]
    if gated:
        qg = qg.view(t, n_q, 2, d)
        q, gate = qg[:, :, 0], qg[:, :, 1]
    else:
        q, gate = qg.view(t, n_q, d), None
    k = qkv[:, q_rows:q_rows + n_kv * d].view(t, n_kv, d)
    v = qkv[:, q_rows + n_kv * d:].view(t, n_kv, d)
    q = rope_partial(rmsnorm(q, q_norm_w, eps), positions, theta, rotary_dim)
    k = rope_partial(rmsnorm(k, k_norm_w, eps), positions, theta, rotary_dim)
    return q, gate, k, v.clone()


def kv_write_fp8(kcache, vcache, kscale, vscale, k, v, slot_mapping):
    """fp8 KV: e4m3 values with one fp32 scale per (token, head) = amax / 448 (K taken after
    RoPE).  Pools ``[blocks, hkv, 16, D]`` fp8, scales ``[blocks, hkv, 16]``."""
    from ..formats import quantize_kv_fp8
    k8, ks = quantize_kv_fp8(k)
    v8, vs = quantize_kv_fp8(v)
    for t in range(k.shape[0]):
        s = int(slot_mapping[t])
        if s < 0:
            continue
        b, o = divmod(s, KV_BLOCK)
        kcache[b, :, o] = k8[t]
        vcache[b, :, o] = v8[t]
        kscale[b, :, o] = ks[t]
        vscale[b, :, o] = vs[t]


def kv_dequant_fp8(cache, scale):
    """The fp32 view of an fp8 pool layer (oracle path: the kernels dequantise at the gather)."""
    return cache.float() * scale.unsqueeze(-1)


def kv_write(kcache, vcache, k, v, slot_mapping):
    """Scatter token rows into the paged pools ``[blocks, hkv, 16, D]``;
    ``slot_mapping[t] = block * 16 + offset`` (negative = skip)."""
    for t in range(k.shape[0]):
        s = int(slot_mapping[t])
        if s < 0:
            continue
        b, o = divmod(s, KV_BLOCK)
        kcache[b, :, o] = k[t].to(kcache.dtype)
        vcache[b, :, o] = v[t].to(vcache.dtype)


def gather_kv(cache, block_row, length: int):
    """``[blocks, hkv, 16, D]`` pool -> ``[length, hkv, D]`` of one sequence."""
    nb = (length + KV_BLOCK - 1) // KV_BLOCK
    pages = cache[block_row[:nb].long()]                # [nb, hkv, 16, D]
    return _f(pages).permute(0, 2, 1, 3).reshape(nb * KV_BLOCK, cache.shape[1], -1)[:length]


def paged_attention(q, gate, kcache, vcache, block_table, seq_ids, positions, scale: float):
    """Causal GQA over paged KV.  Token ``t`` of sequence ``seq_ids[t]`` at position
    ``p`` attends to KV positions ``0..p``.  Output ``[T, hq*D]`` after the sigmoid
    output gate (reference ``src/tilerl/testing.py:229-235``)."""
    q = _f(q)
    t, hq, d = q.shape
    hkv = kcache.shape[1]
    g = hq // hkv
    out = torch.zeros(t, hq, d, dtype=torch.float32, device=q.device)
    for i in range(t):
        row = int(seq_ids[i])
        n = int(positions[i]) + 1
        kk = gather_kv(kcache, block_table[row], n)     # [n, hkv, D]
        vv = gather_kv(vcache, block_table[row], n)
        qi = q[i].view(hkv, g, d)
        s = torch.einsum("hgd,nhd->hgn", qi, kk) * scale
        p = torch.softmax(s, dim=-1)
        out[i] = torch.einsum("hgn,nhd->hgd", p, vv).reshape(hq, d)
    if gate is not None:
        out = out * torch.sigmoid(_f(gate))
    return out.reshape(t, hq * d)


def sparse_paged_attention(q, gate, kcache, vcache, page_lists, page_counts, seq_ids,
                           positions, scale: float):
    """Top-k sparse variant: token ``t`` attends only to the pages listed for its
    sequence, ``page_lists[row, :page_counts[row]]`` holding *logical* page
    numbers already translated to physical blocks in sequence order, together
    with each page's first logical position in ``page_lists[row, :, 1]``."""
    q = _f(q)
    t, hq, d = q.shape
    hkv = kcache.shape[1]
    g = hq // hkv
    out = torch.zeros(t, hq, d, dtype=torch.float32, device=q.device)
    for i in range(t):
        row = int(seq_ids[i])
        pos = int(positions[i])
        ks, vs = [], []
        for j in range(int(page_counts[row])):
            blk, first = int(page_lists[row, j, 0]), int(page_lists[row, j, 1])
            n = min(KV_BLOCK, pos + 1 - first)
            if n <= 0:
                continue
            ks.append(_f(kcache[blk])[:, :n].transpose(0, 1))
            vs.append(_f(vcache[blk])[:, :n].transpose(0, 1))
        kk, vv = torch.cat(ks), torch.cat(vs)
        s = torch.einsum("hgd,nhd->hgn", q[i].view(hkv, g, d), kk) * scale
        out[i] = torch.einsum("hgn,nhd->hgd", torch.softmax(s, -1), vv).reshape(hq, d)
    if gate is not None:
        out = out * torch.sigmoid(_f(gate))
    return out.reshape(t, hq * d)


def dense_attention(q, k, v, gate, scale: float, q_pos=None, k_pos=None):
    """Training-path causal GQA on dense ``[B, T, heads, D]`` tensors.  With
    ``q_pos``/``k_pos`` the mask is ``k_pos <= q_pos`` (context-parallel chunks)."""
    q, k, v = _f(q), _f(k), _f(v)
    b, t, hq, d = q.shape
    hkv = k.shape[2]
    g = hq // hkv
    qq = q.view(b, t, hkv, g, d)
    s = torch.einsum("bthgd,bshd->bhgts", qq, k) * scale
    if q_pos is None:
        q_pos = torch.arange(t, device=q.device)
        k_pos = torch.arange(k.shape[1], device=q.device)
    mask = k_pos[None, :] <= q_pos[:, None]
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bhgts,bshd->bthgd", p, v).reshape(b, t, hq, d)
    if gate is not None:
        o = o * torch.sigmoid(_f(gate))
    return o.reshape(b, t, hq * d)


# ---- Quest-style page index (sparse KV) ---------------------------------------------------
def page_bounds(kcache_block):
    """Per (kv head) element-wise min and max over a page's tokens: ``[hkv, 2, D]``."""
    kb = _f(kcache_block)
    return torch.stack([kb.amin(1), kb.amax(1)], dim=1)


def page_bound_scores(q, bounds):
    """Upper bound of q.k over each page: sum_d max(q*kmin, q*kmax), summed over the
    GQA group and kv heads.  ``q [hq, D]``, ``bounds [P, hkv, 2, D]`` -> ``[P]``."""
    q = _f(q)
    hkv = bounds.shape[1]
    qg = q.view(hkv, -1, q.shape[-1])
    lo = qg[None, :, :, :] * bounds[:, :, None, 0, :]
    hi = qg[None, :, :, :] * bounds[:, :, None, 1, :]
    return torch.maximum(lo, hi).sum(-1).sum((1, 2))


def select_pages(scores, n_pages: int, top_k: int, window: int):
    """top-k pages united with the trailing ``window`` pages, in sequence order."""
    keep = set(range(max(0, n_pages - window), n_pages))
    early = n_pages - len(keep)
    if early > 0 and top_k > 0:
        k = min(top_k, early)
        keep |= set(torch.topk(scores[:early], k).indices.tolist())
    return sorted(keep)


# ---- Gated DeltaNet -------------------------------------------------------------------------
def gdn_split(inp, *, nk, nv, dk, dv):
    """Fused GDN projection rows -> q, k, v (raw, pre-conv), z, a, b."""
    qd, vd = nk * dk, nv * dv
    o = 0
    parts = []
    for w in (qd, qd, vd, vd, nv, nv):
        parts.append(inp[..., o:o + w])
        o += w
    return parts


def gdn_gates(a, b, a_log, dt_bias):
    """log-decay g = -exp(A_log) * softplus(a + dt_bias); beta = sigmoid(b)."""
    g = -torch.exp(_f(a_log)) * F.softplus(_f(a) + _f(dt_bias))
    return g, torch.sigmoid(_f(b))


def gdn_conv_silu(raw_rows, conv_w):
    """Depthwise causal conv over a window of raw rows.  ``raw_rows [W, C]`` holds
    the rows at positions p-(W-1) .. p (older first; zeros before position 0),
    ``conv_w [C, W]`` with tap W-1 multiplying the newest row."""
    return F.silu((_f(raw_rows) * _f(conv_w).t()).sum(0))


def l2norm(x, eps: float = 1e-12):
    return x / torch.sqrt(x.pow(2).sum(-1, keepdim=True) + eps)


def gdn_recurrent_step(state, q, k, v, g, beta):
    """One decay-first delta-rule step on ``state [nv, dk, dv]`` (fp32, updated
    copy returned).  ``q, k [nv, dk]`` already normalised and expanded to value
    heads; ``v [nv, dv]``; ``g, beta [nv]``."""
    s = state * torch.exp(g)[:, None, None]
    p = torch.einsum("hk,hkv->hv", k, s)
    d = (v - p) * beta[:, None]
    s = s + k[:, :, None] * d[:, None, :]
    o = torch.einsum("hk,hkv->hv", q, s)
    return s, o


def gdn_gated_norm(o, z, norm_w, eps: float):
    """RMSNorm over the value dim times weight, gated by silu(z).  ``[.., nv, dv]``."""
    return o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * _f(norm_w) * F.silu(_f(z))


def gdn_sequence(inp, positions, state, ring, *, conv_w, dt_bias, a_log, norm_w,
                 nk, nv, dk, dv, eps, step_states=None):
    """Run the GDN core over the tokens of ONE sequence.

    ``inp [T, rows]`` fused projection output; ``state [nv, dk, dv]`` fp32 (updated
    in place); ``ring [R, C]`` raw-qkv ring buffer indexed by ``position % R``
    (updated in place).  If ``step_states`` (``[>=T, nv, dk, dv]``) is given the
    state after each token is stored there (speculative verify).  Returns
    ``[T, nv*dv]`` fp32."""
    inp = _f(inp)
    t = inp.shape[0]
    kw = conv_w.shape[1]
    r = ring.shape[0]
    q_raw, k_raw, v_raw, z, a, b = gdn_split(inp, nk=nk, nv=nv, dk=dk, dv=dv)
    g_all, beta_all = gdn_gates(a, b, a_log, dt_bias)
    rep = nv // nk
    out = torch.zeros(t, nv, dv, dtype=torch.float32, device=inp.device)
    s = state.clone()
    for i in range(t):
        pos = int(positions[i])
        ring[pos % r] = torch.cat([q_raw[i], k_raw[i], v_raw[i]]).to(ring.dtype)
        rows = []
        for j in range(kw - 1, -1, -1):
            pj = pos - j
            rows.append(_f(ring[pj % r]) if pj >= 0 else torch.zeros_like(_f(ring[0])))
        c = gdn_conv_silu(torch.stack(rows), conv_w)
        qc = c[:nk * dk].view(nk, dk)
        kc = c[nk * dk:2 * nk * dk].view(nk, dk)
        vc = c[2 * nk * dk:].view(nv, dv)
        qn = (l2norm(qc) / math.sqrt(dk)).repeat_interleave(rep, 0)
        kn = l2norm(kc).repeat_interleave(rep, 0)
        s, o = gdn_recurrent_step(s, qn, kn, vc, g_all[i], beta_all[i])
        if step_states is not None:
            step_states[i] = s
        out[i] = gdn_gated_norm(o, z[i].view(nv, dv), norm_w, eps)
    state.copy_(s)
    return out.reshape(t, nv * dv)


def gdn_chunked(q, k, v, g, beta, state, chunk: int = 64):
    """Chunk-parallel (WY) form of the same recurrence, batched.

    ``q, k [B, T, H, dk]`` (normalised), ``v [B, T, H, dv]``, ``g, beta [B, T, H]``,
    ``state [B, H, dk, dv]``.  Returns ``(o [B,T,H,dv], final_state)``.  Built only
    from differentiable torch ops, so it also serves as the autograd twin of the
    hand-written backward."""
    b, t, h, dk = q.shape
    dv = v.shape[-1]
    pad = (-t) % chunk
    if pad:
        q, k, v = (F.pad(x, (0, 0, 0, 0, 0, pad)) for x in (q, k, v))
        g, beta = F.pad(g, (0, 0, 0, pad)), F.pad(beta, (0, 0, 0, pad))
    n = (t + pad) // chunk
    # [B, H, n, C, *]
    q, k, v = (x.transpose(1, 2).reshape(b, h, n, chunk, -1) for x in (q, k, v))
    g = g.transpose(1, 2).reshape(b, h, n, chunk)
    beta = beta.transpose(1, 2).reshape(b, h, n, chunk)
    gc = g.cumsum(-1)                                   # G_i
    eye = torch.eye(chunk, device=q.device, dtype=q.dtype)
    strict = torch.tril(torch.ones(chunk, chunk, device=q.device, dtype=torch.bool), -1)
    incl = torch.tril(torch.ones(chunk, chunk, device=q.device, dtype=torch.bool), 0)
    # e^{G_i - G_j} for j <= i; the exponent is masked *before* exp so the upper
    # triangle (positive, possibly overflowing) never produces inf * 0 in backward
    dec = torch.exp((gc[..., :, None] - gc[..., None, :]).masked_fill(~incl, float("-inf")))
    kk = torch.einsum("bhnik,bhnjk->bhnij", k, k)
    a = (beta[..., :, None] * kk * dec).masked_fill(~strict, 0.0)
    tmat = torch.linalg.solve_triangular(eye + a, eye.expand_as(a), upper=False)
    w = tmat @ (k * (beta * torch.exp(gc))[..., None])
    u = tmat @ (v * beta[..., None])
    qk = (torch.einsum("bhnik,bhnjk->bhnij", q, k) * dec).masked_fill(~incl, 0.0)
    s = state
    outs = []
    for c in range(n):
        v_new = u[:, :, c] - w[:, :, c] @ s
        o = (q[:, :, c] * torch.exp(gc[:, :, c])[..., None]) @ s + qk[:, :, c] @ v_new
        outs.append(o)
        last = gc[:, :, c, -1]
        kd = k[:, :, c] * torch.exp(last[..., None] - gc[:, :, c])[..., None]
        s = s * torch.exp(last)[..., None, None] + kd.transpose(-1, -2) @ v_new
    o = torch.stack(outs, 2).reshape(b, h, n * chunk, dv).transpose(1, 2)[:, :t]
    return o, s


def gdn_recurrent_batched(q, k, v, g, beta, state):
    """Token-serial form on the same batched layout as :func:`gdn_chunked`."""
    b, t, h, dk = q.shape
    s = state.clone()
    outs = []
    for i in range(t):
        s = s * torch.exp(g[:, i])[..., None, None]
        p = torch.einsum("bhk,bhkv->bhv", k[:, i], s)
        d = (v[:, i] - p) * beta[:, i][..., None]
        s = s + k[:, i][..., :, None] * d[..., None, :]
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, i], s))
    return torch.stack(outs, 1), s


def gdn_recurrent_backward(q, k, v, g, beta, state, d_out, d_state_final=None):
    """Hand-derived adjoint of :func:`gdn_recurrent_batched` (reverse-time scan).
    Returns (dq, dk, dv, dg, dbeta, dstate0)."""
    b, t, h, dk = q.shape
    states = [state]
    s = state
    for i in range(t):
        s_t = s * torch.exp(g[:, i])[..., None, None]
        p = torch.einsum("bhk,bhkv->bhv", k[:, i], s_t)
        d = (v[:, i] - p) * beta[:, i][..., None]
        s = s_t + k[:, i][..., :, None] * d[..., None, :]
        states.append(s)
    dq, dkk, dvv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    dg, db = torch.zeros_like(g), torch.zeros_like(beta)
    ds = torch.zeros_like(state) if d_state_final is None else d_state_final.clone()
    for i in range(t - 1, -1, -1):
        s_prev, s_cur = states[i], states[i + 1]
        a = torch.exp(g[:, i])
        s_t = s_prev * a[..., None, None]
        p = torch.einsum("bhk,bhkv->bhv", k[:, i], s_t)
        resid = v[:, i] - p
        d = resid * beta[:, i][..., None]
        do = d_out[:, i]
        ds = ds + q[:, i][..., :, None] * do[..., None, :]
        dq[:, i] = torch.einsum("bhkv,bhv->bhk", s_cur, do)
        dkk[:, i] = torch.einsum("bhkv,bhv->bhk", ds, d)
        dd = torch.einsum("bhkv,bhk->bhv", ds, k[:, i])
        db[:, i] = (dd * resid).sum(-1)
        dvv[:, i] = dd * beta[:, i][..., None]
        dp = -dvv[:, i]
        ds_t = ds + k[:, i][..., :, None] * dp[..., None, :]
        dkk[:, i] += torch.einsum("bhkv,bhv->bhk", s_t, dp)
        dg[:, i] = (ds_t * s_prev).sum((-1, -2)) * a
        ds = ds_t * a[..., None, None]
    return dq, dkk, dvv, dg, db, ds


# ---- linear -----------------------------------------------------------------------------------
def dequant_weight(w) -> torch.Tensor:
    """Any served weight representation -> fp32 ``[N, K]``."""
    if isinstance(w, torch.Tensor):
        return _f(w)
    return w.dequant()


def linear(x, w, residual=None):
    y = _f(x) @ dequant_weight(w).t().to(x.device)
    return y if residual is None else y + _f(residual)


# ---- loss / sampling -----------------------------------------------------------------------------
def cross_entropy_grad(logits, targets, weights):
    """Weighted token CE: ``loss = sum_i w_i * (lse_i - logit_i[target_i])`` and its
    gradient w.r.t. logits.  ``weights`` already carry 1/N and the advantage."""
    lg = _f(logits)
    lse = torch.logsumexp(lg, -1)
    picked = lg.gather(-1, targets.long()[:, None]).squeeze(-1)
    loss = (weights * (lse - picked)).sum()
    grad = torch.softmax(lg, -1)
    grad[torch.arange(lg.shape[0]), targets.long()] -= 1.0
    return loss, grad * weights[:, None]


def cross_entropy_sharded(logits_shards, targets, weights, vocab_starts):
    """Vocab-parallel CE from per-rank partials (max, sum-exp, picked) so the full
    ``[T, V]`` logits are never concatenated.  Returns (loss, [grad per shard])."""
    maxes = torch.stack([_f(l).amax(-1) for l in logits_shards]).amax(0)
    sumexp = sum(torch.exp(_f(l) - maxes[:, None]).sum(-1) for l in logits_shards)
    picked = torch.zeros_like(maxes)
    for l, s in zip(logits_shards, vocab_starts):
        loc = targets.long() - s
        ok = (loc >= 0) & (loc < l.shape[-1])
        picked += torch.where(ok, _f(l).gather(-1, loc.clamp(0, l.shape[-1] - 1)[:, None]).squeeze(-1),
                              torch.zeros_like(picked))
    lse = maxes + torch.log(sumexp)
    loss = (weights * (lse - picked)).sum()
    grads = []
    for l, s in zip(logits_shards, vocab_starts):
        gsh = torch.exp(_f(l) - lse[:, None])
        loc = targets.long() - s
        ok = (loc >= 0) & (loc < l.shape[-1])
        rows = torch.arange(l.shape[0])[ok]
        gsh[rows, loc[ok]] -= 1.0
        grads.append(gsh * weights[:, None])
    return loss, grads


def token_logprobs(logits, targets):
    lg = _f(logits)
    return lg.gather(-1, targets.long()[:, None]).squeeze(-1) - torch.logsumexp(lg, -1)


def sample_seed(seed: int, index: int) -> int:
    """Per-(request, generated-index) stream seed (splitmix-style mix)."""
    x = (seed * 0x9E3779B97F4A7C15 + (index + 1) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    x ^= x >> 31
    return x & 0x7FFFFFFFFFFFFFFF


def sample(logits_row, temperature: float, top_p: float, top_k: int, seed: int,
           allowed: Optional[torch.Tensor] = None) -> Tuple[int, float]:
    """One row: greedy when temperature == 0, else temperature -> allowed-ids /
    top-k restriction -> top-p nucleus (renormalised) -> seeded multinomial.  The
    returned logprob is under the nucleus distribution."""
    lg = _f(logits_row).clone()
    if allowed is not None:
        mask = torch.full_like(lg, float("-inf"))
        mask[allowed.long()] = 0.0
        lg = lg + mask
    if temperature <= 0.0:
        tok = int(torch.argmax(lg))
        return tok, float(torch.log_softmax(lg, -1)[tok])
    lg = lg / temperature
    if top_k and top_k < lg.numel():
        kth = torch.topk(lg, top_k).values[-1]
        lg = torch.where(lg < kth, torch.full_like(lg, float("-inf")), lg)
    probs = torch.softmax(lg, -1)
    if top_p < 1.0:
        sp, si = torch.sort(probs, descending=True)
        cum = sp.cumsum(0)
        cut = (cum - sp) >= top_p
        sp = torch.where(cut, torch.zeros_like(sp), sp)
        probs = torch.zeros_like(probs).scatter_(0, si, sp)
        probs = probs / probs.sum()
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    tok = int(torch.multinomial(probs.cpu(), 1, generator=gen))
    return tok, float(torch.log(probs[tok]))


def sample_nucleus_model(logits_row, temperature: float, top_k: int, top_p: float, u: float):
    """Executable model of the device top-k / top-p sampler (``csrc/misc.cu``:
    ``sample_nucleus_kernel``), which never sorts: every logit is keyed by its distance below the
    row maximum in 2^-19 nat steps (24 bits, clamped) and weighted by an integer mass
    ``exp(-distance) * 2^40``; the k-th key and the nucleus bound are the smallest keys whose
    cumulative count / mass reaches ``k`` / ``top_p * Z``; the draw is the inverse CDF at ``u`` over
    the kept masses in vocabulary order.  Returns ``(kept mask, token, logprob)``.  The kept set
    equals :func:`sample`'s (up to keys closer than 2^-19 nat, which are kept together)."""
    import numpy as np
    s = (np.asarray(logits_row, dtype=np.float32) * np.float32(1.0 / temperature)).astype(np.float32)
    d = (s.max() - s).astype(np.float32)
    qf = d * np.float32(524288.0)
    q = np.where((qf >= 16777215.0) | np.isnan(qf), 0xFFFFFF, qf.astype(np.int64))
    m = np.where(q == 0xFFFFFF, 0, (np.exp(-d.astype(np.float64)).astype(np.float32) * np.float32(2.0 ** 40)).astype(np.int64))

    def select(weight, need, qcap):
        """Smallest key t with weight{q <= t, q <= qcap} >= need, by three 8-bit digits."""
        prefix = 0
        for ps in range(3):
            shift = 16 - 8 * ps
            ok = q <= qcap
            if ps:
                ok &= (q >> (shift + 8)) == prefix
            hist = np.zeros(256, dtype=np.int64)
            np.add.at(hist, (q[ok] >> shift) & 255, weight[ok])
            cum, b = 0, 255
            for j in range(256):
                if cum + hist[j] >= need:
                    b, need = j, need - cum
                    break
                cum += hist[j]
            prefix = (prefix << 8) | b
        return prefix

    v = s.shape[0]
    qcut = 0xFFFFFF
    if 0 < top_k < v:
        qcut = select(np.ones(v, dtype=np.int64), top_k, 0xFFFFFF)
    if top_p < 1.0:
        z = int(m[q <= qcut].sum())
        qcut = min(qcut, select(m, max(1, int(top_p * float(z))), qcut))
    kept = (q <= qcut) & (m > 0)
    mm = np.where(kept, m, 0)
    cs = np.cumsum(mm)
    total = int(cs[-1])
    target = min(total - 1, int(u * float(total)))
    tok = int(np.searchsorted(cs, target, side="right"))
    return torch.from_numpy(kept), tok, float(np.log(mm[tok] / total))
