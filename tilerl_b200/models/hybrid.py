"""The hybrid decoder: embedding -> N x (gated-GQA attention | Gated DeltaNet) +
SwiGLU MLP -> final norm -> lm_head.

``HybridModel`` owns a flat parameter dict and runs the *serving* forward over a
flat-token :class:`~tilerl_b200.batch.Batch` through an ops backend
(:class:`~tilerl_b200.ops.backend.RefOps` on CPU,
:class:`~tilerl_b200.ops.cuda.CudaOps` on B200).  Per layer the backend is
called at the granularity of the fused kernels:

* attention layer: ``norm_linear`` (RMSNorm folded into the qkv GEMV/GEMM) ->
  ``attention`` (q/k norm + RoPE + KV write + paged attention + sigmoid gate) ->
  ``linear_residual`` (o_proj, residual add and the TP reduction in its epilogue)
* GDN layer: ``norm_linear`` (fused q/k/v/z/a/b projection) -> ``gdn`` ->
  ``linear_residual``
* MLP: ``norm_linear_swiglu`` -> ``linear_residual``

Parameter names: ``embed``, ``lm_head``, ``final_norm`` and per layer
``L{i}.norm1|norm2|gate_up|down`` plus ``qkv|q_norm|k_norm|o`` or
``in|conv|dt_bias|a_log|gdn_norm|out``.  Master (bf16/fp32) copies used by
training live under ``master.<name>``.

Parity: reference ``src/tilerl/model.py`` -- ``param_specs:38``,
``_fuse_projections:186``, ``Model.forward:639-721``, ``add_lora:724``,
``build_random:775``, ``requantize_fp4:1255``.
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..config import ATTN, GDN, ModelConfig
from ..formats import (FP8BlockTensor, NVFP4Tensor, quantize_fp8_block, quantize_nvfp4)

LINEAR_KEYS_ATTN = ("qkv", "o")
LINEAR_KEYS_GDN = ("in", "out")
LINEAR_KEYS_MLP = ("gate_up", "down")


def linear_names(cfg: ModelConfig) -> List[str]:
    """Every quantisable projection, in forward order."""
    names = []
    for i, t in enumerate(cfg.layer_types):
        keys = (LINEAR_KEYS_ATTN if t == ATTN else LINEAR_KEYS_GDN) + LINEAR_KEYS_MLP
        names += [f"L{i}.{k}" for k in keys]
    return names


def param_shapes(cfg: ModelConfig, tp: int = 1) -> Dict[str, Tuple[int, ...]]:
    """Logical (unquantised) shape of every parameter at TP degree ``tp``."""
    from ..parallel.mesh import tp_dims
    d = tp_dims(cfg, tp)
    h = cfg.hidden
    shapes: Dict[str, Tuple[int, ...]] = {"embed": (cfg.vocab, h), "final_norm": (h,)}
    if not cfg.tie_embeddings:
        shapes["lm_head"] = (d.vocab_local, h)
    for i, t in enumerate(cfg.layer_types):
        p = f"L{i}."
        shapes[p + "norm1"] = (h,)
        shapes[p + "norm2"] = (h,)
        if t == ATTN:
            shapes[p + "qkv"] = (d.qkv_rows, h)
            shapes[p + "o"] = (h, d.n_q * cfg.head_dim)
            shapes[p + "q_norm"] = (cfg.head_dim,)
            shapes[p + "k_norm"] = (cfg.head_dim,)
        else:
            shapes[p + "in"] = (d.gdn_in_rows, h)
            shapes[p + "out"] = (h, d.gdn_nv * cfg.gdn_head_dim)
            shapes[p + "conv"] = (d.gdn_conv_dim, cfg.gdn_conv)
            shapes[p + "dt_bias"] = (d.gdn_nv,)
            shapes[p + "a_log"] = (d.gdn_nv,)
            shapes[p + "gdn_norm"] = (cfg.gdn_head_dim,)
        shapes[p + "gate_up"] = (2 * d.ffn, h)
        shapes[p + "down"] = (h, d.ffn)
    return shapes


def quantize_weight(w: torch.Tensor, quant: str):
    if quant == "nvfp4":
        return quantize_nvfp4(w)
    if quant == "fp8":
        return quantize_fp8_block(w)
    return w


def random_master(cfg: ModelConfig, seed: int = 0, device="cpu", dtype=torch.float32,
                  std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Full (TP=1) master parameters: projections N(0, std), norm weights 1,
    ``a_log`` = log U(1, 16), ``dt_bias`` small.  Generated on CPU per tensor so the
    stream is identical on every rank and device."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for name, shape in param_shapes(cfg, 1).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2", "final_norm", "q_norm", "k_norm", "gdn_norm"):
            t = torch.ones(shape)
        elif leaf == "a_log":
            t = torch.log(torch.empty(shape).uniform_(1.0, 16.0, generator=g))
        elif leaf == "dt_bias":
            t = torch.empty(shape).uniform_(-1.0, 1.0, generator=g)
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) * 0.3
        else:
            t = torch.randn(shape, generator=g) * std
        out[name] = t.to(device=device, dtype=dtype if t.dim() == 2 and leaf != "conv" else torch.float32)
    return out


class HybridModel:
    def __init__(self, cfg: ModelConfig, params: Dict[str, object], tp_rank: int = 0,
                 tp: int = 1):
        from ..parallel.mesh import tp_dims
        self.cfg = cfg
        self.params = params
        self.tp, self.tp_rank = tp, tp_rank
        self.dims = tp_dims(cfg, tp)
        self.lora: Dict[str, Tuple[torch.Tensor, torch.Tensor, float]] = {}
        self.weights_version = 0

    # ---- construction ---------------------------------------------------------
    @classmethod
    def from_master(cls, cfg: ModelConfig, master: Dict[str, torch.Tensor], *, tp_rank=0, tp=1,
                    device=None, keep_master: bool = False, quant: Optional[str] = None,
                    act_dtype=torch.bfloat16) -> "HybridModel":
        """Shard (TP) and quantise a full master dict into serving parameters."""
        from ..parallel.mesh import shard_param
        quant = quant or cfg.quant
        params: Dict[str, object] = {}
        lin = set(linear_names(cfg))
        for name, w in master.items():
            ws = shard_param(cfg, name, w, tp_rank, tp)
            if device is not None:
                ws = ws.to(device)
            if name in lin or (name == "lm_head" and cfg.lm_head_quant == "nvfp4"):
                if quant == "nvfp4" or name == "lm_head":
                    # quantise the FULL tensor, then cut the packed planes: every TP degree
                    # serves exactly the same quantised values
                    q = shard_param(cfg, name, quantize_nvfp4(w.float()), tp_rank, tp)
                    params[name] = q.to(device) if device is not None else q
                else:
                    params[name] = quantize_weight(ws.float(), quant)
                if keep_master and name in lin:
                    params["master." + name] = ws.clone()
            elif ws.dim() == 2 and name in ("embed", "lm_head"):
                params[name] = ws.to(act_dtype)
            else:
                params[name] = ws.float()
        return cls(cfg, params, tp_rank, tp)

    @classmethod
    def build_random(cls, cfg: ModelConfig, seed: int = 0, device="cpu", *, tp_rank=0, tp=1,
                     keep_master=False, act_dtype=torch.float32, quant=None) -> "HybridModel":
        master = random_master(cfg, seed, "cpu")
        return cls.from_master(cfg, master, tp_rank=tp_rank, tp=tp, device=device,
                               keep_master=keep_master, quant=quant, act_dtype=act_dtype)

    def layer_params(self, i: int) -> Dict[str, object]:
        p = f"L{i}."
        return {k[len(p):]: v for k, v in self.params.items() if k.startswith(p)}

    # ---- LoRA -------------------------------------------------------------------------
    def add_lora(self, rank: int = 16, alpha: float = 32.0, targets: Optional[Iterable[str]] = None,
                 seed: int = 0, dtype=torch.float32) -> List[str]:
        """Attach rank-``rank`` adapters (A ~ N(0, 1/r), B = 0) to the named
        projections (default: every projection).  Returns the adapter keys."""
        from .. import formats
        g = torch.Generator(device="cpu").manual_seed(seed)
        names = linear_names(self.cfg)
        if targets is not None:
            tset = set(targets)
            names = [n for n in names if n.split(".")[-1] in tset]
        keys = []
        for n in names:
            w = self.params[n]
            nn, kk = w.shape
            dev = w.wq.device if isinstance(w, formats.NVFP4Tensor) else (
                w.w8.device if isinstance(w, formats.FP8BlockTensor) else w.device)
            a = (torch.randn(rank, kk, generator=g) / math.sqrt(rank)).to(dev, dtype)
            b = torch.zeros(nn, rank, dtype=dtype, device=dev)
            self.params[n + ".lora_a"], self.params[n + ".lora_b"] = a, b
            self.lora[n] = (a, b, alpha / rank)
            keys += [n + ".lora_a", n + ".lora_b"]
        return keys

    def _lora(self, name: str):
        return self.lora.get(name)

    # ---- serving forward ------------------------------------------------------------------
    def forward(self, batch, ops, kv_pool, state_pool, *, last_only: bool = True,
                aux_layers: Sequence[int] = (), return_hidden: bool = False):
        """Returns logits ``[B or T, vocab]`` (fp32).  ``aux_layers``: also return the
        residual stream after those layers (taps for the block drafter)."""
        cfg, P, d = self.cfg, self.params, self.dims
        eps = cfg.rms_eps
        x = ops.embed(P["embed"], batch.token_ids)
        settle = getattr(ops, "settle", lambda: None)   # tensor parallelism: complete a deferred all-reduce
        taps = {}
        ai = gi = 0
        for i, t in enumerate(cfg.layer_types):
            p = f"L{i}."
            if t == ATTN:
                qkv = ops.norm_linear(x, P[p + "norm1"], P[p + "qkv"], eps, self._lora(p + "qkv"))
                a = ops.attention(qkv, {"q_norm": P[p + "q_norm"], "k_norm": P[p + "k_norm"]},
                                  batch, kv_pool, ai, cfg, d.n_q, d.n_kv)
                x = ops.linear_residual(a, P[p + "o"], x, self._lora(p + "o"))
                ai += 1
            else:
                inp = ops.norm_linear(x, P[p + "norm1"], P[p + "in"], eps, self._lora(p + "in"))
                lp = {k: P[p + k] for k in ("conv", "dt_bias", "a_log", "gdn_norm")}
                a = ops.gdn(inp, lp, batch, state_pool, gi, cfg, d.gdn_nk, d.gdn_nv)
                x = ops.linear_residual(a, P[p + "out"], x, self._lora(p + "out"))
                gi += 1
            act = ops.norm_linear_swiglu(x, P[p + "norm2"], P[p + "gate_up"], eps,
                                         self._lora(p + "gate_up"))
            x = ops.linear_residual(act, P[p + "down"], x, self._lora(p + "down"))
            if i in aux_layers:
                settle()
                taps[i] = x.clone()  # the residual stream is updated in place
        settle()
        xs = x[batch.last_idx.long()] if last_only else x
        head = P["embed"] if cfg.tie_embeddings else P["lm_head"]
        logits = ops.lm_head(xs, P["final_norm"], head, eps)[..., :cfg.vocab]
        if aux_layers or return_hidden:
            return logits, x, taps
        return logits

    # ---- weight maintenance -------------------------------------------------------------------
    def requantize_(self) -> None:
        """Re-pack every projection from its master copy *in place* (device
        addresses stay fixed so captured CUDA graphs keep working)."""
        for n in linear_names(self.cfg):
            m = self.params.get("master." + n)
            if m is None:
                continue
            new = quantize_weight(m.float(), self.cfg.quant)
            cur = self.params[n]
            if isinstance(cur, NVFP4Tensor):
                cur.wq.copy_(new.wq), cur.scale.copy_(new.scale), cur.tscale.copy_(new.tscale)
            elif isinstance(cur, FP8BlockTensor):
                cur.w8.copy_(new.w8), cur.wscale.copy_(new.wscale)
            else:
                cur.copy_(new)
        self.weights_version += 1

    def served_bytes(self) -> int:
        n = 0
        for k, v in self.params.items():
            if k.startswith("master.") or ".lora_" in k:
                continue
            n += v.nbytes() if hasattr(v, "wq") or hasattr(v, "w8") else v.numel() * v.element_size()
        return n

    # ---- dense training forward (on the tape) -----------------------------------------------
    def trainable(self, mode: str = "auto") -> Dict[str, torch.Tensor]:
        """Tensors an optimizer updates: LoRA adapters when present (``auto``/``lora``),
        else every ``master.*`` projection plus norms and GDN vectors (``full``)."""
        if self.lora and mode in ("auto", "lora"):
            return {k: v for k, v in self.params.items() if ".lora_" in k}
        out = {}
        lin = set(linear_names(self.cfg))
        for k, v in self.params.items():
            if k in lin:
                continue  # served copy; its master (if kept) is the trainable one
            if k.startswith("master."):
                out[k] = v
            elif isinstance(v, torch.Tensor) and v.is_floating_point() and ".lora_" not in k \
                    and k not in ("embed", "lm_head"):
                # by kind, not by dtype: a sharded trainer swaps these tensors' storage for
                # working-precision views between steps and they must stay in the set
                out[k] = v
        return out

    def _w(self, name: str):
        """Weight used by the training forward: the master copy if kept, else the
        (frozen) served representation."""
        m = self.params.get("master." + name)
        return (m, False) if m is not None else (self.params[name], True)

    def _tlinear(self, tape, x, name: str):
        from .. import tape as T
        w, frozen = self._w(name)
        y = T.linear(tape, x, w, frozen=frozen)
        lo = self.lora.get(name)
        if lo is not None:
            y = T.lora(tape, y, x, lo[0], lo[1], lo[2])
        return y

    def forward_dense(self, tape, ids: torch.Tensor, *, checkpoint_layers: bool = False,
                      positions: Optional[torch.Tensor] = None, hook=None, cp=None,
                      return_hidden: bool = False):
        """Full-sequence forward on dense ``ids [B, T]`` with every op recorded on
        ``tape``; no KV cache, zero initial GDN state.  Returns this rank's logits
        ``[B, T, vocab_local]`` (full vocab at TP=1).  ``hook`` (a parameter sharder) is told
        when the model starts (``pre_model``), when a layer is about to run -- in the forward
        and again in its backward replay -- (``pre_layer``) and when a layer's forward is over
        (``post_layer``).  ``cp`` (a ``parallel.cp.CPContext``): ``ids`` and ``positions`` hold this
        rank's zigzag slice of the sequence; attention gathers K / V, the GDN layers exchange
        chunk summaries and conv halos."""
        from .. import tape as T
        cfg, P, d = self.cfg, self.params, self.dims
        eps = cfg.rms_eps
        b, t = ids.shape
        pos = positions if positions is not None else torch.arange(t, device=ids.device)
        if hook is not None:
            hook.pre_model()
        x = T.embedding(tape, P["embed"], ids)
        tp = self.tp > 1

        def layer(tape, x, i=0):
            p = f"L{i}."
            if hook is not None:
                hook.pre_layer(i)
            h = T.rmsnorm(tape, x, P[p + "norm1"], eps)
            if tp:
                h = T.tp_fork(tape, h)
            if cfg.layer_types[i] == ATTN:
                qkv = self._tlinear(tape, h, p + "qkv")
                a = T.attention_block(tape, qkv, P[p + "q_norm"], P[p + "k_norm"], pos,
                                      n_q=d.n_q, n_kv=d.n_kv, head_dim=cfg.head_dim,
                                      rotary_dim=cfg.rotary_dim, theta=cfg.rope_theta, eps=eps,
                                      gated=cfg.attn_gated, cp=cp)
                y = self._tlinear(tape, a, p + "o")
            else:
                inp = self._tlinear(tape, h, p + "in")
                a = T.gdn_block(tape, inp, P[p + "conv"], P[p + "dt_bias"], P[p + "a_log"],
                                P[p + "gdn_norm"], nk=d.gdn_nk, nv=d.gdn_nv, dk=cfg.gdn_head_dim,
                                dv=cfg.gdn_head_dim, eps=eps, cp=cp)
                y = self._tlinear(tape, a, p + "out")
            if tp:
                y = T.all_reduce(tape, y)
            x = T.add(tape, x, y)
            h = T.rmsnorm(tape, x, P[p + "norm2"], eps)
            if tp:
                h = T.tp_fork(tape, h)
            act = T.swiglu(tape, self._tlinear(tape, h, p + "gate_up"))
            y = self._tlinear(tape, act, p + "down")
            if tp:
                y = T.all_reduce(tape, y)
            return T.add(tape, x, y)

        for i in range(cfg.n_layers):
            if checkpoint_layers:
                p = f"L{i}."
                leaves = [v for k, v in self.params.items()
                          if (k.startswith(p) or k.startswith("master." + p)) and id(v) in tape.leaves]
                x = tape.checkpoint(lambda tp_, x_, i=i: layer(tp_, x_, i), x, params=leaves)
            else:
                x = layer(tape, x, i)
            if hook is not None and checkpoint_layers:
                hook.post_layer(i)
        h = T.rmsnorm(tape, x, P["final_norm"], eps)
        if tp:
            h = T.tp_fork(tape, h)
        head = "embed" if cfg.tie_embeddings else "lm_head"
        w = P.get("master." + head, P[head])
        frozen = id(w) not in tape.leaves
        if return_hidden:          # the caller fuses the head with its loss (never forms [T, vocab])
            return h, w, frozen
        return T.linear(tape, h, w, frozen=frozen)
