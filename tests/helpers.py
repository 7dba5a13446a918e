"""Shared test fixtures: tiny engines and an autograd twin of the dense forward."""
import math

import torch
import torch.nn.functional as F

from tilerl_b200.config import ATTN
from tilerl_b200.engine import Engine, StepLimits
from tilerl_b200.kv import GdnStatePool, PagedKvPool
from tilerl_b200.models.hybrid import HybridModel
from tilerl_b200.ops import ref
from tilerl_b200.ops.backend import RefOps
from tilerl_b200.tape import gdn_block_torch


def make_engine(cfg, seed=1, blocks=96, slots=12, planes=1, keep_master=False, **kw):
    model = kw.pop("model", None) or HybridModel.build_random(cfg, seed=seed, keep_master=keep_master)
    kv = PagedKvPool(cfg, blocks, dtype=torch.float32)
    st = GdnStatePool(cfg, slots, planes=planes, ring_dtype=torch.float32)
    return Engine(model, RefOps(), kv, st, **kw)


def rand_prompts(cfg, n, length, seed=3):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab, (length,), generator=g).tolist() for _ in range(n)]


def autograd_forward(model, ids, weights):
    """Plain differentiable torch forward (no tape) over ``weights`` (name -> tensor
    requiring grad, falling back to the model's own parameters)."""
    cfg, d = model.cfg, model.dims

    def W(name):
        if name in weights:
            return weights[name]
        if "master." + name in weights:
            return weights["master." + name]
        p = model.params.get("master." + name, model.params[name])
        return p if isinstance(p, torch.Tensor) else p.dequant()

    def lin(x, name):
        y = x @ W(name).float().t()
        if name in model.lora:
            a, b, s = W(name + ".lora_a"), W(name + ".lora_b"), model.lora[name][2]
            y = y + (x @ a.t()) @ b.t() * s
        return y

    b, t = ids.shape
    pos = torch.arange(t)
    x = W("embed").float()[ids]
    for i, kind in enumerate(cfg.layer_types):
        p = f"L{i}."
        h = ref.rmsnorm(x, W(p + "norm1"), cfg.rms_eps)
        if kind == ATTN:
            qkv = lin(h, p + "qkv")
            outs = []
            for bi in range(b):
                q, gate, k, v = ref.attn_prep(qkv[bi], W(p + "q_norm"), W(p + "k_norm"), pos, n_q=d.n_q,
                                              n_kv=d.n_kv, head_dim=cfg.head_dim, rotary_dim=cfg.rotary_dim,
                                              theta=cfg.rope_theta, eps=cfg.rms_eps, gated=cfg.attn_gated)
                outs.append(ref.dense_attention(q[None], k[None], v[None], gate[None],
                                                1 / math.sqrt(cfg.head_dim))[0])
            x = x + lin(torch.stack(outs), p + "o")
        else:
            inp = lin(h, p + "in")
            a = gdn_block_torch(inp, W(p + "conv"), W(p + "dt_bias"), W(p + "a_log"), W(p + "gdn_norm"),
                                nk=d.gdn_nk, nv=d.gdn_nv, dk=cfg.gdn_head_dim, dv=cfg.gdn_head_dim,
                                eps=cfg.rms_eps, chunk=0)
            x = x + lin(a, p + "out")
        h = ref.rmsnorm(x, W(p + "norm2"), cfg.rms_eps)
        x = x + lin(ref.swiglu(lin(h, p + "gate_up")), p + "down")
    h = ref.rmsnorm(x, W("final_norm"), cfg.rms_eps)
    head = "embed" if cfg.tie_embeddings else "lm_head"
    return h @ W(head).float().t()
