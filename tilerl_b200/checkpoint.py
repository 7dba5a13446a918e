"""Checkpoint I/O.

``load_checkpoint`` reads a HuggingFace-style directory (``config.json`` +
``*.safetensors``) in any of these weight dialects and produces the served
parameter dict (TP-sharded if asked):

* bf16 / fp16 / fp32 dense weights (quantised to the model's serving format on load);
* NVFP4 "modelopt" files: ``<w>.weight_packed`` (or ``.weight`` uint8) + ``.weight_scale``
  (e4m3 per 16) + ``.weight_global_scale`` (stored as the *reciprocal* tensor scale);
* official NVFP4 files: ``.weight`` uint8 + ``.weight_scale`` + ``.weight_scale_2``;
* FP8 128x128-block files: ``.weight`` e4m3 + ``.weight_scale_inv``; FP8 per-tensor / per-channel:
  ``.weight`` e4m3 + ``.weight_scale``;
* MLX 4-bit: ``.weight`` uint32 (8 nibbles, low first) + ``.scales`` + ``.biases`` per group of 64;
* AWQ: ``.qweight`` int32 ``[K, N/8]`` (AWQ nibble order) + ``.qzeros`` + ``.scales`` per group;
* this framework's own dialect: ``<name>.wq / .scale / .tscale``.

HF tensor names are mapped onto the fused layouts used here (gate/query interleave for
``qkv``, ``[q;k;v;z;a;b]`` for the GDN input projection, interleaved ``gate_up``).  RMSNorm
weights stored zero-centred are folded ``+1`` on load.  ``config.json`` is validated
against the model config; rope scaling and other unsupported features are refused.

``save_checkpoint`` writes the own dialect; ``save_train_state`` / ``load_train_state``
write one file per rank (parameters or ZeRO shard, optimizer moments, step, RNG state)
with atomic rename, so training resumes exactly.

Parity: reference ``src/tilerl/model.py`` -- ``_LAYER_SUFFIXES:813``,
``_validate_hf_config:865``, ``load_hf:965-1229``, ``requantize_fp4:1255``,
``save_hf:1298``; format maths ``tilerl_kernels/reference.py:189-419``.  The reference
does not checkpoint optimizer state (``src/tilerl/train.py:1233-1260``).
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Optional

import torch

from .config import ATTN, ModelConfig
from .formats import (FP8BlockTensor, NVFP4Tensor, dequantize_fp8_block, dequantize_nvfp4,
                      quantize_nvfp4)
from .models.hybrid import HybridModel, linear_names, quantize_weight


class CheckpointError(ValueError):
    pass


# ---- HF config validation -------------------------------------------------------------------
def validate_hf_config(cfg: ModelConfig, hf: Dict) -> None:
    tc = hf.get("text_config", hf)
    want = {"num_hidden_layers": cfg.n_layers, "hidden_size": cfg.hidden,
            "num_attention_heads": cfg.n_q_heads, "num_key_value_heads": cfg.n_kv_heads}
    for k, v in want.items():
        if tc.get(k) is not None and tc[k] != v:
            raise CheckpointError(f"config.json {k}={tc[k]} but model config expects {v}")
    if tc.get("head_dim") is not None and tc["head_dim"] != cfg.head_dim:
        raise CheckpointError(f"config.json head_dim={tc['head_dim']} != {cfg.head_dim}")
    rs = tc.get("rope_scaling") or tc.get("rope_parameters", {}).get("rope_scaling")
    if rs and rs.get("type", rs.get("rope_type", "default")) not in ("default", None):
        raise CheckpointError(f"rope scaling {rs} is not supported")
    types = tc.get("layer_types")
    if types:
        mine = ["full_attention" if t == ATTN else "linear_attention" for t in cfg.layer_types]
        if list(types) != mine:
            raise CheckpointError("config.json layer_types do not match the model's attention/GDN layout")
    if tc.get("sliding_window") and tc.get("use_sliding_window"):
        raise CheckpointError("sliding-window attention is not supported")


# ---- third-party 4-bit dialects ------------------------------------------------------------------
AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)          # nibble i of a packed int32 holds output column AWQ_ORDER[i]
AWQ_REVERSE = (0, 4, 1, 5, 2, 6, 3, 7)        # column c sits in nibble AWQ_REVERSE[c]


def _nibbles(p: torch.Tensor) -> torch.Tensor:
    """``[..., n]`` int32/uint32 -> ``[..., n, 8]`` nibbles, low bits first."""
    q = p.to(torch.int64) & 0xFFFFFFFF
    sh = torch.arange(0, 32, 4, dtype=torch.int64)
    return (q.unsqueeze(-1) >> sh) & 0xF


def dequantize_mlx4(w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group: int = 64) -> torch.Tensor:
    """MLX affine 4-bit: ``w [N, K/8]`` packed, ``scales / biases [N, K/group]``; value = q * scale + bias."""
    n = w.shape[0]
    q = _nibbles(w).reshape(n, -1).float()
    k = q.shape[1]
    return (q.view(n, k // group, group) * scales.float().unsqueeze(-1) + biases.float().unsqueeze(-1)).view(n, k)


def quantize_mlx4(w: torch.Tensor, group: int = 64):
    """Inverse of :func:`dequantize_mlx4` (used by tests and tools): returns (packed, scales, biases)."""
    n, k = w.shape
    g = w.float().view(n, k // group, group)
    lo, hi = g.amin(-1), g.amax(-1)
    scale = ((hi - lo) / 15.0).clamp_min(1e-12)
    q = torch.clamp(torch.round((g - lo.unsqueeze(-1)) / scale.unsqueeze(-1)), 0, 15).to(torch.int64).view(n, k // 8, 8)
    sh = torch.arange(0, 32, 4, dtype=torch.int64)
    packed = (q << sh).sum(-1)
    packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)
    return packed, scale, lo


def dequantize_awq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """AWQ GEMM layout: ``qweight [K, N/8]``, ``qzeros [K/g, N/8]``, ``scales [K/g, N]`` ->
    dense ``[N, K]`` (this framework keeps weights output-major)."""
    k = qweight.shape[0]
    rev = torch.tensor(AWQ_REVERSE)
    q = _nibbles(qweight)[..., rev].reshape(k, -1).float()                 # [K, N]
    z = _nibbles(qzeros)[..., rev].reshape(qzeros.shape[0], -1).float()     # [K/g, N]
    g = k // z.shape[0]
    w = (q.view(z.shape[0], g, -1) - z.unsqueeze(1)) * scales.float().unsqueeze(1)
    return w.view(k, -1).t().contiguous()


def quantize_awq(w: torch.Tensor, group: int = 128):
    """Inverse of :func:`dequantize_awq` for tests and tools: dense ``[N, K]`` -> (qweight, qzeros, scales)."""
    n, k = w.shape
    wt = w.float().t().contiguous().view(k // group, group, n)               # [K/g, g, N]
    lo, hi = wt.amin(1), wt.amax(1)
    scale = ((hi - lo) / 15.0).clamp_min(1e-12)
    zero = torch.clamp(torch.round(-lo / scale), 0, 15)
    q = torch.clamp(torch.round(wt / scale.unsqueeze(1)) + zero.unsqueeze(1), 0, 15).to(torch.int64).view(k, n)
    order = torch.tensor(AWQ_ORDER)

    def pack(x):                                                             # [R, N] -> [R, N/8]
        x = x.view(x.shape[0], -1, 8)[..., order]
        sh = torch.arange(0, 32, 4, dtype=torch.int64)
        p = (x << sh).sum(-1)
        return torch.where(p >= 2 ** 31, p - 2 ** 32, p).to(torch.int32)
    return pack(q), pack(zero.to(torch.int64)), scale.to(torch.float16)


# ---- tensor-level readers ----------------------------------------------------------------------
class _Reader:
    """All tensors of a directory, lazily, by name."""

    def __init__(self, path: str):
        from safetensors import safe_open
        self.files = {}
        self.index: Dict[str, str] = {}
        for fn in sorted(os.listdir(path)):
            if fn.endswith(".safetensors"):
                f = safe_open(os.path.join(path, fn), framework="pt", device="cpu")
                self.files[fn] = f
                for k in f.keys():
                    self.index[k] = fn
        if not self.index:
            raise CheckpointError(f"no .safetensors files in {path}")

    def has(self, name: str) -> bool:
        return name in self.index

    def get(self, name: str) -> torch.Tensor:
        return self.files[self.index[name]].get_tensor(name)

    def dense(self, base: str) -> torch.Tensor:
        """The fp32 dense value of weight ``base`` (``...proj``), whatever its dialect."""
        if self.has(base + ".wq"):
            return dequantize_nvfp4(NVFP4Tensor(self.get(base + ".wq"), self.get(base + ".scale").view(torch.float8_e4m3fn),
                                                self.get(base + ".tscale").float()))
        if self.has(base + ".qweight"):
            return dequantize_awq(self.get(base + ".qweight"), self.get(base + ".qzeros"), self.get(base + ".scales"))
        packed = base + ".weight_packed" if self.has(base + ".weight_packed") else base + ".weight"
        if not self.has(packed):
            raise CheckpointError(f"missing tensor for {base}")
        w = self.get(packed)
        if w.dtype in (torch.uint32, torch.int32) and self.has(base + ".scales") and self.has(base + ".biases"):
            return dequantize_mlx4(w, self.get(base + ".scales"), self.get(base + ".biases"))
        if w.dtype == torch.uint8 and self.has(base + ".weight_scale"):
            sc = self.get(base + ".weight_scale")
            sc = sc.view(torch.float8_e4m3fn) if sc.dtype == torch.uint8 else sc.to(torch.float8_e4m3fn)
            if self.has(base + ".weight_global_scale"):      # modelopt: reciprocal tensor scale
                ts = 1.0 / self.get(base + ".weight_global_scale").float().reshape(1)
            elif self.has(base + ".weight_scale_2"):         # official: direct tensor scale
                ts = self.get(base + ".weight_scale_2").float().reshape(1)
            else:
                ts = torch.ones(1)
            return dequantize_nvfp4(NVFP4Tensor(w, sc, ts))
        if w.dtype == torch.float8_e4m3fn:
            if self.has(base + ".weight_scale_inv"):
                return dequantize_fp8_block(FP8BlockTensor(w, self.get(base + ".weight_scale_inv").float()))
            if self.has(base + ".weight_scale"):
                s = self.get(base + ".weight_scale").float()
                return w.float() * (s if s.numel() == 1 else s.reshape(-1, 1))
            return w.float()
        return w.float()

    def nvfp4(self, base: str) -> Optional[NVFP4Tensor]:
        """The stored NVFP4 planes when the file already holds them (no requantisation)."""
        if self.has(base + ".wq"):
            return NVFP4Tensor(self.get(base + ".wq"), self.get(base + ".scale").view(torch.float8_e4m3fn),
                               self.get(base + ".tscale").float())
        return None


# ---- HF name mapping ------------------------------------------------------------------------------
def _hf_prefix(reader: _Reader) -> str:
    for p in ("model.language_model.", "language_model.model.", "model."):
        if any(k.startswith(p + "layers.") for k in reader.index):
            return p
    return ""


def _interleave_rows(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return torch.stack([a, b], dim=1).reshape(a.shape[0] * 2, *a.shape[1:])


def assemble_master(cfg: ModelConfig, reader: _Reader) -> Dict[str, torch.Tensor]:
    """HF tensors -> full (TP=1) master dict in this framework's fused layouts."""
    p = _hf_prefix(reader)
    own = reader.has("embed") or reader.has("embed.weight")
    out: Dict[str, torch.Tensor] = {}

    def norm(name: str) -> torch.Tensor:
        # HF checkpoints of this family store these norms zero-centred (y = x_normed * (1 + w)): the
        # +1 is folded in by NAME -- input / post-attention / q / k / final norm always, the GDN output
        # norm never -- as the reference does (src/tilerl/model.py:810-811, :1162), not by looking at
        # the values: a trained weight far from zero must load like any other
        return reader.get(name).float() + 1.0

    if own:
        return {}
    out["embed"] = reader.get(p + "embed_tokens.weight").float()
    out["final_norm"] = norm(p + "norm.weight")
    if not cfg.tie_embeddings:
        head = "lm_head" if reader.has("lm_head.weight") or reader.has("lm_head.weight_packed") else p + "lm_head"
        out["lm_head"] = reader.dense(head)
    for i, t in enumerate(cfg.layer_types):
        L, q = f"{p}layers.{i}.", f"L{i}."
        out[q + "norm1"] = norm(L + "input_layernorm.weight")
        out[q + "norm2"] = norm(L + "post_attention_layernorm.weight")
        if t == ATTN:
            a = L + "self_attn."
            # HF q_proj rows are already [query(D); gate(D)] per head when gated
            out[q + "qkv"] = torch.cat([reader.dense(a + "q_proj"), reader.dense(a + "k_proj"),
                                        reader.dense(a + "v_proj")])
            out[q + "o"] = reader.dense(a + "o_proj")
            out[q + "q_norm"] = norm(a + "q_norm.weight")
            out[q + "k_norm"] = norm(a + "k_norm.weight")
        else:
            g = L + "linear_attn."
            out[q + "in"] = torch.cat([reader.dense(g + "in_proj_qkv"), reader.dense(g + "in_proj_z"),
                                       reader.dense(g + "in_proj_a"), reader.dense(g + "in_proj_b")])
            out[q + "out"] = reader.dense(g + "out_proj")
            conv = reader.get(g + "conv1d.weight").float()
            out[q + "conv"] = conv.reshape(conv.shape[0], -1)
            out[q + "dt_bias"] = reader.get(g + "dt_bias").float()
            out[q + "a_log"] = reader.get(g + "A_log").float()
            out[q + "gdn_norm"] = reader.get(g + "norm.weight").float()
        m = L + "mlp."
        out[q + "gate_up"] = _interleave_rows(reader.dense(m + "gate_proj"), reader.dense(m + "up_proj"))
        out[q + "down"] = reader.dense(m + "down_proj")
    return out


def load_checkpoint(cfg: ModelConfig, path: str, *, device="cpu", tp_rank: int = 0, tp: int = 1,
                    keep_master: bool = False) -> HybridModel:
    cj = os.path.join(path, "config.json")
    if os.path.exists(cj):
        with open(cj) as f:
            validate_hf_config(cfg, json.load(f))
    reader = _Reader(path)
    if reader.has("embed"):
        return _load_own(cfg, reader, device, tp_rank, tp, keep_master)
    master = assemble_master(cfg, reader)
    from .models.hybrid import param_shapes
    shapes = param_shapes(cfg, 1)
    for k, shp in shapes.items():
        if k not in master:
            raise CheckpointError(f"checkpoint lacks parameter {k}")
        if tuple(master[k].shape) != tuple(shp):
            raise CheckpointError(f"{k}: checkpoint shape {tuple(master[k].shape)} != expected {tuple(shp)}")
    act = torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32
    return HybridModel.from_master(cfg, master, tp_rank=tp_rank, tp=tp, device=device,
                                   keep_master=keep_master, act_dtype=act)


def _load_own(cfg, reader: _Reader, device, tp_rank, tp, keep_master) -> HybridModel:
    """Own dialect: NVFP4 planes are adopted bit for bit (no requantisation)."""
    from .parallel.mesh import shard_param
    params: Dict[str, object] = {}
    lin = set(linear_names(cfg))
    names = {k.rsplit(".", 1)[0] if k.endswith((".wq", ".scale", ".tscale")) else k for k in reader.index}
    act = torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32
    for name in sorted(names):
        q = reader.nvfp4(name)
        if q is not None:
            v = shard_param(cfg, name, q, tp_rank, tp).to(device)
        else:
            t = reader.get(name)
            t = shard_param(cfg, name, t, tp_rank, tp)
            if name in lin:
                v = quantize_weight(t.float(), cfg.quant)
                v = v.to(device) if hasattr(v, "to") else v
            elif name in ("embed", "lm_head"):
                v = t.to(device=device, dtype=act)
            else:
                v = t.float().to(device)
        params[name] = v
    return HybridModel(cfg, params, tp_rank, tp)


def save_checkpoint(model: HybridModel, path: str) -> None:
    """Write the served parameters (own dialect) + a config.json describing the model."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    tensors: Dict[str, torch.Tensor] = {}
    for k, v in model.params.items():
        if k.startswith("master."):
            continue
        if isinstance(v, NVFP4Tensor):
            tensors[k + ".wq"] = v.wq.cpu().contiguous()
            tensors[k + ".scale"] = v.scale.view(torch.uint8).cpu().contiguous()
            tensors[k + ".tscale"] = v.tscale.cpu().contiguous()
        elif isinstance(v, FP8BlockTensor):
            tensors[k] = v.dequant().to(torch.bfloat16).cpu().contiguous()
        else:
            tensors[k] = v.detach().cpu().contiguous()
    tmp = os.path.join(path, "model.safetensors.tmp")
    save_file(tensors, tmp)
    os.replace(tmp, os.path.join(path, "model.safetensors"))
    cfg = model.cfg
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump({"model_type": "tilerl_b200_hybrid", "name": cfg.name, "num_hidden_layers": cfg.n_layers,
                   "hidden_size": cfg.hidden, "num_attention_heads": cfg.n_q_heads,
                   "num_key_value_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
                   "layer_types": ["full_attention" if t == ATTN else "linear_attention" for t in cfg.layer_types],
                   "quant": cfg.quant, "tp": model.tp}, f, indent=1)


def save_adapter(model: HybridModel, path: str) -> None:
    from safetensors.torch import save_file
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    tensors = {k: v.detach().cpu().contiguous() for k, v in model.params.items() if ".lora_" in k}
    save_file(tensors, path + ".tmp")
    os.replace(path + ".tmp", path)


def load_adapter(model: HybridModel, path: str) -> None:
    from safetensors.torch import load_file
    for k, v in load_file(path).items():
        if k not in model.params:
            raise CheckpointError(f"adapter tensor {k} has no slot (call add_lora with the same targets first)")
        model.params[k].copy_(v.to(model.params[k].device))


# ---- training state (exact resume) -------------------------------------------------------------------
def save_train_state(path: str, rank: int, *, params: Dict[str, torch.Tensor], optimizer=None, step: int = 0,
                     extra: Optional[Dict] = None) -> str:
    """One file per rank: parameters (or this rank's ZeRO shard), optimizer moments, step
    counter and RNG state; written to a temp name and renamed."""
    os.makedirs(path, exist_ok=True)
    blob = {"step": int(step), "params": {k: v.detach().cpu() for k, v in params.items()},
            "optimizer": None, "rng_cpu": torch.get_rng_state(), "extra": extra or {}}
    if optimizer is not None:
        sd = optimizer.state_dict()
        blob["optimizer"] = {k: ({n: t.cpu() for n, t in v.items()} if isinstance(v, dict) and v and
                                 isinstance(next(iter(v.values())), torch.Tensor) else v) for k, v in sd.items()}
    if torch.cuda.is_available():
        blob["rng_cuda"] = torch.cuda.get_rng_state()
    fn = os.path.join(path, f"rank{rank:03d}.pt")
    torch.save(blob, fn + ".tmp")
    with open(fn + ".tmp", "rb") as f:
        data = f.read()
    with open(fn + ".crc.tmp", "w") as f:      # integrity sidecar: size and CRC32 of the shard
        json.dump({"nbytes": len(data), "crc32": zlib.crc32(data)}, f)
    os.replace(fn + ".tmp", fn)
    os.replace(fn + ".crc.tmp", fn + ".crc")
    return fn


def load_train_state(path: str, rank: int, *, params: Dict[str, torch.Tensor], optimizer=None) -> Dict:
    fn = os.path.join(path, f"rank{rank:03d}.pt")
    if os.path.exists(fn + ".crc"):
        with open(fn + ".crc") as f:
            want = json.load(f)
        with open(fn, "rb") as f:
            data = f.read()
        if len(data) != want["nbytes"] or zlib.crc32(data) != want["crc32"]:
            raise CheckpointError(f"{fn}: size or CRC32 does not match its sidecar (corrupt shard)")
    blob = torch.load(fn, map_location="cpu", weights_only=False)
    for k, v in blob["params"].items():
        if k not in params:
            raise CheckpointError(f"state has parameter {k} that the model lacks")
        params[k].copy_(v.to(params[k].device))
    if optimizer is not None and blob["optimizer"] is not None:
        sd = blob["optimizer"]
        dev = next(iter(params.values())).device
        for key in ("m", "v"):
            if key in sd:
                sd[key] = {n: t.to(dev) for n, t in sd[key].items()}
        optimizer.load_state_dict(sd)
    torch.set_rng_state(blob["rng_cpu"])
    if "rng_cuda" in blob and torch.cuda.is_available():
        torch.cuda.set_rng_state(blob["rng_cuda"])
    return {"step": blob["step"], "extra": blob["extra"]}
