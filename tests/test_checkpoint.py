"""Checkpoint dialects: synthetic safetensors per dialect -> load -> same served values."""
import json
import os

import pytest
import torch
from safetensors.torch import save_file

from helpers import make_engine, rand_prompts
from tilerl_b200 import formats as F
from tilerl_b200.checkpoint import (CheckpointError, load_adapter, load_checkpoint, load_train_state,
                                    save_adapter, save_checkpoint, save_train_state, validate_hf_config)
from tilerl_b200.config import ATTN, tiny_hybrid
from tilerl_b200.engine import SamplingParams
from tilerl_b200.models.hybrid import HybridModel, random_master
from tilerl_b200.optim import AdamW


def _hf_tensors(cfg, master, dialect):
    """Write the master in HF names, projections in the requested dialect."""
    out = {}

    def put(name, w):
        if dialect == "bf16":
            out[name + ".weight"] = w.to(torch.bfloat16)
        elif dialect == "modelopt":
            q = F.quantize_nvfp4(w)
            out[name + ".weight_packed"] = q.wq
            out[name + ".weight_scale"] = q.scale.view(torch.uint8)
            out[name + ".weight_global_scale"] = 1.0 / q.tscale
        elif dialect == "official":
            q = F.quantize_nvfp4(w)
            out[name + ".weight"] = q.wq
            out[name + ".weight_scale"] = q.scale.view(torch.uint8)
            out[name + ".weight_scale_2"] = q.tscale
        elif dialect == "fp8":
            q = F.quantize_fp8_block(w)
            out[name + ".weight"] = q.w8
            out[name + ".weight_scale_inv"] = q.wscale
        elif dialect == "fp8_channel":
            s_ = w.abs().amax(-1).clamp_min(1e-12) / 448.0
            out[name + ".weight"] = (w / s_.unsqueeze(-1)).to(torch.float8_e4m3fn)
            out[name + ".weight_scale"] = s_
        elif dialect == "mlx4":
            from tilerl_b200.checkpoint import quantize_mlx4
            g = 64 if w.shape[1] % 64 == 0 else 32
            pk, sc, bi = quantize_mlx4(w, g)
            out[name + ".weight"], out[name + ".scales"], out[name + ".biases"] = pk, sc, bi
        elif dialect == "awq":
            from tilerl_b200.checkpoint import quantize_awq
            if w.shape[0] % 8 or w.shape[1] % 64 or name == "lm_head":
                out[name + ".weight"] = w.to(torch.bfloat16)      # AWQ files keep the head and odd shapes dense
            else:
                qw, qz, sc = quantize_awq(w, 64)
                out[name + ".qweight"], out[name + ".qzeros"], out[name + ".scales"] = qw, qz, sc
    out["model.embed_tokens.weight"] = master["embed"]
    out["model.norm.weight"] = master["final_norm"] - 1.0        # zero-centred storage
    put("lm_head", master["lm_head"])
    for i, t in enumerate(cfg.layer_types):
        L, q = f"model.layers.{i}.", f"L{i}."
        out[L + "input_layernorm.weight"] = master[q + "norm1"] - 1.0
        out[L + "post_attention_layernorm.weight"] = master[q + "norm2"] - 1.0
        if t == ATTN:
            w = master[q + "qkv"]
            put(L + "self_attn.q_proj", w[:cfg.q_rows])
            put(L + "self_attn.k_proj", w[cfg.q_rows:cfg.q_rows + cfg.kv_rows])
            put(L + "self_attn.v_proj", w[cfg.q_rows + cfg.kv_rows:])
            put(L + "self_attn.o_proj", master[q + "o"])
            out[L + "self_attn.q_norm.weight"] = master[q + "q_norm"] - 1.0
            out[L + "self_attn.k_norm.weight"] = master[q + "k_norm"] - 1.0
        else:
            w = master[q + "in"]
            c, v, nv = cfg.gdn_conv_dim, cfg.gdn_v_dim, cfg.gdn_v_heads
            put(L + "linear_attn.in_proj_qkv", w[:c])
            put(L + "linear_attn.in_proj_z", w[c:c + v])
            put(L + "linear_attn.in_proj_a", w[c + v:c + v + nv])
            put(L + "linear_attn.in_proj_b", w[c + v + nv:])
            put(L + "linear_attn.out_proj", master[q + "out"])
            out[L + "linear_attn.conv1d.weight"] = master[q + "conv"].unsqueeze(1)
            out[L + "linear_attn.dt_bias"] = master[q + "dt_bias"]
            out[L + "linear_attn.A_log"] = master[q + "a_log"]
            out[L + "linear_attn.norm.weight"] = master[q + "gdn_norm"]
        gu = master[q + "gate_up"]
        put(L + "mlp.gate_proj", gu[0::2])
        put(L + "mlp.up_proj", gu[1::2])
        put(L + "mlp.down_proj", master[q + "down"])
    return {k: v.contiguous() for k, v in out.items()}


def test_third_party_4bit_roundtrips():
    from tilerl_b200.checkpoint import dequantize_awq, dequantize_mlx4, quantize_awq, quantize_mlx4
    g = torch.Generator().manual_seed(0)
    w = torch.randn(48, 256, generator=g) * 0.05
    pk, sc, bi = quantize_mlx4(w)
    assert pk.dtype == torch.int32 and pk.shape == (48, 32)
    assert float((dequantize_mlx4(pk, sc, bi) - w).abs().max()) <= float(sc.max()) * 0.51
    qw, qz, s16 = quantize_awq(w, 64)
    assert qw.shape == (256, 6) and qz.shape == (4, 6) and s16.shape == (4, 48)
    assert float((dequantize_awq(qw, qz, s16) - w).abs().max()) <= float(s16.float().max()) * 0.6


@pytest.mark.parametrize("dialect,tol", [("bf16", 0.12), ("modelopt", 0.2), ("official", 0.2), ("fp8", 0.2),
                                         ("fp8_channel", 0.2), ("mlx4", 0.25), ("awq", 0.25)])
def test_load_hf_dialects(tmp_path, dialect, tol):
    cfg = tiny_hybrid()
    master = random_master(cfg, seed=3)
    d = str(tmp_path / dialect)
    os.makedirs(d)
    save_file(_hf_tensors(cfg, master, dialect), os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump({"num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 2,
                   "head_dim": 64, "layer_types": ["linear_attention", "full_attention"]}, f)
    m = load_checkpoint(cfg, d)
    for name in ("L0.in", "L1.qkv", "L1.gate_up", "L0.down"):
        got, want = m.params[name].dequant(), master[name]
        assert (got - want).norm() / want.norm() < tol, name
    assert torch.allclose(m.params["L0.norm1"], master["L0.norm1"])
    assert torch.allclose(m.params["L0.conv"], master["L0.conv"])


def test_config_validation_refuses_mismatch_and_rope_scaling():
    cfg = tiny_hybrid()
    with pytest.raises(CheckpointError):
        validate_hf_config(cfg, {"num_hidden_layers": 3})
    with pytest.raises(CheckpointError):
        validate_hf_config(cfg, {"rope_scaling": {"type": "yarn", "factor": 4}})
    with pytest.raises(CheckpointError):
        validate_hf_config(cfg, {"layer_types": ["full_attention", "full_attention"]})
    validate_hf_config(cfg, {"num_hidden_layers": 2, "rope_scaling": None})


def test_own_dialect_roundtrip_is_bit_exact_and_tp_shardable(tmp_path):
    cfg = tiny_hybrid()
    eng = make_engine(cfg)
    p = rand_prompts(cfg, 1, 20)
    want = eng.generate(p, SamplingParams(max_tokens=6))[0].tokens
    d = str(tmp_path / "own")
    save_checkpoint(eng.model, d)
    m2 = load_checkpoint(cfg, d)
    assert torch.equal(m2.params["L0.in"].wq, eng.model.params["L0.in"].wq)
    assert make_engine(cfg, model=m2).generate(p, SamplingParams(max_tokens=6))[0].tokens == want
    r1 = load_checkpoint(cfg, d, tp_rank=1, tp=2)
    assert r1.params["L1.o"].wq.shape[1] * 2 == cfg.attn_out_dim // 2


def test_adapter_and_train_state_resume(tmp_path):
    cfg = tiny_hybrid()
    m = HybridModel.build_random(cfg, seed=1)
    keys = m.add_lora(rank=2)
    for k in keys:
        m.params[k].normal_()
    save_adapter(m, str(tmp_path / "adapter.safetensors"))
    m2 = HybridModel.build_random(cfg, seed=1)
    m2.add_lora(rank=2)
    load_adapter(m2, str(tmp_path / "adapter.safetensors"))
    assert all(torch.equal(m.params[k], m2.params[k]) for k in keys)
    # optimizer state + step + RNG survive a save/load
    tr = m.trainable()
    opt = AdamW(tr, lr=1e-2)
    opt.step({k: torch.ones_like(v) for k, v in tr.items()})
    torch.manual_seed(5)
    save_train_state(str(tmp_path / "st"), 0, params=tr, optimizer=opt, step=7)
    a = torch.rand(3)
    tr2 = m2.trainable()
    opt2 = AdamW(tr2, lr=1e-2)
    info = load_train_state(str(tmp_path / "st"), 0, params=tr2, optimizer=opt2)
    assert info["step"] == 7 and torch.equal(torch.rand(3), a)
    g = {k: torch.full_like(v, 0.5) for k, v in tr.items()}
    opt.step(g), opt2.step(g)
    assert all(torch.equal(tr[k], tr2[k]) for k in tr)


def test_norm_fold_is_decided_by_name_not_by_value(tmp_path):
    """A trained zero-centred norm far from zero (mean |w| above 0.5) still gets its +1, and the GDN
    output norm, which is stored as is, never does -- whatever its values look like."""
    cfg = tiny_hybrid()
    master = random_master(cfg, seed=3)
    master["L0.norm1"] = torch.full_like(master["L0.norm1"], 1.8)          # stored as 0.8: not "small"
    master["L1.q_norm"] = torch.linspace(0.2, 2.5, master["L1.q_norm"].numel())
    master["final_norm"] = torch.full_like(master["final_norm"], 2.0)
    master["L0.gdn_norm"] = torch.full_like(master["L0.gdn_norm"], 0.05)   # plain norm with small weights
    d = str(tmp_path / "n")
    os.makedirs(d)
    save_file(_hf_tensors(cfg, master, "bf16"), os.path.join(d, "model.safetensors"))
    m = load_checkpoint(cfg, d)
    for k in ("L0.norm1", "L1.q_norm", "final_norm", "L0.gdn_norm", "L1.norm2", "L1.k_norm"):
        assert torch.allclose(m.params[k].float(), master[k].float(), atol=1e-2), k
