"""Hand-written tape vs torch.autograd, optimizers, and one GRPO step (config 1)."""
import torch

from helpers import autograd_forward, make_engine, rand_prompts
from tilerl_b200 import rl
from tilerl_b200 import tape as T
from tilerl_b200.config import tiny, tiny_hybrid
from tilerl_b200.models.hybrid import HybridModel
from tilerl_b200.optim import AdamW, Adafactor, ISO, clip_grad_norm, cosine_warmup
from tilerl_b200.ops import ref


def _autograd_grads(model, ids, targets, w):
    tr = model.trainable()
    leaves = {k: v.detach().clone().requires_grad_(True) for k, v in tr.items()}
    lg = autograd_forward(model, ids, leaves)
    lp = torch.log_softmax(lg, -1).gather(-1, targets[..., None]).squeeze(-1)
    loss = -(w * lp).sum()
    gs = torch.autograd.grad(loss, list(leaves.values()), allow_unused=True)
    return float(loss), dict(zip(leaves, gs))


def _check(model, ckpt=False):
    torch.manual_seed(0)
    cfg = model.cfg
    ids = torch.randint(0, cfg.vocab, (2, 12))
    targets = torch.roll(ids, -1, 1)
    w = torch.rand(2, 12) / 24
    tr = model.trainable()
    loss, grads, _ = rl.forward_backward(model, ids, targets, lambda lg: w, trainable=tr,
                                         checkpoint_layers=ckpt)
    want_loss, want = _autograd_grads(model, ids, targets, w)
    assert abs(loss - want_loss) < 1e-4 * max(1, abs(want_loss))
    assert set(grads) == {k for k, g in want.items() if g is not None}
    for k, g in grads.items():
        assert torch.allclose(g, want[k], rtol=2e-3, atol=2e-6), k


def test_tape_full_param_grads_match_autograd():
    _check(HybridModel.build_random(tiny(), seed=2, keep_master=True))


def test_tape_checkpointed_grads_match_autograd():
    _check(HybridModel.build_random(tiny(), seed=2, keep_master=True), ckpt=True)


def test_tape_lora_on_frozen_nvfp4_base():
    m = HybridModel.build_random(tiny_hybrid(), seed=4)
    keys = m.add_lora(rank=4, alpha=8.0)
    for k in keys:
        if k.endswith("lora_b"):
            m.params[k].normal_(0, 0.02)
    assert set(m.trainable()) == set(keys)
    _check(m)


def test_streaming_on_grad_sees_every_leaf_once():
    m = HybridModel.build_random(tiny(), seed=2, keep_master=True)
    tr = m.trainable()
    seen = []
    name_of = {id(v): k for k, v in tr.items()}
    ids = torch.randint(0, 320, (1, 6))
    rl.forward_backward(m, ids, torch.roll(ids, -1, 1), lambda lg: torch.full((1, 6), 1 / 6),
                        trainable=tr, on_grad=lambda t, g: seen.append(name_of[id(t)]))
    assert sorted(seen) == sorted(tr) and len(set(seen)) == len(seen)
    assert seen.index("master.L1.down") < seen.index("master.L0.qkv")  # reverse layer order


def test_group_advantages():
    a = rl.group_advantages([1, 0, 0, 1, 5, 5, 5, 5], 4)
    assert torch.allclose(a[:4], torch.tensor([1., -1., -1., 1.]), atol=1e-4)
    assert a[4:].abs().sum() == 0  # tied group: no signal
    b = rl.group_advantages([1, 0, 9, 9], 4, live=[True, True, False, False])
    assert b[2] == 0 and b[3] == 0 and b[0] > 0 > b[1]


def test_optimizers_write_in_place_and_descend():
    torch.manual_seed(0)
    for cls in (AdamW, Adafactor, ISO):
        p = {"w": torch.randn(8, 6), "b": torch.randn(6)}
        ptr = {k: v.data_ptr() for k, v in p.items()}
        opt = cls(p, lr=0.05)
        tgt = {"w": torch.zeros(8, 6), "b": torch.zeros(6)}
        l0 = sum((p[k] - tgt[k]).pow(2).sum() for k in p)
        for _ in range(60):
            opt.step({k: 2 * (p[k] - tgt[k]) for k in p})
        l1 = sum((p[k] - tgt[k]).pow(2).sum() for k in p)
        assert l1 < 0.5 * l0, cls.__name__
        assert all(p[k].data_ptr() == ptr[k] for k in p)


def test_clip_and_schedule():
    g = {"a": torch.ones(4) * 3, "b": torch.ones(4) * 4}
    n = clip_grad_norm(g, 1.0)
    assert abs(n - 10.0) < 1e-5
    assert abs(sum(v.pow(2).sum() for v in g.values()).sqrt() - 1.0) < 1e-4
    assert cosine_warmup(0, 100, 10, 1.0) == 0.1 and abs(cosine_warmup(100, 100, 10, 1.0) - 0.1) < 1e-6


def test_config1_grpo_step_grads_match_autograd_and_policy_moves():
    """2 prompts x G=4, reward = fraction of even ids, clip 0.2, lr 1e-5."""
    cfg = tiny_hybrid()
    eng = make_engine(cfg, keep_master=True)
    model = eng.model
    prompts = rand_prompts(cfg, 2, 16)
    reward = lambda p, c: sum(1 for t in c if t % 2 == 0) / max(1, len(c))
    opt = AdamW(model.trainable(), lr=1e-5)
    # gradient check of the objective on a hand-made batch
    ids = rl.pad_batch([p + [2, 4, 5, 7] for p in prompts])
    adv = torch.tensor([1.0, -0.5])
    st = rl.policy_step(model, ids, [16, 16], [20, 20], adv, None, return_grads=True, max_norm=0.0)
    mask = rl._scored_mask(ids, [16, 16], [20, 20])
    w = adv[:, None] * mask / mask.sum()
    _, want = _autograd_grads(model, ids, torch.roll(ids, -1, 1), w)
    for k, g in st["grads"].items():
        assert torch.allclose(g, want[k], rtol=2e-3, atol=2e-6), k
    before = {k: v.clone() for k, v in model.trainable().items()}
    ms = list(rl.grpo_loop(eng, model, prompts, reward, opt, steps=1, group=4, prompts_per_step=2,
                           max_tokens=8, post_step=lambda m: m.requantize_()))
    assert len(ms) == 1 and ms[0]["completion_tokens"] == 64 and 0 <= ms[0]["reward"] <= 1
    moved = sum(float((v - before[k]).abs().sum()) for k, v in model.trainable().items())
    assert (moved > 0) == (ms[0]["tied_groups"] < 2)
    assert eng.kv.used_blocks == 0


def test_clipped_ratio_zeroes_gradient():
    cfg = tiny()
    m = HybridModel.build_random(cfg, seed=2, keep_master=True)
    ids = rl.pad_batch([[1, 2, 3, 4, 5, 6]])
    old = torch.full((1, 6), -50.0)  # rho huge, A > 0 -> every token clipped
    st = rl.policy_step(m, ids, [3], [6], torch.tensor([1.0]), None, old_logprobs=old,
                        return_grads=True, max_norm=0.0)
    assert st["clipped"] == 3 and all(float(g.abs().max()) == 0 for g in st["grads"].values())


def test_fused_head_cross_entropy_equals_the_unfused_path():
    """The chunked lm_head + CE op (never forms [T, V]) gives the same loss, log-probabilities and
    gradients as head -> logits -> cross-entropy, for the SFT mask and for PPO-clip weights, with a
    frozen and with a trainable head."""
    import torch
    from tilerl_b200 import rl
    from tilerl_b200 import tape as T
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.models.hybrid import HybridModel
    from tilerl_b200.ops import ref
    cfg = tiny_hybrid()
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (3, 11), generator=g)
    adv = torch.tensor([1.0, -0.5, 0.25])
    model = HybridModel.build_random(cfg, seed=2, keep_master=True)
    outs = []
    for fused in (False, True):
        st = rl.policy_step(model, ids, [4, 3, 5], [11, 9, 10], adv, None, clip_eps=0.2, micro=2,
                            return_grads=True, fused_ce=fused)
        outs.append(st)
    assert abs(outs[0]["loss"] - outs[1]["loss"]) < 1e-5
    for k, gref in outs[0]["grads"].items():
        assert torch.allclose(outs[1]["grads"][k], gref, atol=2e-5, rtol=1e-4), k
    # the op itself, trainable head, chunk smaller than the token count
    h = torch.randn(2, 7, cfg.hidden, generator=g)
    w = torch.randn(cfg.vocab, cfg.hidden, generator=g) * 0.05
    tg = torch.randint(0, cfg.vocab, (2, 7), generator=g)
    wt = torch.rand(2, 7, generator=g)
    tp = T.Tape()
    tp.watch(h, w)
    loss, lp = T.linear_cross_entropy(tp, h, w, tg, lambda l: wt, frozen=False, chunk=4)
    grads = tp.backward(loss)
    h2, w2 = h.clone().requires_grad_(True), w.clone().requires_grad_(True)
    lg = h2 @ w2.t()
    lp_ref = ref.token_logprobs(lg.reshape(-1, cfg.vocab), tg.reshape(-1)).view(2, 7)
    (-(wt * lp_ref).sum()).backward()
    assert torch.allclose(lp, lp_ref.detach(), atol=1e-5)
    assert torch.allclose(grads[id(h)], h2.grad, atol=1e-5) and torch.allclose(grads[id(w)], w2.grad, atol=1e-5)


def test_group_advantages_signal_and_group_count():
    """A group whose task reward is constant gets zeros even when a length term separates its rows
    (a length-only gradient), and a reward count that is not a whole number of groups, or not the
    number of groups the caller means, is refused."""
    import pytest
    task = [1.0, 1.0, 1.0, 1.0, 0.0, 1.0, 0.0, 1.0]
    lens = [3, 9, 5, 7, 4, 4, 8, 8]
    shaped = [t - 0.01 * n for t, n in zip(task, lens)]
    adv = rl.group_advantages(shaped, 4, signal=task, groups=2)
    assert torch.all(adv[:4] == 0)                       # constant signal: silent group
    assert adv[4] < 0 < adv[5] and adv[6] < 0 < adv[7]   # the other group keeps its ordering
    plain = rl.group_advantages(shaped, 4)               # without the signal the length term fills the advantage
    assert plain[:4].abs().max() > 0.5
    with pytest.raises(ValueError):
        rl.group_advantages(shaped[:7], 4)
    with pytest.raises(ValueError):
        rl.group_advantages(shaped, 4, groups=1)
    # dead rows do not make a constant-signal group look ordered
    adv = rl.group_advantages([1.0, 1.0, 0.0, 1.0], 4, live=[True, True, False, True], signal=[1.0, 1.0, 0.0, 1.0])
    assert torch.all(adv == 0)


def test_opd_loop_teacher_generates_student_trains_and_weights_are_restored():
    """On-policy distillation on the tiny model: every step yields a finite loss, the student's
    adapters move, the EMA teacher follows them more slowly, the live tensors hold the STUDENT after
    each step (the teacher was only swapped in for the rollout), and the engine's prefix store holds
    nothing computed under the other set of weights."""
    cfg = tiny_hybrid()
    eng = make_engine(cfg, seed=3)
    model = eng.model
    keys = model.add_lora(rank=4, alpha=8.0)
    for k in keys:
        if k.endswith("lora_b"):
            model.params[k].normal_(0, 0.02)
    before = {k: v.detach().clone() for k, v in model.trainable().items()}
    opt = AdamW(model.trainable(), lr=1e-2)
    prompts = rand_prompts(cfg, 4, 12)
    out = list(rl.opd_loop(eng, model, prompts, opt, steps=3, max_tokens=6, ema=0.5, prompts_per_step=2))
    assert len(out) == 3 and all(torch.isfinite(torch.tensor(m["loss"])) for m in out)
    assert all(m["tokens"] > 0 for m in out)
    after = model.trainable()
    moved = sum(float((after[k] - before[k]).abs().sum()) for k in before)
    assert moved > 0
    assert len(eng.prefix) == 0          # nothing cached under either set of weights survives a step


def test_grpo_judge_orders_a_tied_group_and_leaves_decided_groups_alone():
    """A judge sees each group's completions after the rule-based reward: a tie becomes a signal (non-zero
    advantages, a finite loss), and the rewards handed to it are what the rule produced."""
    from helpers import make_engine, rand_prompts
    from tilerl_b200 import evals, rl
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.optim import make_optimizer
    cfg = tiny_hybrid()
    eng = make_engine(cfg, blocks=96)
    model = eng.model
    model.add_lora(rank=2)
    opt = make_optimizer("adamw", model.trainable(), 1e-4)
    prompts = rand_prompts(cfg, 2, 8, seed=3)
    seen = []

    def judge(prompt, comps, rewards):
        seen.append((list(prompt), [list(c) for c in comps], list(rewards)))
        return evals.judge_tiebreak(rewards, ["x" * len(set(c)) for c in comps], lambda a, b: 1.0 if len(a) > len(b) else (0.0 if len(a) < len(b) else 0.5))

    tie = lambda p, c: 1.0                                    # every rollout "right": the rule alone gives no gradient
    m_plain = next(rl.grpo_loop(eng, model, prompts, tie, opt, steps=1, group=4, prompts_per_step=1, max_tokens=6))
    m_judge = next(rl.grpo_loop(eng, model, prompts, tie, opt, steps=1, group=4, prompts_per_step=1, max_tokens=6, judge=judge))
    assert len(seen) == 1 and seen[0][2] == [1.0] * 4 and len(seen[0][1]) == 4
    assert m_plain["loss"] == 0.0 or abs(m_plain["loss"]) < 1e-12
    assert m_judge["loss"] == m_judge["loss"]                  # finite
    # the policy as its own judge: deterministic, symmetric in the order it is asked
    from tilerl_b200.tokenizer import ByteTokenizer
    cmp = evals.policy_compare(eng, ByteTokenizer(cfg.vocab), question="2+2=")
    a, b = cmp("4", "5"), cmp("5", "4")
    assert 0.0 <= a <= 1.0 and abs(a + b - 1.0) < 1e-9
