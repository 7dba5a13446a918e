"""Training loops on the hand-written tape: SFT, GRPO, on-policy distillation.

``policy_step`` implements the clipped GRPO surrogate with the rollout
log-probabilities as ``pi_old``:

    L = -1/N * sum_i min(rho_i A_i, clip(rho_i, 1-eps, 1+eps) A_i) + beta * KL_k3

Its gradient w.r.t. the logits is a weighted cross-entropy gradient with
per-token weight ``w_i = (A_i rho_i [unclipped_i] - beta (1 - exp(ref_i - logp_i))) / N``,
so the tape's ``cross_entropy`` op (which emits loss and gradient together and
never differentiates a softmax twice) is the whole objective.  With one
on-policy update ``rho == 1`` and the weights reduce to ``A_i / N`` -- exactly the
REINFORCE-with-baseline form of the reference.  ``N`` is the batch-wide scored
token count, not the micro-batch's.

``grpo_loop`` rolls out through the *same* engine that serves (P prompts x G
samples with per-sample seeds), scores, normalises advantages per group, runs
``policy_step``, re-quantises the served weights in place and invalidates the
engine's caches.

Parity: reference ``src/tilerl/train.py`` -- ``_step:164-310``,
``train_step:716``, ``group_advantages:740``, ``rl_step:805``,
``_require_on_policy:864``, ``grpo_loop:936-1135``, ``opd_loop:1138``,
``pretrain:1222``.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass
from typing import Callable, Dict, Iterator, List, Optional, Sequence

import torch

from . import tape as T
from .engine import Engine, SamplingParams
from .optim import clip_grad_norm, cosine_warmup
from .ops import ref


def group_advantages(rewards: Sequence[float], group: int, live: Optional[Sequence[bool]] = None,
                     eps: float = 1e-6, signal: Optional[Sequence[float]] = None,
                     groups: Optional[int] = None) -> torch.Tensor:
    """``(r - mean_g) / std_g`` within each group of ``group`` consecutive samples.
    A group whose live samples all tie gets zeros (no signal); dead samples (empty
    completions) get zero and do not enter the statistics.

    ``signal``: the reward without shaping terms (the length penalty).  A group whose signal is
    constant over its live rows has no ordering left except the shaping term, and normalisation
    would blow that up to a full-size advantage (a length-only gradient); such a group gets zeros.
    ``groups``: how many groups the caller means to pass; checked, because the count is otherwise
    inferred from the length.  The number of rewards must be a whole number of groups.
    Parity: reference ``group_advantages`` (``src/tilerl/train.py:740-801``)."""
    r = torch.tensor(list(rewards), dtype=torch.float32)
    if group < 1 or len(r) % group:
        raise ValueError(f"group_advantages: {len(r)} rewards are not a whole number of groups of {group}")
    if groups is not None and len(r) // group != groups:
        raise ValueError(f"group_advantages: {len(r)} rewards make {len(r) // group} groups of {group}, "
                         f"the caller expected {groups}")
    lv = torch.ones_like(r, dtype=torch.bool) if live is None else torch.tensor(list(live), dtype=torch.bool)
    sg = r if signal is None else torch.tensor(list(signal), dtype=torch.float32)
    adv = torch.zeros_like(r)
    for g0 in range(0, len(r), group):
        sl = slice(g0, g0 + group)
        m = lv[sl]
        if m.sum() < 2:
            continue
        x = r[sl][m]
        sd = x.std(unbiased=False)
        if float(sd) < eps:
            continue
        sx = sg[sl][m]
        if float(sx.max()) == float(sx.min()):
            continue                       # constant signal: what differs is shaping only
        a = torch.zeros(m.shape[0])
        a[m] = (x - x.mean()) / (sd + eps)
        adv[sl] = a
    return adv


def require_on_policy(p: SamplingParams) -> None:
    if not p.untruncated:
        raise ValueError("GRPO rollouts must sample the untruncated policy "
                         "(temperature 1, top_p 1, top_k 0, no allowed_ids)")


def pad_batch(seqs: Sequence[Sequence[int]], pad: int = 0, pow2: bool = False):
    width = max(len(s) for s in seqs)
    if pow2:
        w = 1
        while w < width:
            w *= 2
        width = w
    ids = torch.full((len(seqs), width), pad, dtype=torch.long)
    for i, s in enumerate(seqs):
        ids[i, :len(s)] = torch.tensor(list(s), dtype=torch.long)
    return ids


def _named_grads(trainable: Dict[str, torch.Tensor], grads_by_id) -> Dict[str, torch.Tensor]:
    return {n: grads_by_id[id(t)] for n, t in trainable.items() if id(t) in grads_by_id}


TP_PARTIAL_REPLICATED = ("q_norm", "k_norm", "gdn_norm")


def tp_sync_replicated_grads(grads: Dict[str, torch.Tensor], group) -> None:
    """Per-head norm weights are replicated over the TP ranks but each rank applies them to its own
    heads only, so its gradient is a partial sum: add the ranks' parts (sorted names: same order
    everywhere).  Every other replicated tensor sees complete gradients thanks to ``tp_fork``."""
    import torch.distributed as dist
    for k in sorted(grads):
        if k.split(".")[-1] in TP_PARTIAL_REPLICATED:
            g = grads[k].contiguous()
            dist.all_reduce(g, group=group)
            grads[k] = g


def _clip(grads: Dict[str, torch.Tensor], max_norm: float, fb: Dict[str, object]) -> float:
    """Global-norm clip with the SAME coefficient on every TP rank: sharded gradients add their
    squares over the ranks, replicated ones count once; without this each rank would clip by its
    own shard's norm and the replicated parameters (norms, embeddings) would drift apart."""
    world = int(fb.get("tp_world", 1) or 1)
    if world > 1:
        from .parallel.mesh import grad_is_sharded
        return clip_grad_norm(grads, max_norm, sharded=grad_is_sharded, tp_group=fb.get("tp_group"), tp_world=world)
    return clip_grad_norm(grads, max_norm)


def _scored_mask(ids: torch.Tensor, prompt_lens, seq_lens) -> torch.Tensor:
    """Positions i whose *next* token is a completion token: plen-1 <= i < slen-1."""
    b, t = ids.shape
    pos = torch.arange(t)[None, :]
    pl = torch.as_tensor(prompt_lens)[:, None]
    sl = torch.as_tensor(seq_lens)[:, None]
    return (pos >= pl - 1) & (pos < sl - 1)


def forward_backward(model, ids: torch.Tensor, targets: torch.Tensor, weights_fn, *,
                     trainable: Dict[str, torch.Tensor], tp_group=None, tp_world: int = 1,
                     checkpoint_layers: bool = False, on_grad=None, hook=None, fused_ce: bool = False,
                     lp_weights_fn=None):
    """One micro-batch: dense forward on a fresh tape, weights from ``weights_fn(logits)``,
    cross-entropy op, backward.  Returns (loss, named grads, logits).  With ``fused_ce`` the head
    and the loss run chunked (``tape.linear_cross_entropy``): ``lp_weights_fn(logprobs [B, T])``
    gives the weights and the third return value is the target log-probabilities."""
    tp = T.Tape(tp_group, tp_world)
    tp.watch(*trainable.values())
    if fused_ce and tp_world == 1:
        h, w, frozen = model.forward_dense(tp, ids, checkpoint_layers=checkpoint_layers, hook=hook, return_hidden=True)
        loss, lp = T.linear_cross_entropy(tp, h, w, targets, lp_weights_fn, frozen=frozen)
        grads = tp.backward(loss, on_grad=on_grad)
        return float(loss), _named_grads(trainable, grads), lp
    logits = model.forward_dense(tp, ids, checkpoint_layers=checkpoint_layers, hook=hook)
    if tp_world > 1:
        # vocab-parallel logits: the loss and the weights come from the sharded CE
        if lp_weights_fn is None:
            raise ValueError("tensor-parallel training needs lp_weights_fn (weights from target log-probabilities)")
        loss, lp = T.cross_entropy_tp(tp, logits, targets, lp_weights_fn)
        grads = tp.backward(loss, on_grad=on_grad)
        named = _named_grads(trainable, grads)
        tp_sync_replicated_grads(named, tp_group)
        return float(loss), named, lp
    w = weights_fn(logits)
    loss = T.cross_entropy(tp, logits, targets, w)
    grads = tp.backward(loss, on_grad=on_grad)
    return float(loss), _named_grads(trainable, grads), logits


def train_step(model, ids: torch.Tensor, optimizer, *, seq_lens=None, max_norm: float = 1.0,
               lr: Optional[float] = None, micro: int = 0, **fb) -> Dict[str, float]:
    """Supervised next-token CE, mean over the B*(T-1) (or valid) positions."""
    b, t = ids.shape
    sl = torch.full((b,), t) if seq_lens is None else torch.as_tensor(seq_lens)
    mask = torch.arange(t)[None, :] < (sl[:, None] - 1)
    n = float(mask.sum())
    targets = torch.roll(ids, -1, 1)
    trainable = model.trainable()
    total, acc = 0.0, {}
    mb = micro or b
    for s in range(0, b, mb):
        m = mask[s:s + mb].float() / n
        loss, grads, _ = forward_backward(model, ids[s:s + mb], targets[s:s + mb],
                                          lambda lg, m=m: m.to(lg.device), trainable=trainable,
                                          lp_weights_fn=lambda lp, m=m: m.to(lp.device), **fb)
        total += loss
        for k, g in grads.items():
            acc[k] = g if k not in acc else acc[k] + g
    norm = _clip(acc, max_norm, fb)
    optimizer.step(acc, lr)
    return dict(loss=total, grad_norm=norm, tokens=n)


def policy_step(model, ids: torch.Tensor, prompt_lens, seq_lens, advantages: torch.Tensor,
                optimizer, *, old_logprobs: Optional[torch.Tensor] = None, clip_eps: float = 0.2,
                kl_coef: float = 0.0, ref_logprobs: Optional[torch.Tensor] = None,
                max_norm: float = 1.0, lr: Optional[float] = None, micro: int = 0,
                return_grads: bool = False, **fb) -> Dict[str, object]:
    """One GRPO update on padded ``ids [B, T]``.  ``old_logprobs [B, T]`` holds
    log pi_old of token i+1 at position i (None: on-policy, rho = 1)."""
    b, t = ids.shape
    mask = _scored_mask(ids, prompt_lens, seq_lens)
    n = max(1.0, float(mask.sum()))
    targets = torch.roll(ids, -1, 1)
    trainable = model.trainable()
    acc: Dict[str, torch.Tensor] = {}
    stats = dict(loss=0.0, clipped=0.0, ratio_mean=0.0)
    mb = micro or b
    for s in range(0, b, mb):
        sl = slice(s, s + mb)
        adv = advantages[sl, None].float()

        def weights_lp(lp, sl=sl, adv=adv):
            if old_logprobs is None:
                rho = torch.ones_like(lp)
            else:
                rho = torch.exp(lp - old_logprobs[sl].to(lp.device))
            a = adv.to(lp.device)
            unclipped = ~(((rho > 1 + clip_eps) & (a > 0)) | ((rho < 1 - clip_eps) & (a < 0)))
            w = a * rho * unclipped
            if kl_coef and ref_logprobs is not None:
                w = w - kl_coef * (1 - torch.exp(ref_logprobs[sl].to(lp.device) - lp))
            m = mask[sl].to(lp.device)
            stats["clipped"] += float((~unclipped & m).sum())
            stats["ratio_mean"] += float((rho * m).sum())
            return w * m / n

        def weights(lg, sl=sl):
            lp = ref.token_logprobs(lg.reshape(-1, lg.shape[-1]), targets[sl].reshape(-1)).view(lg.shape[:2])
            return weights_lp(lp)

        loss, grads, _ = forward_backward(model, ids[sl], targets[sl], weights, trainable=trainable,
                                          lp_weights_fn=weights_lp, **fb)
        stats["loss"] += loss
        for k, g in grads.items():
            acc[k] = g if k not in acc else acc[k] + g
    stats["ratio_mean"] /= n
    stats["grad_norm"] = _clip(acc, max_norm, fb)
    stats["tokens"] = n
    if optimizer is not None:
        optimizer.step(acc, lr)
    if return_grads:
        stats["grads"] = acc
    return stats


def drain(engine: Engine, rids: Sequence[int], max_ticks: int = 1 << 30) -> List:
    """Step the engine until every request finished.  A request the pool could not
    hold comes back empty (dead sample) instead of aborting the step."""
    ticks = 0
    while ticks < max_ticks:
        if all(engine.poll(r)["state"] == "done" for r in rids):
            break
        if not engine.step():
            break
        ticks += 1
    return [engine.take(r) for r in rids]


ROLLOUT_HEADROOM = 0.8      # mean completion length above this share of the cap: rollouts are being cut off


def refuse_short_rollouts(mean_len: Optional[float], cap: int, allow: bool = False) -> None:
    """Stop before training when rollouts cannot reach an answer: the policy's measured mean completion
    length against the rollout cap.  Truncated rollouts never state the answer, every sample of a group
    scores the floor, and the run trains on a constant reward -- which reads like a hard task, not like
    a wrong flag.  ``allow`` is for runs that want the truncation (smoke recipes).  Reference
    ``src/tilerl/train.py:1841`` (``_refuse_short_rollouts``)."""
    if not mean_len or allow or mean_len <= ROLLOUT_HEADROOM * cap:
        return
    raise SystemExit(f"error: the policy averages {mean_len:.0f} completion tokens but the rollout cap is {cap}. "
                     f"Rollouts would be cut off before they answer, so every group ties at the floor and no "
                     f"gradient flows. Raise --max-tokens above {mean_len / ROLLOUT_HEADROOM:.0f}, pick an easier "
                     f"task, or pass --allow-short-rollouts if the truncation is deliberate.")


class RolloutDrift:
    """The same check inside the loop: the mean completion length of the last ``window`` steps against the
    cap (reference ``src/tilerl/train.py:2448``).  ``update`` returns False once the window mean passes
    the headroom; ``reason`` then says what to change."""

    def __init__(self, cap: int, window: int = 5):
        self.cap, self.window, self.threshold = cap, window, ROLLOUT_HEADROOM * cap
        self.values: List[float] = []
        self.reason: Optional[str] = None
        self.mean: Optional[float] = None

    def update(self, mean_len: float, step: int) -> bool:
        self.values.append(float(mean_len))
        if len(self.values) < self.window:
            return True
        self.mean = sum(self.values[-self.window:]) / self.window
        if self.mean <= self.threshold:
            return True
        self.reason = (f"error: at step {step} the last {self.window} steps average {self.mean:.1f} completion "
                       f"tokens but the rollout cap is {self.cap}. Rollouts risk being cut off before they answer. "
                       f"Raise --max-tokens above {self.mean / ROLLOUT_HEADROOM:.0f}, pick an easier task, or pass "
                       f"--allow-short-rollouts if the truncation is deliberate.")
        return False


def grpo_loop(engine: Engine, model, prompts: Sequence[Sequence[int]], reward_fn: Callable,
              optimizer, *, steps: int, group: int = 4, prompts_per_step: int = 2,
              max_tokens: int = 16, clip_eps: float = 0.2, kl_coef: float = 0.0, lr: Optional[float] = None,
              micro: int = 0, seed: int = 0, on_policy_updates: int = 1, post_step: Optional[Callable] = None,
              length_penalty: float = 0.0, judge: Optional[Callable] = None,
              max_think_tokens: Optional[int] = None, **fb) -> Iterator[Dict[str, object]]:
    """Yields one metrics dict per RL step (mean reward, loss, seconds by phase).  ``judge(prompt,
    completions, rewards) -> rewards``: called per group after the rule-based reward, it may order the
    completions that tie (the rule decides first; see ``evals.judge_tiebreak``)."""
    engine.invalidate_weights()
    cursor = 0
    for step in range(steps):
        t0 = time.perf_counter()
        batch_prompts = [prompts[(cursor + i) % len(prompts)] for i in range(prompts_per_step)]
        cursor += prompts_per_step
        rids = []
        for pi, p in enumerate(batch_prompts):
            for g in range(group):
                sp = SamplingParams(max_tokens=max_tokens, temperature=1.0, top_p=1.0, top_k=0,
                                    seed=seed + ((step * 1009 + pi) * 131 + g), logprobs=True,
                                    max_think_tokens=max_think_tokens)
                require_on_policy(sp)
                rids.append(engine.submit(p, sp))
        results = drain(engine, rids)
        t1 = time.perf_counter()
        comps = [r.tokens if r is not None else [] for r in results]
        live = [len(c) > 0 for c in comps]
        task = [float(reward_fn(batch_prompts[i // group], c)) for i, c in enumerate(comps)]
        if judge is not None:
            for gi in range(prompts_per_step):
                sl = slice(gi * group, (gi + 1) * group)
                task[sl] = [float(x) for x in judge(batch_prompts[gi], comps[sl], task[sl])]
        rewards = [t - length_penalty * len(c) for t, c in zip(task, comps)]
        # the task reward is the signal: a group that only differs in length gets no gradient
        adv = group_advantages(rewards, group, live, signal=task, groups=prompts_per_step)
        seqs = [list(batch_prompts[i // group]) + c for i, c in enumerate(comps)]
        plens = [len(batch_prompts[i // group]) for i in range(len(seqs))]
        slens = [len(s) for s in seqs]
        ids = pad_batch(seqs, pow2=False)
        old = None
        if on_policy_updates > 1:
            old = torch.zeros(ids.shape, dtype=torch.float32)
            for i, r in enumerate(results):
                if r is not None and r.logprobs:
                    old[i, plens[i] - 1:plens[i] - 1 + len(r.logprobs)] = torch.tensor(r.logprobs)
        t2 = time.perf_counter()
        stats = {}
        for _ in range(on_policy_updates):
            stats = policy_step(model, ids.to(engine.device), plens, slens, adv, optimizer,
                                old_logprobs=old, clip_eps=clip_eps, kl_coef=kl_coef, lr=lr,
                                micro=micro, **fb)
        t3 = time.perf_counter()
        if post_step is not None:
            post_step(model)
        engine.invalidate_weights()
        t4 = time.perf_counter()
        n_tied = sum(1 for g0 in range(0, len(rewards), group)
                     if len(set(rewards[g0:g0 + group])) == 1)
        yield dict(step=step, reward=sum(rewards) / len(rewards), loss=stats.get("loss", 0.0),
                   grad_norm=stats.get("grad_norm", 0.0), tokens=stats.get("tokens", 0),
                   tied_groups=n_tied, completion_tokens=sum(len(c) for c in comps),
                   mean_completion_tokens=sum(len(c) for c in comps) / max(1, len(comps)),
                   # one row per completion, so that length and reward stay paired (group means per step
                   # confound them with the difficulty of the step's prompts)
                   rollouts=[dict(prompt=i // group, tokens=len(c), reward=rewards[i], task=task[i],
                                  finish=(results[i].finish_reason if results[i] is not None else "lost"))
                             for i, c in enumerate(comps)],
                   timings=dict(rollout=t1 - t0, score=t2 - t1, train=t3 - t2,
                                invalidate=t4 - t3, total=t4 - t0))


def opd_loop(engine: Engine, model, prompts, optimizer, *, steps: int, max_tokens: int = 16,
             ema: float = 0.99, prompts_per_step: int = 2, lr=None, seed: int = 0, **fb):
    """On-policy distillation with an EMA teacher: the engine generates each completion under an
    exponential moving average of the trainable tensors (the teacher: the same model, only
    adapter-sized memory is duplicated), then the student weights are swapped back in and take one
    supervised :func:`train_step` on prompt + completion.  The swaps copy INTO the live tensors and
    never rebind them -- the engine and captured graphs read those objects -- and the engine's
    cached state is invalidated around every swap, because a prefix entry or a captured graph made
    under one set of weights must not be replayed under the other.

    Parity: reference ``opd_loop`` (``src/tilerl/train.py:1138-1200``): teacher generates under the
    EMA adapters, student runs ``train_step``; here ``prompts_per_step`` prompts form one batch."""
    trainable = model.trainable()
    teacher = {k: v.detach().clone() for k, v in trainable.items()}
    student = {k: v.detach().clone() for k, v in trainable.items()}

    def swap_in(src):
        with torch.no_grad():
            for k, v in trainable.items():
                v.copy_(src[k])
        model.requantize_()
        engine.invalidate_weights()

    engine.invalidate_weights()
    cursor = 0
    for step in range(steps):
        ps = [prompts[(cursor + i) % len(prompts)] for i in range(prompts_per_step)]
        cursor += prompts_per_step
        swap_in(teacher)                                   # the teacher generates
        rids = [engine.submit(p, SamplingParams(max_tokens=max_tokens, temperature=1.0, seed=seed + step * 131 + i))
                for i, p in enumerate(ps)]
        results = drain(engine, rids)
        seqs = [list(p) + (r.tokens if r else []) for p, r in zip(ps, results)]
        swap_in(student)                                   # the student learns from it
        ids = pad_batch(seqs).to(engine.device)
        m = train_step(model, ids, optimizer, seq_lens=[len(s) for s in seqs], lr=lr, **fb)
        with torch.no_grad():
            for k, v in trainable.items():
                student[k].copy_(v)
                teacher[k].mul_(ema).add_(v.detach(), alpha=1 - ema)
        model.requantize_()
        engine.invalidate_weights()
        yield dict(step=step, loss=m["loss"], tokens=m["tokens"], grad_norm=m["grad_norm"],
                   completion_tokens=sum(len(r.tokens) if r else 0 for r in results))


def pretrain(model, data: Iterator[torch.Tensor], optimizer, *, steps: int, lr: float, warmup: int = 0,
             ckpt_every: int = 0, ckpt_dir: Optional[str] = None, log: Optional[Callable] = None, **fb):
    """SFT/pre-training loop with cosine schedule and periodic checkpoints."""
    from .checkpoint import save_checkpoint
    history = []
    for step in range(steps):
        ids = next(data)
        cur = cosine_warmup(step, steps, warmup, lr)
        m = train_step(model, ids, optimizer, lr=cur, **fb)
        m.update(step=step, lr=cur)
        history.append(m)
        if log:
            log(json.dumps(m))
        if ckpt_every and ckpt_dir and (step + 1) % ckpt_every == 0:
            save_checkpoint(model, os.path.join(ckpt_dir, f"step_{step + 1}"))
    if ckpt_dir:
        save_checkpoint(model, os.path.join(ckpt_dir, "final"))
    return history


def eval_reward(engine: Engine, prompts: Sequence[Sequence[int]], reward_fn: Callable, *, max_tokens: int = 16,
                seed: int = 12345) -> float:
    """Mean reward of greedy completions on held-out prompts (the eval signal of adapter runs)."""
    res = engine.generate([list(p) for p in prompts], SamplingParams(max_tokens=max_tokens, seed=seed))
    return sum(float(reward_fn(p, r.tokens)) for p, r in zip(prompts, res)) / max(1, len(prompts))


def train_adapters(engine: Engine, model, prompts: Sequence[Sequence[int]], reward_fn: Callable, optimizer, *,
                   steps: int, eval_prompts: Optional[Sequence[Sequence[int]]] = None, eval_every: int = 0,
                   patience: int = 3, save_dir: Optional[str] = None, run=None, opd: bool = False,
                   **loop_kw) -> Dict[str, object]:
    """Adapter (LoRA) GRPO / OPD run with periodic evals, early stopping on the eval reward, the
    best adapter kept on disk and every step logged to the run manifest.

    Parity: reference ``_train_adapters`` (``src/tilerl/train.py:1920-2535``): evals, early stop,
    ``adapter.safetensors`` + ``adapter-best.safetensors``, run manifest with gates."""
    from .checkpoint import save_adapter
    from .ledger import EarlyStop
    stop = EarlyStop(patience=patience)
    history: List[Dict[str, object]] = []
    evals: List[Dict[str, float]] = []
    if opd:
        loop = opd_loop(engine, model, prompts, optimizer, steps=steps, **loop_kw)
    else:
        loop = grpo_loop(engine, model, prompts, reward_fn, optimizer, steps=steps, **loop_kw)
    stopped = False
    for m in loop:
        history.append(m)
        if run is not None:
            run.log(**{k: v for k, v in m.items() if not isinstance(v, (dict, list))})
        step = int(m["step"])
        if eval_every and eval_prompts and (step + 1) % eval_every == 0:
            score = eval_reward(engine, eval_prompts, reward_fn, max_tokens=loop_kw.get("max_tokens", 16))
            evals.append(dict(step=step, reward=score))
            if run is not None:
                run.log(step=step, eval_reward=score)
            done = stop.update(score, step)
            if stop.improved and save_dir:
                os.makedirs(save_dir, exist_ok=True)
                save_adapter(model, os.path.join(save_dir, "adapter-best.safetensors"))
            if done:
                stopped = True
                break
    if save_dir:
        os.makedirs(save_dir, exist_ok=True)
        save_adapter(model, os.path.join(save_dir, "adapter.safetensors"))
    out = dict(steps=len(history), evals=evals, best_eval=stop.best, best_step=stop.best_step,
               early_stopped=stopped, history=history)
    if run is not None:
        if stop.best is not None and evals:
            run.gate("eval_reward_not_worse", stop.best, evals[0]["reward"])
        if save_dir:
            run.artifacts["adapter"] = os.path.join(save_dir, "adapter.safetensors")
    return out
