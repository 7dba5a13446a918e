"""Evaluation and reward functions: multiple-choice accuracy (MMLU style), GSM8K-style
numeric answers, boxed-answer matching, synthetic rewards for the RL gates, and a pairwise
self-judge with Copeland tie-breaking.

Parity: reference ``src/tilerl/eval.py``, ``src/tilerl/math_answer.py``, ``src/tilerl/judge.py``.
"""
from __future__ import annotations

import re
from fractions import Fraction
from typing import Callable, Dict, List, Optional, Sequence


# ---- answer extraction -------------------------------------------------------------------------
def last_boxed(text: str) -> Optional[str]:
    i = text.rfind("\\boxed{")
    if i < 0:
        return None
    depth, j = 0, i + 7
    start = j
    while j < len(text):
        if text[j] == "{":
            depth += 1
        elif text[j] == "}":
            if depth == 0:
                return text[start:j]
            depth -= 1
        j += 1
    return None


def _num(s: str) -> Optional[Fraction]:
    s = s.strip().replace(",", "").replace("$", "").rstrip(".")
    m = re.fullmatch(r"\\?d?frac\{(-?\d+)\}\{(-?\d+)\}", s)
    if m:
        return Fraction(int(m.group(1)), int(m.group(2)))
    try:
        return Fraction(s)
    except (ValueError, ZeroDivisionError):
        return None


def answers_match(pred: Optional[str], gold: str) -> bool:
    if pred is None:
        return False
    a, b = _num(pred), _num(gold)
    if a is not None and b is not None:
        return a == b
    norm = lambda s: re.sub(r"\s+", "", s).lower()
    return norm(pred) == norm(gold)


def gsm8k_answer(text: str) -> Optional[str]:
    b = last_boxed(text)
    if b is not None:
        return b
    m = re.findall(r"####\s*(-?[\d,\.]+)", text)
    if m:
        return m[-1]
    m = re.findall(r"-?\d[\d,]*\.?\d*", text)
    return m[-1] if m else None


def choice_answer(text: str, letters: str = "ABCD") -> Optional[str]:
    m = re.findall(rf"\b([{letters}])\b", text.upper())
    return m[-1] if m else None


# ---- rewards for GRPO ---------------------------------------------------------------------------------
def reward_even(prompt: Sequence[int], completion: Sequence[int]) -> float:
    """Fraction of generated ids that are even (tiny-config gate)."""
    return sum(1 for t in completion if t % 2 == 0) / max(1, len(completion))


def reward_mod7(prompt: Sequence[int], completion: Sequence[int]) -> float:
    """1 if the sum of the last 4 generated ids is divisible by 7, else 0."""
    return 1.0 if len(completion) >= 1 and sum(completion[-4:]) % 7 == 0 else 0.0


def make_text_reward(tokenizer, gold: Dict[str, str], kind: str = "gsm8k") -> Callable:
    extract = gsm8k_answer if kind == "gsm8k" else last_boxed

    def fn(prompt_ids, completion_ids) -> float:
        p = tokenizer.decode(prompt_ids)
        g = next((v for k, v in gold.items() if k in p), None)
        return 1.0 if g is not None and answers_match(extract(tokenizer.decode(completion_ids)), g) else 0.0
    return fn


REWARDS = {"even": reward_even, "mod7": reward_mod7}


# ---- engine-driven evaluation -------------------------------------------------------------------------------
def evaluate(engine, tokenizer, items: List[Dict[str, str]], *, kind: str = "gsm8k", max_tokens: int = 256,
             batch: int = 8, render: Optional[Callable[[str], str]] = None) -> Dict[str, float]:
    """``items``: dicts with ``question`` and ``answer`` (and ``choices`` for multiple choice)."""
    from .engine import SamplingParams
    correct = total = gen = 0
    for i in range(0, len(items), batch):
        chunk = items[i:i + batch]
        texts = []
        for it in chunk:
            q = it["question"]
            if kind == "choice":
                q += "\n" + "\n".join(f"{l}. {c}" for l, c in zip("ABCD", it["choices"])) + "\nAnswer:"
            texts.append(render(q) if render else q)
        res = engine.generate([tokenizer.encode(t) for t in texts], SamplingParams(max_tokens=max_tokens))
        for it, r in zip(chunk, res):
            out = tokenizer.decode(r.tokens)
            pred = choice_answer(out) if kind == "choice" else gsm8k_answer(out)
            correct += int(answers_match(pred, it["answer"]))
            total += 1
            gen += len(r.tokens)
    return {"accuracy": correct / max(1, total), "n": total, "mean_tokens": gen / max(1, total)}


# ---- pairwise self-judge --------------------------------------------------------------------------------------
def copeland_scores(n: int, wins: Dict[tuple, float]) -> List[float]:
    """``wins[(i, j)]`` in [0, 1]: how strongly i beat j.  Copeland score = wins - losses."""
    s = [0.0] * n
    for (i, j), w in wins.items():
        if w > 0.5:
            s[i] += 1
            s[j] -= 1
        elif w < 0.5:
            s[i] -= 1
            s[j] += 1
    return s


def judge_tiebreak(rewards: Sequence[float], completions: Sequence[str], compare: Callable[[str, str], float],
                   eps: float = 0.05) -> List[float]:
    """Within a group whose rule-based rewards tie, add a small pairwise-judge bonus so the
    group still carries a signal.  ``compare(a, b)`` returns P(a better than b)."""
    out = list(rewards)
    groups: Dict[float, List[int]] = {}
    for i, r in enumerate(rewards):
        groups.setdefault(r, []).append(i)
    for idx in groups.values():
        if len(idx) < 2:
            continue
        wins = {(a, b): compare(completions[idx[a]], completions[idx[b]])
                for a in range(len(idx)) for b in range(a + 1, len(idx))}
        sc = copeland_scores(len(idx), wins)
        top = max(abs(x) for x in sc) or 1.0
        for k, i in enumerate(idx):
            out[i] += eps * sc[k] / top
    return out


def policy_compare(engine, tokenizer, question: str = "", max_tokens: int = 2) -> Callable[[str, str], float]:
    """``compare(a, b)`` for :func:`judge_tiebreak` answered by the policy itself: the two completions are
    shown as answers A and B, the engine decodes greedily and the first ``A`` / ``B`` of its reply decides
    (1.0: a is better, 0.0: b is, 0.5: neither letter).  Both orders are asked and averaged, so a policy
    that always says "A" ranks nothing.  Parity: the reference's self-judge (src/tilerl/judge.py)."""
    from .engine import SamplingParams

    def ask(first: str, second: str) -> float:
        text = (f"{question}\nAnswer A:\n{first}\nAnswer B:\n{second}\n"
                "Which answer is better? Reply with A or B.\n")
        out = tokenizer.decode(engine.generate([tokenizer.encode(text)], SamplingParams(max_tokens=max_tokens))[0].tokens)
        for ch in out:
            if ch in "AB":
                return 1.0 if ch == "A" else 0.0
        return 0.5

    def compare(a: str, b: str) -> float:
        return 0.5 * (ask(a, b) + (1.0 - ask(b, a)))
    return compare
