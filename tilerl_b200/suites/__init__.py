"""Measurement suites behind ``python -m tilerl_b200.cli bench --suite NAME [args...]``.

Each suite is a module with ``main(argv)`` that builds the named model with random-init weights,
runs one workload of the benchmark configurations on the GPU(s) it is started on and prints one
JSON line:

* ``spec`` / ``batch`` / ``sparse`` (:mod:`.serve`): speculative decode with the block drafter,
  continuous batching of long prompts, sparse top-k KV decode at long context;
* ``tick`` (:mod:`.tick`): eager decode ticks (and one prefill) with a per-op event breakdown, the
  command profiler captures of single kernels are taken on;
* ``grpo`` (:mod:`.grpo`): one-GPU GRPO step with LoRA adapters, split rollout / train;
* ``grpo-zero3`` (:mod:`.grpo_zero3`, started under ``torchrun``): GRPO step with ZeRO-3 training
  and a tensor-parallel NVFP4 rollout engine on the same GPUs.

Parity: the reference's ``tilerl bench --suite`` (``src/tilerl/bench.py:215-230``) hands the name to
its harness script; here the suites are importable modules.
"""
from __future__ import annotations

import importlib
from typing import List, Optional

SUITES = {
    "spec": ("serve", ["--what", "spec"]),
    "batch": ("serve", ["--what", "batch"]),
    "sparse": ("serve", ["--what", "sparse"]),
    "tick": ("tick", []),
    "grpo": ("grpo", []),
    "grpo-zero3": ("grpo_zero3", []),
}


def run(name: str, argv: Optional[List[str]] = None) -> int:
    if name not in SUITES:
        raise SystemExit(f"unknown suite {name!r}; known: {', '.join(sorted(SUITES))}")
    mod, fixed = SUITES[name]
    m = importlib.import_module(f"{__name__}.{mod}")
    m.main(fixed + list(argv or []))
    return 0
