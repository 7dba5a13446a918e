"""A forward as data: an instruction table for one tick and its interpreter.

``compile_program(model)`` turns the serving forward of a model into an int32 table
``program[ip, 8]`` over numbered activation buffers and numbered parameters; ``interpret``
walks the table against any op backend.  On the reference backend the interpreter is the
oracle of the table (it must equal :meth:`HybridModel.forward` bit for bit), which is what a
persistent single-launch tick would be checked against: the table is exactly the work list
such a kernel loops over, with a grid-wide barrier between instructions.

Instruction row: ``(opcode, dst, src, aux_src, p0, p1, p2, layer_slot)``.

=============  =====================================================================
opcode         meaning (buffers ``b*``, parameters ``p*`` by index into ``params``)
=============  =====================================================================
EMBED          ``b[dst] = params[p0][token_ids]``
NORM_LINEAR    ``b[dst] = rmsnorm(b[src], params[p0]) @ params[p1]^T``
ATTENTION      ``b[dst] = attention(b[src]; q_norm p0, k_norm p1; attention layer layer_slot)``
GDN            ``b[dst] = gdn(b[src]; conv p0, dt_bias p1, a_log p2, gdn_norm in aux_src; GDN layer layer_slot)``
LINEAR_RES     ``b[dst] += b[src] @ params[p0]^T``  (in place on the residual stream)
NORM_SWIGLU    ``b[dst] = swiglu(rmsnorm(b[src], params[p0]) @ params[p1]^T)``
GATHER_LAST    ``b[dst] = b[src][last token of every sequence]``
LM_HEAD        ``b[dst] = rmsnorm(b[src], params[p0]) @ params[p1]^T`` in fp32, cut to the vocabulary
=============  =====================================================================

Parity: the instruction-table forward of the reference's experimental megakernel
(``tilerl_kernels/mega.py:8`` ``MegaForward``, ``mega_loader.py``, the CPU interpreter oracle
``mega_reference.py``; opcodes ``kernels_mega.py:31``).  The reference measured its persistent
kernel 9.2x slower than its serial path; the persistent kernel is not built here, the table and
its oracle are.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

import torch

from .config import ATTN

EMBED, NORM_LINEAR, ATTENTION, GDN, LINEAR_RES, NORM_SWIGLU, GATHER_LAST, LM_HEAD = range(8)
OPCODE_NAMES = ("EMBED", "NORM_LINEAR", "ATTENTION", "GDN", "LINEAR_RES", "NORM_SWIGLU", "GATHER_LAST", "LM_HEAD")
# activation buffers of a tick
B_X, B_PROJ, B_MIX, B_ACT, B_LAST, B_LOGITS = range(6)
N_BUFFERS = 6


@dataclass
class Program:
    table: torch.Tensor          # int32 [n_instructions, 8]
    param_names: List[str]       # index -> parameter name
    last_only: bool

    def __len__(self) -> int:
        return int(self.table.shape[0])

    def listing(self) -> str:
        rows = []
        for ip, r in enumerate(self.table.tolist()):
            ps = [self.param_names[i] if i >= 0 else "-" for i in r[4:7]]
            rows.append(f"{ip:4d} {OPCODE_NAMES[r[0]]:12s} b{r[1]} <- b{r[2]}  {' '.join(ps)}  slot {r[7]}")
        return "\n".join(rows)


def compile_program(model, last_only: bool = True) -> Program:
    """The serving forward of ``model`` (no LoRA, no taps) as an instruction table."""
    if model.lora:
        raise ValueError("the instruction table covers the base forward: merge or drop the adapters first")
    cfg = model.cfg
    names: List[str] = []
    index: Dict[str, int] = {}

    def pid(name: str) -> int:
        if name not in index:
            index[name] = len(names)
            names.append(name)
        return index[name]

    rows = [(EMBED, B_X, -1, -1, pid("embed"), -1, -1, 0)]
    ai = gi = 0
    for i, t in enumerate(cfg.layer_types):
        p = f"L{i}."
        if t == ATTN:
            rows.append((NORM_LINEAR, B_PROJ, B_X, -1, pid(p + "norm1"), pid(p + "qkv"), -1, 0))
            rows.append((ATTENTION, B_MIX, B_PROJ, -1, pid(p + "q_norm"), pid(p + "k_norm"), -1, ai))
            rows.append((LINEAR_RES, B_X, B_MIX, -1, pid(p + "o"), -1, -1, 0))
            ai += 1
        else:
            rows.append((NORM_LINEAR, B_PROJ, B_X, -1, pid(p + "norm1"), pid(p + "in"), -1, 0))
            rows.append((GDN, B_MIX, B_PROJ, pid(p + "gdn_norm"), pid(p + "conv"), pid(p + "dt_bias"),
                         pid(p + "a_log"), gi))
            rows.append((LINEAR_RES, B_X, B_MIX, -1, pid(p + "out"), -1, -1, 0))
            gi += 1
        rows.append((NORM_SWIGLU, B_ACT, B_X, -1, pid(p + "norm2"), pid(p + "gate_up"), -1, 0))
        rows.append((LINEAR_RES, B_X, B_ACT, -1, pid(p + "down"), -1, -1, 0))
    src = B_X
    if last_only:
        rows.append((GATHER_LAST, B_LAST, B_X, -1, -1, -1, -1, 0))
        src = B_LAST
    head = "embed" if cfg.tie_embeddings else "lm_head"
    rows.append((LM_HEAD, B_LOGITS, src, -1, pid("final_norm"), pid(head), -1, 0))
    return Program(torch.tensor(rows, dtype=torch.int32), names, last_only)


def interpret(program: Program, model, batch, ops, kv_pool, state_pool) -> torch.Tensor:
    """Runs the table instruction by instruction on ``ops``; returns the logits buffer."""
    cfg, d, P = model.cfg, model.dims, model.params
    eps = cfg.rms_eps
    prm = [P[n] for n in program.param_names]
    buf: List = [None] * N_BUFFERS
    for op, dst, src, aux, p0, p1, p2, slot in program.table.tolist():
        if op == EMBED:
            buf[dst] = ops.embed(prm[p0], batch.token_ids)
        elif op == NORM_LINEAR:
            buf[dst] = ops.norm_linear(buf[src], prm[p0], prm[p1], eps, None)
        elif op == ATTENTION:
            buf[dst] = ops.attention(buf[src], {"q_norm": prm[p0], "k_norm": prm[p1]}, batch, kv_pool, slot, cfg,
                                     d.n_q, d.n_kv)
        elif op == GDN:
            lp = {"conv": prm[p0], "dt_bias": prm[p1], "a_log": prm[p2], "gdn_norm": prm[aux]}
            buf[dst] = ops.gdn(buf[src], lp, batch, state_pool, slot, cfg, d.gdn_nk, d.gdn_nv)
        elif op == LINEAR_RES:
            buf[dst] = ops.linear_residual(buf[src], prm[p0], buf[dst], None)
        elif op == NORM_SWIGLU:
            buf[dst] = ops.norm_linear_swiglu(buf[src], prm[p0], prm[p1], eps, None)
        elif op == GATHER_LAST:
            getattr(ops, "settle", lambda: None)()     # queued projections write the row before it is gathered
            buf[dst] = buf[src][batch.last_idx.long()]
        elif op == LM_HEAD:
            buf[dst] = ops.lm_head(buf[src], prm[p0], prm[p1], eps)[..., :cfg.vocab]
        else:
            raise ValueError(f"unknown opcode {op}")
    return buf[B_LOGITS]
