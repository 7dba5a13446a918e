"""The instruction-table forward (tilerl_b200/mega.py): its interpreter on the reference backend
equals the model's own forward bit for bit, for a ragged prefill and the decode ticks after it."""
import torch

from helpers import rand_prompts
from tilerl_b200 import mega
from tilerl_b200.batch import Batch
from tilerl_b200.config import tiny_hybrid
from tilerl_b200.kv import GdnStatePool, PagedKvPool
from tilerl_b200.models.hybrid import HybridModel
from tilerl_b200.ops.backend import RefOps


def _pools(cfg):
    return PagedKvPool(cfg, 16, dtype=torch.float32), GdnStatePool(cfg, 4, ring_dtype=torch.float32)


def test_interpreter_equals_the_forward_for_prefill_and_decode():
    cfg = tiny_hybrid()
    model = HybridModel.build_random(cfg, seed=2)
    prog = mega.compile_program(model)
    n_layers = len(cfg.layer_types)
    assert len(prog) == 1 + 5 * n_layers + 2
    assert "NORM_SWIGLU" in prog.listing() and "L0.norm1" in prog.listing()
    prompts = rand_prompts(cfg, 2, 19)
    prompts[1] = prompts[1][:7]
    ops = RefOps()
    pools = {k: _pools(cfg) for k in ("fwd", "prog")}
    ticks = [[dict(tokens=p, start=0, blocks=[1 + 2 * i, 2 + 2 * i], slot=i + 1) for i, p in enumerate(prompts)]]
    for step in range(3):
        ticks.append([dict(tokens=[5 + step + i], start=len(p) + step, blocks=[1 + 2 * i, 2 + 2 * i], slot=i + 1)
                      for i, p in enumerate(prompts)])
    for seqs in ticks:
        batch = Batch.build(seqs, "cpu")
        want = model.forward(batch, ops, *pools["fwd"])
        got = mega.interpret(prog, model, batch, ops, *pools["prog"])
        assert torch.equal(got, want)
    assert torch.equal(pools["fwd"][1].states, pools["prog"][1].states)


def test_all_rows_program_and_adapter_refusal():
    cfg = tiny_hybrid()
    model = HybridModel.build_random(cfg, seed=3)
    prog = mega.compile_program(model, last_only=False)
    assert mega.OPCODE_NAMES[int(prog.table[-2, 0])] != "GATHER_LAST"
    batch = Batch.build([dict(tokens=[1, 2, 3, 4, 5], start=0, blocks=[1], slot=1)], "cpu")
    ops = RefOps()
    a, b = _pools(cfg), _pools(cfg)
    assert torch.equal(mega.interpret(prog, model, batch, ops, *a), model.forward(batch, ops, *b, last_only=False))
    model.add_lora(rank=2)
    try:
        mega.compile_program(model)
    except ValueError:
        pass
    else:
        raise AssertionError("adapters must be refused")
