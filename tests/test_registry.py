"""The declared support matrix (ops/registry.py) against the tree: every registered kernel exists
in the file it names, every entry point is declared by the module that binds it, and cells that
nobody registered refuse loudly.  Counterpart of the reference's tests/test_support_matrix.py."""
import importlib
import os
import re

import pytest

from tilerl_b200.ops import registry as R

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cells():
    for (precision, arch), table in R._CELLS.items():
        for op, k in table.items():
            yield precision, arch, op, k


def test_every_registered_kernel_exists_where_it_says():
    for precision, arch, op, k in _cells():
        path = os.path.join(ROOT, k.source)
        assert os.path.exists(path), (op, k.source)
        text = open(path).read()
        if k.entry is None and arch == "cpu":
            assert re.search(rf"^def {re.escape(k.name)}\(", text, re.M), (op, k.name)
        elif k.entry is not None:
            for name in re.split(r"\s*[+/]\s*", k.name):
                name = re.sub(r"<.*>", "", name).rstrip("*").strip()
                if name.endswith("_kernel") or name.startswith("trl_"):
                    assert name in text, (op, name, k.source)
            assert k.entry in text, (op, k.entry)


def test_every_entry_point_is_bound_by_the_module_it_names():
    for _, _, op, k in _cells():
        if k.entry is None:
            continue
        mod = importlib.import_module(k.binds)
        assert k.entry in open(mod.__file__).read(), (op, k.entry, k.binds)


def test_resolution_falls_through_and_refuses_unknown_cells():
    assert R.resolve("attn_prep", "fp8", "sm100").entry == "trl_attn_prep_fp8"
    assert R.resolve("attn_prep", "nvfp4", "sm100").entry == "trl_attn_prep"      # (any, sm100)
    assert R.resolve("attn_prep", "nvfp4", "cpu").source.endswith("ref.py")
    with pytest.raises(NotImplementedError):
        R.resolve("linear_nvfp4_gemm", "nvfp4", "sm90")
    with pytest.raises(NotImplementedError):
        R.resolve("no_such_op", "nvfp4", "sm100")
    assert "gdn" in R.ops("nvfp4", "sm100") and "gdn" in R.ops("any", "cpu")


def test_linear_bands_follow_the_dispatch_of_the_cuda_backend():
    assert [R.linear_kernel_for(m) for m in (1, 2, 3, 8, 64, 512)] == \
        ["linear_nvfp4_gemv"] * 2 + ["linear_nvfp4_gemm"] * 4
    assert [R.linear_kernel_for(m, mma_rows=True) for m in (2, 3, 16, 17)] == \
        ["linear_nvfp4_gemv", "linear_nvfp4_rows16", "linear_nvfp4_rows16", "linear_nvfp4_gemm"]
    R.resolve("linear_nvfp4_rows16", "nvfp4", "sm100")
    assert R.linear_kernel_for(8, gemv_tokens=8) == "linear_nvfp4_gemv"
    assert R.arch_for("cpu") == "cpu"
    for m in (1, 8, 512):
        R.resolve(R.linear_kernel_for(m), "nvfp4", "sm100")
        R.resolve(R.linear_kernel_for(m, precision="bf16"), "bf16", "sm100")
