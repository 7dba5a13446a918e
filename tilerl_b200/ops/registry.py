"""Kernel registry: which kernel serves which op, per (precision, target).

The dispatch itself is by shape inside :class:`tilerl_b200.ops.cuda.CudaOps` (one GPU target, so
no indirection on the hot path); this table is the declared support matrix that tools and tests
read: ``resolve(op, precision, arch)`` falls through exact cell -> ``(precision, "any")`` ->
``("any", "any")`` and raises ``NotImplementedError`` for a cell nobody registered, and
``linear_kernel_for(m)`` names the projection kernel of a launch of ``m`` token rows.

Every ``sm100`` entry names the kernel, its source file under ``csrc/`` and the C entry point of
``_C.so`` that launches it; ``tests/test_registry.py`` checks that the sources exist and that the
entry points are declared in :mod:`tilerl_b200.ops.native` (or by the module named in ``binds``).

Parity: reference ``packages/tilerl-kernels/src/tilerl_kernels/registry.py:12-40`` (``_register`` /
``_resolve``), ``:198-209`` (MMA-dtype bands by launch M); its sm100 cell is empty (``:188-189``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple


@dataclass(frozen=True)
class Kernel:
    name: str                 # kernel (or oracle function) name
    source: str               # file that defines it
    entry: Optional[str] = None   # C entry point in _C.so (None: a Python function)
    binds: str = "tilerl_b200.ops.native"   # module that declares the entry point's signature
    note: str = ""


_CELLS: Dict[Tuple[str, str], Dict[str, Kernel]] = {}


def register(precision: str, arch: str, table: Dict[str, Kernel]) -> None:
    _CELLS.setdefault((precision, arch), {}).update(table)


def resolve(op: str, precision: str = "any", arch: str = "any") -> Kernel:
    for cell in ((precision, arch), (precision, "any"), ("any", arch), ("any", "any")):
        k = _CELLS.get(cell, {}).get(op)
        if k is not None:
            return k
    raise NotImplementedError(f"no kernel registered for op {op!r} at ({precision}, {arch})")


def ops(precision: str = "any", arch: str = "any") -> List[str]:
    """Every op name that resolves for the cell."""
    names = set()
    for (p, a), table in _CELLS.items():
        if p in (precision, "any") and a in (arch, "any"):
            names |= set(table)
    return sorted(names)


def arch_for(device) -> str:
    """``cpu`` or ``sm100``; any other GPU has no cell (single target by design)."""
    import torch
    device = torch.device(device)
    if device.type != "cuda":
        return "cpu"
    major, minor = torch.cuda.get_device_capability(device)
    if major == 10:
        return "sm100"
    raise NotImplementedError(f"no kernels for compute capability {major}.{minor}: this build targets sm_100a only")


# Projection kernel by launch M (token rows): the weight-streaming GEMV up to `gemv_tokens`
# rows, the tcgen05 block-scaled GEMM above; with `mma_rows` (the backend's TRL_GEMV_MMA switch, off by
# default) 3..16 rows go to the mma.sync kernel with f16 activations.
def linear_kernel_for(m: int, gemv_tokens: int = 2, precision: str = "nvfp4", mma_rows: bool = False) -> str:
    if precision == "bf16":
        return "linear_bf16_gemv" if m <= 8 else "linear_bf16_gemm"
    if m <= gemv_tokens:
        return "linear_nvfp4_gemv"
    return "linear_nvfp4_rows16" if (mma_rows and m <= 16) else "linear_nvfp4_gemm"


_REF = "tilerl_b200/ops/ref.py"
register("any", "cpu", {op: Kernel(fn, _REF) for op, fn in {
    "embed": "embedding", "rmsnorm": "rmsnorm", "linear": "linear", "swiglu": "swiglu", "attn_prep": "attn_prep",
    "kv_write": "kv_write", "kv_write_fp8": "kv_write_fp8", "paged_attention_decode": "paged_attention",
    "paged_attention_prefill": "paged_attention", "gdn": "gdn_sequence", "gdn_chunked": "gdn_chunked",
    "gdn_backward": "gdn_recurrent_backward", "sample": "sample", "sample_nucleus": "sample_nucleus_model",
    "cross_entropy": "cross_entropy_grad", "cross_entropy_sharded": "cross_entropy_sharded",
    "page_bounds": "page_bounds", "select_pages": "select_pages",
}.items()})
register("any", "cpu", {
    "quantize_nvfp4": Kernel("quantize_nvfp4", "tilerl_b200/formats.py"),
    "dequantize_nvfp4": Kernel("dequantize_nvfp4", "tilerl_b200/formats.py"),
})

register("nvfp4", "sm100", {
    "linear_nvfp4_gemv": Kernel("gemv_nvfp4_kernel / gemv_nvfp4_sk_kernel", "csrc/gemv.cu", "trl_gemv_nvfp4",
                                note="M <= 8; RMSNorm prologue; residual / SwiGLU / fp32 / TP-push epilogues"),
    "linear_nvfp4_rows16": Kernel("gemv_nvfp4_mma_kernel", "csrc/gemv_mma.cu", "trl_gemv_nvfp4_mma",
                                  note="3..16 rows: weights as the mma.sync A operand, f16 activations, every epilogue"),
    "linear_nvfp4_gemm": Kernel("gemm_nvfp4_kernel", "csrc/gemm_tc.cu", "trl_gemm_nvfp4", "tilerl_b200.ops.gemm_tc",
                                note="tcgen05.mma kind::mxf4nvf4.block_scale, TMA, TMEM accumulator, stream-K"),
    "quant_act_nvfp4": Kernel("quant_act_kernel", "csrc/gemm_tc.cu", "trl_quant_act_nvfp4", "tilerl_b200.ops.gemm_tc",
                              note="RMSNorm / SwiGLU + J NVFP4 residual terms per token"),
    "quantize_nvfp4": Kernel("quant_nvfp4_kernel", "csrc/misc.cu", "trl_quant_nvfp4", note="weights, in place (resync)"),
    "dequantize_nvfp4": Kernel("dequant_nvfp4_kernel", "csrc/misc.cu", "trl_dequant_nvfp4"),
})
register("bf16", "sm100", {
    "linear_bf16_gemv": Kernel("gemv_bf16_kernel", "csrc/gemv.cu", "trl_gemv_bf16"),
    "linear_bf16_gemv_rows16": Kernel("gemv_bf16_mma_kernel", "csrc/gemv.cu", "trl_gemv_bf16",
                                      note="3..16 rows (batched / verify lm_head): one mma.sync pass over the weights"),
    "linear_bf16_gemm": Kernel("torch.matmul (cuBLAS)", "tilerl_b200/ops/gemm.py", note="plain library GEMM"),
})
register("fp8", "sm100", {
    "linear_fp8": Kernel("gemm_fp8_kernel", "csrc/gemm_fp8.cu", "trl_gemm_fp8",
                         note="tcgen05 kind::f8f6f4, 128x128 weight blocks, per-128-k promotion from TMEM"),
    "linear_fp8_gemv": Kernel("gemv_fp8_kernel", "csrc/gemm_fp8.cu", "trl_gemv_fp8"),
    "quant_fp8": Kernel("quant_act_fp8_kernel", "csrc/gemm_fp8.cu", "trl_quant_act_fp8",
                        note="RMSNorm / SwiGLU + e4m3 with one scale per token and 128 k"),
    "attn_prep": Kernel("attn_prep_fp8_kernel", "csrc/attn_fp8.cu", "trl_attn_prep_fp8", note="e4m3 KV pool"),
    "paged_attention_decode_fused": Kernel("attn_decode_mma_kernel<true>", "csrc/attn.cu", "trl_attn_decode_fused",
                                           note="decode ticks, optional: prep + split-KV attention + split merge in one launch"),
    "paged_attention_decode": Kernel("attn_split_fp8_kernel", "csrc/attn_fp8.cu", "trl_attn_paged_fp8"),
    "paged_attention_prefill": Kernel("attn_prefill_kernel<true>", "csrc/attn.cu", "trl_attn_prefill_fp8"),
})
register("any", "sm100", {
    "embed": Kernel("embedding_kernel", "csrc/misc.cu", "trl_embedding"),
    "gather_rows": Kernel("gather_rows_kernel", "csrc/misc.cu", "trl_gather_rows"),
    "rmsnorm": Kernel("rmsnorm_kernel", "csrc/misc.cu", "trl_rmsnorm"),
    "swiglu": Kernel("swiglu_kernel", "csrc/misc.cu", "trl_swiglu"),
    "add": Kernel("add_kernel", "csrc/misc.cu", "trl_add"),
    "attn_prep": Kernel("attn_prep_kernel", "csrc/attn.cu", "trl_attn_prep"),
    "paged_attention_decode": Kernel("attn_decode_mma_kernel + attn_combine_kernel", "csrc/attn.cu", "trl_attn_decode_mma",
                                     note="decode, verify width W, short chunks: kv-group x window rows as one mma tile"),
    "paged_attention_decode_scalar": Kernel("attn_split_kernel + attn_combine_kernel", "csrc/attn.cu", "trl_attn_paged",
                                            note="head dims other than 256; TRL_ATTN_MMA=0"),
    "paged_attention_prefill": Kernel("attn_prefill_kernel<false>", "csrc/attn.cu", "trl_attn_prefill"),
    "gdn": Kernel("gdn_prep_kernel + gdn_scan_kernel / gdn_scan_wy_kernel / gdn_recur_kernel", "csrc/gdn.cu", "trl_gdn"),
    "argmax": Kernel("argmax_stage1_kernel + argmax_stage2_kernel", "csrc/misc.cu", "trl_argmax"),
    "sample": Kernel("sample_softmax_kernel", "csrc/misc.cu", "trl_sample_softmax"),
    "sample_nucleus": Kernel("sample_nucleus_kernel", "csrc/misc.cu", "trl_sample_nucleus"),
    "page_bounds": Kernel("quest_score_kernel", "csrc/sparse.cu", "trl_quest_scores",
                          note="min / max of a K page per dimension in registers + Quest upper bound, one CTA per page"),
    "learned_index_scores": Kernel("page_mean_kernel + index_score_kernel", "csrc/sparse.cu", "trl_index_scores",
                                   note="page mean keys from the K pages, relu-dot scores; the projections are library GEMMs"),
    "select_pages": Kernel("topk_pages_kernel", "csrc/sparse.cu", "trl_topk_pages",
                           note="k-th largest by radix select, kept page indices ascending"),
    "spec_accept": Kernel("spec_accept_kernel", "csrc/misc.cu", "trl_spec_accept",
                          note="greedy accept length + GDN state-plane selection of a verify tick, inside its graph"),
    "lora": Kernel("lora_a_kernel + lora_b_kernel", "csrc/misc.cu", "trl_lora_add"),
    "adamw": Kernel("adamw_kernel", "csrc/misc.cu", "trl_adamw"),
    "decode_advance": Kernel("decode_advance_kernel", "csrc/misc.cu", "trl_decode_advance"),
    "zero_all_gather": Kernel("zero_allgather_kernel", "csrc/zero.cu", "trl_zero_allgather", "tilerl_b200.parallel.zero3"),
    "zero_reduce_scatter": Kernel("zero_reduce_scatter_kernel", "csrc/zero.cu", "trl_zero_reduce_scatter",
                                  "tilerl_b200.parallel.zero3"),
    "batch_fill": Kernel("trl_batch_fill", "csrc/runtime.cpp", "trl_batch_fill", note="host runtime"),
    "pager": Kernel("trl_pager_*", "csrc/runtime.cpp", "trl_pager_alloc", note="host runtime"),
})
