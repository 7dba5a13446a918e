"""Symmetric peer memory and the tensor-parallel kernels that use it.

``SymmComm.create(group, device)`` allocates one workspace per rank with ``cudaMalloc``
(inside the extension, so it can be exported with CUDA IPC), exchanges the IPC handles
over the process group (``all_gather_object``: bootstrap only) and opens every peer's
workspace.  After that no library collective is on the decode path:

* ``linear_allreduce_residual`` -- row-parallel projection + all-reduce + residual add.
  Up to 8 tokens: the GEMV pushes fp32 partial rows into every peer's slot from its
  epilogue (one-shot); the sum is completed by the NEXT projection's prologue
  (``consume_pending``: the streamed GEMV polls the slots, adds the residual and stores the
  row before it normalises it) or, where the next reader of the residual stream is another
  kind of kernel, by ``allreduce_finish`` (``settle``).  More tokens: the GEMM writes
  its partial into the symmetric ``big`` region and one two-shot kernel reduce-scatters
  by peer loads and all-gathers by peer stores straight into every rank's residual stream.
* ``argmax`` -- vocab-parallel argmax with a (max, index) exchange.
* ``all_gather_logits`` -- full-vocab logits for sampling (NCCL; off the greedy path).

The residual stream (workspace buffer ``x``) and the row-parallel GEMM output
(``rowout``) are views of the symmetric workspace so peers can address them.

Parity: the reference has only ``torch.distributed`` collectives
(``packages/tilerl-kernels/src/tilerl_kernels/backend.py:165-364``); this replaces
``Backend.all_reduce`` ``:260`` and the logits ``all_gather`` ``:272``.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import native as N

for _name, _sig in {
    "trl_symm_bytes": [N.I, N.I], "trl_symm_big_offset": [N.I], "trl_symm_out_offset": [N.I, N.I],
    "trl_symm_alloc": [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)], "trl_symm_free": [N.P],
    "trl_ipc_get": [N.P, N.P], "trl_ipc_open": [N.P, ctypes.POINTER(ctypes.c_void_p)], "trl_ipc_close": [N.P],
    "trl_allreduce_finish": [N.P, N.I, N.I, N.I, N.P, N.I, N.P, N.I, N.I, N.I, N.P],
    "trl_allreduce_twoshot": [N.P, N.I, N.I, N.I, N.I, N.P, N.I, N.I, N.I, N.I, N.P],
    "trl_argmax_tp": [N.P, N.I, N.I, N.I, N.P, N.P, N.I, N.I, N.P, N.I, N.P],
    "trl_gemv_nvfp4_push": [N.P, N.I, N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.I, N.I, N.P],
    "trl_gemv2_nvfp4_coop": [N.P, N.I, N.P, N.P, N.P, N.F, N.P, N.I, N.I, N.I, N.I, N.I, N.P, N.I, N.I, N.I, N.P],
}.items():
    N.register(_name, _sig)


class _DevMem:
    """Expose a raw device allocation to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class SymmComm:
    def __init__(self, rank: int, world: int, group, device, hmax: int, tmax: int):
        self.rank, self.world, self.group, self.device = rank, world, group, torch.device(device)
        self.hmax, self.tmax = hmax, tmax
        self.lib = N.lib()
        for fn in ("trl_symm_bytes", "trl_symm_big_offset", "trl_symm_out_offset"):
            getattr(self.lib, fn).restype = ctypes.c_size_t
        self.nbytes = self.lib.trl_symm_bytes(hmax, tmax)
        p = ctypes.c_void_p()
        N.check(self.lib.trl_symm_alloc(self.nbytes, ctypes.byref(p)), "symm_alloc")
        self.local_ptr = p.value
        handle = (ctypes.c_ubyte * 64)()
        N.check(self.lib.trl_ipc_get(self.local_ptr, handle), "ipc_get")
        handles: List[Optional[bytes]] = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.ptrs: List[int] = []
        for r, h in enumerate(handles):
            if r == rank:
                self.ptrs.append(self.local_ptr)
                continue
            q = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            N.check(self.lib.trl_ipc_open(buf, ctypes.byref(q)), "ipc_open")
            self.ptrs.append(q.value)
        self.table = (ctypes.c_void_p * 8)(*(self.ptrs + [None] * (8 - world)))
        self.mem = torch.as_tensor(_DevMem(self.local_ptr, self.nbytes), device=self.device)
        big0 = self.lib.trl_symm_big_offset(hmax)
        out0 = self.lib.trl_symm_out_offset(hmax, tmax)
        self.big = self.mem[big0:big0 + tmax * hmax * 2].view(torch.bfloat16)
        self.xres = self.mem[out0:out0 + tmax * hmax * 2].view(torch.bfloat16)
        # a one-shot all-reduce whose partial rows are pushed but not yet summed into the residual
        # stream: (rows, columns, residual tensor)
        self.pending = None
        self.fuse_finish = __import__("os").environ.get("TRL_FUSE_FINISH", "1") != "0"
        self.stream_push = __import__("os").environ.get("TRL_GEMV_STREAM_PUSH", "1") != "0"
        dist.barrier(group=group)

    @classmethod
    def create(cls, group, device, hmax: int = 8192, tmax: int = 8192) -> "SymmComm":
        return cls(dist.get_rank(group), dist.get_world_size(group), group, device, hmax, tmax)

    # ---- workspace views handed to CudaOps ----------------------------------------------------
    def attach(self, ops) -> None:
        """Place the residual stream and the row-parallel GEMM output in symmetric memory."""
        self.ops = ops
        ops.ws.bufs["x"] = self.xres
        ops.ws.bufs["rowout"] = self.big

    # ---- fused ops ------------------------------------------------------------------------------
    def linear_allreduce_residual(self, ops, a, w, residual, lora=None):
        from ..formats import NVFP4Tensor
        t, k = a.shape
        n = w.shape[0]
        st = N.stream()
        self.settle()
        if t <= min(8, getattr(ops, "gemv_tokens", 8)) and isinstance(w, NVFP4Tensor) and lora is None:
            if t <= 2 and getattr(ops, "gemv_stream", False) and self.stream_push and ops._stream_ok(w) and t * k * 2 <= 88 * 1024 and k <= 18432:
                from ..ops.gemm_tc import w_stream
                if getattr(ops, "chain", False) and n <= self.hmax:
                    from ..ops.cuda import EPI_PUSH
                    ops._enqueue(t, a, w_stream(w), w.tscale, None, 0.0, None, None, n, k, EPI_PUSH)
                    self.pending = (t, n, residual)
                    if not self.fuse_finish:
                        self.settle()
                    return residual
                N.check(self.lib.trl_gemv2_nvfp4_push(a.data_ptr(), a.stride(0), w_stream(w).data_ptr(),
                                                      w.tscale.data_ptr(), self.table, self.rank, self.world,
                                                      self.hmax, t, n, k, st), "gemv2_push")
            else:
                N.check(self.lib.trl_gemv_nvfp4_push(a.data_ptr(), a.stride(0), w.wq.data_ptr(), w.scale.data_ptr(),
                                                     w.tscale.data_ptr(), self.table, self.rank, self.world, self.hmax,
                                                     t, n, k, st), "gemv_push")
            self.pending = (t, n, residual)
            N.count((t + 3) // 4)
            if not self.fuse_finish:
                self.settle()
            return residual
        # large-M: local partial into the symmetric region, then one two-shot kernel
        assert residual.data_ptr() == self.xres.data_ptr(), "residual stream must live in symmetric memory"
        assert t <= self.tmax and n <= self.hmax
        part = self.big[: t * n].view(t, n)
        ops._linear(a, w, part)
        if lora is not None:
            ops._lora_add(part, a, lora)
        N.check(self.lib.trl_allreduce_twoshot(self.table, self.rank, self.world, self.hmax, self.tmax,
                                               residual.data_ptr(), residual.stride(0), residual.stride(0), t, n, st),
                "allreduce_twoshot")
        N.count()
        return residual

    def pending_is(self, x) -> bool:
        """True when ``x`` is exactly the residual rows whose all-reduce is pending."""
        if self.pending is None:
            return False
        t, n, residual = self.pending
        return (x.data_ptr() == residual.data_ptr() and x.shape[0] == t and x.shape[1] == n and n <= self.hmax
                and x.stride(0) == residual.stride(0))

    def settle(self) -> None:
        """Complete a pending one-shot all-reduce with the stand-alone finishing kernel."""
        if self.pending is None:
            return
        if getattr(self, "ops", None) is not None:
            self.ops.flush()          # the pushing projection may still sit in the launch queue
        t, n, residual = self.pending
        self.pending = None
        N.check(self.lib.trl_allreduce_finish(self.table, self.rank, self.world, self.hmax, residual.data_ptr(),
                                              residual.stride(0), residual.data_ptr(), residual.stride(0),
                                              t, n, N.stream()), "allreduce_finish")
        N.count()

    def consume_pending(self, x, wst, tscale, norm_w, eps, y, n_out: int, epi: int) -> bool:
        """Run ``y = epi(norm(x) @ W^T)`` with the pending all-reduce into ``x`` completed by the same
        kernel.  False (nothing launched) when ``x`` is not the pending residual rows."""
        if self.pending is None:
            return False
        t, n, residual = self.pending
        if (x.data_ptr() != residual.data_ptr() or x.shape[0] != t or x.shape[1] != n or n > self.hmax
                or x.stride(0) != residual.stride(0)):
            return False
        rc = self.lib.trl_gemv2_nvfp4_coop(x.data_ptr(), x.stride(0), wst.data_ptr(), tscale.data_ptr(),
                                           norm_w.data_ptr(), eps, y.data_ptr(), y.stride(0), t, n_out, n, epi,
                                           self.table, self.rank, self.world, self.hmax, N.stream())
        if rc != 0:
            return False      # shape outside the fused kernel's limits: the caller settles and falls back
        self.pending = None
        N.count()
        return True

    def argmax(self, ops, logits, v_valid: int):
        """Global argmax over vocab-parallel fp32 logits ``[M, V_local]``."""
        m, v_local = logits.shape
        out = ops.ws.get("argmax", (m,), torch.int32)
        scratch = ops.ws.get("argmax_scratch", (m * 128,), torch.float32)
        pv = scratch
        pi = scratch[m * 64:]
        N.check(ops.lib.trl_argmax_stage1(logits.data_ptr(), logits.stride(0), m, max(0, min(v_local, v_valid)),
                                          pv.data_ptr(), pi.data_ptr(), N.stream()), "argmax_stage1")
        N.check(self.lib.trl_argmax_tp(self.table, self.rank, self.world, self.hmax, pv.data_ptr(), pi.data_ptr(),
                                       64, v_local, out.data_ptr(), m, N.stream()), "argmax_tp")
        N.count(2)
        return out

    def all_gather_logits(self, logits: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(logits) for _ in range(self.world)]
        dist.all_gather(parts, logits.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    def close(self) -> None:
        for r, p in enumerate(self.ptrs):
            if r != self.rank and p:
                self.lib.trl_ipc_close(p)
        self.lib.trl_symm_free(self.local_ptr)


class NcclComm:
    """The unfused control: the same tensor-parallel op surface as :class:`SymmComm`, but every
    collective is a library call -- ``dist.all_reduce`` after each row-parallel projection, an
    all-gather of the vocabulary shards for the argmax -- on top of this repository's own
    single-GPU kernels.  It is what the fused peer-memory kernels are measured against on the same
    box (``bench.py --impl unfused``); NCCL calls are not captured by the decode graph here, so
    its ticks run eagerly, as the reference's TP ticks do
    (``src/tilerl/tensor_parallel.py:20-24``; collectives ``tilerl_kernels/backend.py:260-281``)."""
    graph_capturable = False

    def __init__(self, group, device):
        self.group, self.device = group, torch.device(device)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.pending = None

    def attach(self, ops) -> None:
        pass

    def settle(self) -> None:
        pass

    def consume_pending(self, *a, **k) -> bool:
        return False

    def pending_is(self, x) -> bool:
        return False

    def linear_allreduce_residual(self, ops, a, w, residual, lora=None):
        t, n = a.shape[0], w.shape[0]
        part = ops.ws.get("nccl_part", (t, n), torch.bfloat16)
        ops._linear(a, w, part)
        if lora is not None:
            ops._lora_add(part, a, lora)
        ops.flush()
        dist.all_reduce(part, group=self.group)
        residual.add_(part)
        N.count(2)
        return residual

    def all_gather_logits(self, logits: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(logits) for _ in range(self.world)]
        dist.all_gather(parts, logits.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    def argmax(self, ops, logits, v_valid: int):
        full = self.all_gather_logits(logits)
        if ops.vocab:
            full = full[..., :ops.vocab]
        out = ops.ws.get("argmax", (logits.shape[0],), torch.int32)
        out.copy_(full.argmax(-1).to(torch.int32))
        return out

    def close(self) -> None:
        pass
