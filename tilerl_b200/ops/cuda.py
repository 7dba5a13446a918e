"""B200 implementation of the model's op surface on the hand-written kernels.

Shapes decide the kernel, not flags: up to ``GEMV_MAX_M`` tokens a projection
is a weight-streaming NVFP4 GEMV with RMSNorm folded into its prologue and the
residual add / SwiGLU folded into its epilogue; above that it is the tcgen05
block-scaled GEMM (:mod:`tilerl_b200.ops.gemm`).  All intermediate buffers live
in a workspace allocated once per ``max_tokens`` so every launch of a decode tick
sees fixed addresses and the tick can be captured in a CUDA graph.

With a tensor-parallel group the row-parallel projections end in the fused
one-shot all-reduce of :mod:`tilerl_b200.parallel.symm` instead of a separate
collective.

Parity: the ``Backend`` op surface of reference
``packages/tilerl-kernels/src/tilerl_kernels/backend.py:559-1797`` (dispatch by
launch M ``:733-905``).
"""
from __future__ import annotations

import math
import ctypes
import os
from typing import Dict, Optional

import torch

from ..formats import FP8BlockTensor, NVFP4Tensor
from . import native as N

EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU, EPI_STORE_F32 = 0, 1, 2, 3
EPI_PUSH = 4            # tensor-parallel row-parallel projection: partial rows pushed to every rank
CHAIN_MAX = 4


class ChainOp(ctypes.Structure):
    """One projection of a chained launch (``TrlChainOp`` of ``csrc/gemv2.cu``)."""
    _fields_ = [("x", ctypes.c_void_p), ("wst", ctypes.c_void_p), ("tscale", ctypes.c_void_p),
                ("norm_w", ctypes.c_void_p), ("residual", ctypes.c_void_p), ("out", ctypes.c_void_p),
                ("ldx", ctypes.c_int), ("ldr", ctypes.c_int), ("ldy", ctypes.c_int), ("N", ctypes.c_int),
                ("K", ctypes.c_int), ("epi", ctypes.c_int), ("coop", ctypes.c_int), ("eps", ctypes.c_float)]
GEMV_MAX_M = 8
MMA_MAX_M = 16     # rows served by the mma.sync NVFP4 kernel (csrc/gemv_mma.cu)


class Workspace:
    """Named, lazily created device buffers.  A buffer that has to grow is replaced, but the old
    allocation is kept alive: CUDA graphs captured earlier hold its address (a decode graph
    captured at start-up must survive the first long prefill growing the shared buffers)."""

    def __init__(self, device):
        self.device = device
        self.bufs: Dict[str, torch.Tensor] = {}
        self.retired: list = []

    def get(self, name: str, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        t = self.bufs.get(name)
        if t is None or t.numel() < n or t.dtype != dtype:
            if t is not None and torch.cuda.is_current_stream_capturing():
                raise RuntimeError(f"workspace buffer {name!r} would be reallocated during graph capture")
            if t is not None:
                self.retired.append(t)
            t = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self.bufs[name] = t
        return t[:n].view(*shape)


class CudaOps:
    name = "cuda"

    def __init__(self, device="cuda", tp=None, comm=None, attn_splits: int = 0, use_tc_gemm: bool = True,
                 decode_tc: Optional[bool] = None, terms_small: int = 4, terms_large: int = 2):
        if not torch.cuda.is_available():
            raise RuntimeError("CudaOps needs a CUDA device")
        self.lib = N.lib()
        self.device = torch.device(device)
        self.ws = Workspace(self.device)
        self.tp = tp
        self.comm = comm          # parallel.symm.SymmComm or None
        self.attn_splits = attn_splits
        self.use_tc_gemm = use_tc_gemm and os.environ.get("TRL_GEMM", "tc") == "tc"
        # small-M projections: the SIMT weight-streaming GEMV (default; measured faster at
        # B=1) or the tcgen05 GEMM with `terms_small` residual terms (TRL_DECODE=tc)
        self.decode_tc = (os.environ.get("TRL_DECODE", "simt") == "tc") if decode_tc is None else decode_tc
        self.gemv_tokens = int(os.environ.get("TRL_GEMV_TOKENS", 2))
        # rows <= 2: the ring-streamed GEMV on the weight's stream-layout copy (TRL_GEMV_STREAM=0: the
        # register-streamed kernels on the checkpoint layout)
        self.gemv_stream = os.environ.get("TRL_GEMV_STREAM", "1") != "0"
        self.prefill_attn = os.environ.get("TRL_PREFILL_ATTN", "1") != "0"   # tiled kernel for q_len >= 16
        self.gdn_fused_decode = os.environ.get("TRL_GDN_FUSED", "1") != "0"    # decode ticks: prep inside the scan kernel
        from .. import tape as _tape
        _tape.set_dequant(self.dequantize_nvfp4)   # frozen-base linears of the training forward
        self.terms_small = int(os.environ.get("TRL_TERMS_SMALL", terms_small))
        self.terms_large = int(os.environ.get("TRL_TERMS_LARGE", terms_large))
        self.act_dtype = torch.bfloat16
        self.attn_mma = os.environ.get("TRL_ATTN_MMA", "1") != "0" and hasattr(self.lib, "trl_attn_decode_mma")
        # TRL_GEMV_MMA=1: 3..16 rows against NVFP4 weights go to the mma.sync kernel with f16 activations
        # (csrc/gemv_mma.cu) instead of the activation quantiser + tcgen05 GEMM.  Off by default: launch for
        # launch it ties with that pair on the 27B shapes (gate_up at 8 rows 34.1 us against 34.6), but inside
        # a B = 8 decode tick it loses, 14.5 ms against 10.65: decoding e2m1 on the CUDA cores costs 23.5
        # instructions per MMA (issue slots 45 % busy, no pipe saturated), and its staging of the activation rows
        # sits behind the dependency of every launch where the GEMM's prologue does not.
        self.gemv_mma = os.environ.get("TRL_GEMV_MMA", "0") == "1" and hasattr(self.lib, "trl_gemv_nvfp4_mma")
        # TRL_ATTN_FUSED=1: decode ticks run prep, split-KV attention and the merge of the splits as ONE launch
        # (325 instead of 357 launches per 27B tick).  Off by default: measured 4.47 ms per tick against 4.32 ms
        # for the three launches -- every CTA repeats the query prep behind the dependency and the last CTA's
        # merge is serial, where the three small kernels overlap their neighbours' tails.
        self.attn_fused = os.environ.get("TRL_ATTN_FUSED", "0") == "1" and hasattr(self.lib, "trl_attn_decode_fused")
        self._attn_counters = None
        self.mma_tokens = int(os.environ.get("TRL_GEMV_MMA_TOKENS", "8"))      # rows it serves (the kernel takes up to 16)
        self.mma_kmax = int(os.environ.get("TRL_GEMV_MMA_KMAX", "8192"))      # longer rows go to the tcgen05 GEMM
        # TRL_GEMV_CHAIN=1: consecutive 1-2 row projections are queued and go out as one chained launch
        # (grid barriers between them, weight rings refilled across the barriers); anything else
        # flushes the queue.  Off by default: measured on the 27B tick a grid barrier costs more than the
        # kernel boundary it replaces (the CTAs of one projection finish 6-9 us apart and the barrier
        # waits for the last, where separate launches let the next kernel's CTAs move in as slots free up):
        # 5.54 ms per tick chained, 4.37 ms as separate launches.
        self.chain = os.environ.get("TRL_GEMV_CHAIN", "0") == "1" and hasattr(self.lib, "trl_gemv2_chain")
        self._queue = []          # [(ChainOp fields, rows, tensors kept alive)]
        self._chain_bar = torch.zeros(64, dtype=torch.int32, device=self.device)
        self.chain_kmax = int(os.environ.get("TRL_GEMV_CHAIN_KMAX", "65536"))   # longer rows are launched alone
        self.sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.vocab = None   # set by the engine builder: real vocabulary size (TP pads it)
        if comm is not None:
            comm.attach(self)

    # ---- helpers ------------------------------------------------------------------
    def _f32(self, t: torch.Tensor) -> torch.Tensor:
        assert t.dtype == torch.float32 and t.is_cuda, "norm/vector parameters must be fp32 on device"
        return t

    def settle(self) -> None:
        """Make every buffer current: launch the queued projections and complete an all-reduce
        that a row-parallel projection left pending for its consumer (tensor parallelism only)."""
        self.flush()
        if self.comm is not None and getattr(self.comm, "pending", None) is not None:
            self.comm.settle()

    # ---- chained projections ------------------------------------------------------------
    def _enqueue(self, m, x, wst, tscale, norm_w, eps, residual, out, n, k, epi, coop=0) -> None:
        if self._queue and (self._queue[0][1] != m or k > self.chain_kmax or self._queue[-1][0]["K"] > self.chain_kmax):
            self.flush()
        f = dict(x=x.data_ptr(), wst=wst.data_ptr(), tscale=tscale.data_ptr(), norm_w=N.ptr(norm_w),
                 residual=N.ptr(residual), out=N.ptr(out), ldx=x.stride(0),
                 ldr=residual.stride(0) if residual is not None else 0, ldy=out.stride(0) if out is not None else 0,
                 N=n, K=k, epi=epi, coop=coop, eps=float(eps))
        self._queue.append((f, m, (x, wst, tscale, norm_w, residual, out)))
        if len(self._queue) == CHAIN_MAX:
            self.flush()

    def gemv_now(self, x, w, y, **kw) -> None:
        """``_gemv`` launched at once (tests, probes): the queued form leaves ``y`` unwritten until
        ``flush`` / ``settle`` or the next op that is not a 1-2 row projection."""
        self._gemv(x, w, y, **kw)
        self.flush()

    def flush(self) -> None:
        """Launch what ``_enqueue`` collected: one chained launch, or the single-projection kernels
        when the chain is one op long or the chained launch is refused (grid not co-resident)."""
        q = self._queue
        if not q:
            return
        self._queue = []
        comm = self.comm if (self.comm is not None and hasattr(self.comm, "table")) else None
        if len(q) > 1:
            arr = (ChainOp * len(q))(*[ChainOp(**f) for f, _, _ in q])
            rc = self.lib.trl_gemv2_chain(arr, len(q), q[0][1], self._chain_bar.data_ptr(),
                                          comm.table if comm else None, comm.rank if comm else 0,
                                          comm.world if comm else 0, comm.hmax if comm else 0, N.stream())
            if rc == 0:
                N.count()
                return
        for f, m, _ in q:
            self._launch_single(f, m, comm)

    def _launch_single(self, f, m, comm) -> None:
        st = N.stream()
        if f["epi"] == EPI_PUSH:
            N.check(self.lib.trl_gemv2_nvfp4_push(f["x"], f["ldx"], f["wst"], f["tscale"], comm.table, comm.rank,
                                                  comm.world, comm.hmax, m, f["N"], f["K"], st), "gemv2_push")
        elif f["coop"]:
            rc = self.lib.trl_gemv2_nvfp4_coop(f["x"], f["ldx"], f["wst"], f["tscale"], f["norm_w"], f["eps"],
                                               f["out"], f["ldy"], m, f["N"], f["K"], f["epi"], comm.table,
                                               comm.rank, comm.world, comm.hmax, st)
            if rc != 0:     # outside the cooperative kernel's limits: finishing kernel, then the plain projection
                N.check(self.lib.trl_allreduce_finish(comm.table, comm.rank, comm.world, comm.hmax, f["x"], f["ldx"],
                                                      f["x"], f["ldx"], m, f["K"], st), "allreduce_finish")
                N.check(self.lib.trl_gemv2_nvfp4(f["x"], f["ldx"], f["wst"], f["tscale"], f["norm_w"], f["eps"],
                                                 None, 0, f["out"], f["ldy"], m, f["N"], f["K"], f["epi"], st),
                        "gemv2_nvfp4")
                N.count()
        else:
            N.check(self.lib.trl_gemv2_nvfp4(f["x"], f["ldx"], f["wst"], f["tscale"], f["norm_w"], f["eps"],
                                             f["residual"], f["ldr"], f["out"], f["ldy"], m, f["N"], f["K"],
                                             f["epi"], st), "gemv2_nvfp4")
        N.count()

    def _gemv(self, x, w, y, *, norm_w=None, eps=0.0, residual=None, epi=EPI_STORE):
        m, k = x.shape
        stream = isinstance(w, NVFP4Tensor) and m <= 2 and self.gemv_stream and self._stream_ok(w) \
            and (m * k * 2 <= 88 * 1024) and k <= 18432
        if self.comm is not None and getattr(self.comm, "pending", None) is not None:
            if stream and norm_w is not None and residual is None and epi in (EPI_STORE, EPI_SWIGLU):
                from .gemm_tc import w_stream
                if self.chain and self.comm.pending_is(x):
                    # the consumer completes the all-reduce itself, inside the chained launch
                    self.comm.pending = None
                    self._enqueue(m, x, w_stream(w), w.tscale, norm_w, eps, None, y, w.wq.shape[0], k, epi, coop=1)
                    return
                if not self.chain and self.comm.consume_pending(x, w_stream(w), w.tscale, norm_w, eps, y, w.wq.shape[0], epi):
                    return
            self.settle()
        if stream:
            from .gemm_tc import w_stream
            n = w.wq.shape[0]
            if self.chain:
                self._enqueue(m, x, w_stream(w), w.tscale, norm_w, eps, residual, y, n, k, epi)
                return
            N.check(self.lib.trl_gemv2_nvfp4(
                x.data_ptr(), x.stride(0), w_stream(w).data_ptr(), w.tscale.data_ptr(),
                N.ptr(norm_w), eps, N.ptr(residual), residual.stride(0) if residual is not None else 0,
                y.data_ptr(), y.stride(0), m, n, k, epi, N.stream()), "gemv2_nvfp4")
            N.count()
            return
        self.flush()
        if isinstance(w, NVFP4Tensor):
            n = w.wq.shape[0]
            N.check(self.lib.trl_gemv_nvfp4(
                x.data_ptr(), x.stride(0), w.wq.data_ptr(), w.scale.data_ptr(), w.tscale.data_ptr(),
                N.ptr(norm_w), eps, N.ptr(residual), residual.stride(0) if residual is not None else 0,
                y.data_ptr(), y.stride(0), m, n, k, epi, N.stream()), "gemv_nvfp4")
            N.count((m + 3) // 4)
        elif isinstance(w, torch.Tensor) and w.dtype == torch.bfloat16:
            n = w.shape[0]
            assert epi != EPI_SWIGLU
            N.check(self.lib.trl_gemv_bf16(
                x.data_ptr(), x.stride(0), w.data_ptr(), N.ptr(norm_w), eps, N.ptr(residual),
                residual.stride(0) if residual is not None else 0, y.data_ptr(), y.stride(0),
                m, n, k, epi, N.stream()), "gemv_bf16")
            # 3..16 rows whose activations fit shared memory: one tensor-core pass over the weights
            one_pass = 2 < m <= 16 and k % 32 == 0 and (8 if m <= 8 else 16) * (k + 32) * 2 <= 200 * 1024
            N.count(1 if one_pass else (m + 3) // 4)
        elif isinstance(w, FP8BlockTensor):
            from . import gemm_fp8
            gemm_fp8.gemv(self, x, w, y, norm_w=norm_w, eps=eps, residual=residual, epi=epi)
        else:
            raise TypeError(f"no GEMV for weight type {type(w)}")

    @staticmethod
    def _stream_ok(w) -> bool:
        n, k = w.shape
        return n % 2 == 0 and k % 128 == 0

    def _tc(self, w, t: int) -> bool:
        # measured on the 27B shapes (gate_up): 1 token GEMV 27.5 us; 2 tokens GEMV 35.6 / tensor-core
        # GEMM incl. its activation quantiser 36.0; 4 tokens 58.5 / 36.1; 8 tokens 115 / 40.5.  So
        # the GEMV serves up to `gemv_tokens` = 2 rows and the tensor-core kernel everything above
        # (batched decode, verify ticks).  The two kernels round activations differently; set
        # `gemv_tokens = 8` where batch-size-independent bits matter more than speed.
        return isinstance(w, NVFP4Tensor) and self.use_tc_gemm and (t > self.gemv_tokens or self.decode_tc)

    def _linear(self, x, w, y, *, norm_w=None, eps=0.0, residual=None, epi=EPI_STORE):
        """``y = epi(norm(x) @ W^T)`` with everything fused into one or two kernels."""
        t = x.shape[0]
        if not (t <= GEMV_MAX_M and not self._tc(w, t)):
            self.settle()     # only the GEMV path can finish a pending all-reduce itself
        if isinstance(w, FP8BlockTensor) and w.shape[1] % 128 == 0:
            from . import gemm_fp8
            self.settle()
            gemm_fp8.linear(self, x, w, y, norm_w=norm_w, eps=eps, residual=residual, epi=epi)
            return
        if (self._tc(w, t) and self.gemv_mma and t <= self.mma_tokens and x.shape[1] <= self.mma_kmax
                and not self.decode_tc and x.stride(0) % 8 == 0):
            # 3..16 rows (batched decode, verify windows): f16 activations against the NVFP4 weights on
            # mma.sync, weights streamed once, no activation quantiser; shapes it does not take
            # (cudaErrorNotSupported) go on to the quantiser + tcgen05 GEMM below
            rc = self.lib.trl_gemv_nvfp4_mma(
                x.data_ptr(), x.stride(0), w.wq.data_ptr(), w.scale.data_ptr(), w.tscale.data_ptr(),
                N.ptr(norm_w), eps, N.ptr(residual), residual.stride(0) if residual is not None else 0,
                y.data_ptr(), y.stride(0), t, w.wq.shape[0], x.shape[1], epi, N.stream())
            if rc == 0:
                N.count()
                return
            if rc != 801:
                N.check(rc, "gemv_nvfp4_mma")
        if self._tc(w, t):
            from .gemm_tc import gemm_nvfp4
            terms = self.terms_small if t <= GEMV_MAX_M else self.terms_large
            gemm_nvfp4(self, x, w, y, terms=terms, norm_w=norm_w, eps=eps, residual=residual, epi=epi)
            return
        if t <= GEMV_MAX_M:
            self._gemv(x, w, y, norm_w=norm_w, eps=eps, residual=residual, epi=epi)
            return
        # unfused large-M path (non-NVFP4 weights, or TRL_GEMM=dequant for bisecting numerics)
        from . import gemm
        h = self._rmsnorm(x, norm_w, eps) if norm_w is not None else x
        n = w.shape[0]
        tmp = self.ws.get("gemm_tmp", (t, n), torch.bfloat16)
        gemm.linear(self, h, w, tmp)
        if epi == EPI_SWIGLU:
            N.check(self.lib.trl_swiglu(tmp.data_ptr(), y.data_ptr(), y.numel(), N.stream()), "swiglu")
        elif epi == EPI_RESIDUAL:
            N.check(self.lib.trl_add(tmp.data_ptr(), residual.data_ptr(), y.data_ptr(), tmp.numel(), N.stream()), "add")
        else:
            y.copy_(tmp)
        N.count()

    def _rmsnorm(self, x, w, eps, name="h"):
        self.settle()
        t, h = x.shape
        out = self.ws.get(name, (t, h), torch.bfloat16)
        N.check(self.lib.trl_rmsnorm(x.data_ptr(), w.data_ptr(), out.data_ptr(), t, h, eps, N.stream()), "rmsnorm")
        N.count()
        return out

    def _lora_add(self, y, x, lora, norm_w=None, eps=0.0):
        """``y += s * (norm(x) A^T) B^T`` in place (two small kernels; the norm is recomputed
        inside the first, so no normalised copy of x is materialised)."""
        if lora is not None:
            self.settle()
            a, b, s = lora
            t, k = x.shape
            n, r = b.shape
            if a.dtype == torch.float32 and b.dtype == torch.float32 and r <= 64 and k % 2 == 0 \
                    and a.is_contiguous() and b.is_contiguous():
                tmp = self.ws.get("lora_t", (t, r), torch.float32)
                N.check(self.lib.trl_lora_add(x.data_ptr(), x.stride(0), N.ptr(self._f32(norm_w) if norm_w is not None else None),
                                              eps, a.data_ptr(), b.data_ptr(), tmp.data_ptr(), y.data_ptr(), y.stride(0),
                                              t, n, k, r, float(s), N.stream()), "lora_add")
                N.count(2)
            else:
                xn = self._rmsnorm(x, norm_w, eps) if norm_w is not None else x
                y.add_(((xn.float() @ a.float().t()) @ b.float().t() * s).to(y.dtype))
        return y

    # ---- op surface --------------------------------------------------------------------
    def embed(self, table, ids):
        self.settle()
        t, h = ids.shape[0], table.shape[1]
        x = self.ws.get("x", (t, h), torch.bfloat16)
        N.check(self.lib.trl_embedding(table.data_ptr(), ids.data_ptr(), x.data_ptr(), t, h, table.shape[0],
                                       N.stream()), "embedding")
        N.count()
        return x

    def norm_linear(self, x, norm_w, w, eps, lora=None):
        t, n = x.shape[0], w.shape[0]
        y = self.ws.get("proj", (t, n), torch.bfloat16)
        self._linear(x, w, y, norm_w=self._f32(norm_w), eps=eps)
        if lora is not None:
            self._lora_add(y, x, lora, norm_w, eps)
        return y

    def norm_linear_swiglu(self, x, norm_w, w, eps, lora=None):
        t, n = x.shape[0], w.shape[0]
        act = self.ws.get("act", (t, n // 2), torch.bfloat16)
        if lora is None:
            self._linear(x, w, act, norm_w=self._f32(norm_w), eps=eps, epi=EPI_SWIGLU)
            return act
        gu = self.ws.get("proj", (t, n), torch.bfloat16)
        self._linear(x, w, gu, norm_w=self._f32(norm_w), eps=eps)
        self._lora_add(gu, x, lora, norm_w, eps)
        N.check(self.lib.trl_swiglu(gu.data_ptr(), act.data_ptr(), act.numel(), N.stream()), "swiglu")
        N.count()
        return act

    def linear_residual(self, a, w, residual, lora=None):
        """``residual += a @ W^T`` (in place on the residual stream).  Under TP the
        partial products are summed across ranks inside the fused kernel."""
        if self.comm is not None and self.comm.world > 1:
            return self.comm.linear_allreduce_residual(self, a, w, residual, lora)
        self._linear(a, w, residual, residual=residual, epi=EPI_RESIDUAL)
        if lora is not None:
            self._lora_add(residual, a, lora)
        return residual

    def attention(self, qkv, lp, batch, pool, attn_idx, cfg, n_q, n_kv):
        self.flush()
        t = qkv.shape[0]
        d = cfg.head_dim
        q = self.ws.get("q", (t, n_q, d), torch.bfloat16)
        out = self.ws.get("act", (t, n_q * d), torch.bfloat16)
        kc, vc = pool.layer(attn_idx)
        st = N.stream()
        if getattr(pool, "fp8", False):
            return self._attention_fp8(qkv, lp, batch, pool, attn_idx, cfg, n_q, n_kv, q, out, kc, vc, st)
        sp = batch.sparse
        if (self.attn_fused and self.attn_mma and batch.max_q_len == 1 and t == batch.n_seqs and d == 256
                and cfg.rotary_dim == 64 and n_q % n_kv == 0 and n_q // n_kv <= 16 and qkv.stride(0) % 8 == 0
                and not (sp is not None and sp.active(attn_idx))):
            # decode tick: prep, split-KV attention and the merge of the splits in one launch
            splits = min(64, self.attn_splits or self._pick_splits(batch, t, n_kv, 64))
            po = self.ws.get("attn_po", (t * n_q * splits * d,), torch.float32)
            pm = self.ws.get("attn_pm", (t * n_q * splits,), torch.float32)
            pl = self.ws.get("attn_pl", (t * n_q * splits,), torch.float32)
            if self._attn_counters is None or self._attn_counters.numel() < t * n_kv:
                self._attn_counters = torch.zeros(max(4096, t * n_kv), dtype=torch.int32, device=self.device)
            N.check(self.lib.trl_attn_decode_fused(
                qkv.data_ptr(), qkv.stride(0), self._f32(lp["q_norm"]).data_ptr(), self._f32(lp["k_norm"]).data_ptr(),
                batch.positions.data_ptr(), batch.slot_mapping.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                batch.block_table.data_ptr(), batch.block_table.stride(0), kc.shape[0], batch.seq_ids.data_ptr(),
                po.data_ptr(), pm.data_ptr(), pl.data_ptr(), self._attn_counters.data_ptr(), out.data_ptr(),
                t, n_q, n_kv, d, cfg.rotary_dim, float(cfg.rope_theta), cfg.rms_eps, splits, 1.0 / math.sqrt(d),
                int(cfg.attn_gated), st), "attn_decode_fused")
            N.count()
            return out
        N.check(self.lib.trl_attn_prep(
            qkv.data_ptr(), qkv.stride(0), self._f32(lp["q_norm"]).data_ptr(),
            self._f32(lp["k_norm"]).data_ptr(), batch.positions.data_ptr(),
            batch.slot_mapping.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), t, n_q, n_kv, d,
            cfg.rotary_dim, float(cfg.rope_theta), cfg.rms_eps, int(cfg.attn_gated), kc.shape[0], st), "attn_prep")
        table, pos = batch.block_table, batch.positions
        sp = batch.sparse
        sparse_now = sp is not None and sp.active(attn_idx)
        if (not sparse_now and self.prefill_attn and batch.max_q_len >= 16 and d == 256 and n_q % n_kv == 0
                and n_q // n_kv <= 8 and not getattr(batch, "keep_steps", 0)):
            # prefill chunks (and whatever decode rows ride along): K / V tiles are read once per
            # 16 query tokens by the tiled tensor-core kernel
            N.check(self.lib.trl_attn_prefill(
                q.data_ptr(), qkv.data_ptr(), qkv.stride(0), kc.data_ptr(), vc.data_ptr(), table.data_ptr(),
                table.stride(0), kc.shape[0], batch.q_start.data_ptr(), batch.q_len.data_ptr(), pos.data_ptr(),
                out.data_ptr(), batch.n_seqs, batch.max_q_len, n_q, n_kv, d, 1.0 / math.sqrt(d), int(cfg.attn_gated),
                st), "attn_prefill")
            N.count(2)
            return out
        if sparse_now:
            table, pos = sp.packed(attn_idx, q, kc, ops=self)    # same kernel on [selected pages ; trailing window]
        mma = self.attn_mma and d == 256 and n_q % n_kv == 0 and n_q // n_kv <= 16
        tpg = self._tokens_per_group(batch, t, n_q // n_kv) if mma else 1
        splits = self.attn_splits or self._pick_splits(batch, t // tpg if mma else t, n_kv, 64 if mma else 32)
        po = self.ws.get("attn_po", (t * n_q * splits * d,), torch.float32)
        pm = self.ws.get("attn_pm", (t * n_q * splits,), torch.float32)
        pl = self.ws.get("attn_pl", (t * n_q * splits,), torch.float32)
        if mma:
            # decode / verify rows: the heads of a kv group (times the rows of a verify window) are one
            # tensor-core tile, K / V rows are read once per group
            N.check(self.lib.trl_attn_decode_mma(
                q.data_ptr(), qkv.data_ptr(), qkv.stride(0), kc.data_ptr(), vc.data_ptr(),
                table.data_ptr(), table.stride(0), kc.shape[0], batch.seq_ids.data_ptr(),
                pos.data_ptr(), po.data_ptr(), pm.data_ptr(), pl.data_ptr(), out.data_ptr(),
                t, n_q, n_kv, d, splits, tpg, 1.0 / math.sqrt(d), int(cfg.attn_gated), st), "attn_decode_mma")
        else:
            N.check(self.lib.trl_attn_paged(
                q.data_ptr(), qkv.data_ptr(), qkv.stride(0), kc.data_ptr(), vc.data_ptr(),
                table.data_ptr(), table.stride(0), batch.seq_ids.data_ptr(),
                pos.data_ptr(), po.data_ptr(), pm.data_ptr(), pl.data_ptr(), out.data_ptr(),
                t, n_q, n_kv, d, splits, 1.0 / math.sqrt(d), int(cfg.attn_gated), st), "attn_paged")
        N.count(2 + (1 if splits > 1 else 0))
        return out

    def _attention_fp8(self, qkv, lp, batch, pool, attn_idx, cfg, n_q, n_kv, q, out, kc, vc, st):
        """e4m3 KV pool with per-(token, head) scales: quantising prep kernel, then the split-KV
        kernel reading fp8 rows (decode, verify and prefill chunks alike)."""
        sp = batch.sparse
        if sp is not None and sp.active(attn_idx):
            raise NotImplementedError("sparse page selection reads a bf16 KV pool")
        t = qkv.shape[0]
        d = cfg.head_dim
        ks, vs = pool.k_scale[attn_idx], pool.v_scale[attn_idx]
        N.check(self.lib.trl_attn_prep_fp8(
            qkv.data_ptr(), qkv.stride(0), self._f32(lp["q_norm"]).data_ptr(),
            self._f32(lp["k_norm"]).data_ptr(), batch.positions.data_ptr(),
            batch.slot_mapping.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), ks.data_ptr(),
            vs.data_ptr(), t, n_q, n_kv, d, cfg.rotary_dim, float(cfg.rope_theta), cfg.rms_eps,
            int(cfg.attn_gated), st), "attn_prep_fp8")
        if (self.prefill_attn and batch.max_q_len >= 16 and d == 256 and n_q % n_kv == 0 and n_q // n_kv <= 8
                and not getattr(batch, "keep_steps", 0)):
            N.check(self.lib.trl_attn_prefill_fp8(
                q.data_ptr(), qkv.data_ptr(), qkv.stride(0), kc.data_ptr(), vc.data_ptr(), ks.data_ptr(),
                vs.data_ptr(), batch.block_table.data_ptr(), batch.block_table.stride(0),
                batch.q_start.data_ptr(), batch.q_len.data_ptr(), batch.positions.data_ptr(), out.data_ptr(),
                batch.n_seqs, batch.max_q_len, n_q, n_kv, d, 1.0 / math.sqrt(d), int(cfg.attn_gated), st),
                "attn_prefill_fp8")
            N.count(2)
            return out
        splits = self.attn_splits or self._pick_splits(batch, t, n_kv)
        po = self.ws.get("attn_po", (t * n_q * splits * d,), torch.float32)
        pm = self.ws.get("attn_pm", (t * n_q * splits,), torch.float32)
        pl = self.ws.get("attn_pl", (t * n_q * splits,), torch.float32)
        N.check(self.lib.trl_attn_paged_fp8(
            q.data_ptr(), qkv.data_ptr(), qkv.stride(0), kc.data_ptr(), vc.data_ptr(), ks.data_ptr(),
            vs.data_ptr(), batch.block_table.data_ptr(), batch.block_table.stride(0),
            batch.seq_ids.data_ptr(), batch.positions.data_ptr(), po.data_ptr(), pm.data_ptr(),
            pl.data_ptr(), out.data_ptr(), t, n_q, n_kv, d, splits, 1.0 / math.sqrt(d),
            int(cfg.attn_gated), st), "attn_paged_fp8")
        N.count(2 + (1 if splits > 1 else 0))
        return out

    def _pick_splits(self, batch, t: int, n_kv: int, keys: int = 32) -> int:
        """Enough CTAs to fill the GPU when few tokens attend to long contexts; a split covers at
        least ``keys`` keys (scalar kernel: 32 = four keys per warp; tensor-core kernel: one 64-key
        tile)."""
        longest = max(batch.host_kv_len) if batch.host_kv_len else 1
        if keys >= 64:
            # tensor-core kernel: one CTA is resident per SM (its K / V ring takes the shared memory), so
            # one wave of CTAs: more splits than that only queue behind the first wave
            if t * n_kv >= self.sms:
                return 1
            return max(1, min(self.sms // max(1, t * n_kv), 64, (longest + keys - 1) // keys))
        if t * n_kv >= self.sms:
            return 1
        want = max(1, self.sms // max(1, t * n_kv))
        return max(1, min(want, 32, (longest + keys - 1) // keys))

    @staticmethod
    def _tokens_per_group(batch, t: int, g: int) -> int:
        """Rows of one sequence that may share a tile of the tensor-core decode kernel: a divisor of the
        (uniform) rows per sequence with ``rows * g <= 16``; 1 when the batch is ragged."""
        w = batch.max_q_len
        if w <= 1 or t != batch.n_seqs * w:
            return 1
        best = 1
        for c in range(1, w + 1):
            if w % c == 0 and c * g <= 16:
                best = c
        return best

    def gdn(self, inp, lp, batch, spool, gdn_idx, cfg, nk, nv):
        self.flush()
        t = inp.shape[0]
        d = cfg.gdn_head_dim
        f32 = torch.float32
        qn = self.ws.get("gdn_qn", (t * nk * d,), f32)
        kn = self.ws.get("gdn_kn", (t * nk * d,), f32)
        vc = self.ws.get("gdn_vc", (t * nv * d,), f32)
        g = self.ws.get("gdn_g", (t * nv,), f32)
        beta = self.ws.get("gdn_b", (t * nv,), f32)
        osc = self.ws.get("gdn_o", (t * nv * d,), f32)
        out = self.ws.get("act", (t, nv * d), torch.bfloat16)
        states, ring = spool.states, spool.ring
        s_l = states[:, gdn_idx]
        r_l = ring[:, gdn_idx]
        keep = batch.keep_flags if batch.keep_steps else None
        if self.gdn_fused_decode and keep is None and t == batch.n_seqs and batch.max_q_len == 1 \
                and nv % nk == 0 and d in (64, 128):
            # decode tick: one launch per layer (state prefetched before the dependency wait, prep,
            # step and gated norm in one kernel)
            N.check(self.lib.trl_gdn_decode(
                inp.data_ptr(), inp.stride(0), self._f32(lp["conv"]).data_ptr(),
                self._f32(lp["dt_bias"]).data_ptr(), self._f32(lp["a_log"]).data_ptr(),
                self._f32(lp["gdn_norm"]).data_ptr(), s_l.data_ptr(), spool.cur.data_ptr(), r_l.data_ptr(),
                batch.positions.data_ptr(), batch.q_start.data_ptr(), batch.state_slots.data_ptr(),
                states.stride(0), states.stride(2), ring.stride(0), out.data_ptr(), batch.n_seqs, nk, nv, d,
                cfg.gdn_conv, cfg.rms_eps, N.stream()), "gdn_decode")
            N.count()
            return out
        N.check(self.lib.trl_gdn(
            inp.data_ptr(), inp.stride(0), self._f32(lp["conv"]).data_ptr(),
            self._f32(lp["dt_bias"]).data_ptr(), self._f32(lp["a_log"]).data_ptr(),
            self._f32(lp["gdn_norm"]).data_ptr(), s_l.data_ptr(), spool.cur.data_ptr(), r_l.data_ptr(),
            batch.positions.data_ptr(), batch.seq_ids.data_ptr(), batch.q_start.data_ptr(),
            batch.q_len.data_ptr(), batch.state_slots.data_ptr(), N.ptr(keep),
            states.stride(0), states.stride(2), ring.stride(0),
            qn.data_ptr(), kn.data_ptr(), vc.data_ptr(), g.data_ptr(), beta.data_ptr(), osc.data_ptr(),
            out.data_ptr(), t, batch.n_seqs, nk, nv, d, cfg.gdn_conv, spool.planes, cfg.rms_eps,
            N.stream()), "gdn")
        N.count(2)
        return out

    def lm_head(self, x, norm_w, w, eps):
        self.settle()
        m = x.shape[0]
        n = w.shape[0]
        logits = self.ws.get("logits", (m, n), torch.float32)
        if m <= GEMV_MAX_M or (m <= 16 and isinstance(w, torch.Tensor) and w.dtype == torch.bfloat16):
            # bf16 head: up to 16 rows share one pass over the vocabulary matrix (tensor-core GEMV)
            self._gemv(x.contiguous(), w, logits, norm_w=self._f32(norm_w), eps=eps, epi=EPI_STORE_F32)
        else:
            xc = x.contiguous()
            if (isinstance(w, NVFP4Tensor) and self.use_tc_gemm) or isinstance(w, FP8BlockTensor):
                self._linear(xc, w, logits, norm_w=self._f32(norm_w), eps=eps, epi=EPI_STORE_F32)
            else:
                h = self._rmsnorm(xc, norm_w, eps, name="h_head")
                hb = self.ws.get("head_bf16", (m, n), torch.bfloat16)
                torch.matmul(h, (w if isinstance(w, torch.Tensor) else w.dequant().to(torch.bfloat16)).t(), out=hb)
                logits.copy_(hb)
        return logits   # vocab-parallel under TP: [M, V_local]

    def full_logits(self, logits):
        """Full-vocabulary logits (gathers the vocab shards under TP)."""
        self.flush()
        if self.comm is not None and self.comm.world > 1:
            full = self.comm.all_gather_logits(logits)
            return full[..., :self.vocab] if self.vocab else full
        return logits

    def quest_select(self, q, kcache, table_early, k: int):
        """Indices (ascending, int64) of the ``k`` early pages with the largest Quest upper bound for the
        token whose prepared query rows are ``q [n_q, D]``: one scoring kernel that reads each page's K rows
        once (min / max per dimension in registers) and one radix-select kernel; ``None`` for shapes the
        kernels do not take (the caller then scores with torch)."""
        n = int(table_early.numel())
        n_kv, d = kcache.shape[1], kcache.shape[-1]
        if d != 256 or kcache.dtype != torch.bfloat16 or q.dtype != torch.bfloat16 or n == 0 or k <= 0:
            return None
        self.flush()
        scores = self.ws.get("quest_scores", (n,), torch.float32)
        tab = table_early.to(torch.int32).contiguous()
        N.check(self.lib.trl_quest_scores(q.contiguous().data_ptr(), kcache.data_ptr(), tab.data_ptr(), scores.data_ptr(),
                                          n, q.shape[0], n_kv, d, N.stream()), "quest_scores")
        sel = torch.empty(min(k, n), dtype=torch.int64, device=kcache.device)
        N.check(self.lib.trl_topk_pages(scores.data_ptr(), n, k, sel.data_ptr(), N.stream()), "topk_pages")
        N.count(2)
        return sel

    def index_select(self, indexer, layer: int, q, kcache, table_early, k: int):
        """The learned indexer's selection on the device: page mean keys by one kernel that reads each K
        page once, the indexer's two small projections as library GEMMs, scores and the ascending top-k
        by kernels.  ``None`` for shapes the kernels do not take."""
        n = int(table_early.numel())
        n_kv, d = kcache.shape[1], kcache.shape[-1]
        if d != 256 or kcache.dtype != torch.bfloat16 or n == 0 or k <= 0:
            return None
        self.flush()
        tab = table_early.to(torch.int32).contiguous()
        pooled = self.ws.get("index_pooled", (n, n_kv * d), torch.float32)
        N.check(self.lib.trl_page_mean(kcache.data_ptr(), tab.data_ptr(), pooled.data_ptr(), n, n_kv, d, N.stream()), "page_mean")
        k_idx = (pooled @ indexer.wk[layer].float()).contiguous()                 # [n, H * dim]
        q_idx = (q.float().reshape(-1) @ indexer.wq[layer].float()).contiguous()   # [H * dim]
        scores = self.ws.get("quest_scores", (n,), torch.float32)
        N.check(self.lib.trl_index_scores(q_idx.data_ptr(), k_idx.data_ptr(), scores.data_ptr(), n, indexer.heads,
                                          indexer.dim, N.stream()), "index_scores")
        sel = torch.empty(min(k, n), dtype=torch.int64, device=kcache.device)
        N.check(self.lib.trl_topk_pages(scores.data_ptr(), n, k, sel.data_ptr(), N.stream()), "topk_pages")
        N.count(3)
        return sel

    def spec_accept(self, tok, batch, cur, pack) -> None:
        """Greedy acceptance of a verify tick on the device: ``pack[:B*W]`` gets the argmax tokens,
        ``pack[B*W:]`` the number of drafts each sequence's trunk reproduced, and ``cur`` (the GDN pool's
        current-plane index) is set to it for every sequence of the tick."""
        self.flush()
        b = batch.n_seqs
        w = batch.n_tokens // b
        N.check(self.lib.trl_spec_accept(tok.data_ptr(), batch.token_ids.data_ptr(), batch.q_len.data_ptr(),
                                         batch.state_slots.data_ptr(), cur.data_ptr(), pack.data_ptr(), b, w,
                                         N.stream()), "spec_accept")
        N.count()

    def argmax(self, logits):
        self.flush()
        m, v = logits.shape
        if self.comm is not None and self.comm.world > 1:
            v_valid = (self.vocab or v * self.comm.world) - self.comm.rank * v
            return self.comm.argmax(self, logits, v_valid)
        out = self.ws.get("argmax", (m,), torch.int32)
        scratch = self.ws.get("argmax_scratch", (m * 128,), torch.float32)
        N.check(self.lib.trl_argmax(logits.data_ptr(), logits.stride(0), m, v, out.data_ptr(), scratch.data_ptr(),
                                    N.stream()), "argmax")
        N.count(2)
        return out

    def sample_rows(self, logits: torch.Tensor, rows, seeds, temps, top_ks=None, top_ps=None):
        """Seeded sampling of the listed logits rows on the device: plain temperature sampling, or
        with per-row ``top_ks`` (0 = off) / ``top_ps`` (>= 1 = off) the top-k / nucleus sampler.
        One pinned staging block and one host-to-device copy carry all per-row arguments, one
        kernel draws every row, one device-to-host copy brings tokens and log-probabilities back.
        Returns ``(tokens, logprobs)`` as Python lists."""
        self.flush()
        import numpy as np
        n = len(rows)
        nucleus = top_ks is not None and any(k or p < 1.0 for k, p in zip(top_ks, top_ps))
        pin = getattr(self, "_samp_pin", None)
        if pin is None or pin.numel() < 8 * n:
            pin = self._samp_pin = torch.empty(max(8 * n, 1024), dtype=torch.int32).pin_memory()
        a = pin.numpy()          # int32 words: [seeds 2n][rows n][1/T n][top_k n][top_p n] | [tokens n][logprobs n]
        a[:2 * n].view(np.int64)[:] = np.fromiter((s & 0x7FFFFFFFFFFFFFFF for s in seeds), dtype=np.int64, count=n)
        a[2 * n:3 * n] = np.asarray(rows, dtype=np.int32)
        a[3 * n:4 * n].view(np.float32)[:] = (1.0 / np.asarray(temps, dtype=np.float64)).astype(np.float32)
        a[4 * n:5 * n] = np.asarray(top_ks, dtype=np.int32) if nucleus else 0
        a[5 * n:6 * n].view(np.float32)[:] = np.asarray(top_ps, dtype=np.float32) if nucleus else 1.0
        dev = torch.empty(8 * n, dtype=torch.int32, device=self.device)
        dev[:6 * n].copy_(pin[:6 * n], non_blocking=True)
        base = dev.data_ptr()
        seeds_p, rows_p, it_p, k_p, p_p = base, base + 8 * n, base + 12 * n, base + 16 * n, base + 20 * n
        tok_p, lp_p = base + 24 * n, base + 28 * n
        lg = logits if logits.dtype == torch.float32 else logits.float()
        if nucleus:
            N.check(self.lib.trl_sample_nucleus(lg.data_ptr(), lg.stride(0), rows_p, seeds_p, it_p, k_p, p_p,
                                                tok_p, lp_p, n, lg.shape[1], N.stream()), "sample_nucleus")
        else:
            N.check(self.lib.trl_sample_softmax(lg.data_ptr(), lg.stride(0), rows_p, seeds_p, it_p, tok_p, lp_p, n,
                                                lg.shape[1], N.stream()), "sample_softmax")
        N.count()
        pin[6 * n:8 * n].copy_(dev[6 * n:], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return a[6 * n:7 * n].tolist(), a[7 * n:8 * n].view(np.float32).tolist()

    # ---- training / maintenance kernels ------------------------------------------------------
    def quantize_nvfp4_(self, w: torch.Tensor, dst: NVFP4Tensor, keep_tscale: bool = False) -> None:
        """Re-pack ``w`` (fp32 or bf16 ``[N, K]``) into ``dst`` in place."""
        n, k = w.shape
        tmp = self.ws.get("amax_tmp", (1,), torch.float32)
        dt = {torch.float32: 0, torch.bfloat16: 1}[w.dtype]
        N.check(self.lib.trl_quant_nvfp4(w.data_ptr(), dt, n, k, dst.wq.data_ptr(), dst.scale.data_ptr(),
                                         dst.tscale.data_ptr(), tmp.data_ptr(), int(keep_tscale), N.stream()),
                "quant_nvfp4")
        N.count(4)

    def quantize_new(self, w: torch.Tensor) -> NVFP4Tensor:
        """Quantise a full ``[N, K]`` fp32 / bf16 tensor into a fresh NVFP4 tensor (kernel)."""
        n, k = w.shape
        dst = NVFP4Tensor(torch.empty(n, k // 2, dtype=torch.uint8, device=self.device),
                          torch.empty(n, k // 16, dtype=torch.float8_e4m3fn, device=self.device),
                          torch.empty(1, dtype=torch.float32, device=self.device))
        self.quantize_nvfp4_(w.contiguous(), dst)
        return dst

    def read_device_error(self, clear: bool = True):
        """``(code, a, b, c)`` of the device error word: non-zero code when a bounded wait of a kernel
        (a peer's partial rows, an mbarrier) ran out since the last read.  Synchronises the stream."""
        torch.cuda.current_stream(self.device).synchronize()
        return N.read_error(clear)

    def device_alive(self) -> bool:
        """Synchronising probe: False when the context no longer answers (sticky error).  The engine
        loop polls it and exits the process on False so a supervisor restarts it.
        Parity: ``Backend.device_alive`` (``tilerl_kernels/backend.py:442-465``)."""
        try:
            t = torch.zeros(1, device=self.device)
            t.add_(1)
            torch.cuda.synchronize(self.device)
            return bool(t.item() == 1.0)
        except RuntimeError:
            return False

    def refresh_weight(self, w: NVFP4Tensor) -> None:
        """Bring the GEMM's tile-contiguous copies of a rewritten weight up to date (in place)."""
        from .gemm_tc import sf_tiled, w_stream, wq_tiled
        if getattr(w, "wq_tiled", None) is not None:
            wq_tiled(w)
        if getattr(w, "sf_tiled", None) is not None:
            sf_tiled(w)
        if getattr(w, "w_stream", None) is not None:
            w_stream(w)

    def dequantize_nvfp4(self, w: NVFP4Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        n, k = w.shape
        if out is None:
            out = torch.empty(n, k, dtype=torch.bfloat16, device=self.device)
        N.check(self.lib.trl_dequant_nvfp4(w.wq.data_ptr(), w.scale.data_ptr(), w.tscale.data_ptr(),
                                           out.data_ptr(), n, k, N.stream()), "dequant_nvfp4")
        N.count()
        return out

    def adamw_step(self, p, m, v, g, *, lr, betas, eps, wd, step, gscale=1.0, p_bf16=None) -> None:
        N.check(self.lib.trl_adamw(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), N.ptr(p_bf16),
                                   p.numel(), lr, betas[0], betas[1], eps, wd, step, gscale, N.stream()), "adamw")
        N.count()
