"""ZeRO-3 for the full-parameter training path: fp32 master weights, Adam moments and
gradients are sharded over the data-parallel group; a layer's working weights exist in full
only while that layer runs.

* A *unit* is one decoder layer (all of its trainable tensors, flattened and padded to a
  multiple of the world size) plus one unit for everything outside the layers.
* Forward (the tape's checkpointed ``forward_dense``): ``pre_layer(i)`` gathers unit ``i`` and
  prefetches the next one (on a side stream on CUDA), ``post_layer(i)`` drops it again.
  Backward replays a layer, so ``pre_layer(i)`` gathers once more and prefetches ``i - 1``.
* ``on_grad`` receives each leaf gradient as soon as the layer's backward has produced it;
  when a unit is complete its flat gradient is reduce-scattered with the 1/world scale and the
  cast to fp32 fused, accumulated into the local gradient shard, and the unit is dropped.
* ``step`` clips by the global norm (one all-reduce of a scalar) and runs AdamW on the shards.
* ``state_dict`` / ``load_state_dict`` are per rank (sharded checkpoint): master shard, both
  moments, step count.

The collectives go through a small comm object: :class:`TorchComm` (torch.distributed; gloo on
CPU, NCCL on CUDA) or :class:`P2PComm` (hand-written kernels over NVLink peer memory, see
``csrc/zero.cu``).  With ``group=None`` the world is 1 and both collectives are copies.

The reference has no ZeRO/FSDP (its data parallelism replicates parameters and all-reduces
every gradient: ``packages/tilerl-kernels/src/tilerl_kernels/backend.py:216-247``,
``src/tilerl/train.py:254-302``); this is the sharded replacement for that path.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

_LAYER = re.compile(r"^(?:master\.)?L(\d+)\.")


class TorchComm:
    """Collectives through torch.distributed.  gloo has no reduce-scatter, so that one is an
    all-reduce followed by a slice there."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.backend = dist.get_backend(group) if group is not None else "none"

    def grad_buffer(self, numel: int, dtype, device) -> torch.Tensor:
        return torch.zeros(numel, dtype=dtype, device=device)

    def all_gather(self, shard: torch.Tensor, full: torch.Tensor, stream=None) -> None:
        """``shard`` may be the fp32 master shard: it is cast to ``full``'s dtype on the way."""
        shard = shard.to(full.dtype)
        if self.world == 1:
            full.copy_(shard)
            return
        if self.backend == "nccl":
            dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
        else:
            parts = list(full.view(self.world, -1).unbind(0))
            dist.all_gather(parts, shard.contiguous(), group=self.group)

    def reduce_scatter(self, full: torch.Tensor, shard_out: torch.Tensor, scale: float, accumulate: bool) -> None:
        n = shard_out.numel()
        if self.world == 1:
            red = full.float() * scale
        elif self.backend == "nccl":
            tmp = torch.empty(n, dtype=full.dtype, device=full.device)
            dist.reduce_scatter_tensor(tmp, full.contiguous(), group=self.group)
            red = tmp.float() * scale
        else:
            buf = full.float().clone()
            dist.all_reduce(buf, group=self.group)
            red = buf[self.rank * n:(self.rank + 1) * n] * scale
        if accumulate:
            shard_out.add_(red)
        else:
            shard_out.copy_(red)

    def all_reduce_scalar(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t


@dataclass
class _Unit:
    index: int
    names: List[str] = field(default_factory=list)
    shapes: List[Tuple[int, ...]] = field(default_factory=list)
    offsets: List[int] = field(default_factory=list)
    numel: int = 0
    padded: int = 0
    full: Optional[torch.Tensor] = None        # gathered working weights (flat), None when dropped
    grad: Optional[torch.Tensor] = None        # flat gradient being filled by on_grad
    pending: int = 0                           # leaves of this unit still to arrive
    prefetched: bool = False


class Zero3:
    def __init__(self, model, group=None, *, lr: float = 1e-6, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, max_norm: float = 1.0, work_dtype: Optional[torch.dtype] = None,
                 comm=None, mode: str = "full"):
        self.model = model
        self.comm = comm or TorchComm(group)
        self.world, self.rank = self.comm.world, self.comm.rank
        self.lr, self.betas, self.eps, self.wd, self.max_norm = lr, betas, eps, weight_decay, max_norm
        self.params = model.trainable(mode)
        dev = next(iter(self.params.values())).device
        self.device = dev
        self.work_dtype = work_dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32)
        n_layers = model.cfg.n_layers
        self.units: List[_Unit] = [_Unit(i) for i in range(n_layers + 1)]
        self.where: Dict[int, Tuple[int, int]] = {}     # id(param) -> (unit, slot)
        for name, p in self.params.items():
            m = _LAYER.match(name)
            u = self.units[int(m.group(1)) if m else n_layers]
            self.where[id(p)] = (u.index, len(u.names))
            u.names.append(name)
            u.shapes.append(tuple(p.shape))
            u.offsets.append(u.numel)
            u.numel += p.numel()
        self.master: List[torch.Tensor] = []
        self.gshard: List[Optional[torch.Tensor]] = []
        self.m: List[torch.Tensor] = []
        self.v: List[torch.Tensor] = []
        self.t = 0
        with torch.no_grad():
            for u in self.units:
                q = self.world * getattr(self.comm, "align", 1)
                u.padded = (u.numel + q - 1) // q * q
                flat = torch.zeros(max(u.padded, q), dtype=torch.float32, device=dev)
                for name, off in zip(u.names, u.offsets):
                    p = self.params[name]
                    flat[off:off + p.numel()] = p.detach().float().reshape(-1)
                n = flat.numel() // self.world
                self.master.append(flat[self.rank * n:(self.rank + 1) * n].clone())
                self.gshard.append(None)
                self.m.append(torch.zeros(n, dtype=torch.float32, device=dev))
                self.v.append(torch.zeros(n, dtype=torch.float32, device=dev))
                self._drop(u)
        self._last_layer = -1
        self.side = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        self.stats = dict(gathers=0, reduce_scatters=0, prefetch_hits=0)

    # ---- memory ---------------------------------------------------------------------------
    def shard_bytes(self) -> int:
        """Persistent bytes on this rank: master + two moments + gradient shards."""
        return sum(4 * t.numel() * 4 for t in self.master)

    def _drop(self, u: _Unit) -> None:
        empty = torch.empty(0, dtype=self.work_dtype, device=self.device)
        for name in u.names:
            self.params[name].data = empty
        u.full, u.prefetched = None, False

    def _gather(self, u: _Unit) -> None:
        if u.full is not None or not u.names:
            return
        shard = self.master[u.index]                 # fp32; the comm casts it into the working dtype
        full = torch.empty(shard.numel() * self.world, dtype=self.work_dtype, device=self.device)
        self.comm.all_gather(shard, full)
        u.full = full
        self.stats["gathers"] += 1
        for name, off, shape in zip(u.names, u.offsets, u.shapes):
            n = 1
            for s in shape:
                n *= s
            self.params[name].data = full[off:off + n].view(shape)

    def _prefetch(self, i: int) -> None:
        if not 0 <= i < len(self.units) - 1:
            return
        u = self.units[i]
        if u.full is not None:
            return
        if self.side is None:
            return                      # CPU: nothing to overlap with; gather on demand
        self.side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.side):
            self._gather(u)
        u.prefetched = True

    # ---- hooks used by forward_dense ----------------------------------------------------------
    def pre_model(self) -> None:
        self._gather(self.units[-1])
        self._last_layer = -1

    def pre_layer(self, i: int) -> None:
        u = self.units[i]
        if u.prefetched and self.side is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.side)
            self.stats["prefetch_hits"] += 1
            u.prefetched = False
        self._gather(u)
        step = 1 if i > self._last_layer else -1
        self._last_layer = i
        self._prefetch(i + step)

    def post_layer(self, i: int) -> None:
        """End of a layer's forward (not of its backward replay: the gradients still need it)."""
        self._drop(self.units[i])

    # ---- gradients ------------------------------------------------------------------------------
    def on_grad(self, param: torch.Tensor, grad: torch.Tensor) -> None:
        loc = self.where.get(id(param))
        if loc is None:
            return
        u = self.units[loc[0]]
        if u.grad is None:
            n_flat = self.master[u.index].numel() * self.world
            if u.index == len(self.units) - 1:
                # tensors outside the layers get their gradients at both ends of the backward; they
                # must not sit in the area the layers (one in flight at a time) take turns in
                u.grad = torch.zeros(n_flat, dtype=self.work_dtype, device=self.device)
            else:
                u.grad = self.comm.grad_buffer(n_flat, self.work_dtype, self.device)
            u.pending = len(u.names)
        off = u.offsets[loc[1]]
        u.grad[off:off + grad.numel()] = grad.reshape(-1).to(self.work_dtype)
        u.pending -= 1
        if u.pending == 0:
            self._reduce(u)

    def _reduce(self, u: _Unit) -> None:
        acc = self.gshard[u.index] is not None
        if not acc:
            self.gshard[u.index] = torch.empty_like(self.master[u.index])
        self.comm.reduce_scatter(u.grad, self.gshard[u.index], 1.0 / self.world, acc)
        self.stats["reduce_scatters"] += 1
        u.grad = None
        if u.index != len(self.units) - 1:
            self._drop(u)

    def flush(self) -> None:
        """Reduce units whose leaves did not all receive a gradient (unused tensors)."""
        staged = getattr(self.comm, "is_staged", lambda t: False)
        # the unit that borrowed the comm's staging area goes first: the others pass through it
        for u in sorted(self.units, key=lambda u: not (u.grad is not None and staged(u.grad))):
            if u.grad is not None:
                self.stats["flushed"] = self.stats.get("flushed", 0) + 1
                self._reduce(u)
        wait = getattr(self.comm, "wait", None)
        if wait is not None:
            wait()                 # the reduced shards are read next (norm, optimizer)

    # ---- optimizer --------------------------------------------------------------------------------
    def grad_norm(self) -> float:
        sq = torch.zeros(1, dtype=torch.float64, device=self.device)
        for g in self.gshard:
            if g is not None:
                sq += g.double().pow(2).sum()
        return float(self.comm.all_reduce_scalar(sq).sqrt())

    def step(self, grads=None, lr: Optional[float] = None) -> float:
        """AdamW on the shards.  ``grads`` (the dict a non-streaming caller collected) is fed
        through ``on_grad`` first so both call styles work.  Returns the global gradient norm."""
        if grads:
            for name, g in grads.items():
                self.on_grad(self.params[name], g)
        self.flush()
        norm = self.grad_norm()
        clip = min(1.0, self.max_norm / (norm + 1e-6)) if self.max_norm else 1.0
        self.t += 1
        lr = self.lr if lr is None else lr
        b1, b2 = self.betas
        fused = None
        if self.device.type == "cuda":
            from ..ops import native as N
            if N.available():
                fused = N
        for i, g in enumerate(self.gshard):
            if g is None:
                continue
            m, v, w = self.m[i], self.v[i], self.master[i]
            if fused is not None and g.dtype == torch.float32 and g.is_contiguous():
                # one kernel per unit: the clip coefficient rides along as the gradient scale, no
                # temporaries of the shard's size
                fused.check(fused.lib().trl_adamw(w.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), None,
                                                  w.numel(), lr, b1, b2, self.eps, self.wd, self.t, clip,
                                                  fused.stream()), "adamw")
                fused.count()
                self.gshard[i] = None
                continue
            g = g * clip
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            mhat = m / (1 - b1 ** self.t)
            vhat = v / (1 - b2 ** self.t)
            if self.wd:
                w.mul_(1 - lr * self.wd)
            w.sub_(lr * mhat / (vhat.sqrt() + self.eps))
            self.gshard[i] = None
        self._drop(self.units[-1])
        self.check_device()
        return norm

    def check_device(self) -> None:
        """Raise ``CommTimeout`` when a bounded wait of a peer-memory collective ran out during the
        step (the kernels record it in the device error word and return)."""
        if self.device.type == "cuda" and getattr(self.comm, "device_waits", False):
            from ..ops import native as N
            from .health import raise_on_device_error
            torch.cuda.synchronize(self.device)
            raise_on_device_error(lambda: N.read_error(True))

    # ---- whole-model views --------------------------------------------------------------------------
    def gather_all(self) -> None:
        """Materialise every unit (evaluation, export, re-quantisation for the rollout engine)."""
        for u in self.units:
            self._gather(u)

    def drop_all(self) -> None:
        for u in self.units:
            self._drop(u)

    def unit_tensors(self, i: int) -> Dict[str, torch.Tensor]:
        u = self.units[i]
        self._gather(u)
        return {n: self.params[n] for n in u.names}

    # ---- sharded checkpoint ----------------------------------------------------------------------------
    def state_dict(self) -> Dict[str, object]:
        return dict(rank=self.rank, world=self.world, t=self.t, master=[t.cpu() for t in self.master],
                    m=[t.cpu() for t in self.m], v=[t.cpu() for t in self.v],
                    numel=[u.numel for u in self.units])

    def load_state_dict(self, sd) -> None:
        if sd["world"] != self.world or sd["rank"] != self.rank:
            raise ValueError(f"shard of rank {sd['rank']}/{sd['world']} loaded on rank {self.rank}/{self.world}")
        if list(sd["numel"]) != [u.numel for u in self.units]:
            raise ValueError("checkpoint was written for a different parameter layout")
        self.t = int(sd["t"])
        for dst, src in ((self.master, sd["master"]), (self.m, sd["m"]), (self.v, sd["v"])):
            for d, s in zip(dst, src):
                d.copy_(s.to(d.device))
        self.drop_all()


class P2PComm:
    """ZeRO collectives by the kernels of ``csrc/zero.cu`` over NVLink peer memory.

    One symmetric region per rank, exported with CUDA IPC, with the staging areas: the
    parameter shard in the working dtype (the fp32 master shard is cast straight into it) and TWO
    areas for the full flat gradient of a unit (``grad_buffer`` hands them out in turn, so the
    backward writes gradients where the peers will read them -- no staging copy -- and the
    backward of the next layer fills one area while the reduce-scatter of the previous layer still
    reads the other).  Every collective is enqueued on this object's own stream, in program order
    on every rank, so at most one of them runs per GPU and a prefetch never meets a
    reduce-scatter half way.  The caller's stream is joined before every collective; after an
    all-gather it is joined again (the parameters are about to be used), after a reduce-scatter it
    is NOT: the reduced shard is awaited by ``wait()`` (``Zero3.flush``) or by the event of its
    area, so the reduction overlaps the backward that follows."""
    align = 8          # elements: shards are moved in 16-byte vectors
    device_waits = True      # its kernels wait on peers with a bound and record a give-up on the device

    def __init__(self, group, device, cap_bytes: int):
        """``cap_bytes``: the largest unit's flat gradient in the working dtype."""
        import ctypes

        from ..ops import native as N
        from .symm import _DevMem
        self.group, self.device = group, torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.backend = "p2p"
        self.lib = N.lib()
        for name, sig in {"trl_zero_allgather": [N.P, N.I, N.I, ctypes.c_long, ctypes.c_long, N.P, N.P],
                          "trl_zero_reduce_scatter": [N.P, N.I, N.I, ctypes.c_long, ctypes.c_long, N.I, ctypes.c_float,
                                                      N.P, N.I, N.P],
                          }.items():
            N.register(name, sig)
        self.lib.trl_zero_data_offset.restype = ctypes.c_size_t
        off = self.lib.trl_zero_data_offset()
        self.cap_grad = (cap_bytes + 255) // 256 * 256
        self.cap_shard = (cap_bytes // self.world + 4096 + 255) // 256 * 256
        self.off_shard, self.off_grad = off, off + self.cap_shard
        self.off_grads = [self.off_grad, self.off_grad + self.cap_grad]
        self.nbytes = self.off_grad + 2 * self.cap_grad
        p = ctypes.c_void_p()
        N.check(self.lib.trl_symm_alloc(self.nbytes, ctypes.byref(p)), "symm_alloc")
        self.local_ptr = p.value
        handle = (ctypes.c_ubyte * 64)()
        N.check(self.lib.trl_ipc_get(self.local_ptr, handle), "ipc_get")
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.ptrs: List[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local_ptr)
                continue
            q = ctypes.c_void_p()
            N.check(self.lib.trl_ipc_open((ctypes.c_ubyte * 64).from_buffer_copy(h), ctypes.byref(q)), "ipc_open")
            self.ptrs.append(q.value)
        self.table = (ctypes.c_void_p * 8)(*(self.ptrs + [None] * (8 - self.world)))
        self.mem = torch.as_tensor(_DevMem(self.local_ptr, self.nbytes), device=self.device)
        self.stage_shard = self.mem[self.off_shard:self.off_shard + self.cap_shard]
        self.stage_grads = [self.mem[o:o + self.cap_grad] for o in self.off_grads]
        self.stage_grad = self.stage_grads[0]
        self._lent = [False, False]            # area handed to a unit's backward, not yet reduced
        self._read_done = [None, None]         # event: the last reduce-scatter has read the area
        self._next_area = 0
        self.stream = torch.cuda.Stream(device=self.device)
        self._check = N.check
        dist.barrier(group=group)

    def _enter(self):
        cur = torch.cuda.current_stream(self.device)
        self.stream.wait_stream(cur)
        return cur

    def grad_buffer(self, numel: int, dtype, device) -> torch.Tensor:
        """A gradient staging area as a zeroed tensor (ordinary memory if the unit is larger than an
        area or both areas are lent out)."""
        nb = numel * torch.empty(0, dtype=dtype).element_size()
        k = self._next_area
        if self._lent[k]:
            k ^= 1
        if nb > self.cap_grad or self._lent[k]:
            return torch.zeros(numel, dtype=dtype, device=device)
        self._lent[k] = True
        self._next_area = k ^ 1
        if self._read_done[k] is not None:           # the reduce-scatter that last used this area has read it
            torch.cuda.current_stream(self.device).wait_event(self._read_done[k])
        buf = self.stage_grads[k][:nb].view(dtype)
        buf.zero_()
        return buf

    def _area_of(self, t: torch.Tensor) -> int:
        for k, a in enumerate(self.stage_grads):
            if t.data_ptr() == a.data_ptr():
                return k
        return -1

    def is_staged(self, t: torch.Tensor) -> bool:
        return self._area_of(t) >= 0

    def wait(self) -> None:
        """Join the caller's stream with everything enqueued here (the reduced shards are read next)."""
        torch.cuda.current_stream(self.device).wait_stream(self.stream)

    def all_gather(self, shard: torch.Tensor, full: torch.Tensor, stream=None) -> None:
        nb = shard.numel() * full.element_size()
        if nb > self.cap_shard or nb % 16:
            raise ValueError(f"shard of {nb} B does not fit the staging area ({self.cap_shard} B) or is not 16-byte sized")
        cur = self._enter()
        with torch.cuda.stream(self.stream):
            self.stage_shard[:nb].view(full.dtype).copy_(shard)          # cast (fp32 master -> working dtype) and stage
            self._check(self.lib.trl_zero_allgather(self.table, self.rank, self.world, self.off_shard, nb,
                                                    full.data_ptr(), self.stream.cuda_stream), "zero_allgather")
        shard.record_stream(self.stream)
        full.record_stream(self.stream)
        cur.wait_stream(self.stream)

    def reduce_scatter(self, full: torch.Tensor, shard_out: torch.Tensor, scale: float, accumulate: bool) -> None:
        nb = full.numel() * full.element_size()
        if nb > self.cap_grad or shard_out.numel() % 8 or full.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("gradient does not fit the staging area, or shard not a multiple of 8 elements")
        self._enter()
        k = self._area_of(full)
        with torch.cuda.stream(self.stream):
            if k < 0:
                k = 0 if not self._lent[0] else 1
                if self._lent[k]:
                    # both areas are lent to units whose backward is still running: cannot happen with
                    # at most two layers in flight
                    raise RuntimeError("both gradient staging areas are lent out while another unit is reduced")
                self.stage_grads[k][:nb].copy_(full.contiguous().view(torch.uint8))   # ordered on this stream
                full.record_stream(self.stream)
            else:
                self._lent[k] = False
            self._check(self.lib.trl_zero_reduce_scatter(self.table, self.rank, self.world, self.off_grads[k],
                                                         shard_out.numel(), int(full.dtype == torch.bfloat16),
                                                         float(scale), shard_out.data_ptr(), int(accumulate),
                                                         self.stream.cuda_stream), "zero_reduce_scatter")
            ev = torch.cuda.Event()
            ev.record(self.stream)
            self._read_done[k] = ev
        shard_out.record_stream(self.stream)

    def all_reduce_scalar(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                self.lib.trl_ipc_close(p)
        self.lib.trl_symm_free(self.local_ptr)
