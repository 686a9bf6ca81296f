"""Parameter-sharded data parallelism (ZeRO-3 / FULL_SHARD), the regime of the reference's
``train_distributed.py`` (reference: train_distributed.py:275-333 wraps every ``TransformerBlock`` in
FSDP FULL_SHARD with bf16 all-gather / reduce-scatter, optional CPU offload, AdamW only).

The default data-parallel plan of this framework (:mod:`.zero`) keeps the bf16 parameters replicated
and shards only gradients and optimizer state, which is the faster choice while the model fits in a
GPU.  This module is the memory-lean alternative for models that do not fit:

* a *unit* is one ``TransformerBlock`` (plus one root unit for embeddings, final norm and heads);
  its parameters are laid out back to back in one flat vector, padded to a multiple of the world size;
  each rank keeps 1/world of it (the *shard*) plus fp32 AdamW moments for that shard - optionally in
  pinned host memory (``cpu_offload``);
* before a unit runs (forward, and again before its backward) its flat vector is all-gathered into
  one of two rotating device buffers and the module's parameters are pointed at views of it; after
  the unit's forward, and after its gradients are complete, the parameters are released again;
* when the last gradient of a unit arrives, the unit's gradients are flattened, reduce-scattered
  (mean) into the rank's gradient shard, and dropped;
* the step clips by the global norm of all gradient shards and runs AdamW on the shards (one fused
  kernel per unit on a GPU).

Transport.  ``nccl``/``gloo``: library all-gather and reduce-scatter.  ``p2p`` (the default on NVLink
machines): the two rotating parameter buffers and the two gradient staging buffers live in symmetric
memory; a gather is this library's push kernel (every rank stores its shard into all peers' buffers
through peer pointers, or once through the NVLink switch's multicast address) between two flag
barriers, and the reduce-scatter is the peer-load kernel of the replicated plan.  The GEMMs of a unit
then read the gathered weights from local memory only.

Overlap.  On a GPU the gather of the unit that runs next (the following block in the forward pass, the
preceding one in the backward pass) is issued on a side stream as soon as its buffer is free, and the
reduce-scatter of a finished unit runs on a second side stream, so that both hide behind the compute
of the neighbouring unit.  ``KMOE_FSDP_OVERLAP=0`` keeps everything on the compute stream.

Expert parallelism.  Tensors already split over an expert-parallel group (``_kmoe_expert_parallel``) are
not sharded again: they stay resident, and a second pool (``zero.ShardedDataParallel(expert_params=True)``
over the ranks that hold the same experts) reduces and steps them.  ``zero.ParallelPlan([this plan, that
pool])`` drives both through ``reduce / owned_sq_norm / scale_owned / finish`` with one global-norm clip -
the combination the reference cannot run (its expert-parallel layer has no backward and clashes with its
FSDP wrapping, moe_arch/model/sparse_moe.py:540-603).

Muon needs whole matrices on one rank and is therefore offered by the replicated plan only, as in the
reference, whose distributed launcher is AdamW-only (train_distributed.py:336-397).
"""
from __future__ import annotations

import contextlib
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class _Unit:
    def __init__(self, name: str, module: Optional[torch.nn.Module], params: List[torch.nn.Parameter],
                 names: List[str]):
        self.name, self.module, self.params, self.names = name, module, params, names
        self.offsets: List[int] = []
        self.total = 0
        self.padded = 0
        self.shard: Optional[torch.Tensor] = None          # this rank's slice of the flat parameters
        self.grad_shard: Optional[torch.Tensor] = None     # accumulated, reduced gradient slice
        self.m: Optional[torch.Tensor] = None              # AdamW moments (fp32)
        self.v: Optional[torch.Tensor] = None
        self.gathered = False                              # parameters point into the buffer
        self.inflight = False                              # gather enqueued, parameters not yet pointed
        self.ready = None                                  # event: the enqueued gather has finished
        self.buffer: Optional[torch.Tensor] = None
        self.slot = -1                                     # which rotating buffer (-1: the root's own)
        self.index = -1                                    # position among the block units
        self.pending = 0
        self.reduced = False


class FullyShardedDataParallel:
    """``model`` must already be on its device in its training dtype.  ``unit_cls``: module class whose
    instances become units (default: the framework's ``TransformerBlock``)."""

    def __init__(self, model: torch.nn.Module, group=None, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.01, unit_cls=None, cpu_offload: bool = False,
                 broadcast_from_rank0: bool = True, transport: Optional[str] = None,
                 overlap: Optional[bool] = None):
        if unit_cls is None:
            from ..models.layers import TransformerBlock
            unit_cls = TransformerBlock
        self.model, self.group = model, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.cpu_offload = cpu_offload
        first = next(p for p in model.parameters() if p.requires_grad)
        self.device, self.dtype = first.device, first.dtype
        self.backend = dist.get_backend(group) if dist.is_initialized() else "none"
        self.hyper = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        self.step_count = 0
        self.early_gathers = 0                  # gathers issued ahead of their use (diagnostic)
        self._in_backward = False

        # ---- units
        seen = set()
        self.units: List[_Unit] = []
        for mname, mod in model.named_modules():
            if isinstance(mod, unit_cls):
                ps, ns = [], []
                for n, p in mod.named_parameters():
                    if p.requires_grad and id(p) not in seen:
                        seen.add(id(p))
                        if getattr(p, "_kmoe_expert_parallel", False):
                            continue            # already split over the expert-parallel group: its own pool steps it
                        ps.append(p)
                        ns.append(f"{mname}.{n}")
                if ps:
                    self.units.append(_Unit(mname, mod, ps, ns))
        rp, rn = [], []
        for n, p in model.named_parameters():
            if p.requires_grad and id(p) not in seen and not getattr(p, "_kmoe_expert_parallel", False):
                seen.add(id(p))
                rp.append(p)
                rn.append(n)
        self.root = _Unit("", None, rp, rn) if rp else None
        all_units = self.units + ([self.root] if self.root else [])
        align = 8 * self.world
        for u in all_units:
            off = 0
            for p in u.params:
                assert p.dtype == self.dtype, "parameters must share one dtype"
                p._kmoe_shape, p._kmoe_numel = tuple(p.shape), p.numel()
                u.offsets.append(off)
                off += _round_up(p.numel(), 8)
            u.total, u.padded = off, _round_up(off, align)
        # ---- transport and streams
        cuda = self.device.type == "cuda"
        self.transport = self._pick_transport(transport)
        if overlap is None:
            overlap = cuda and self.world > 1 and os.environ.get("KMOE_FSDP_OVERLAP", "1") != "0"
        self.overlap = bool(overlap)            # without a GPU the early gathers simply run in program order
        self._ag_stream = torch.cuda.Stream(self.device) if self.overlap and cuda else None
        self._rs_stream = torch.cuda.Stream(self.device) if self.overlap and cuda and not cpu_offload else None
        # ---- buffers: two rotating ones for the block units (parameters, and gradients on their way to
        # the reduce-scatter), permanent ones for the root unit
        big = max([u.padded for u in self.units], default=0)
        self._big = big
        self._sym = None
        if self.transport == "p2p" and big > 0:
            from .p2p import SymmetricBuffers
            try:
                self._sym = SymmetricBuffers(2 * big, self.dtype, self.device, group,
                                             barrier_timeout_s=float(os.environ.get("KMOE_FSDP_BARRIER_S", "20")))
            except Exception as e:
                if transport == "p2p":
                    raise
                print(f"[kmoe] symmetric-memory set-up failed ({type(e).__name__}: {e}); using NCCL collectives",
                      flush=True)
            flag = torch.tensor([1.0 if self._sym is not None else 0.0], device=self.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)        # every rank takes the same branch
            if flag.item() == 0.0:
                self._sym = None
        if self._sym is None and self.transport == "p2p":
            self.transport = self.backend
        if self._sym is not None:
            self._pool = [self._sym.param[:big], self._sym.param[big:]]
            self._grad_bufs = [self._sym.grad[:big], self._sym.grad[big:]]
        else:
            self._pool = [torch.zeros(big, dtype=self.dtype, device=self.device) for _ in range(2 if big else 0)]
            self._grad_bufs = [torch.zeros(big, dtype=self.dtype, device=self.device) for _ in range(2 if big else 0)]
        # grids of the two peer kernels while they run beside compute kernels (0 = whole device)
        self._ag_blocks = int(os.environ.get("KMOE_FSDP_AG_BLOCKS", "32")) if self.overlap else 0
        self._rs_blocks = int(os.environ.get("KMOE_FSDP_RS_BLOCKS", "148"))
        self._p2p_rs = os.environ.get("KMOE_FSDP_P2P_RS", "1") != "0"
        self._red_bufs = ([torch.empty(big // self.world, dtype=self.dtype, device=self.device) for _ in range(2)]
                          if (self._sym is None or not self._p2p_rs) and self.backend == "nccl" and big else None)
        self._rs_done = [None, None]
        self._rs_slot = 0
        for i, u in enumerate(self.units):
            u.index, u.slot = i, i % 2
            u.buffer = self._pool[u.slot][: u.padded]
        if self.root:
            self.root.buffer = torch.zeros(self.root.padded, dtype=self.dtype, device=self.device)
            self._root_grad = torch.zeros(self.root.padded, dtype=self.dtype, device=self.device)
        self._placeholder = torch.empty(0, dtype=self.dtype, device=self.device)
        # ---- shards from the initial parameters (rank 0's values when asked to broadcast)
        store = torch.device("cpu") if cpu_offload else self.device
        for u in all_units:
            flat = torch.zeros(u.padded, dtype=self.dtype, device=self.device)
            for p, off in zip(u.params, u.offsets):
                flat[off: off + p.numel()].copy_(p.data.reshape(-1))
            if broadcast_from_rank0 and self.world > 1:
                dist.broadcast(flat, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            chunk = u.padded // self.world
            sl = flat[self.rank * chunk: (self.rank + 1) * chunk]
            u.shard = sl.to(store).clone()
            if cpu_offload and torch.cuda.is_available():
                u.shard = u.shard.pin_memory()
            u.grad_shard = torch.zeros(chunk, dtype=torch.float32, device=store)
            u.m = torch.zeros(chunk, dtype=torch.float32, device=store)
            u.v = torch.zeros(chunk, dtype=torch.float32, device=store)
            for p in u.params:
                p.data = self._placeholder
                p.grad = None
            del flat
        # ---- hooks
        for u in self.units:
            u.module.register_forward_pre_hook(lambda m, a, u=u: self._before_forward(u))
            u.module.register_forward_hook(lambda m, a, o, u=u: self._after_forward(u))
            u.module.register_full_backward_pre_hook(lambda m, g, u=u: self._before_backward(u))
        model.register_forward_pre_hook(lambda m, a: self._begin_forward())
        for u in all_units:
            for p in u.params:
                p.register_post_accumulate_grad_hook(lambda p, u=u: self._grad_arrived(u))
        self.optimizer = _ShardOptimizer(self)
        self._arm()

    def _pick_transport(self, transport: Optional[str]) -> str:
        if self.world == 1:
            return "none"
        if transport in ("nccl", "gloo"):
            return self.backend
        want = transport or os.environ.get("KMOE_FSDP_TRANSPORT", "p2p")
        if want == "p2p" and self.backend == "nccl" and self.dtype == torch.bfloat16:
            from .p2p import p2p_available
            if p2p_available(self.device):
                return "p2p"
        if transport == "p2p":
            raise RuntimeError("p2p transport asked for: it needs bf16 parameters on GPUs of an NCCL group "
                               "with symmetric memory")
        return self.backend

    @contextlib.contextmanager
    def _side(self, stream):
        """Run the body on ``stream`` after everything the compute stream holds so far (no-op without one)."""
        if stream is None:
            yield
            return
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            yield

    # ------------------------------------------------------------------ gather / release
    def _launch_gather(self, u: _Unit) -> None:
        """Enqueue the all-gather of ``u``'s flat parameters into its buffer (on the gather stream when
        overlapping).  The buffer's previous user must already be enqueued on the compute stream."""
        if u.gathered or u.inflight:
            return
        chunk = u.padded // self.world
        with self._side(self._ag_stream):
            shard = u.shard.to(self.device, non_blocking=True) if u.shard.device != self.device else u.shard
            out = u.buffer.data                 # alias with its own version counter: autograd never sees the write
            if self.world == 1:
                out.copy_(shard)
            elif self._sym is not None and u is not self.root:
                # one kernel stores this rank's shard into every rank's buffer (its own included); the first
                # barrier says that every rank is done with what the buffer held before, the second that
                # every store has landed
                off = u.slot * self._big + self.rank * chunk
                self._sym.barrier(2)
                self._sym.all_gather_range(off, chunk, src=shard, max_blocks=self._ag_blocks)
                self._sym.barrier(2)
            else:
                dist.all_gather_into_tensor(out, shard.contiguous(), group=self.group)
            if self._ag_stream is not None:
                u.ready = torch.cuda.Event()
                u.ready.record(self._ag_stream)
        u.inflight = True

    def _gather(self, u: _Unit) -> None:
        if u.gathered:
            return
        self._launch_gather(u)
        if u.ready is not None:
            torch.cuda.current_stream(self.device).wait_event(u.ready)
            u.ready = None
        for p, off in zip(u.params, u.offsets):
            p.data = u.buffer[off: off + p._kmoe_numel].view(p._kmoe_shape)
        u.gathered, u.inflight = True, False
        from ..ops import mxfp8
        mxfp8.invalidate_weight_cache()         # the same addresses now hold another unit's weights

    def _prefetch(self, index: int) -> None:
        """Start gathering block ``index`` if its buffer is free (its other users are neither resident nor
        on their way)."""
        if not self.overlap or not (0 <= index < len(self.units)):
            return
        u = self.units[index]
        for o in self.units[u.slot::2]:
            if o is not u and (o.gathered or o.inflight):
                return
        self.early_gathers += 1
        self._launch_gather(u)

    def _release(self, u: _Unit) -> None:
        if not u.gathered or u is self.root:
            return
        for p in u.params:
            p.data = self._placeholder
        u.gathered = False

    def _drop_all(self) -> None:
        """Forget every gathered or in-flight copy (the shards have changed under them)."""
        if self._ag_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._ag_stream)
        for u in self.units:
            self._release(u)
            u.inflight, u.ready = False, None
        if self.root is not None:
            self.root.gathered, self.root.inflight, self.root.ready = False, False, None

    def _begin_forward(self) -> None:
        if self._in_backward:                   # a new micro-batch: its gradients are reduced and added again
            self._arm()
        self._in_backward = False
        if self.root is not None:
            self._gather(self.root)
        self._prefetch(0)

    def _before_forward(self, u: _Unit) -> None:
        self._gather(u)
        if not self._in_backward:
            self._prefetch(u.index + 1)

    def _after_forward(self, u: _Unit) -> None:
        # a forward that runs inside the backward pass (activation recomputation) keeps the unit for its
        # backward; otherwise the buffer goes to the unit two positions on, and this unit's backward
        # gathers it again into the same addresses (which tensors saved by autograd still point at)
        if not self._in_backward:
            self._release(u)

    def _before_backward(self, u: _Unit) -> None:
        self._in_backward = True
        # the other unit of this buffer may still be resident
        for o in self.units[u.slot::2]:
            if o is not u and o.gathered:
                self._release(o)
        self._gather(u)
        self._prefetch(u.index - 1)

    # ------------------------------------------------------------------ gradients
    def _grad_arrived(self, u: _Unit) -> None:
        u.pending -= 1
        if u.pending <= 0 and not u.reduced and u is not self.root:
            self._reduce_unit(u)
            self._release(u)

    def _reduce_unit(self, u: _Unit) -> None:
        """Flatten the unit's gradients, average them over the ranks, add this rank's slice to its
        gradient shard.  Block units alternate between two staging buffers so that the collective of one
        (on the reduce stream when overlapping) runs beside the backward pass of the next."""
        chunk = u.padded // self.world
        cur = torch.cuda.current_stream(self.device) if self.device.type == "cuda" else None
        if u is self.root:
            slot, g = -1, self._root_grad
        else:
            slot = self._rs_slot
            self._rs_slot ^= 1
            g = self._grad_bufs[slot][: u.padded]
            if self._rs_done[slot] is not None:            # the collective that last read this buffer
                cur.wait_event(self._rs_done[slot])
                self._rs_done[slot] = None
        g.zero_()
        for p, off in zip(u.params, u.offsets):
            if p.grad is not None:
                g[off: off + p._kmoe_numel].copy_(p.grad.reshape(-1))
                p.grad = None
        side = self._rs_stream if slot >= 0 else None
        with self._side(side):
            if self.world == 1:
                red = g
            elif self._sym is not None and slot >= 0 and self._p2p_rs:
                off = slot * self._big + self.rank * chunk
                self._sym.barrier(3)                       # every rank's gradients are in place
                self._sym.reduce_scatter_mean(off, chunk, None, self._rs_blocks if side is not None else 0)
                self._sym.barrier(3)                       # every rank has read what it needs from this buffer
                red = g[self.rank * chunk: (self.rank + 1) * chunk]
            elif self.backend == "nccl":
                red = (self._red_bufs[slot][:chunk] if slot >= 0 and self._red_bufs is not None
                       else torch.empty(chunk, dtype=g.dtype, device=g.device))
                dist.reduce_scatter_tensor(red, g, op=dist.ReduceOp.AVG, group=self.group)
            else:                                   # gloo has no reduce-scatter
                dist.all_reduce(g, group=self.group)
                red = g[self.rank * chunk: (self.rank + 1) * chunk] / self.world
            if u.grad_shard.device == red.device:
                u.grad_shard.add_(red)
            else:
                u.grad_shard.add_(red.to(u.grad_shard.device).float())
            if side is not None:
                self._rs_done[slot] = torch.cuda.Event()
                self._rs_done[slot].record(side)
        u.reduced = True

    # ------------------------------------------------------------------ step
    def set_sync(self, flag: bool) -> None:
        pass                                    # every micro-batch is reduced, like the reference's FSDP use

    def _arm(self) -> None:
        for u in self.units + ([self.root] if self.root else []):
            u.pending = len(u.params)
            u.reduced = False

    def _fused_adamw_ok(self) -> bool:
        if self.device.type != "cuda" or self.cpu_offload or self.dtype != torch.bfloat16:
            return False
        if os.environ.get("KMOE_FSDP_FUSED_ADAMW", "1") == "0":
            return False
        from ..ops.loader import require_ext
        require_ext()                           # a GPU run without the extension is an error, not a slow path
        return True

    # The step in the four phases a ``ParallelPlan`` drives (so that this plan and the pool of the
    # expert-parallel tensors clip by one global norm): reduce, owned_sq_norm, scale_owned, finish.
    def reduce(self) -> None:
        for u in self.units + ([self.root] if self.root else []):     # the root unit, and units whose
            if not u.reduced:                                          # parameters got no gradient
                self._reduce_unit(u)
                self._release(u)
        if self._rs_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._rs_stream)

    def owned_sq_norm(self) -> torch.Tensor:
        all_units = self.units + ([self.root] if self.root else [])
        norms = torch._foreach_norm([u.grad_shard for u in all_units])
        return torch.stack([n.to(self.device) for n in norms]).pow(2).sum()

    def scale_owned(self, coef) -> None:
        self._coef = coef

    def reduce_clip_and_step(self, optimizer=None, max_norm: Optional[float] = 1.0) -> torch.Tensor:
        self.reduce()
        sq = self.owned_sq_norm().reshape(1)
        if self.world > 1:
            dist.all_reduce(sq, group=self.group)
        total = sq.sqrt()[0]
        self._coef = None
        if max_norm is not None and max_norm > 0:
            self._coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
        self.finish()
        return total

    def finish(self) -> None:
        all_units = self.units + ([self.root] if self.root else [])
        coef, self._coef = getattr(self, "_coef", None), None
        self.step_count += 1
        h = self.hyper
        b1, b2 = h["betas"]
        bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
        if self._fused_adamw_ok():
            # one kernel per unit: clip, moments, decoupled weight decay, bf16 parameters written in place
            from ..ops import cuda_ops
            cdev = coef.reshape(1).float() if coef is not None else None
            for u in all_units:
                n = u.shard.numel()
                torch.ops.kmoe.p2p_adamw_allgather([u.shard.data_ptr()], u.grad_shard.to(torch.bfloat16), u.m, u.v,
                                                   0, 1, 0, n, h["lr"], b1, b2, h["eps"], h["weight_decay"],
                                                   self.step_count, cdev, 0)
                cuda_ops._count()
                u.grad_shard.zero_()
        else:
            for u in all_units:
                g = u.grad_shard
                if coef is not None:
                    g = g * coef.to(g.device)
                u.m.mul_(b1).add_(g, alpha=1 - b1)
                u.v.mul_(b2).addcmul_(g, g, value=1 - b2)
                p32 = u.shard.float()
                p32.mul_(1 - h["lr"] * h["weight_decay"])
                p32.addcdiv_(u.m / bc1, (u.v / bc2).sqrt_().add_(h["eps"]), value=-h["lr"])
                u.shard.copy_(p32.to(u.shard.dtype))
                u.grad_shard.zero_()
        self._drop_all()                        # new values: everything is gathered again at its next use
        self._arm()

    # ------------------------------------------------------------------ whole-model access
    def full_state_dict(self, to_cpu: bool = True) -> Dict[str, torch.Tensor]:
        """Every parameter in full, gathered unit by unit (call on all ranks)."""
        out: Dict[str, torch.Tensor] = {}
        for u in self.units + ([self.root] if self.root else []):
            was = u.gathered
            self._gather(u)
            for p, n in zip(u.params, u.names):
                t = p.data.detach().clone()
                out[n] = t.cpu() if to_cpu else t
            if not was:
                self._release(u)
        # tied parameters appear under every name they have in the model (e.g. lm_heads.0 = embedding)
        primary = {id(p): n for u in self.units + ([self.root] if self.root else []) for p, n in zip(u.params, u.names)}
        for n, p in self.model.named_parameters(remove_duplicate=False):
            if n not in out and id(p) in primary:
                out[n] = out[primary[id(p)]]
        return out

    def load_full_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        for u in self.units + ([self.root] if self.root else []):
            flat = torch.zeros(u.padded, dtype=self.dtype, device=self.device)
            for p, n, off in zip(u.params, u.names, u.offsets):
                flat[off: off + p._kmoe_numel].copy_(sd[n].reshape(-1).to(self.device, self.dtype))
            chunk = u.padded // self.world
            u.shard.copy_(flat[self.rank * chunk: (self.rank + 1) * chunk].to(u.shard.device))
        self._drop_all()

    def shard_state_dict(self) -> Dict:
        return {"rank": self.rank, "world": self.world, "step": self.step_count,
                "units": {u.name: {"shard": u.shard, "m": u.m, "v": u.v}
                          for u in self.units + ([self.root] if self.root else [])}}

    def load_shard_state_dict(self, sd: Dict) -> None:
        assert sd["world"] == self.world and sd["rank"] == self.rank, "shard file belongs to another rank layout"
        self.step_count = sd["step"]
        for u in self.units + ([self.root] if self.root else []):
            s = sd["units"][u.name]
            u.shard.copy_(s["shard"])
            u.m.copy_(s["m"])
            u.v.copy_(s["v"])
        self._drop_all()

    def param_bytes_per_rank(self) -> int:
        es = torch.empty(0, dtype=self.dtype).element_size()
        return sum(u.shard.numel() for u in self.units + ([self.root] if self.root else [])) * es


class _ShardOptimizer:
    """Optimizer-shaped handle (``param_groups`` for LR schedulers, state dicts)."""

    def __init__(self, plan: FullyShardedDataParallel):
        self.plan = plan
        self.param_groups = [plan.hyper]
        plan.hyper.setdefault("params", [])

    def state_dict(self):
        return self.plan.shard_state_dict()

    def load_state_dict(self, sd):
        self.plan.load_shard_state_dict(sd)

    def zero_grad(self, set_to_none: bool = True):
        for u in self.plan.units + ([self.plan.root] if self.plan.root else []):
            u.grad_shard.zero_()

    def step(self):
        raise RuntimeError("step through FullyShardedDataParallel.reduce_clip_and_step")
